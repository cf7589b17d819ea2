// Causal GQA flash-attention forward for sm_100a (head_dim 64): TMA -> smem, QK^T and PV on tcgen05 with
// S/P/O in tensor memory, online softmax by one thread per query row.
//
// A persistent kernel, two CTAs per SM. A CTA owns one softmax group (128 threads, one per query row of a 128-row tile) and
// draws (batch, head, query tile) work items from a device-wide counter, heavy tiles first. Its other warpgroup holds the
// single-thread roles: a TMA producer, a thread that issues the score products and a thread that issues the PV products;
// it gives up most of its registers (`setmaxnreg`) so that a softmax thread can hold its 128 scores.
//   TMEM (256 columns per CTA): S [0,128) fp32 scores; P [128,192) bf16 probabilities (fed to the PV MMA straight from
//   tensor memory); O [192,256).
// P has its own columns so that the scores of tile j+1 can be issued as soon as the softmax group has pulled tile j
// into registers (`s_free`), long before P(j) exists: the MMA round trip is off the softmax group's critical path.
// The running maximum is updated lazily: probabilities are taken relative to a stale maximum and O is
// rescaled in TMEM only when a row's maximum grows by more than 2^8, so the common iteration has no
// accumulator traffic. Replaces the cuDNN SDPA graph of the reference
// (parameter-golf-rs/crates/pg-kernels/cpp/cudnn_sdpa.cu:312-362) and its SIMT fallback
// (pg-kernels/src/gpu_kernels.rs:4751-4843).
#include "common.cuh"
#include "pgb.h"
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "tma_host.h"

namespace pgb {

constexpr int AT_BM = 128;   // query rows per tile
constexpr int AT_BN = 128;   // keys per tile
constexpr int AT_HD = 64;
constexpr int AT_TILE_BYTES = 128 * AT_HD * 2;   // 16 KB: one Q, K or V tile

struct AttnFwdParams {
  int B, S, H, Hkv, n_qt;
  float scale_log2;
  __nv_bfloat16* Y;
  long long ldy;
  float* lse;
  int* status;
  unsigned* sched;                   // {next work item, CTAs finished}: both zero between launches
  // Optional second output z_h = y_h - (<y_h, v> / (|v|^2 + eps)) v with the token's own value vector of the head's KV group
  // (exclusive self attention); null when the layer does not use it.
  __nv_bfloat16* Z;
  long long ldz;
  const __nv_bfloat16* V;
  long long ldv;
  float xsa_eps;
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));      // one half-rate instruction instead of two
  return r;
}

// Between work items nothing is torn down: the producer is already fetching the next item's Q/K/V while the last tiles of
// the current one are in flight, the next item's first score product is issued as soon as the last scores of this item have
// been pulled into registers, and an item's output is read out of tensor memory and stored while the next item's first tile
// is being processed, when its last PV product has long completed. Work items are drawn from a counter because the two CTAs
// of an SM do not run at the same speed. K and V tiles are fetched once per head (not once per KV head); the heads of a KV
// group are neighbours in the item order, so the repeated fetches hit L2.
//   warps 0-3: TMA producer (warp 0), score-product issuer (warp 1), PV issuer (warp 2), one idle; warps 4-7: softmax, one
//   thread per query row.
//   TMEM (256 columns): S [0,128) fp32 scores, P [128,192) bf16 probabilities, O [192,256).
//   Shared memory: 2 Q tiles (this item's and the next one's), a ring of 2 K tiles (a K tile is free once its score product
//   has completed) and a ring of 2 V tiles.
constexpr int A1_THREADS = 256;
constexpr int A1_KST = 2, A1_VST = 2;
constexpr int A1_SMEM = (2 + A1_KST + A1_VST) * AT_TILE_BYTES + 1024 + 256;
// Register budget: 2 CTAs x 256 threads => 128 registers per thread at launch. `setmaxnreg.inc` can only take what the
// role warps released; a request for more never completes, so the two sides must balance exactly.
constexpr int A1_REG_LAUNCH = 128, A1_REG_ROLE = 40, A1_REG_SOFTMAX = 216;
static_assert(128 * A1_REG_ROLE + 128 * A1_REG_SOFTMAX == A1_THREADS * A1_REG_LAUNCH, "setmaxnreg: released and requested registers must balance");
static_assert(2 * (A1_SMEM + 1024) <= 227 * 1024, "two CTAs must fit the shared memory of one SM");

struct FwdItem {
  int qt, b, head, kvh, n_kv, row0;
};
__device__ __forceinline__ FwdItem fwd_item(const AttnFwdParams& p, int item) {
  FwdItem w;
  const int per_qt = p.B * p.H;
  w.qt = p.n_qt - 1 - item / per_qt;         // heavy (long KV range) query tiles first
  const int rem = item % per_qt;
  w.b = rem / p.H;
  w.head = rem % p.H;                        // the heads of a KV group are neighbours, so their K/V fetches share L2 lines
  w.kvh = w.head / (p.H / p.Hkv);
  w.n_kv = w.qt + 1;
  w.row0 = w.b * p.S + w.qt * AT_BM;
  return w;
}

// Work counters of the persistent kernel, one pair per launch in flight: consecutive launches rotate through the slots, and the
// last CTA of a launch zeroes its pair again. Launches that run concurrently on one device must therefore be fewer than the
// number of slots apart in issue order (the engine issues all attention calls on one stream).
constexpr int A1_SCHED_SLOTS = 64;
__device__ unsigned g_fwd_sched[A1_SCHED_SLOTS * 2];

__global__ void __launch_bounds__(A1_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // two tiles: the next item's Q lands while this item's score products still read theirs
  uint8_t* sK = smem + 2 * AT_TILE_BYTES;
  uint8_t* sV = sK + A1_KST * AT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + A1_VST * AT_TILE_BYTES);
  uint64_t* q_full = bars;                 // 2: Q of the item has landed
  uint64_t* q_empty = bars + 2;            // 2: the item's last score product has completed, its Q tile may be overwritten
  uint64_t* k_full = bars + 4;             // KST
  uint64_t* k_empty = k_full + A1_KST;     // KST
  uint64_t* v_full = k_empty + A1_KST;     // VST
  uint64_t* v_empty = v_full + A1_VST;     // VST
  uint64_t* s_full = v_empty + A1_VST;     // scores in tensor memory
  uint64_t* p_full = s_full + 1;           // probabilities in tensor memory
  uint64_t* o_full = p_full + 1;           // one commit per PV
  uint64_t* s_free = o_full + 1;           // scores pulled into registers
  uint64_t* sched_full = s_free + 1;       // 2: the slot holds the next work item
  uint64_t* sched_empty = sched_full + 2;  // 2: every consumer has read the slot
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sched_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched_item = abort_flag + 1;   // 2 slots; -1 ends the list

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = p.n_qt * p.B * p.H;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    for (int s = 0; s < A1_KST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < A1_VST; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);                  // one arrival per softmax warp
    mbar_init(o_full, 1);
    mbar_init(s_free, 4);
    for (int s = 0; s < 2; ++s) { mbar_init(&sched_full[s], 1); mbar_init(&sched_empty[s], 6); }   // readers: two issuers, four softmax warps
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(A1_REG_ROLE));
    if (warp == 0 && lane == 0) {
      // ---- TMA producer ----
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0, ic = 0, q_issued = 0;
      bool ok = true;
      for (;; ++ic) {
        // work items are handed out by a device-wide counter: the two CTAs of an SM do not run at the same speed (the warp
        // scheduler favours one of them), and a fixed split would leave the fast half of the grid idle at the end
        const int slot = ic & 1;
        if (!mbar_wait(&sched_empty[slot], ((ic >> 1) & 1) ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, -3)) { ok = false; break; }
        int item = (int)atomicAdd(p.sched, 1u);
        if (item >= n_items) item = -1;
        sched_item[slot] = item;
        mbar_arrive(&sched_full[slot]);
        if (item < 0) break;
        const FwdItem w = fwd_item(p, item);
        if (!mbar_wait(&q_empty[slot], ((ic >> 1) & 1) ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, -1)) { ok = false; break; }
        mbar_expect_tx(&q_full[slot], AT_TILE_BYTES);
        tma_load_2d(sQ + slot * AT_TILE_BYTES, &map_q, &q_full[slot], w.head * AT_HD, w.row0);
        ++q_issued;
        for (int j = 0; j < w.n_kv; ++j) {
          if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, j)) { ok = false; break; }
          mbar_expect_tx(&k_full[ks], AT_TILE_BYTES);
          tma_load_2d(sK + ks * AT_TILE_BYTES, &map_k, &k_full[ks], w.kvh * AT_HD, w.b * p.S + j * AT_BN);
          if (++ks == A1_KST) { ks = 0; kph ^= 1; }
          if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, j)) { ok = false; break; }
          mbar_expect_tx(&v_full[vs], AT_TILE_BYTES);
          tma_load_2d(sV + vs * AT_TILE_BYTES, &map_v, &v_full[vs], w.kvh * AT_HD, w.b * p.S + j * AT_BN);
          if (++vs == A1_VST) { vs = 0; vph ^= 1; }
        }
      }
      if (!ok) {
        // copies still in flight must land before the CTA's shared memory is given back: the most recent phase of every
        // barrier a copy was issued on (stages below the ring position are in the current phase, the rest in the previous one)
        for (int s = 0; s < 2; ++s) {
          const uint32_t n = (q_issued + 1 - s) / 2;       // Q loads issued on this slot
          if (n > 0) mbar_drain(&q_full[s], (n - 1) & 1);
        }
        for (int s = 0; s < A1_KST; ++s) mbar_drain(&k_full[s], (s < ks) ? kph : (kph ^ 1));
        for (int s = 0; s < A1_VST; ++s) mbar_drain(&v_full[s], (s < vs) ? vph : (vph ^ 1));
      }
    } else if (warp == 1 && lane == 0) {
      // ---- score products: S = Q K^T as soon as K has landed and the previous scores have been pulled into registers ----
      constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);    // both operands K-major
      int ks = 0;
      uint32_t kph = 0, it = 0, ic = 0;
      bool ok = true;
      for (; ok; ++ic) {
        const int slot = ic & 1;
        if (!mbar_wait(&sched_full[slot], (ic >> 1) & 1, abort_flag, p.status, ST_WAIT_FULL, -3)) break;
        const int item = sched_item[slot];
        mbar_arrive(&sched_empty[slot]);
        if (item < 0) break;
        const int n_kv = fwd_item(p, item).n_kv;
        if (!mbar_wait(&q_full[slot], (ic >> 1) & 1, abort_flag, p.status, ST_WAIT_FULL, -1)) break;
        const uint32_t sq = smem_u32(sQ + slot * AT_TILE_BYTES);
        for (int j = 0; j < n_kv; ++j, ++it) {
          if (!mbar_wait(&k_full[ks], kph, abort_flag, p.status, ST_WAIT_FULL, j)) { ok = false; break; }
          if (it > 0 && !mbar_wait(s_free, (it - 1) & 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY, j)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sk = smem_u32(sK + ks * AT_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < AT_HD / 16; ++k)
            umma_ss(tmem_base, make_smem_desc(sq + k * 32, 16, 1024), make_smem_desc(sk + k * 32, 16, 1024), IDESC_S, k > 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(&k_empty[ks]);
          if (++ks == A1_KST) { ks = 0; kph ^= 1; }
        }
        umma_commit(&q_empty[slot]);
      }
    } else if (warp == 2 && lane == 0) {
      // ---- O += P V: its own issuing thread, so that a score product never queues behind a wait for probabilities ----
      constexpr uint32_t IDESC_O = make_idesc_bf16(128, AT_HD, 0, 1);  // A from TMEM, V is N-contiguous
      int vs = 0;
      uint32_t vph = 0, it = 0, ic = 0;
      bool ok = true;
      for (; ok; ++ic) {
        const int slot = ic & 1;
        if (!mbar_wait(&sched_full[slot], (ic >> 1) & 1, abort_flag, p.status, ST_WAIT_FULL, -3)) break;
        const int item = sched_item[slot];
        mbar_arrive(&sched_empty[slot]);
        if (item < 0) break;
        const int n_kv = fwd_item(p, item).n_kv;
        for (int j = 0; j < n_kv; ++j, ++it) {
          if (!mbar_wait(&v_full[vs], vph, abort_flag, p.status, ST_WAIT_FULL, j)) { ok = false; break; }
          // the first product of an item overwrites O; the softmax group reads the previous item's output out of tensor
          // memory before it releases these probabilities
          if (!mbar_wait(p_full, it & 1, abort_flag, p.status, ST_WAIT_MISC, j)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sv = smem_u32(sV + vs * AT_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < AT_BN / 16; ++k)
            umma_ts(tmem_base + 192, tmem_base + 128 + k * 8, make_smem_desc(sv + k * 2048, 8192, 1024), IDESC_O, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(o_full);
          umma_commit(&v_empty[vs]);
          if (++vs == A1_VST) { vs = 0; vph ^= 1; }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(A1_REG_SOFTMAX));
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;             // query row within the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_off;
    const uint32_t tP = tmem_base + 128 + lane_off;
    const uint32_t tO = tmem_base + 192 + lane_off;
    uint32_t it = 0, ic = 0;                       // tiles / items processed by this CTA: the phases of the barriers
    bool ok = true;
    // The output of an item is written while the next item's first tile is in flight: its last PV product has long completed
    // by the time that tile's probabilities are ready, so no wait for the tensor core is exposed between items.
    bool pend = false;
    FwdItem wp = {};
    float m_p = 0.f, l_p = 1.f;
    auto store_out = [&](const uint32_t* o, const FwdItem& w, float m, float lsum) {
      const float inv = 1.f / lsum;
      __nv_bfloat16* yrow = p.Y + (size_t)(w.row0 + r) * p.ldy + w.head * AT_HD;
#pragma unroll
      for (int c = 0; c < 64; c += 8)
        *reinterpret_cast<uint4*>(yrow + c) =
            make_uint4(pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv),
                       pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv),
                       pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv),
                       pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv));
      p.lse[((size_t)w.b * p.H + w.head) * p.S + w.qt * AT_BM + r] = -(m + log2f(lsum));   // negated, log2 domain: what the backward consumes
      if (p.Z != nullptr) {
        // the row's own value vector: the diagonal V tile held it a moment ago, so these 128 bytes come from L2
        const uint4* vp = reinterpret_cast<const uint4*>(p.V + (size_t)(w.row0 + r) * p.ldv + w.kvh * AT_HD);
        uint32_t vv[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 t = __ldg(vp + c);
          vv[4 * c] = t.x; vv[4 * c + 1] = t.y; vv[4 * c + 2] = t.z; vv[4 * c + 3] = t.w;
        }
        float n = p.xsa_eps, dot = 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float2 f = unpack_bf16x2(vv[c]);
          n += f.x * f.x + f.y * f.y;
          dot += __uint_as_float(o[2 * c]) * f.x + __uint_as_float(o[2 * c + 1]) * f.y;
        }
        const float coef = dot * inv / n;
        __nv_bfloat16* zrow = p.Z + (size_t)(w.row0 + r) * p.ldz + w.head * AT_HD;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          uint32_t out[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(vv[c + e]);
            out[e] = pack_bf16x2(__uint_as_float(o[2 * (c + e)]) * inv - coef * f.x, __uint_as_float(o[2 * (c + e) + 1]) * inv - coef * f.y);
          }
          *reinterpret_cast<uint4*>(zrow + 2 * c) = make_uint4(out[0], out[1], out[2], out[3]);
        }
      }
    };
    for (; ok; ++ic) {
      const int slot = ic & 1;
      if (!mbar_wait(&sched_full[slot], (ic >> 1) & 1, abort_flag, p.status, ST_WAIT_FULL, -3)) { ok = false; break; }
      const int item = sched_item[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sched_empty[slot]);
      if (item < 0) break;
      const FwdItem w = fwd_item(p, item);
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < w.n_kv; ++j, ++it) {
        if (!mbar_wait(s_full, it & 1, abort_flag, p.status, ST_WAIT_TMEM_FULL, j)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[128];
        PGB_TMEM_LD32(tS, (s));
        PGB_TMEM_LD32(tS + 32, (s + 32));
        PGB_TMEM_LD32(tS + 64, (s + 64));
        PGB_TMEM_LD32(tS + 96, (s + 96));
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);          // the scores are in registers: the next tile's may overwrite them
        if (j == w.qt) {
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if (c > r) s[c] = 0xff800000u;            // -inf
        }
        float mx8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) mx8[c] = max3(__uint_as_float(s[c]), __uint_as_float(s[8 + c]), __uint_as_float(s[16 + c]));
#pragma unroll
        for (int c = 24; c < 120; c += 16)
#pragma unroll
          for (int e = 0; e < 8; ++e) mx8[e] = max3(mx8[e], __uint_as_float(s[c + e]), __uint_as_float(s[c + 8 + e]));      // 8 independent chains
#pragma unroll
        for (int e = 0; e < 8; ++e) mx8[e] = fmaxf(mx8[e], __uint_as_float(s[120 + e]));
        float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
        mx *= p.scale_log2;
        // lazy running maximum: probabilities stay relative to a stale maximum until a row's maximum has grown by more than 2^8
        const bool need = mx > m_used + 8.0f;
        const bool any_need = __any_sync(0xffffffffu, need);
        float alpha = 1.f;
        if (any_need) {
          const float m_new = need ? mx : m_used;
          alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
        }
        float2 sum2 = make_float2(0.f, 0.f), sum2b = make_float2(0.f, 0.f);
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_used, -m_used);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float2 t = __ffma2_rn(make_float2(__uint_as_float(s[q * 32 + 2 * c]), __uint_as_float(s[q * 32 + 2 * c + 1])), sc2, nm2);
            const float2 pr = make_float2(ex2(t.x), ex2(t.y));
            if (c & 1) sum2b = __fadd2_rn(sum2b, pr); else sum2 = __fadd2_rn(sum2, pr);
            pk[c] = pack_bf16x2(pr.x, pr.y);
          }
          if (q == 0 && it > 0) {
            // The previous PV product reads P and writes O: it must be finished before P is stored again / O rescaled.
            // It was released a whole softmax phase ago, so this wait is normally already satisfied.
            if (!mbar_wait(o_full, (it - 1) & 1, abort_flag, p.status, ST_WAIT_MISC, j)) { ok = false; break; }
            tc_fence_after();
            if (any_need && j > 0) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint32_t o[32];
                PGB_TMEM_LD32(tO + h * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                PGB_TMEM_ST16(tO + h * 32, (o));
                PGB_TMEM_ST16(tO + h * 32 + 16, (o + 16));
              }
            }
          }
          PGB_TMEM_ST16(tP + q * 16, pk);
        }
        if (!ok) break;
        l += (sum2.x + sum2.y) + (sum2b.x + sum2b.y);
        if (j == 0 && pend) {
          // the previous item's O is still in tensor memory (the PV product that overwrites it needs the arrival below)
          uint32_t o[64];
          PGB_TMEM_LD32(tO, (o));
          PGB_TMEM_LD32(tO + 32, (o + 32));
          tmem_wait_ld();
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full);
          store_out(o, wp, m_p, l_p);
          pend = false;
        } else {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full);
        }
      }
      if (!ok) break;
      pend = true;
      wp = w;
      m_p = m_used;
      l_p = l;
    }
    if (ok && pend) {
      if (mbar_wait(o_full, (it - 1) & 1, abort_flag, p.status, ST_WAIT_MISC, -4)) {
        tc_fence_after();
        uint32_t o[64];
        PGB_TMEM_LD32(tO, (o));
        PGB_TMEM_LD32(tO + 32, (o + 32));
        tmem_wait_ld();
        store_out(o, wp, m_p, l_p);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  // the last CTA to leave puts the work counter back for the next launch (every CTA has drawn its end marker by now)
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

static CUtensorMap attn_map(const void* ptr, long long ld, int cols, long long rows) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld * 2};
  uint32_t box[2] = {AT_HD, 128};
  return make_tmap_bf16(ptr, 2, dims, strides, box);
}

void attn_fwd(const void* q, const void* k, const void* v, void* y, float* lse, long long ldq, long long ldk, long long ldv, long long ldy, int B,
              int S, int H, int Hkv, int hd, int* status, cudaStream_t st, void* z, long long ldz, float xsa_eps) {
  if (hd != AT_HD) throw std::runtime_error("attention kernel is specialised for head_dim 64");
  if (S % 128) throw std::runtime_error("attention kernel needs seq_len to be a multiple of 128");
  if (H % Hkv) throw std::runtime_error("num_heads must be divisible by num_kv_heads");
  const long long T = (long long)B * S;
  const CUtensorMap mq = attn_map(q, ldq, H * hd, T), mk = attn_map(k, ldk, Hkv * hd, T), mv = attn_map(v, ldv, Hkv * hd, T);
  AttnFwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.n_qt = S / AT_BM;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  p.Y = (__nv_bfloat16*)y;
  p.ldy = ldy;
  p.lse = lse;
  p.status = status;
  if (z && ((ldz % 8) || (ldv % 8) || (reinterpret_cast<uintptr_t>(z) & 15) || (reinterpret_cast<uintptr_t>(v) & 15)))
    throw std::runtime_error("attention: the second output and the value rows must be 16-byte aligned");
  p.Z = (__nv_bfloat16*)z;
  p.ldz = ldz;
  p.V = (const __nv_bfloat16*)v;
  p.ldv = ldv;
  p.xsa_eps = xsa_eps;
  static bool configured[64] = {};          // the attribute is a per-device property of the kernel
  static unsigned* sched_base[64] = {};
  static std::atomic<unsigned> sched_next{0};     // host threads launching on different streams must not share a slot
  static int sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cached = dev >= 0 && dev < 64;
  if (!cached || !configured[dev]) {
    cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A1_SMEM);
    cudaFuncAttributes fa;
    // the register hand-over inside the kernel is balanced for exactly this launch allocation; anything else would never complete
    if (cudaFuncGetAttributes(&fa, attn_fwd_kernel) != cudaSuccess || fa.numRegs != A1_REG_LAUNCH)
      throw std::runtime_error("attn_fwd_kernel was not built with the register allocation its setmaxnreg hand-over assumes");
  }
  unsigned* base = cached ? sched_base[dev] : nullptr;
  int sms = cached ? sm_count[dev] : 0;
  if (!base || !sms) {
    if (cudaGetSymbolAddress((void**)&base, g_fwd_sched) != cudaSuccess) throw std::runtime_error("attn_fwd: no scheduler counters");
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cached) {
      sched_base[dev] = base;
      sm_count[dev] = sms;
      configured[dev] = true;
    }
  }
  p.sched = base + 2 * (sched_next.fetch_add(1, std::memory_order_relaxed) % A1_SCHED_SLOTS);
  const int grid = std::min(p.n_qt * B * H, 2 * sms);
  attn_fwd_kernel<<<grid, A1_THREADS, A1_SMEM, st>>>(mq, mk, mv, p);
}

}  // namespace pgb
