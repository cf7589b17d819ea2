// Causal GQA flash-attention forward for sm_100a (head_dim 64): TMA -> smem, QK^T and PV on tcgen05 with
// S/P/O in tensor memory, online softmax by one thread per query row.
//
// One CTA handles one 128-row query tile of TWO query heads that share a KV head, so every K/V tile is
// loaded once and used by both. Warp roles (384 threads = three warpgroups): warpgroup 0 holds the TMA producer
// (warp 0) and one MMA-issuing warp per head (warps 1, 2); warpgroups 1 and 2 are the softmax groups of head 0 and
// head 1, one thread per query row. Warpgroup 0 gives up most of its registers (`setmaxnreg`) so that a softmax
// thread can hold its 128 scores and still leave the scheduler room to overlap MUFU, FMA and conversion latencies.
//   TMEM: S0 [0,128) S1 [128,256) fp32 scores; P0 [256,320) P1 [320,384) bf16 probabilities (fed to the PV MMA straight
//         from tensor memory); O0 [384,448) O1 [448,512).
// P has its own columns so that the scores of tile j+1 can be issued as soon as the softmax group has pulled tile j
// into registers (`s_free`), long before P(j) exists: the MMA round trip is off the softmax group's critical path.
// The running maximum is updated lazily: probabilities are taken relative to a stale maximum and O is
// rescaled in TMEM only when a row's maximum grows by more than 2^8, so the common iteration has no
// accumulator traffic. Replaces the cuDNN SDPA graph of the reference
// (parameter-golf-rs/crates/pg-kernels/cpp/cudnn_sdpa.cu:312-362) and its SIMT fallback
// (pg-kernels/src/gpu_kernels.rs:4751-4843).
#include "common.cuh"
#include "pgb.h"
#include <cstdlib>

#include "tma_host.h"

namespace pgb {

constexpr int AT_THREADS = 384;   // warpgroup 0: warp 0 TMA, warps 1 and 2 issue the MMAs of head 0 / head 1, warp 3 idle; warpgroups 1, 2: softmax
constexpr int AT_BM = 128;   // query rows per tile
constexpr int AT_BN = 128;   // keys per tile
constexpr int AT_HD = 64;
constexpr int AT_STAGES = 4;
constexpr int AT_TILE_BYTES = 128 * AT_HD * 2;   // 16 KB: one Q, K or V tile
constexpr int AT_SMEM = (2 + 2 * AT_STAGES) * AT_TILE_BYTES + 1024 + 256;

struct AttnFwdParams {
  int B, S, H, Hkv, n_qt, pairs;     // pairs = ceil(group / 2)
  float scale_log2;
  int head1_delay_clk;               // head start of head 0's softmax group over head 1's, in SM clocks
  __nv_bfloat16* Y;
  long long ldy;
  float* lse;
  int* status;
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

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // 2 tiles
  uint8_t* sKV = smem + 2 * AT_TILE_BYTES;              // stages of {K, V}
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * AT_STAGES) * AT_TILE_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // STAGES
  uint64_t* kv_empty = kv_full + AT_STAGES;
  uint64_t* s_full = kv_empty + AT_STAGES; // 2
  uint64_t* p_full = s_full + 2;           // 2
  uint64_t* o_full = p_full + 2;           // 2: one commit per PV
  uint64_t* s_free = o_full + 2;           // 2: scores pulled into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item: heavy (long KV range) tiles first
  const int per_qt = p.B * p.Hkv * p.pairs;
  const int qt = p.n_qt - 1 - (int)(blockIdx.x / per_qt);
  int rem = (int)(blockIdx.x % per_qt);
  const int b = rem / (p.Hkv * p.pairs);
  rem -= b * p.Hkv * p.pairs;
  const int kvh = rem / p.pairs, pair = rem % p.pairs;
  const int group = p.H / p.Hkv;
  const int head0 = kvh * group + pair * 2;
  const int n_active = min(2, group - pair * 2);
  const int n_kv = qt + 1;
  const int row0 = b * p.S + qt * AT_BM;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], n_active);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&p_full[w], 128);
      mbar_init(&o_full[w], 1);
      mbar_init(&s_free[w], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
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
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, n_active * AT_TILE_BYTES);
      for (int w = 0; w < n_active; ++w) tma_load_2d(sQ + w * AT_TILE_BYTES, &map_q, q_full, (head0 + w) * AT_HD, row0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, j)) { ok = false; break; }
        uint8_t* sk = sKV + stage * 2 * AT_TILE_BYTES;
        mbar_expect_tx(&kv_full[stage], 2 * AT_TILE_BYTES);
        tma_load_2d(sk, &map_k, &kv_full[stage], kvh * AT_HD, b * p.S + j * AT_BN);
        tma_load_2d(sk + AT_TILE_BYTES, &map_v, &kv_full[stage], kvh * AT_HD, b * p.S + j * AT_BN);
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        mbar_drain(q_full, 0);
        for (int s = 0; s < AT_STAGES; ++s) mbar_drain(&kv_full[s], (s < stage) ? phase : (phase ^ 1));
      }
    }
  } else if (warp == 1 || warp == 2) {
    const int w = warp - 1;                     // each head of the pair has its own issuing thread
    if (lane == 0 && w < n_active) {
      constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);    // Q K^T : both K-major
      constexpr uint32_t IDESC_O = make_idesc_bf16(128, AT_HD, 0, 1);  // P V   : A from TMEM, V is N-contiguous
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_WAIT_FULL, -1);
      auto issue_s = [&](int stage) {
        const uint32_t sq = smem_u32(sQ + w * AT_TILE_BYTES);
        const uint32_t sk = smem_u32(sKV + stage * 2 * AT_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k)
          umma_ss(tmem_base + w * 128, make_smem_desc(sq + k * 32, 16, 1024), make_smem_desc(sk + k * 32, 16, 1024), IDESC_S, k > 0 ? 1u : 0u);
        umma_commit(&s_full[w]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag, p.status, ST_WAIT_FULL, 0);
      if (ok) {
        tc_fence_after();
        if (w == 1 && p.head1_delay_clk > 0) {
          // The two softmax groups share the MUFU. Started together they stay in lock step and the unit idles while both
          // load scores and take row maxima; started half a tile period apart, one group's exponentials cover the other's
          // loads, maxima and hand-overs.
          const long long t0 = clock64();
          while (clock64() - t0 < p.head1_delay_clk) {}
        }
        issue_s(0);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        int nstage = stage + 1;
        uint32_t nphase = phase;
        if (nstage == AT_STAGES) { nstage = 0; nphase ^= 1; }
        if (j + 1 < n_kv) {
          if (!mbar_wait(&kv_full[nstage], nphase, abort_flag, p.status, ST_WAIT_FULL, j + 1)) { ok = false; break; }
          // scores of the next tile: only need the current ones to have been pulled into registers
          if (!mbar_wait(&s_free[w], j & 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY, j)) { ok = false; break; }
          tc_fence_after();
          issue_s(nstage);
        }
        const uint32_t sv = smem_u32(sKV + stage * 2 * AT_TILE_BYTES + AT_TILE_BYTES);
        if (!mbar_wait(&p_full[w], j & 1, abort_flag, p.status, ST_WAIT_MISC, j)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT_BN / 16; ++k)
          umma_ts(tmem_base + 384 + w * AT_HD, tmem_base + 256 + w * 64 + k * 8, make_smem_desc(sv + k * 2048, 8192, 1024), IDESC_O,
                  (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&o_full[w]);
        umma_commit(&kv_empty[stage]);
        stage = nstage;
        phase = nphase;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int w = (warp - 4) >> 2;                 // softmax group / head within the pair
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;             // query row within the tile
    if (w < n_active) {
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      const uint32_t tS = tmem_base + w * 128 + lane_off;
      const uint32_t tO = tmem_base + 384 + w * AT_HD + lane_off;
      const uint32_t tP = tmem_base + 256 + w * 64 + lane_off;
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait(&s_full[w], j & 1, abort_flag, p.status, ST_WAIT_TMEM_FULL, j)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[128];
        PGB_TMEM_LD32(tS, (s));
        PGB_TMEM_LD32(tS + 32, (s + 32));
        PGB_TMEM_LD32(tS + 64, (s + 64));
        PGB_TMEM_LD32(tS + 96, (s + 96));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_free[w]);                   // S(j) is in registers: the next tile's scores may overwrite it
        if (j == qt) {
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if (c > r) s[c] = 0xff800000u;          // -inf
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
          if (q == 0 && j > 0) {
            // P(j-1) is read by PV(j-1) and O is written by it: both must be finished before P(j) is stored / O rescaled.
            // PV(j-1) was released a whole softmax phase ago, so this wait is normally already satisfied.
            if (!mbar_wait(&o_full[w], (j - 1) & 1, abort_flag, p.status, ST_WAIT_MISC, j)) { ok = false; break; }
            tc_fence_after();
            if (any_need) {
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
        const float sum = (sum2.x + sum2.y) + (sum2b.x + sum2b.y);
        l += sum;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[w]);
      }
      if (ok && mbar_wait(&o_full[w], (n_kv - 1) & 1, abort_flag, p.status, ST_WAIT_MISC, n_kv)) {
        tc_fence_after();
        const float inv = 1.f / l;
        const int head = head0 + w;
        __nv_bfloat16* yrow = p.Y + (size_t)(row0 + r) * p.ldy + head * AT_HD;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t o[32];
          PGB_TMEM_LD32(tO + h * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            *reinterpret_cast<uint4*>(yrow + h * 32 + c) =
                make_uint4(pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv),
                           pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv),
                           pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv),
                           pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv));
        }
        p.lse[((size_t)b * p.H + head) * p.S + qt * AT_BM + r] = -(m_used + log2f(l));   // negated, log2 domain: what the backward FMAs consume
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static CUtensorMap attn_map(const void* ptr, long long ld, int cols, long long rows) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld * 2};
  uint32_t box[2] = {AT_HD, 128};
  return make_tmap_bf16(ptr, 2, dims, strides, box);
}

void attn_fwd(const void* q, const void* k, const void* v, void* y, float* lse, long long ldq, long long ldk, long long ldv, long long ldy, int B,
              int S, int H, int Hkv, int hd, int* status, cudaStream_t st) {
  if (hd != AT_HD) throw std::runtime_error("attention kernel is specialised for head_dim 64");
  if (S % 128) throw std::runtime_error("attention kernel needs seq_len to be a multiple of 128");
  if (H % Hkv) throw std::runtime_error("num_heads must be divisible by num_kv_heads");
  const long long T = (long long)B * S;
  const CUtensorMap mq = attn_map(q, ldq, H * hd, T), mk = attn_map(k, ldk, Hkv * hd, T), mv = attn_map(v, ldv, Hkv * hd, T);
  AttnFwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.n_qt = S / AT_BM;
  p.pairs = (H / Hkv + 1) / 2;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  {
    static int delay = -1;
    if (delay < 0) {
      const char* e = getenv("PGB_ATTN_FWD_DELAY");
      delay = e ? atoi(e) : 800;      // measured plateau 600-1200 clk at B=48, S=2048: 0.398 -> 0.381 ms
    }
    p.head1_delay_clk = delay;
  }
  p.Y = (__nv_bfloat16*)y;
  p.ldy = ldy;
  p.lse = lse;
  p.status = status;
  static bool configured[64] = {};          // the attribute is a per-device property of the kernel
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int grid = p.n_qt * B * Hkv * p.pairs;
  attn_fwd_kernel<<<grid, AT_THREADS, AT_SMEM, st>>>(mq, mk, mv, p);
}

}  // namespace pgb
