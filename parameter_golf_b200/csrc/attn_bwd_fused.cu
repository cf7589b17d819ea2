// Causal GQA flash-attention backward for sm_100a (head_dim 64) in ONE pass over the score tiles.
//
//   attn_bwd_prep_kernel    D = rowsum(dO * O) per (token, head), stored negated.
//   attn_bwd_fused_kernel   key-stationary and persistent: a CTA holds the K/V tile of one KV head and streams the
//                           128-row Q/dO tiles of every query head of the group that attend to it.  Per tile pair it
//                           computes the transposed scores S^T = K Q^T and dP^T = V dO^T once, forms P^T and dS^T once,
//                           and issues all three gradient products from them:
//                               dV += P^T dO      A = P^T  from tensor memory
//                               dK += dS^T Q      A = dS^T from shared memory, read K-major
//                               dQ_part = dS K    A = the same dS^T tile, read MN-major (M = queries)
//                           dK / dV stay in tensor memory for the whole key tile; each 128x64 partial dQ is pulled into
//                           registers and added to an fp32 accumulator in global memory with vector `red.add`.
//   attn_bwd_finish_kernel  dq = bf16(scale * accumulator); the accumulator is left zeroed for the next call.
//
// Five MMA products per tile pair (the two-kernel form in attn_bwd.cu needs seven because both of its kernels recompute
// the scores) and one exponential per score instead of two.  The price is the fp32 accumulator (B*H*S*64 floats of
// scratch) and an order of summation in dQ that depends on scheduling, so dQ is reproducible to fp32 rounding, not bit
// for bit; attn_bwd.cu remains the bit-reproducible form.
//
// Scheduling: work items are (batch, KV head, key tile); key tiles j and n-1-j of one (batch, KV head) are handed to the
// same CTA one after the other, so every CTA-level item has the same length, and items are numbered (batch, KV head)
// first so that the CTAs running at any time add into a few MB of the accumulator, which therefore stays in L2 between
// the contributions of different key tiles.
//
// The per-query terms ride on the tensor core. P^T = exp2(c S^T - lse[q]) and dS^T = P^T (dP^T - D[q]) need one lse and one
// D per query COLUMN of the transposed tiles, i.e. every thread would need every value: broadcast loads from shared memory
// whose register write-back (128 B per value and warp) cost as many shared-memory data-pipe cycles per unit as the MMA
// operand reads, and that pipe is what bounds this kernel. Instead a fifth 16-wide K step is appended to each score
// product: A = a constant 128x16 tile whose first two columns are 1, B = a 128x16 tile per unit whose first two columns
// hold the value split into a bf16 high and low part (-lse / c for S^T, -D for dP^T). The sums come out of the fp32
// accumulator with the term already added (error of the split: 2^-17 relative), and the softmax threads read no shared
// memory at all. The two small tiles are built by the fourth warp of the data-movement warpgroup.
//
// The accumulator uses a tile-local layout chosen for the adds: for each (batch, head, 128-row query tile) a 32 KB
// block of 16 column chunks x 128 rows x 4 floats, so a warp's vector add covers 512 contiguous bytes.
//
// Same role as the cuDNN SDPA backward graph of the reference
// (parameter-golf-rs/crates/pg-kernels/cpp/cudnn_sdpa.cu:364-435).
#include "common.cuh"
#include "pgb.h"
#include "tma_host.h"

namespace pgb {
namespace {

constexpr int F_HD = 64;
constexpr int F_TILE = 128 * F_HD * 2;       // 16 KB: one 128-row bf16 tile of one head
constexpr float F_LOG2E = 1.4426950408889634f;
constexpr uint32_t F_BACKOFF_NS = 96;         // sleep between barrier polls of the single-thread roles
constexpr int F_STAGES = 3;                  // {Q, dO, lse, D} stages
// Two softmax warpgroups of 64 query columns each is the measured optimum at B=48, S=2048 (0.934 ms): four groups of 32
// columns (640 threads, 104 registers) took 1.009 ms, and two groups plus a fourth warpgroup that only drains dQ partials
// (512 threads, softmax at 200 registers) 1.033 ms.
#ifndef PGB_ATTN_BWD_GROUPS
#define PGB_ATTN_BWD_GROUPS 2
#endif
constexpr int F_GROUPS = PGB_ATTN_BWD_GROUPS;   // softmax warpgroups (2 or 4); each owns 128 / F_GROUPS query columns of every unit
constexpr int F_GCOLS = 128 / F_GROUPS;         // 64 or 32
constexpr int F_DQCOLS = 64 / F_GROUPS;         // dQ columns each group moves from tensor memory to the accumulator
constexpr int F_SOFTMAX_THREADS = 128 * F_GROUPS;
constexpr int F_THREADS = 128 + F_SOFTMAX_THREADS;   // warpgroup 0: warp 0 TMA, warp 1 score MMAs, warp 2 gradient MMAs
// Register hand-over. The kernel is launched with F_REGS_LAUNCH registers per thread (the most 640 threads can have);
// warpgroup 0 drops to F_REGS_MOVE and the softmax warpgroups rise to F_REGS_SOFTMAX. `setmaxnreg.inc` blocks until the
// registers exist, and the only pool it can draw from is what this CTA's own warps released, so the rise must fit in it.
constexpr int F_REGS_LAUNCH = F_GROUPS == 4 ? 96 : 168, F_REGS_MOVE = F_GROUPS == 4 ? 40 : 56, F_REGS_SOFTMAX = F_GROUPS == 4 ? 104 : 224;
static_assert(F_THREADS * F_REGS_LAUNCH <= 65536, "launch register count");
static_assert(128 * (F_REGS_LAUNCH - F_REGS_MOVE) >= F_SOFTMAX_THREADS * (F_REGS_SOFTMAX - F_REGS_LAUNCH),
              "the softmax warpgroups would wait forever for registers nobody released");
constexpr int F_BIAS_TILE = 128 * 16 * 2;    // 4 KB: 128 rows x 16 bf16, un-swizzled K-major core matrices (8 rows x 16 B)
// K/V double-buffered, Q/dO stages, one dS^T tile (128 keys x 128 queries), the bias-step tiles (one constant A tile,
// {lse, D} B tiles per stage), barriers, alignment slack
constexpr int F_SMEM = 4 * F_TILE + F_STAGES * 2 * F_TILE + 2 * F_TILE + (1 + 2 * F_STAGES) * F_BIAS_TILE + 256 + 1024;

__device__ __forceinline__ void f_tma2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ float f_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_v4(float* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
               "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}
// A shared-memory descriptor whose start address has moved by `bytes`: only the low word changes (the address field is
// 14 bits of 16-byte units and shared memory is smaller than that), so the issuing thread spends one 32-bit add per operand.
__device__ __forceinline__ uint64_t desc_at(uint64_t base, uint32_t bytes) {
  return (base & 0xFFFFFFFF00000000ull) | (uint64_t)((uint32_t)base + (bytes >> 4));
}

// Un-swizzled K-major operand of one 16-wide K step: core matrices of 8 rows x 16 bytes; the two matrices of a row group
// that are adjacent along K sit `lbo` bytes apart, consecutive 8-row groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// byte offset of (row, first 16-byte K chunk) inside a bias tile
__device__ __forceinline__ int bias_row_off(int r) { return (r >> 3) * 256 + (r & 7) * 16; }

struct FusedParams {
  int B, S, H, Hkv, n_qt, group;
  int n_pairs, n_super;          // key-tile pairs per (batch, KV head); CTA-level items
  float scale, scale_log2;
  const float* lse;              // [B, H, S]  -(log2-domain log-sum-exp)
  const float* Dsum;             // [B, H, S]  -rowsum(dO * O)
  float* dq_acc;                 // [B, H, n_qt] blocks of 16 x 128 x 4 floats
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long lddk, lddv;
  int accumulate_dv;
  int* status;
};

struct FItem { int j, b, kvh, nu, key0; };

// The seq-th item of this CTA: 0 = valid, 1 = nothing at this position (odd tile count, middle tile already done), 2 = end.
__device__ __forceinline__ int f_decode(const FusedParams& p, int seq, FItem& it) {
  const int super = (int)blockIdx.x + (seq >> 1) * (int)gridDim.x;
  if (super >= p.n_super) return 2;
  const int bk = super / p.n_pairs, pr = super - bk * p.n_pairs;
  const int j = (seq & 1) ? p.n_qt - 1 - pr : pr;
  if ((seq & 1) && j == pr) return 1;
  it.j = j;
  it.b = bk / p.Hkv;
  it.kvh = bk - it.b * p.Hkv;
  it.nu = (p.n_qt - j) * p.group;        // units: (query tile >= j, head of the group)
  it.key0 = it.b * p.S + j * 128;
  return 0;
}

// Position in the ring of Q/dO stages: stage index, phase parity of that stage's barriers, and the parity of the
// once-per-unit barriers. Advanced once per unit by every role, so all roles agree without 64-bit arithmetic.
struct UnitPos {
  int stage = 0;
  uint32_t phase = 0, par = 0;
  bool first = true;
  __device__ __forceinline__ void next() {
    if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
    par ^= 1;
    first = false;
  }
};

__global__ void __launch_bounds__(F_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __grid_constant__ CUtensorMap map_do, const FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;                                            // 2 buffers of {K, V}
  uint8_t* sQD = smem + 4 * F_TILE;                               // stages of {Q, dO}
  uint8_t* sDS = sQD + F_STAGES * 2 * F_TILE;                     // dS^T: 2 blocks (64 queries each) of 128 key rows x 128 B
  uint8_t* sAX = sDS + 2 * F_TILE;                                // constant A tile of the bias step: columns 0, 1 = 1
  uint8_t* sBX = sAX + F_BIAS_TILE;                               // stages of {lse tile, D tile}: columns 0, 1 = high, low part
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBX + 2 * F_STAGES * F_BIAS_TILE);
  uint64_t* kv_full = bars;                   // 2
  uint64_t* kv_empty = kv_full + 2;           // 2
  uint64_t* st_full = kv_empty + 2;           // F_STAGES
  uint64_t* st_empty = st_full + F_STAGES;    // F_STAGES
  uint64_t* s_full = st_empty + F_STAGES;     // 1
  uint64_t* s_free = s_full + 1;              // 1
  uint64_t* p_full = s_free + 1;              // 1
  uint64_t* acc_full = p_full + 1;            // 1
  uint64_t* acc_empty = acc_full + 1;         // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(&st_full[s], 2);                 // the TMA thread (with the tile bytes) and the bias-tile warp
      mbar_init(&st_empty[s], 1);
    }
    mbar_init(s_full, 1);
    // one arrival per softmax WARP (its lanes meet at __syncwarp first): hundreds of per-thread arrivals on one barrier
    // word serialise in shared memory
    mbar_init(s_free, F_SOFTMAX_THREADS / 32);
    mbar_init(p_full, F_SOFTMAX_THREADS / 32);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, F_SOFTMAX_THREADS / 32);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp >= 4) {
    // bias-step tiles: everything zero except columns 0 and 1 of the constant A tile, which are 1
    const int t = threadIdx.x - 128;
    uint4* z = reinterpret_cast<uint4*>(sAX);
    for (int i = t; i < (1 + 2 * F_STAGES) * F_BIAS_TILE / 16; i += F_SOFTMAX_THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  if (threadIdx.x >= 128 && threadIdx.x < 256)
    *reinterpret_cast<uint32_t*>(sAX + bias_row_off(threadIdx.x - 128)) = 0x3F803F80u;       // bf16 (1, 1)
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S^T [0,128)  dP^T [128,256)  P^T bf16 [256,320)  dK [320,384)  dV [384,448)  dQ [448,512)

  if (warp < 4) {
    // the data-movement warpgroup hands most of its registers to the softmax warpgroups
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(F_REGS_MOVE));
    if (warp == 0) {
      if (lane == 0) {
        bool ok = true;
        UnitPos up;
        int il = 0;
        for (int seq = 0; ok; ++seq) {
          FItem it;
          const int rc = f_decode(p, seq, it);
          if (rc == 2) break;
          if (rc == 1) continue;
          const int kvb = il & 1;
          if (!mbar_wait(&kv_empty[kvb], (uint32_t)(((il >> 1) & 1) ^ 1), abort_flag, p.status, ST_WAIT_EMPTY, -1, F_BACKOFF_NS)) { ok = false; break; }
          uint8_t* sk = sKV + kvb * 2 * F_TILE;
          mbar_expect_tx(&kv_full[kvb], 2 * F_TILE);
          f_tma2d(sk, &map_k, &kv_full[kvb], it.kvh * F_HD, it.key0);
          f_tma2d(sk + F_TILE, &map_v, &kv_full[kvb], it.kvh * F_HD, it.key0);
          int head = it.kvh * p.group, qi = it.j, g = 0;
          for (int u = 0; u < it.nu; ++u, up.next()) {
            const int stage = up.stage;
            if (!mbar_wait(&st_empty[stage], up.phase ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, u, F_BACKOFF_NS)) { ok = false; break; }
            const int qrow = it.b * p.S + qi * 128;
            mbar_expect_tx(&st_full[stage], 2 * F_TILE);
            f_tma2d(sQD + stage * 2 * F_TILE, &map_q, &st_full[stage], head * F_HD, qrow);
            f_tma2d(sQD + stage * 2 * F_TILE + F_TILE, &map_do, &st_full[stage], head * F_HD, qrow);
            if (++g == p.group) { g = 0; head -= p.group - 1; ++qi; } else { ++head; }
          }
          ++il;
        }
        if (!ok) {
          for (int i = 0; i < 2; ++i) mbar_drain(&kv_full[i], 0), mbar_drain(&kv_full[i], 1);
          for (int s = 0; s < F_STAGES; ++s) mbar_drain(&st_full[s], 0), mbar_drain(&st_full[s], 1);
        }
      }
    } else if (warp == 1) {
      // scores: S^T(u) and dP^T(u) as soon as the previous unit's scores have been pulled into registers
      if (lane == 0) {
        constexpr uint32_t IDESC_T = make_idesc_bf16(128, 128, 0, 0);    // K Q^T and V dO^T
        bool ok = true;
        UnitPos up;
        int il = 0;
        for (int seq = 0; ok; ++seq) {
          FItem it;
          const int rc = f_decode(p, seq, it);
          if (rc == 2) break;
          if (rc == 1) continue;
          const int kvb = il & 1;
          if (!mbar_wait(&kv_full[kvb], (uint32_t)((il >> 1) & 1), abort_flag, p.status, ST_WAIT_FULL, -1, F_BACKOFF_NS)) { ok = false; break; }
          const uint32_t sk = smem_u32(sKV + kvb * 2 * F_TILE);
          const uint64_t dk0 = make_smem_desc(sk, 16, 1024), dv0 = make_smem_desc(sk + F_TILE, 16, 1024);
          const uint64_t dax = make_smem_desc_plain(smem_u32(sAX), 128, 256);
          for (int u = 0; u < it.nu; ++u, up.next()) {
            const int stage = up.stage;
            if (!up.first && !mbar_wait(s_free, up.par ^ 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY, u, F_BACKOFF_NS)) { ok = false; break; }
            if (!mbar_wait(&st_full[stage], up.phase, abort_flag, p.status, ST_WAIT_FULL, u, F_BACKOFF_NS)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sq = smem_u32(sQD + stage * 2 * F_TILE);
            const uint64_t dq0 = make_smem_desc(sq, 16, 1024), ddo0 = make_smem_desc(sq + F_TILE, 16, 1024);
            const uint64_t dbl = make_smem_desc_plain(smem_u32(sBX + stage * 2 * F_BIAS_TILE), 128, 256);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(tmem_base, desc_at(dk0, k * 32), desc_at(dq0, k * 32), IDESC_T, k > 0);
            umma_ss(tmem_base, dax, dbl, IDESC_T, 1u);                                    // S^T += 1 (-lse / c)^T
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(tmem_base + 128, desc_at(dv0, k * 32), desc_at(ddo0, k * 32), IDESC_T, k > 0);
            umma_ss(tmem_base + 128, dax, desc_at(dbl, F_BIAS_TILE), IDESC_T, 1u);        // dP^T += 1 (-D)^T
            umma_commit(s_full);
          }
          ++il;
        }
      }
    } else if (warp == 2) {
      // gradients, once every softmax group has stored its part of P^T (tensor memory) and dS^T (shared memory)
      if (lane == 0) {
        constexpr uint32_t IDESC_DV = make_idesc_bf16(128, 64, 0, 1);    // A = P^T from TMEM; B = dO read N(=hd)-contiguous
        constexpr uint32_t IDESC_DK = make_idesc_bf16(128, 64, 0, 1);    // A = dS^T K-major (rows = keys); B = Q read N-contiguous
        constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, 64, 1, 1);    // A = dS^T read MN-major (M = queries); B = K read N-contiguous
        const uint32_t sds = smem_u32(sDS);
        const uint64_t dsq0 = make_smem_desc(sds, 16384, 1024);          // dS^T as the MN-major A of dQ: 64-query blocks 16 KB apart
        const uint64_t dsk0 = make_smem_desc(sds, 16, 1024);             // dS^T as the K-major A of dK
        bool ok = true;
        UnitPos up;
        int il = 0;
        for (int seq = 0; ok; ++seq) {
          FItem it;
          const int rc = f_decode(p, seq, it);
          if (rc == 2) break;
          if (rc == 1) continue;
          const int kvb = il & 1;
          const uint64_t kb0 = make_smem_desc(smem_u32(sKV + kvb * 2 * F_TILE), 8192, 1024);
          for (int u = 0; u < it.nu; ++u, up.next()) {
            const int stage = up.stage;
            if (!mbar_wait(&st_full[stage], up.phase, abort_flag, p.status, ST_WAIT_FULL, u, F_BACKOFF_NS)) { ok = false; break; }
            if (!mbar_wait(p_full, up.par, abort_flag, p.status, ST_WAIT_MISC, u, F_BACKOFF_NS)) { ok = false; break; }
            if (u == 0) {          // the previous item's dK/dV must have been read out before they are overwritten
              if (!mbar_wait(acc_empty, (uint32_t)((il & 1) ^ 1), abort_flag, p.status, ST_WAIT_TMEM_EMPTY, seq, F_BACKOFF_NS)) { ok = false; break; }
            }
            tc_fence_after();
            const uint32_t sq = smem_u32(sQD + stage * 2 * F_TILE);
            const uint64_t qb0 = make_smem_desc(sq, 8192, 1024), dob0 = make_smem_desc(sq + F_TILE, 8192, 1024);
            const uint32_t acc = u > 0 ? 1u : 0u;
#pragma unroll
            for (int k = 0; k < 8; ++k)   // dQ_part = dS K  (k-th group of 16 keys)
              umma_ss(tmem_base + 448, desc_at(dsq0, k * 2048), desc_at(kb0, k * 2048), IDESC_DQ, k > 0 ? 1u : 0u);
#pragma unroll
            for (int k = 0; k < 8; ++k)   // dV += P^T dO  (k-th group of 16 queries)
              umma_ts(tmem_base + 384, tmem_base + 256 + k * 8, desc_at(dob0, k * 2048), IDESC_DV, k > 0 ? 1u : acc);
#pragma unroll
            for (int k = 0; k < 8; ++k)   // dK += dS^T Q
              umma_ss(tmem_base + 320, desc_at(dsk0, (k >> 2) * 16384 + (k & 3) * 32), desc_at(qb0, k * 2048), IDESC_DK, k > 0 ? 1u : acc);
            umma_commit(&st_empty[stage]);      // frees the Q/dO stage, P^T and dS^T, and says that dQ_part is complete
          }
          if (ok) {
            umma_commit(acc_full);
            umma_commit(&kv_empty[kvb]);        // every MMA that reads this K/V buffer has completed by then
          }
          ++il;
        }
      }
    }
    else {
      // warp 3: the B tiles of the bias step. Lane l owns query rows 4 l .. 4 l + 3 of every unit.
      bool ok = true;
      UnitPos up;
      const float inv_c = 1.f / p.scale_log2;
      for (int seq = 0; ok; ++seq) {
        FItem it;
        const int rc = f_decode(p, seq, it);
        if (rc == 2) break;
        if (rc == 1) continue;
        int head = it.kvh * p.group, qi = it.j, g = 0;
        for (int u = 0; u < it.nu; ++u, up.next()) {
          const int stage = up.stage;
          const size_t vidx = ((size_t)it.b * p.H + head) * p.S + qi * 128 + lane * 4;
          const float4 l4 = *reinterpret_cast<const float4*>(p.lse + vidx), d4 = *reinterpret_cast<const float4*>(p.Dsum + vidx);
          if (!mbar_wait(&st_empty[stage], up.phase ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, u, F_BACKOFF_NS)) { ok = false; break; }
          uint8_t* tl = sBX + stage * 2 * F_BIAS_TILE;
          const float lv[4] = {l4.x * inv_c, l4.y * inv_c, l4.z * inv_c, l4.w * inv_c}, dv4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int off = bias_row_off(lane * 4 + e);
            const __nv_bfloat16 lh = __float2bfloat16_rn(lv[e]), dh = __float2bfloat16_rn(dv4[e]);
            const __nv_bfloat16 ll = __float2bfloat16_rn(lv[e] - __bfloat162float(lh)), dl = __float2bfloat16_rn(dv4[e] - __bfloat162float(dh));
            *reinterpret_cast<uint32_t*>(tl + off) = (uint32_t)__bfloat16_as_ushort(lh) | ((uint32_t)__bfloat16_as_ushort(ll) << 16);
            *reinterpret_cast<uint32_t*>(tl + F_BIAS_TILE + off) = (uint32_t)__bfloat16_as_ushort(dh) | ((uint32_t)__bfloat16_as_ushort(dl) << 16);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&st_full[stage]);
          if (++g == p.group) { g = 0; head -= p.group - 1; ++qi; } else { ++head; }
        }
      }
      if (!ok) __syncwarp();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(F_REGS_SOFTMAX));
    const int w = (warp - 4) >> 2;                 // this group owns query columns [w F_GCOLS, (w + 1) F_GCOLS) of every unit
    const int quarter = warp & 3;
    const int kk = quarter * 32 + lane;            // key row within the tile (and query row of the dQ partial)
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + w * F_GCOLS + lane_off, tdP = tmem_base + 128 + w * F_GCOLS + lane_off;
    const uint32_t tPt = tmem_base + 256 + w * (F_GCOLS / 2) + lane_off;
    const uint32_t tDQ = tmem_base + 448 + w * F_DQCOLS + lane_off;      // this group's share of the 64 dQ columns
    // this thread's part of its dS^T row: 64-query block (w * F_GCOLS) / 64, 16-byte chunks from ch0 on
    uint8_t* ds_row = sDS + ((w * F_GCOLS) >> 6) * F_TILE + kk * 128;
    const int swz = kk & 7, ch0 = ((w * F_GCOLS) & 63) >> 3;
    const int qbase = w * F_GCOLS;
    bool ok = true;
    UnitPos up;
    int prev_stage = 0;
    uint32_t prev_phase = 0;
    int il = 0;
    float* prev_dq = nullptr;                      // accumulator block of the previous unit (its dQ partial is still in TMEM)
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    for (int seq = 0; ok; ++seq) {
      FItem it;
      const int rc = f_decode(p, seq, it);
      if (rc == 2) break;
      if (rc == 1) continue;
      const int j = it.j, kvh = it.kvh, key0 = it.key0, nu = it.nu;
      int head = kvh * p.group, qi = j, g = 0;
      float* dq_blk = p.dq_acc + (((size_t)it.b * p.H + head) * p.n_qt + qi) * 8192;
      for (int u = 0; u < nu; ++u, up.next()) {
        const int stage = up.stage;
        if (!mbar_wait(s_full, up.par, abort_flag, p.status, ST_WAIT_TMEM_FULL, u)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[F_GCOLS], dp[F_GCOLS];
        PGB_TMEM_LD32(tS, s);
        if constexpr (F_GCOLS == 64) PGB_TMEM_LD32(tS + 32, (s + 32));
        PGB_TMEM_LD32(tdP, dp);
        if constexpr (F_GCOLS == 64) PGB_TMEM_LD32(tdP + 32, (dp + 32));
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);        // the score buffers may take the next unit
        const bool diag = qi == j;
        uint32_t pp[F_GCOLS / 2], pd[F_GCOLS / 2];
        if (!diag) {
#pragma unroll
          for (int c = 0; c < F_GCOLS; c += 2) {
            const float2 tt = __fmul2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2);   // the tile already holds S - lse / c
            const float2 pr = make_float2(f_ex2(tt.x), f_ex2(tt.y));
            const float2 dd = __fmul2_rn(pr, make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])));   // ... and dP - D
            pp[c >> 1] = pack_bf16x2(pr.x, pr.y);
            pd[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        } else {
#pragma unroll
          for (int c = 0; c < F_GCOLS; c += 2) {
            const float2 tt = __fmul2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2);   // the tile already holds S - lse / c
            float2 pr = make_float2(f_ex2(tt.x), f_ex2(tt.y));
            if (qbase + c < kk) pr.x = 0.f;              // query position before the key: masked
            if (qbase + c + 1 < kk) pr.y = 0.f;
            const float2 dd = __fmul2_rn(pr, make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])));   // ... and dP - D
            pp[c >> 1] = pack_bf16x2(pr.x, pr.y);
            pd[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        }
        uint32_t o[F_DQCOLS];
        if (!up.first) {
          // The gradient MMAs of the previous unit read P^T / dS^T until their commit arrives; the same commit says that
          // the previous unit's dQ partial is complete: pull this group's 16 columns of it before the next one may start.
          if (!mbar_wait(&st_empty[prev_stage], prev_phase, abort_flag, p.status, ST_WAIT_EMPTY, u)) { ok = false; break; }
          tc_fence_after();
          if constexpr (F_DQCOLS == 32) { PGB_TMEM_LD32(tDQ, o); } else { PGB_TMEM_LD16(tDQ, o); }
        }
        PGB_TMEM_ST16(tPt, pp);
        if constexpr (F_GCOLS == 64) PGB_TMEM_ST16(tPt + 16, (pp + 16));
#pragma unroll
        for (int c = 0; c < F_GCOLS / 8; ++c)
          *reinterpret_cast<uint4*>(ds_row + (((ch0 + c) ^ swz) << 4)) = make_uint4(pd[4 * c], pd[4 * c + 1], pd[4 * c + 2], pd[4 * c + 3]);
        tmem_wait_st();
        tmem_wait_ld();
        fence_proxy_async();                       // the dS^T stores must be visible to the tensor core's reads of shared memory
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        if (!up.first) {
          float* dst = prev_dq + (size_t)(w * (F_DQCOLS / 4)) * 512 + kk * 4;
#pragma unroll
          for (int c = 0; c < F_DQCOLS / 4; ++c) red_add_v4(dst + c * 512, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        prev_dq = dq_blk;
        prev_stage = stage;
        prev_phase = up.phase;
        if (++g == p.group) {                      // next unit: the next head of the group, then the next query tile
          g = 0;
          head -= p.group - 1;
          ++qi;
          dq_blk += 8192 - (size_t)(p.group - 1) * p.n_qt * 8192;
        } else {
          ++head;
          dq_blk += (size_t)p.n_qt * 8192;
        }
      }
      if (!ok) break;
      if (mbar_wait(acc_full, (uint32_t)(il & 1), abort_flag, p.status, ST_WAIT_MISC, nu)) {
        tc_fence_after();
        // dK and dV (64 columns each) are split evenly over the softmax groups: the first half of the groups writes dK
        constexpr int EC = 128 / F_GROUPS;               // columns per group: 64 or 32
        const bool is_dk = w < F_GROUPS / 2;
        const int col0 = (w % (F_GROUPS / 2)) * EC;
        const uint32_t tA = tmem_base + (is_dk ? 320 : 384) + col0 + lane_off;
        __nv_bfloat16* out = (is_dk ? p.dk + (size_t)(key0 + kk) * p.lddk : p.dv + (size_t)(key0 + kk) * p.lddv) + kvh * F_HD + col0;
        const bool acc = !is_dk && p.accumulate_dv;
        const float mul = is_dk ? p.scale : 1.f;
        uint32_t v[EC];
        PGB_TMEM_LD32(tA, v);
        if constexpr (EC == 64) PGB_TMEM_LD32(tA + 32, (v + 32));
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);     // the values are in registers: the next key tile may start accumulating
#pragma unroll
        for (int c = 0; c < EC; c += 8) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[c + e]) * mul;
          if (acc) {
            uint4 q = *reinterpret_cast<const uint4*>(out + c);
            float2 a0 = unpack_bf16x2(q.x), a1 = unpack_bf16x2(q.y), a2 = unpack_bf16x2(q.z), a3 = unpack_bf16x2(q.w);
            f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y; f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
          }
          *reinterpret_cast<uint4*>(out + c) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        }
      } else {
        ok = false;
      }
      ++il;
    }
    if (ok && !up.first) {
      // the last unit's dQ partial
      if (mbar_wait(&st_empty[prev_stage], prev_phase, abort_flag, p.status, ST_WAIT_EMPTY, -2)) {
        tc_fence_after();
        uint32_t o[F_DQCOLS];
        if constexpr (F_DQCOLS == 32) { PGB_TMEM_LD32(tDQ, o); } else { PGB_TMEM_LD16(tDQ, o); }
        tmem_wait_ld();
        float* dst = prev_dq + (size_t)(w * (F_DQCOLS / 4)) * 512 + kk * 4;
#pragma unroll
        for (int c = 0; c < F_DQCOLS / 4; ++c) red_add_v4(dst + c * 512, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
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

// D = rowsum(dO * O) per (token, head), stored negated in [B, H, S] order. Eight lanes share one head's 64 columns.
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, long long ldo,
                                                            long long lddo, float* __restrict__ dsum, long long T, int S, int H) {
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  const int chunk = (int)(idx & 7);
  const long long rh = idx >> 3;
  const int head = (int)(rh % H);
  const long long row = rh / H;
  float dot = 0.f;
  if (row < T) {
    const uint4 a = *reinterpret_cast<const uint4*>(O + row * ldo + head * F_HD + chunk * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + row * lddo + head * F_HD + chunk * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    dot = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y + a3.x * g3.x + a3.y * g3.y;
  }
  dot += __shfl_xor_sync(0xffffffffu, dot, 1);
  dot += __shfl_xor_sync(0xffffffffu, dot, 2);
  dot += __shfl_xor_sync(0xffffffffu, dot, 4);
  if (chunk == 0 && row < T) {
    const long long b = row / S, s = row - b * S;
    dsum[(b * H + head) * S + s] = -dot;
  }
}

// dq = bf16(scale * accumulator), and the accumulator block is zeroed for the next call. One CTA per (batch, head, query tile):
// the 32 KB block is read in its own order (512 contiguous bytes per warp load), turned into bf16 in a padded shared-memory
// tile, and written out one 128-byte head row per 8 lanes.
__global__ void __launch_bounds__(256) attn_bwd_finish_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long lddq, int S, int H,
                                                              int n_qt, float scale) {
  constexpr int PITCH = 136;                        // bytes per staged row: 128 + 8, so that rows start in different banks
  __shared__ __align__(16) uint8_t tile[128 * PITCH];
  const int blk = blockIdx.x;                       // (b * H + head) * n_qt + qi
  const int qi = blk % n_qt;
  const int bh = blk / n_qt;
  const int head = bh % H, b = bh / H;
  float4* base = reinterpret_cast<float4*>(acc + (size_t)blk * 8192);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = it * 256 + threadIdx.x;         // chunk cc = idx / 128 (4 columns), row r = idx % 128
    const int r = idx & 127, cc = idx >> 7;
    const float4 x = base[idx];
    base[idx] = zero;
    *reinterpret_cast<uint2*>(tile + r * PITCH + cc * 8) = make_uint2(pack_bf16x2(x.x * scale, x.y * scale), pack_bf16x2(x.z * scale, x.w * scale));
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int oc = idx & 7, r = idx >> 3;           // 8 lanes write the 128 bytes of one row
    const uint2 lo = *reinterpret_cast<const uint2*>(tile + r * PITCH + oc * 16), hi = *reinterpret_cast<const uint2*>(tile + r * PITCH + oc * 16 + 8);
    *reinterpret_cast<uint4*>(dq + ((size_t)b * S + qi * 128 + r) * lddq + head * F_HD + oc * 8) = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
}

CUtensorMap fused_map(const void* ptr, long long ld, int cols, long long rows) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld * 2};
  uint32_t box[2] = {F_HD, 128};
  return make_tmap_bf16(ptr, 2, dims, strides, box);
}

}  // namespace

size_t attn_bwd_fused_scratch_floats(int B, int S, int H) { return (size_t)B * H * S * F_HD; }

void attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, float* dsum, float* dq_acc, void* dq,
                    void* dk, void* dv, long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk,
                    long long lddv, int B, int S, int H, int Hkv, int hd, int accumulate_dv, int* status, cudaStream_t st, int dsum_ready) {
  if (hd != F_HD) throw std::runtime_error("attention kernel is specialised for head_dim 64");
  if (S % 128) throw std::runtime_error("attention kernel needs seq_len to be a multiple of 128");
  if (H % Hkv) throw std::runtime_error("attention: the number of KV heads must divide the number of query heads");
  if ((ldo % 8) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) throw std::runtime_error("attention: row strides must be multiples of 8 elements");
  const long long T = (long long)B * S;
  FusedParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.n_qt = S / 128;
  p.group = H / Hkv;
  p.n_pairs = (p.n_qt + 1) / 2;
  p.n_super = B * Hkv * p.n_pairs;
  p.scale = 1.f / sqrtf((float)hd);
  p.scale_log2 = p.scale * F_LOG2E;
  p.lse = lse; p.Dsum = dsum; p.dq_acc = dq_acc;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.lddk = lddk; p.lddv = lddv;
  p.accumulate_dv = accumulate_dv;
  p.status = status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  static bool configured[64] = {};          // the attribute is a per-device property of the kernel
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const long long n_chunks = T * H * 8;
  if (!dsum_ready)          // otherwise the producer of d_o has already written -rowsum(d_o * o) (`xsa_bwd` does)
    attn_bwd_prep_kernel<<<(unsigned)((n_chunks + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, ldo, lddo, dsum, T, S, H);
  const CUtensorMap mq = fused_map(q, ldq, H * hd, T), mk = fused_map(k, ldk, Hkv * hd, T), mv = fused_map(v, ldv, Hkv * hd, T),
                    mdo = fused_map(d_o, lddo, H * hd, T);
  attn_bwd_fused_kernel<<<std::min(p.n_super, sms), F_THREADS, F_SMEM, st>>>(mq, mk, mv, mdo, p);
  attn_bwd_finish_kernel<<<B * H * p.n_qt, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, lddq, S, H, p.n_qt, p.scale);
}

}  // namespace pgb
