// Causal GQA flash-attention backward for sm_100a (head_dim 64), two kernels, no atomics:
//
//   attn_bwd_dq_kernel    query-stationary: for a 128-row query tile of one head, streams the K/V tiles,
//                         recomputes P from the saved log-sum-exp, forms dS and accumulates dQ += dS K in tensor
//                         memory. Also produces D = rowsum(dO * O).
//   attn_bwd_dkdv_kernel  key-stationary: for a 128-key tile of one KV head, streams the 128-row Q/dO tiles of
//                         every query head of the group, computes the TRANSPOSED scores S^T = K Q^T and
//                         dP^T = V dO^T (one thread per key row and half of the query columns), and accumulates
//                         dV += P^T dO, dK += dS^T Q.
//
// In both kernels the bf16 P / dS operands are written to TMEM columns of their own and consumed by tcgen05.mma
// straight from there, so probabilities never touch shared or global memory, and the fp32 score buffers are handed
// back to the MMA-issuing thread as soon as they have been read. Accumulating dQ in
// a second pass costs two extra small GEMMs per tile but removes the fp32 atomics a single-pass design
// needs (tens of GB of L2 atomic traffic per layer at this problem size).
// Same role as the cuDNN SDPA backward graph of the reference
// (parameter-golf-rs/crates/pg-kernels/cpp/cudnn_sdpa.cu:364-435).
#include "common.cuh"
#include "pgb.h"
#include "tma_host.h"

namespace pgb {

constexpr int AB_HD = 64;
constexpr int AB_TILE = 128 * AB_HD * 2;     // 16 KB
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void tma2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(gsrc),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnBwdParams {
  int B, S, H, Hkv, n_qt, group;
  int n_items_q, n_items_kv;
  float scale, scale_log2;
  const __nv_bfloat16* O;      // [T, H*hd]
  const __nv_bfloat16* dO;
  long long ldo, lddo;
  const float* lse;            // [B, H, S]
  float* Dsum;                 // [B, H, S]
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long lddq, lddk, lddv;
  int accumulate_dv;
  int* status;
};


// ------------------------------------------------------------------------------------------------------------------
// Query-stationary kernel.  One item = a 128-row query tile of one head; it streams the key tiles 0..qt.  Per key tile:
// S = Q K^T and dP = dO V^T (128 x 128, N = 128 MMAs) land in TMEM; the two softmax groups each take 64 key columns,
// pull them into registers and release the score buffers at once (`s_free`), so the next tile's scores are computed
// while this tile's dS is; dS goes to its own TMEM columns as bf16 and feeds dQ += dS K.  Two issuing threads (scores /
// dQ) keep the tensor pipe fed; Q/dO are double-buffered across items.
// TMEM: S [0,128) dP [128,256) dS [256,320) dQ [320,384).
constexpr int DQ_STAGES = 3;
constexpr int DQ_THREADS = 384;              // warpgroup 0: warp 0 TMA, warp 1 score MMAs, warp 2 dQ MMAs, warp 3 idle; warpgroups 1, 2: softmax
constexpr int DQ_SMEM = (4 + 2 * DQ_STAGES) * AB_TILE + 1024 + 256;

__global__ void __launch_bounds__(DQ_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_do, const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQD = smem;                      // 2 buffers of {Q, dO}
  uint8_t* sKV = smem + 4 * AB_TILE;        // stages {K, V}
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (4 + 2 * DQ_STAGES) * AB_TILE);
  uint64_t* q_full = bars;                   // 2
  uint64_t* q_empty = q_full + 2;            // 2
  uint64_t* kv_full = q_empty + 2;
  uint64_t* kv_empty = kv_full + DQ_STAGES;
  uint64_t* s_full = kv_empty + DQ_STAGES;   // 1
  uint64_t* s_free = s_full + 1;             // 1
  uint64_t* p_full = s_free + 1;             // 1
  uint64_t* dq_full = p_full + 1;            // 1
  uint64_t* dq_empty = dq_full + 1;          // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_qt = p.B * p.H;
  struct Item { int qt, b, head, kvh, n_kv, row0; };
  auto decode = [&](int item) {
    Item it;
    it.qt = p.n_qt - 1 - item / per_qt;     // long key ranges first
    const int rem = item % per_qt;
    it.b = rem / p.H;
    it.head = rem % p.H;
    it.kvh = it.head / p.group;
    it.n_kv = it.qt + 1;
    it.row0 = it.b * p.S + it.qt * 128;
    return it;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int s = 0; s < DQ_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 256);
    mbar_init(p_full, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 256);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
  // the data-movement warpgroup hands most of its registers to the two softmax warpgroups (128 live values per thread)
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {
      long long tg = 0;                     // key tiles loaded by this CTA so far
      int il = 0;                           // items handled by this CTA so far
      bool ok = true;
      for (int item = blockIdx.x; item < p.n_items_q && ok; item += gridDim.x, ++il) {
        const Item it = decode(item);
        const int qb = il & 1;
        if (!mbar_wait(&q_empty[qb], (uint32_t)(((il >> 1) & 1) ^ 1), abort_flag, p.status, ST_WAIT_EMPTY, -1)) { ok = false; break; }
        mbar_expect_tx(&q_full[qb], 2 * AB_TILE);
        tma2d(sQD + qb * 2 * AB_TILE, &map_q, &q_full[qb], it.head * AB_HD, it.row0);
        tma2d(sQD + qb * 2 * AB_TILE + AB_TILE, &map_do, &q_full[qb], it.head * AB_HD, it.row0);
        for (int j = 0; j < it.n_kv; ++j, ++tg) {
          const int stage = (int)(tg % DQ_STAGES);
          if (!mbar_wait(&kv_empty[stage], (uint32_t)(((tg / DQ_STAGES) & 1) ^ 1), abort_flag, p.status, ST_WAIT_EMPTY, j)) { ok = false; break; }
          uint8_t* sk = sKV + stage * 2 * AB_TILE;
          mbar_expect_tx(&kv_full[stage], 2 * AB_TILE);
          tma2d(sk, &map_k, &kv_full[stage], it.kvh * AB_HD, it.b * p.S + j * 128);
          tma2d(sk + AB_TILE, &map_v, &kv_full[stage], it.kvh * AB_HD, it.b * p.S + j * 128);
        }
      }
      if (!ok) {
        for (int i = 0; i < 2; ++i) mbar_drain(&q_full[i], 0), mbar_drain(&q_full[i], 1);
        for (int s = 0; s < DQ_STAGES; ++s) mbar_drain(&kv_full[s], 0), mbar_drain(&kv_full[s], 1);
      }
    }
  } else if (warp == 1) {
    // scores: S(j) and dP(j) as soon as the previous tile's scores have been pulled into registers
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);    // Q K^T, dO V^T
      long long tg = 0;
      int il = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.n_items_q && ok; item += gridDim.x, ++il) {
        const Item it = decode(item);
        const int qb = il & 1;
        if (!mbar_wait(&q_full[qb], (uint32_t)((il >> 1) & 1), abort_flag, p.status, ST_WAIT_FULL, -1)) { ok = false; break; }
        const uint32_t sq = smem_u32(sQD + qb * 2 * AB_TILE), sdo = sq + AB_TILE;
        for (int j = 0; j < it.n_kv && ok; ++j, ++tg) {
          const int stage = (int)(tg % DQ_STAGES);
          if (tg > 0 && !mbar_wait(s_free, (uint32_t)((tg - 1) & 1), abort_flag, p.status, ST_WAIT_TMEM_EMPTY, j)) { ok = false; break; }
          if (!mbar_wait(&kv_full[stage], (uint32_t)((tg / DQ_STAGES) & 1), abort_flag, p.status, ST_WAIT_FULL, j)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sk = smem_u32(sKV + stage * 2 * AB_TILE), sv = sk + AB_TILE;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem_base, make_smem_desc(sq + k * 32, 16, 1024), make_smem_desc(sk + k * 32, 16, 1024), IDESC_S, k > 0);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + 128, make_smem_desc(sdo + k * 32, 16, 1024), make_smem_desc(sv + k * 32, 16, 1024), IDESC_S, k > 0);
          umma_commit(s_full);
        }
        if (ok) umma_commit(&q_empty[qb]);    // Q / dO of this item are read by the score MMAs only
      }
    }
  } else if (warp == 2) {
    // dQ += dS K once both softmax groups have stored their halves of dS
    if (lane == 0) {
      constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, 64, 0, 1);    // dS (TMEM) x K, K read N(=hd)-contiguous
      long long tg = 0;
      int il = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.n_items_q && ok; item += gridDim.x, ++il) {
        const Item it = decode(item);
        for (int j = 0; j < it.n_kv && ok; ++j, ++tg) {
          const int stage = (int)(tg % DQ_STAGES);
          if (!mbar_wait(&kv_full[stage], (uint32_t)((tg / DQ_STAGES) & 1), abort_flag, p.status, ST_WAIT_FULL, j)) { ok = false; break; }
          if (!mbar_wait(p_full, (uint32_t)(tg & 1), abort_flag, p.status, ST_WAIT_MISC, j)) { ok = false; break; }
          if (j == 0) {        // the previous item's dQ must have been read out before it is overwritten
            if (!mbar_wait(dq_empty, (uint32_t)((il & 1) ^ 1), abort_flag, p.status, ST_WAIT_TMEM_EMPTY, item)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sk = smem_u32(sKV + stage * 2 * AB_TILE);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ts(tmem_base + 320, tmem_base + 256 + k * 8, make_smem_desc(sk + k * 2048, 8192, 1024), IDESC_DQ, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(&kv_empty[stage]);      // frees the K/V stage and tells the softmax groups that dS may be overwritten
        }
        if (ok) umma_commit(dq_full);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int w = (warp - 4) >> 2;                 // this group owns key columns [64 w, 64 w + 64) of every tile
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;             // query row within the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + w * 64 + lane_off, tdP = tmem_base + 128 + w * 64 + lane_off;
    const uint32_t tdS = tmem_base + 256 + w * 32 + lane_off, tDQ = tmem_base + 320 + w * 32 + lane_off;
    long long tg = 0;
    int il = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.n_items_q && ok; item += gridDim.x, ++il) {
      const Item it = decode(item);
      const int head = it.head, qt = it.qt, row0 = it.row0, b = it.b;
      // D = rowsum(dO * O) for this query row; also published for the dK/dV kernel
      float Dr = 0.f;
      {
        const __nv_bfloat16* op = p.O + (size_t)(row0 + r) * p.ldo + head * AB_HD;
        const __nv_bfloat16* dop = p.dO + (size_t)(row0 + r) * p.lddo + head * AB_HD;
#pragma unroll
        for (int c = 0; c < AB_HD; c += 8) {
          uint4 a = *reinterpret_cast<const uint4*>(op + c), g = *reinterpret_cast<const uint4*>(dop + c);
          float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
          float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
          Dr += a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y + a3.x * g3.x + a3.y * g3.y;
        }
      }
      {
        // the next item's O / dO rows are read the same way: start them on their way into L2/L1 now
        const int nitem = item + (int)gridDim.x;
        if (nitem < p.n_items_q) {
          const Item nx = decode(nitem);
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.O + (size_t)(nx.row0 + r) * p.ldo + nx.head * AB_HD));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.dO + (size_t)(nx.row0 + r) * p.lddo + nx.head * AB_HD));
        }
      }
      const size_t sidx = ((size_t)b * p.H + head) * p.S + qt * 128 + r;
      if (w == 0) p.Dsum[sidx] = -Dr;          // negated: the dK/dV kernel adds it
      const float nlse2 = p.lse[sidx];         // -(log2-domain log-sum-exp), as written by the forward
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(nlse2, nlse2), nd2 = make_float2(-Dr, -Dr);
      for (int j = 0; j < it.n_kv; ++j, ++tg) {
        if (!mbar_wait(s_full, (uint32_t)(tg & 1), abort_flag, p.status, ST_WAIT_TMEM_FULL, j)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[64], dp[64];
        PGB_TMEM_LD32(tS, (s));
        PGB_TMEM_LD32(tS + 32, (s + 32));
        PGB_TMEM_LD32(tdP, (dp));
        PGB_TMEM_LD32(tdP + 32, (dp + 32));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(s_free);                       // the score buffers may take the next tile
        const bool diag = j == qt;
        const int kbase = w * 64;                           // key offset of this group's columns inside the tile
        uint32_t pk[32];
        if (!diag) {
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, nl2);
            const float2 pr = make_float2(ex2f(tt.x), ex2f(tt.y));
            const float2 dd = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), nd2));
            pk[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, nl2);
            float2 pr = make_float2(ex2f(tt.x), ex2f(tt.y));
            if (kbase + c > r) pr.x = 0.f;
            if (kbase + c + 1 > r) pr.y = 0.f;
            const float2 dd = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), nd2));
            pk[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        }
        if (tg > 0) {            // the dQ MMAs of the previous tile still read dS until their commit arrives
          const long long pg = tg - 1;
          if (!mbar_wait(&kv_empty[(int)(pg % DQ_STAGES)], (uint32_t)((pg / DQ_STAGES) & 1), abort_flag, p.status, ST_WAIT_EMPTY, j)) { ok = false; break; }
          tc_fence_after();
        }
        PGB_TMEM_ST16(tdS, (pk));
        PGB_TMEM_ST16(tdS + 16, (pk + 16));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full);
      }
      if (ok && mbar_wait(dq_full, (uint32_t)(il & 1), abort_flag, p.status, ST_WAIT_MISC, it.n_kv)) {
        tc_fence_after();
        // each group writes 32 of the 64 columns of its row
        __nv_bfloat16* out = p.dq + (size_t)(row0 + r) * p.lddq + head * AB_HD + w * 32;
        uint32_t o[32];
        PGB_TMEM_LD32(tDQ, o);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; c += 8)
          *reinterpret_cast<uint4*>(out + c) =
              make_uint4(pack_bf16x2(__uint_as_float(o[c]) * p.scale, __uint_as_float(o[c + 1]) * p.scale),
                         pack_bf16x2(__uint_as_float(o[c + 2]) * p.scale, __uint_as_float(o[c + 3]) * p.scale),
                         pack_bf16x2(__uint_as_float(o[c + 4]) * p.scale, __uint_as_float(o[c + 5]) * p.scale),
                         pack_bf16x2(__uint_as_float(o[c + 6]) * p.scale, __uint_as_float(o[c + 7]) * p.scale));
        tc_fence_before();
        mbar_arrive(dq_empty);
      } else {
        ok = false;
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

// ------------------------------------------------------------------------------------------------------------------
// Key-stationary kernel.  One item = a 128-key tile of one KV head; its units are the (128-row query tile, query head)
// pairs that attend to it.  Per unit: S^T = K Q^T and dP^T = V dO^T (128 x 128 each, N = 128 MMAs) land in TMEM; the two
// softmax groups each take 64 query columns, pull them into registers and release the score buffers at once
// (`s_free`), so the next unit's scores are computed while this unit's probabilities are; P^T and dS^T go back to
// their own TMEM columns as bf16 and feed dV += P^T dO and dK += dS^T Q.  Two issuing threads (scores / gradients) keep
// the tensor pipe fed.  TMEM: S^T [0,128) dP^T [128,256) P^T [256,320) dS^T [320,384) dK [384,448) dV [448,512).
constexpr int KV_STAGES = 4;
constexpr int KV_THREADS = 384;              // warpgroup 0: warp 0 TMA, warp 1 score MMAs, warp 2 gradient MMAs, warp 3 idle; warpgroups 1, 2: softmax
// one stage holds a 128-row Q tile, a 128-row dO tile, lse[128] and D[128]
constexpr int KV_SMEM = 2 * AB_TILE + KV_STAGES * (2 * AB_TILE) + KV_STAGES * 1024 + 1024 + 256;

__global__ void __launch_bounds__(KV_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                     const __grid_constant__ CUtensorMap map_do, const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + AB_TILE;
  uint8_t* sQD = smem + 2 * AB_TILE;                                   // stages of {Q, dO}
  float* sVec = reinterpret_cast<float*>(smem + 2 * AB_TILE + KV_STAGES * 2 * AB_TILE);   // stages of {lse[128], D[128]}
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sVec) + KV_STAGES * 1024);
  uint64_t* kv_full = bars;
  uint64_t* st_full = bars + 1;
  uint64_t* st_empty = st_full + KV_STAGES;
  uint64_t* s_full = st_empty + KV_STAGES;    // 1
  uint64_t* s_free = s_full + 1;              // 1
  uint64_t* p_full = s_free + 1;              // 1
  uint64_t* acc_full = p_full + 1;            // 1
  uint64_t* acc_empty = acc_full + 1;         // 1
  uint64_t* kv_empty = acc_empty + 1;         // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_kt = p.B * p.Hkv;
  struct Item { int j, b, kvh, nu, key0; };
  auto decode = [&](int item) {
    Item it;
    it.j = item / per_kt;                                   // key tile; low j = long query range = scheduled first
    const int rem = item % per_kt;
    it.b = rem / p.Hkv;
    it.kvh = rem % p.Hkv;
    it.nu = (p.n_qt - it.j) * p.group;                      // units: (query tile, head)
    it.key0 = it.b * p.S + it.j * 128;
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&st_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 256);
    mbar_init(p_full, 256);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    mbar_init(kv_empty, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto unit_coords = [&](const Item& it, int u, int& qi, int& head) {
    head = it.kvh * p.group + (u % p.group);
    qi = it.j + u / p.group;
  };

  if (warp < 4) {
  // the data-movement warpgroup hands most of its registers to the two softmax warpgroups (128 live values per thread)
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t item_par = 0;
      long long ubase = 0;
      for (int item = blockIdx.x; item < p.n_items_kv && ok; item += gridDim.x, item_par ^= 1) {
        const Item it = decode(item);
        if (!mbar_wait(kv_empty, item_par ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, -1)) { ok = false; break; }
        mbar_expect_tx(kv_full, 2 * AB_TILE);
        tma2d(sK, &map_k, kv_full, it.kvh * AB_HD, it.key0);
        tma2d(sV, &map_v, kv_full, it.kvh * AB_HD, it.key0);
        for (int u = 0; u < it.nu && ok; ++u) {
          const long long ug = ubase + u;
          const int stage = (int)(ug % KV_STAGES);
          const uint32_t phase = (uint32_t)((ug / KV_STAGES) & 1);
          if (!mbar_wait(&st_empty[stage], phase ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, u)) { ok = false; break; }
          int qi, head;
          unit_coords(it, u, qi, head);
          const int qrow = it.b * p.S + qi * 128;
          const size_t vidx = ((size_t)it.b * p.H + head) * p.S + qi * 128;
          mbar_expect_tx(&st_full[stage], 2 * AB_TILE + 1024);
          tma2d(sQD + stage * 2 * AB_TILE, &map_q, &st_full[stage], head * AB_HD, qrow);
          tma2d(sQD + stage * 2 * AB_TILE + AB_TILE, &map_do, &st_full[stage], head * AB_HD, qrow);
          bulk_g2s(sVec + stage * 256, p.lse + vidx, 512, &st_full[stage]);
          bulk_g2s(sVec + stage * 256 + 128, p.Dsum + vidx, 512, &st_full[stage]);
        }
        ubase += it.nu;
      }
      if (!ok) {
        mbar_drain(kv_full, 0);
        mbar_drain(kv_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) mbar_drain(&st_full[s], 0), mbar_drain(&st_full[s], 1);
      }
    }
  } else if (warp == 1) {
    // scores: S^T(u) and dP^T(u) as soon as the previous unit's scores have been pulled into registers
    if (lane == 0) {
      constexpr uint32_t IDESC_T = make_idesc_bf16(128, 128, 0, 0);    // K Q^T and V dO^T
      const uint32_t sk = smem_u32(sK), sv = smem_u32(sV);
      bool ok = true;
      uint32_t item_par = 0;
      long long ubase = 0;
      for (int item = blockIdx.x; item < p.n_items_kv && ok; item += gridDim.x, item_par ^= 1) {
        const Item it = decode(item);
        if (!mbar_wait(kv_full, item_par, abort_flag, p.status, ST_WAIT_FULL, -1)) { ok = false; break; }
        for (int u = 0; u < it.nu && ok; ++u) {
          const long long ug = ubase + u;
          const int stage = (int)(ug % KV_STAGES);
          if (ug > 0 && !mbar_wait(s_free, (uint32_t)((ug - 1) & 1), abort_flag, p.status, ST_WAIT_TMEM_EMPTY, u)) { ok = false; break; }
          if (!mbar_wait(&st_full[stage], (uint32_t)((ug / KV_STAGES) & 1), abort_flag, p.status, ST_WAIT_FULL, u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sq = smem_u32(sQD + stage * 2 * AB_TILE), sdo = sq + AB_TILE;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem_base, make_smem_desc(sk + k * 32, 16, 1024), make_smem_desc(sq + k * 32, 16, 1024), IDESC_T, k > 0);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem_base + 128, make_smem_desc(sv + k * 32, 16, 1024), make_smem_desc(sdo + k * 32, 16, 1024), IDESC_T, k > 0);
          umma_commit(s_full);
        }
        ubase += it.nu;
      }
    }
  } else if (warp == 2) {
    // gradients: dV += P^T dO and dK += dS^T Q once both softmax groups have stored their halves of P^T / dS^T
    if (lane == 0) {
      constexpr uint32_t IDESC_A = make_idesc_bf16(128, 64, 0, 1);     // A from TMEM; B (dO, Q) read N(=hd)-contiguous
      bool ok = true;
      uint32_t item_par = 0;
      long long ubase = 0;
      for (int item = blockIdx.x; item < p.n_items_kv && ok; item += gridDim.x, item_par ^= 1) {
        const Item it = decode(item);
        for (int u = 0; u < it.nu && ok; ++u) {
          const long long ug = ubase + u;
          const int stage = (int)(ug % KV_STAGES);
          if (!mbar_wait(&st_full[stage], (uint32_t)((ug / KV_STAGES) & 1), abort_flag, p.status, ST_WAIT_FULL, u)) { ok = false; break; }
          if (!mbar_wait(p_full, (uint32_t)(ug & 1), abort_flag, p.status, ST_WAIT_MISC, u)) { ok = false; break; }
          if (u == 0) {          // the previous item's dK/dV must have been read out before they are overwritten
            if (!mbar_wait(acc_empty, item_par ^ 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY, item)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sq = smem_u32(sQD + stage * 2 * AB_TILE), sdo = sq + AB_TILE;
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dV += P^T dO
            umma_ts(tmem_base + 448, tmem_base + 256 + k * 8, make_smem_desc(sdo + k * 2048, 8192, 1024), IDESC_A, (u > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dK += dS^T Q
            umma_ts(tmem_base + 384, tmem_base + 320 + k * 8, make_smem_desc(sq + k * 2048, 8192, 1024), IDESC_A, (u > 0 || k > 0) ? 1u : 0u);
          umma_commit(&st_empty[stage]);      // frees the Q/dO stage and tells the softmax groups that P^T / dS^T may be overwritten
        }
        if (ok) {
          umma_commit(acc_full);
          umma_commit(kv_empty);        // every score MMA of the item finished before its probabilities existed, so K_j / V_j are free too
        }
        ubase += it.nu;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int w = (warp - 4) >> 2;                 // this group owns query columns [64 w, 64 w + 64) of every unit
    const int quarter = warp & 3;
    const int kk = quarter * 32 + lane;            // key row within the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + w * 64 + lane_off, tdP = tmem_base + 128 + w * 64 + lane_off;
    const uint32_t tPt = tmem_base + 256 + w * 32 + lane_off, tdSt = tmem_base + 320 + w * 32 + lane_off;
    bool ok = true;
    uint32_t item_par = 0;
    long long ubase = 0;
    for (int item = blockIdx.x; item < p.n_items_kv && ok; item += gridDim.x, item_par ^= 1) {
      const Item it = decode(item);
      const int j = it.j, kvh = it.kvh, key0 = it.key0, nu = it.nu;
      for (int u = 0; u < nu; ++u) {
        const long long ug = ubase + u;
        const int stage = (int)(ug % KV_STAGES);
        if (!mbar_wait(&st_full[stage], (uint32_t)((ug / KV_STAGES) & 1), abort_flag, p.status, ST_WAIT_FULL, u)) { ok = false; break; }
        if (!mbar_wait(s_full, (uint32_t)(ug & 1), abort_flag, p.status, ST_WAIT_TMEM_FULL, u)) { ok = false; break; }
        tc_fence_after();
        int qi, head;
        unit_coords(it, u, qi, head);
        uint32_t s[64], dp[64];
        PGB_TMEM_LD32(tS, (s));
        PGB_TMEM_LD32(tS + 32, (s + 32));
        PGB_TMEM_LD32(tdP, (dp));
        PGB_TMEM_LD32(tdP + 32, (dp + 32));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(s_free);                       // the score buffers may take the next unit
        const float* vl = sVec + stage * 256 + w * 64;
        const float* vd = sVec + stage * 256 + 128 + w * 64;
        const bool diag = qi == j;
        const int qbase = w * 64;
        uint32_t pp[32], pd[32];
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        const float2* vl2 = reinterpret_cast<const float2*>(vl);     // -(log2 lse) of this group's 64 query rows
        const float2* vd2 = reinterpret_cast<const float2*>(vd);     // -D of the same rows
        if (!diag) {
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, vl2[c >> 1]);
            const float2 pr = make_float2(ex2f(tt.x), ex2f(tt.y));
            const float2 dd = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), vd2[c >> 1]));
            pp[c >> 1] = pack_bf16x2(pr.x, pr.y);
            pd[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, vl2[c >> 1]);
            float2 pr = make_float2(ex2f(tt.x), ex2f(tt.y));
            if (qbase + c < kk) pr.x = 0.f;              // query position before the key: masked
            if (qbase + c + 1 < kk) pr.y = 0.f;
            const float2 dd = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), vd2[c >> 1]));
            pp[c >> 1] = pack_bf16x2(pr.x, pr.y);
            pd[c >> 1] = pack_bf16x2(dd.x, dd.y);
          }
        }
        if (ug > 0) {            // the gradient MMAs of the previous unit still read P^T / dS^T until their commit arrives
          const long long pg = ug - 1;
          if (!mbar_wait(&st_empty[(int)(pg % KV_STAGES)], (uint32_t)((pg / KV_STAGES) & 1), abort_flag, p.status, ST_WAIT_EMPTY, u)) { ok = false; break; }
          tc_fence_after();
        }
        PGB_TMEM_ST16(tPt, (pp));
        PGB_TMEM_ST16(tPt + 16, (pp + 16));
        PGB_TMEM_ST16(tdSt, (pd));
        PGB_TMEM_ST16(tdSt + 16, (pd + 16));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full);
      }
      if (ok && mbar_wait(acc_full, item_par, abort_flag, p.status, ST_WAIT_MISC, nu)) {
        tc_fence_after();
        // group 0 writes dK, group 1 writes dV
        const uint32_t tA = tmem_base + (w == 0 ? 384 : 448) + lane_off;
        __nv_bfloat16* out = (w == 0 ? p.dk + (size_t)(key0 + kk) * p.lddk : p.dv + (size_t)(key0 + kk) * p.lddv) + kvh * AB_HD;
        const bool acc = (w == 1) && p.accumulate_dv;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t o[32];
          PGB_TMEM_LD32(tA + h * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[c + e]) * (w == 0 ? p.scale : 1.f);
            if (acc) {
              uint4 q = *reinterpret_cast<const uint4*>(out + h * 32 + c);
              float2 a0 = unpack_bf16x2(q.x), a1 = unpack_bf16x2(q.y), a2 = unpack_bf16x2(q.z), a3 = unpack_bf16x2(q.w);
              f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y; f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
            }
            *reinterpret_cast<uint4*>(out + h * 32 + c) =
                make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          }
        }
        tc_fence_before();
        mbar_arrive(acc_empty);
      } else {
        ok = false;
      }
      ubase += nu;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static CUtensorMap bwd_map(const void* ptr, long long ld, int cols, long long rows, int box_rows) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld * 2};
  uint32_t box[2] = {AB_HD, (uint32_t)box_rows};
  return make_tmap_bf16(ptr, 2, dims, strides, box);
}

void attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, float* dsum, void* dq, void* dk, void* dv,
              long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk, long long lddv, int B, int S,
              int H, int Hkv, int hd, int accumulate_dv, int* status, cudaStream_t st) {
  if (hd != AB_HD) throw std::runtime_error("attention kernel is specialised for head_dim 64");
  if (S % 128) throw std::runtime_error("attention kernel needs seq_len to be a multiple of 128");
  const long long T = (long long)B * S;
  AttnBwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.n_qt = S / 128;
  p.group = H / Hkv;
  p.scale = 1.f / sqrtf((float)hd);
  p.scale_log2 = p.scale * LOG2E;
  p.O = (const __nv_bfloat16*)o; p.dO = (const __nv_bfloat16*)d_o;
  p.ldo = ldo; p.lddo = lddo;
  p.lse = lse; p.Dsum = dsum;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.lddq = lddq; p.lddk = lddk; p.lddv = lddv;
  p.accumulate_dv = accumulate_dv;
  p.status = status;
  p.n_items_q = p.n_qt * B * H;
  p.n_items_kv = p.n_qt * B * Hkv;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  static bool configured[64] = {};          // the attribute is a per-device property of the kernel
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  {
    const CUtensorMap mq = bwd_map(q, ldq, H * hd, T, 128), mk = bwd_map(k, ldk, Hkv * hd, T, 128), mv = bwd_map(v, ldv, Hkv * hd, T, 128),
                      mdo = bwd_map(d_o, lddo, H * hd, T, 128);
    attn_bwd_dq_kernel<<<std::min(p.n_items_q, sms), DQ_THREADS, DQ_SMEM, st>>>(mq, mk, mv, mdo, p);
  }
  {
    const CUtensorMap mq = bwd_map(q, ldq, H * hd, T, 128), mk = bwd_map(k, ldk, Hkv * hd, T, 128), mv = bwd_map(v, ldv, Hkv * hd, T, 128),
                      mdo = bwd_map(d_o, lddo, H * hd, T, 128);
    attn_bwd_dkdv_kernel<<<std::min(p.n_items_kv, sms), KV_THREADS, KV_SMEM, st>>>(mq, mk, mv, mdo, p);
  }
}

}  // namespace pgb
