// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   D[b][m][n] = epilogue( sum_k A[b][m][k] * B[b][n][k] )
//
// Both operands may be stored K-contiguous ("K-major", [rows][K]) or row-contiguous along M/N
// ("MN-major", [K][rows]); the tensor core reads either through the shared-memory descriptor, so the
// three GEMMs of a linear layer need no transposes:
//   forward  Y = X W^T         A = X  [T][K]  K-major     B = W  [N][K]  K-major
//   dX = dY W                  A = dY [T][N]  K-major     B = W  [N][K]  MN-major (reduction over N)
//   dW = dY^T X                A = dY [T][N]  MN-major    B = X  [T][K]  MN-major (reduction over T, split-K)
// It replaces the cuBLAS calls of the reference's GEMM engine
// (parameter-golf-rs/crates/pg-kernels/src/gemm.rs:158-179,501-698) and the elementwise kernels that
// follow them, which become epilogues here.
//
// CTA = 10 warps: warp 0 issues TMA loads, warp 1 owns TMEM and issues the MMAs (one elected lane),
// warps 2..9 read the accumulator back (tcgen05.ld, one row per thread) and run the epilogue. Two
// accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
// Tile 128 x BN x 64, BN in {128, 256}; grid = min(#tiles, #SMs); tile index = n fastest so CTAs
// working at the same time share the rows of the large operand in L2.
#include "common.cuh"
#include "pgb.h"
#include "tma_host.h"

namespace pgb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 320;     // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)

struct GemmKernelParams {
  int M, N, K, batch;
  int tiles_m, tiles_n, splits, kb_per_split, kb_total;
  long long ldd, stride_d;
  long long ld_aux, stride_aux;
  void* D;
  void* D2;
  const void* aux;
  const float* colscale;
  float alpha, beta, slope;
  int* status;
  const int* wait_flag;   // optional: B (the weights) is valid once *wait_flag >= wait_value (peer ranks push it)
  int wait_value;
  int seg_rows[2];        // fp32 epilogues: rows >= seg_rows[k] (> 0) are written to seg_D[k] as row m - seg_rows[k]
  float* seg_D[2];
  int aux_l2_prefetch;     // the producer warp pulls the next tile's second operand into L2 through `map_x`
  const float* batch_sumsq;   // optional: alpha and beta of batch b are multiplied by 1 / (sqrt(batch_sumsq[b]) + 1e-7) ^ sumsq_pow
  int sumsq_pow;
  const float* rope_cos;      // EPI_QKV_NORM_ROPE
  const float* rope_sin;
  const float* head_gain;
  int q_heads, qk_heads, rope_half, seq_len;
  float norm_eps;
};

constexpr int STG_PITCH = 64;
constexpr int STG_WARP_BYTES = 32 * STG_PITCH;      // one 32-row x 32-column bf16 chunk

// Epilogue staging: two chunk-sized slots per epilogue warp. A slot first receives a chunk of the epilogue's second
// operand (cp.async, two chunks ahead of its use), is read, then stages the output chunk in place.
template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STG_BYTES = 8 * 2 * STG_WARP_BYTES;
  static constexpr int TOTAL = TILE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + STG_BYTES;
};

__device__ __forceinline__ float act_fn(float x, float slope) { return x >= 0.f ? x : slope * x; }

template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const GemmKernelParams& p, float alpha, float beta, int b, int m, int n0, const uint32_t (&r)[32]) {
  // One thread: row m, columns n0 .. n0+31 of batch b. Caller guarantees m < M.
  const bool full = (n0 + 32 <= p.N);
  const long long off = (long long)b * p.stride_d + (long long)m * p.ldd + n0;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);

  if constexpr (EPI == EPI_F32 || EPI == EPI_F32_ATOMIC) {
    float* d = reinterpret_cast<float*>(p.D) + off;
    // one product, several output matrices (e.g. the packed QKV weight gradient lands in three gradient banks)
    if (p.seg_rows[1] > 0 && m >= p.seg_rows[1]) d = p.seg_D[1] + (long long)b * p.stride_d + (long long)(m - p.seg_rows[1]) * p.ldd + n0;
    else if (p.seg_rows[0] > 0 && m >= p.seg_rows[0]) d = p.seg_D[0] + (long long)b * p.stride_d + (long long)(m - p.seg_rows[0]) * p.ldd + n0;
    if (full && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 q = make_float4(v[i] * alpha, v[i + 1] * alpha, v[i + 2] * alpha, v[i + 3] * alpha);
        if constexpr (EPI == EPI_F32) *reinterpret_cast<float4*>(d + i) = q;
        else atomicAdd(reinterpret_cast<float4*>(d + i), q);
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (n0 + i < p.N) {
          if constexpr (EPI == EPI_F32) d[i] = v[i] * alpha;
          else atomicAdd(d + i, v[i] * alpha);
        }
    }
    return;
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + off;
    const long long aoff = (long long)b * p.stride_aux + (long long)m * p.ld_aux + n0;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
    float a[32];
    if constexpr (EPI == EPI_AXPBY_BF16 || EPI == EPI_RESID_BF16 || EPI == EPI_MUL_ACTGRAD) {
      const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(p.aux) + aoff;
      if (vec && ((reinterpret_cast<uintptr_t>(ap) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const uint4 q = *reinterpret_cast<const uint4*>(ap + i);
          float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
          a[i] = f0.x; a[i + 1] = f0.y; a[i + 2] = f1.x; a[i + 3] = f1.y;
          a[i + 4] = f2.x; a[i + 5] = f2.y; a[i + 6] = f3.x; a[i + 7] = f3.y;
        }
      } else {
        for (int i = 0; i < 32; ++i) a[i] = (n0 + i < p.N) ? __bfloat162float(ap[i]) : 0.f;
      }
    }
    float o[32];
    float o2[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if constexpr (EPI == EPI_BF16) o[i] = v[i] * alpha;
      if constexpr (EPI == EPI_AXPBY_BF16) o[i] = alpha * v[i] + beta * a[i];
      if constexpr (EPI == EPI_RESID_BF16) o[i] = a[i] + ((n0 + i < p.N) ? p.colscale[n0 + i] : 0.f) * v[i];
      if constexpr (EPI == EPI_ACT_SQ) {
        // the pre-activation is stored in bf16 and the activation is computed from that stored value,
        // so the backward pass (which reads it back) sees exactly the same argument
        float h = __bfloat162float(__float2bfloat16(v[i]));
        float t = act_fn(h, p.slope);
        o[i] = h;
        o2[i] = t * t;
      }
      if constexpr (EPI == EPI_MUL_ACTGRAD) {
        float h = a[i];
        o[i] = v[i] * 2.f * act_fn(h, p.slope) * (h >= 0.f ? 1.f : p.slope);
      }
    }
    if (vec) {
#pragma unroll
      for (int i = 0; i < 32; i += 8)
        *reinterpret_cast<uint4*>(d + i) = make_uint4(pack_bf16x2(o[i], o[i + 1]), pack_bf16x2(o[i + 2], o[i + 3]),
                                                      pack_bf16x2(o[i + 4], o[i + 5]), pack_bf16x2(o[i + 6], o[i + 7]));
      if constexpr (EPI == EPI_ACT_SQ) {
        __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(p.D2) + off;
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(d2 + i) = make_uint4(pack_bf16x2(o2[i], o2[i + 1]), pack_bf16x2(o2[i + 2], o2[i + 3]),
                                                         pack_bf16x2(o2[i + 4], o2[i + 5]), pack_bf16x2(o2[i + 6], o2[i + 7]));
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (n0 + i < p.N) {
          d[i] = __float2bfloat16(o[i]);
          if constexpr (EPI == EPI_ACT_SQ) (reinterpret_cast<__nv_bfloat16*>(p.D2) + off)[i] = __float2bfloat16(o2[i]);
        }
    }
  }
}

// Aligned bf16 epilogue with coalesced global traffic. A thread owns one accumulator row, but 16-byte accesses of 32
// different rows per instruction touch half a sector each; here rows are exchanged through a per-warp shared-memory
// tile (32 rows x 64 B) so that every global load/store instruction covers 8 rows x 64 contiguous bytes.
// `auxs` is this chunk of the second operand, already in shared memory in the same swizzled layout (cp.async wrote it).
// The tile is XOR-swizzled: the 16-byte piece p of row r sits at piece p ^ ((r >> 1) & 3). Both access patterns are
// then free of bank conflicts (8 consecutive rows x one piece, and 2 consecutive rows x 4 pieces, each cover all 32
// banks once); a padded pitch can only satisfy one of the two.
__device__ __forceinline__ int stg_off(int row, int piece) { return row * STG_PITCH + ((piece ^ ((row >> 1) & 3)) << 4); }

template <int EPI>
__device__ __forceinline__ void epilogue_chunk_staged(const GemmKernelParams& p, float alpha, float beta, int b, int m_base, int lane, int n0, const uint32_t (&r)[32],
                                                      const uint8_t* auxs, uint8_t* stg) {
  constexpr bool HAS_AUX = (EPI == EPI_AXPBY_BF16 || EPI == EPI_RESID_BF16 || EPI == EPI_MUL_ACTGRAD);
  const int srow = lane >> 2, spc = lane & 3;
  float a[32];
  if constexpr (HAS_AUX) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 q = *reinterpret_cast<const uint4*>(auxs + stg_off(lane, i));
      const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
      a[8 * i] = f0.x; a[8 * i + 1] = f0.y; a[8 * i + 2] = f1.x; a[8 * i + 3] = f1.y;
      a[8 * i + 4] = f2.x; a[8 * i + 5] = f2.y; a[8 * i + 6] = f3.x; a[8 * i + 7] = f3.y;
    }
  }
  float o[32], o2[32];
  float cs[32];
  if constexpr (EPI == EPI_RESID_BF16) {
    if ((reinterpret_cast<uintptr_t>(p.colscale + n0) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(p.colscale + n0) + i);
        cs[4 * i] = t.x; cs[4 * i + 1] = t.y; cs[4 * i + 2] = t.z; cs[4 * i + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) cs[i] = p.colscale[n0 + i];
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float v = __uint_as_float(r[i]);
    if constexpr (EPI == EPI_BF16) o[i] = v * alpha;
    if constexpr (EPI == EPI_AXPBY_BF16) o[i] = alpha * v + beta * a[i];
    if constexpr (EPI == EPI_RESID_BF16) o[i] = a[i] + cs[i] * v;
    if constexpr (EPI == EPI_MUL_ACTGRAD) {
      const float h = a[i];
      o[i] = v * 2.f * act_fn(h, p.slope) * (h >= 0.f ? 1.f : p.slope);
    }
  }
  uint32_t pk[16], pk2[16];
  bool packed = false;
  if constexpr (EPI == EPI_ACT_SQ) {
    // With a slope that is zero or a power of two, slope*h is exact in bf16 and the square of a bf16 value rounds
    // once either way, so the whole activation can run on packed bf16 pairs with bit-identical results.
    if ((__float_as_uint(p.slope) & 0x007fffffu) == 0u && p.slope >= 0.f && p.slope < 1.f) {
      packed = true;
      const __nv_bfloat162 sl = __float2bfloat162_rn(p.slope);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 hb = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        const __nv_bfloat162 t = __hmax2(hb, __hmul2(hb, sl));
        const __nv_bfloat162 sq = __hmul2(t, t);
        pk[i] = *reinterpret_cast<const uint32_t*>(&hb);
        pk2[i] = *reinterpret_cast<const uint32_t*>(&sq);
      }
    }
  }
  if (!packed) {
    if constexpr (EPI == EPI_ACT_SQ) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float h = __bfloat162float(__float2bfloat16(__uint_as_float(r[i])));
        const float t = act_fn(h, p.slope);
        o[i] = h;
        o2[i] = t * t;
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      pk[i] = pack_bf16x2(o[2 * i], o[2 * i + 1]);
      if constexpr (EPI == EPI_ACT_SQ) pk2[i] = pack_bf16x2(o2[2 * i], o2[2 * i + 1]);
    }
  }
  auto put = [&](const uint32_t (&x)[16], void* base) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<uint4*>(stg + stg_off(lane, i)) = make_uint4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    __syncwarp();
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(base) + (long long)b * p.stride_d + n0 + spc * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = m_base + i * 8 + srow;
      if (row < p.M) *reinterpret_cast<uint4*>(d + (long long)row * p.ldd) = *reinterpret_cast<const uint4*>(stg + stg_off(i * 8 + srow, spc));
    }
    __syncwarp();
  };
  put(pk, p.D);
  if constexpr (EPI == EPI_ACT_SQ) put(pk2, p.D2);
}

// Half-split rotary on the first 2*HALF of a head's 64 values, tables [seq_len][HALF] (the layout of `qk_norm_rope_fwd`).
template <int HALF>
__device__ __forceinline__ void rope_head(float (&x)[64], const float* __restrict__ cosT, const float* __restrict__ sinT, int pos) {
  if constexpr (HALF > 0) {
    const float4* c4 = reinterpret_cast<const float4*>(cosT + (size_t)pos * HALF);
    const float4* s4 = reinterpret_cast<const float4*>(sinT + (size_t)pos * HALF);
#pragma unroll
    for (int i = 0; i < HALF; i += 4) {
      const float4 c = __ldg(c4 + i / 4), sn = __ldg(s4 + i / 4);
      const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x1 = x[i + e], x2 = x[i + e + HALF];
        x[i + e] = x1 * cc[e] + x2 * ss[e];
        x[i + e + HALF] = x2 * cc[e] - x1 * ss[e];
      }
    }
  }
}

// EPI_QKV_NORM_ROPE on one head (two 32-column chunks) of 32 rows: the raw projection goes to D; for query and key heads the
// RMS-normalised, rotated and (queries) gain-scaled head goes to D2. The norm is taken of the bf16-rounded projection, the
// values the backward recomputes it from. Replaces a pass over the projection (`qk_norm_rope_fwd`, kept for the LoRA path);
// same math as the reference's fused QK kernels (parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:2640-2822).
__device__ __forceinline__ void epilogue_qkv_head_staged(const GemmKernelParams& p, int b, int m_base, int lane, int n0, const uint32_t (&ra)[32],
                                                         const uint32_t (&rb)[32], uint8_t* stg) {
  const int srow = lane >> 2, spc = lane & 3;
  auto put = [&](const uint32_t* x, void* base, int col0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<uint4*>(stg + stg_off(lane, i)) = make_uint4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    __syncwarp();
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(base) + (long long)b * p.stride_d + col0 + spc * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = m_base + i * 8 + srow;
      if (row < p.M) *reinterpret_cast<uint4*>(d + (long long)row * p.ldd) = *reinterpret_cast<const uint4*>(stg + stg_off(i * 8 + srow, spc));
    }
    __syncwarp();
  };
  uint32_t pk[32];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    pk[i] = pack_bf16x2(__uint_as_float(ra[2 * i]) * p.alpha, __uint_as_float(ra[2 * i + 1]) * p.alpha);
    pk[16 + i] = pack_bf16x2(__uint_as_float(rb[2 * i]) * p.alpha, __uint_as_float(rb[2 * i + 1]) * p.alpha);
  }
  put(pk, p.D, n0);
  put(pk + 16, p.D, n0 + 32);
  const int head = n0 >> 6;
  if (head >= p.qk_heads) return;                  // value heads: the projection as it is (warp-uniform)
  float x[64];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float2 f = unpack_bf16x2(pk[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
    ss += f.x * f.x + f.y * f.y;
  }
  const float inv = rsqrtf(ss * (1.f / 64.f) + p.norm_eps);
#pragma unroll
  for (int i = 0; i < 64; ++i) x[i] *= inv;
  const int row = min(m_base + lane, p.M - 1);
  const int pos = row % p.seq_len;
  switch (p.rope_half) {
    case 8: rope_head<8>(x, p.rope_cos, p.rope_sin, pos); break;
    case 16: rope_head<16>(x, p.rope_cos, p.rope_sin, pos); break;
    case 32: rope_head<32>(x, p.rope_cos, p.rope_sin, pos); break;
    default: break;
  }
  const float g = (head < p.q_heads && p.head_gain != nullptr) ? p.head_gain[head] : 1.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) pk[i] = pack_bf16x2(x[2 * i] * g, x[2 * i + 1] * g);     // one rounding, at the store
  put(pk, p.D2, n0);
  put(pk + 16, p.D2, n0 + 32);
}

template <int BN, bool A_KMAJOR, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_x, const GemmKernelParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = 2 * BN;            // 256 or 512: two accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::TILE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 256);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n * p.splits;
  const int total_tiles = tiles_per_batch * p.batch;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (p.wait_flag != nullptr) {
        // The weight operand is written by peer GPUs (parameter all-gather fused here): poll the per-layer
        // ready counter, bounded, then order the peer's generic-proxy stores before this CTA's TMA reads.
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.wait_flag) : "memory");
        if (seen < p.wait_value) {
          const uint64_t t0 = globaltimer_ns();
          while (true) {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.wait_flag) : "memory");
            if (seen >= p.wait_value) break;
            if (globaltimer_ns() - t0 > PGB_WAIT_LIMIT_NS) {
              *abort_flag = 1;
              report(p.status, ST_WAIT_FLAG, p.wait_value);
              ok = false;
              break;
            }
            __nanosleep(128);
          }
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        int r = tile - b * tiles_per_batch;
        const int split = r / (p.tiles_m * p.tiles_n);
        r -= split * p.tiles_m * p.tiles_n;
        const int tm = r / p.tiles_n, tn = r - tm * p.tiles_n;
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        if (p.aux_l2_prefetch && tile + (int)gridDim.x < total_tiles) {
          // The epilogue warps read the second operand of this CTA's NEXT tile while they finish this one; ask for it now
          // so that those reads find it in L2.
          const int nt = tile + gridDim.x;
          const int pb = nt / tiles_per_batch;
          int pr = nt - pb * tiles_per_batch;
          pr -= (pr / (p.tiles_m * p.tiles_n)) * p.tiles_m * p.tiles_n;
          const int ptm = pr / p.tiles_n, ptn = pr - ptm * p.tiles_n;
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            if (ptn * BN + 64 * j < p.N) tma_prefetch_l2_3d(&map_x, ptn * BN + 64 * j, ptm * BM, pb);
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, ST_WAIT_EMPTY, kb)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if constexpr (A_KMAJOR) {
            tma_load_3d(sa, &map_a, &full_bar[stage], kb * BK, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sa + j * 8192, &map_a, &full_bar[stage], m0 + 64 * j, kb * BK, b);
          }
          if constexpr (B_KMAJOR) {
            tma_load_3d(sb, &map_b, &full_bar[stage], kb * BK, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * 8192, &map_b, &full_bar[stage], n0 + 64 * j, kb * BK, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: every stage whose load may still be in flight
        for (int s = 0; s < STAGES; ++s) mbar_drain(&full_bar[s], (s < stage) ? phase : (phase ^ 1));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, A_KMAJOR ? 0 : 1, B_KMAJOR ? 0 : 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int r = tile % tiles_per_batch;
        const int split = r / (p.tiles_m * p.tiles_n);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY, tile)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, ST_WAIT_FULL, kb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_KMAJOR ? make_smem_desc(sa + k * 32, 16, 1024) : make_smem_desc(sa + k * 2048, 8192, 1024);
            const uint64_t db = B_KMAJOR ? make_smem_desc(sb + k * 32, 16, 1024) : make_smem_desc(sb + k * 2048, 8192, 1024);
            umma_ss(tmem_d, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;             // which half of the tile's columns
    uint8_t* slots = smem + S::TILE_BYTES + 256 + (warp - 2) * 2 * STG_WARP_BYTES;
    const bool staged_ok = (p.ldd % 8 == 0) && (p.stride_d % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                           (p.aux == nullptr || ((p.ld_aux % 8 == 0) && (p.stride_aux % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.aux) & 15) == 0))) &&
                           (p.D2 == nullptr || ((reinterpret_cast<uintptr_t>(p.D2) & 15) == 0));
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr bool HAS_AUX = (EPI == EPI_AXPBY_BF16 || EPI == EPI_RESID_BF16 || EPI == EPI_MUL_ACTGRAD);
    constexpr int CH = BN / 64;                   // 32-column chunks per epilogue warp (the two warps of a quarter split the columns)
    constexpr bool BF16_OUT = !(EPI == EPI_F32 || EPI == EPI_F32_ATOMIC);
    const int c_begin = half * CH;
    auto tile_coords = [&](int tile, int& b, int& tm, int& tn) {
      b = tile / tiles_per_batch;
      int r = tile - b * tiles_per_batch;
      const int split = r / (p.tiles_m * p.tiles_n);
      r -= split * p.tiles_m * p.tiles_n;
      tm = r / p.tiles_n;
      tn = r - tm * p.tiles_n;
    };
    // Second operand: a 32-row x 32-column chunk goes into one of this warp's two staging slots with 16-byte asynchronous
    // copies (8 rows x 64 contiguous bytes per instruction), one commit group per chunk, two chunks ahead of its use
    // (across the tile boundary too), so its DRAM latency hides behind the chunks processed meanwhile. cp.async is used
    // rather than loads into registers because pending register loads share the warp's few scoreboard counters with the
    // shared-memory and tensor-memory traffic of those chunks, which then wait for DRAM as well. The slot is read by the
    // thread that owns the row, reused in place to stage the output chunk, and refilled once the stores have read it.
    const bool aux_async = HAS_AUX && staged_ok;
    auto issue_aux = [&](int b, int tm, int tn, int cc, uint8_t* slot) {
      if constexpr (HAS_AUX) {
        const int n0 = tn * BN + (c_begin + cc) * 32;
        if (n0 + 32 <= p.N) {
          const int m_base = tm * BM + quarter * 32;
          const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)b * p.stride_aux + n0 + (lane & 3) * 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = m_base + i * 8 + (lane >> 2);
            if (row < p.M) cp_async16(slot + stg_off(i * 8 + (lane >> 2), lane & 3), ap + (long long)row * p.ld_aux);
          }
        }
        cp_async_commit();          // one group per chunk, also when nothing was copied: the wait below counts groups
      }
    };
    static_assert(CH % 2 == 0, "slot parity follows the chunk index within the tile");
    if (aux_async && blockIdx.x < total_tiles) {
      int b0, tm0, tn0;
      tile_coords(blockIdx.x, b0, tm0, tn0);
      issue_aux(b0, tm0, tn0, 0, slots);
      issue_aux(b0, tm0, tn0, 1, slots + STG_WARP_BYTES);
    }
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int b, tm, tn;
      tile_coords(tile, b, tm, tn);
      const int next = tile + gridDim.x;
      int nb = 0, ntm = 0, ntn = 0;
      if (next < total_tiles) tile_coords(next, nb, ntm, ntn);
      const int m = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      const int m_base = tm * BM + quarter * 32;
      float alpha = p.alpha, beta = p.beta;
      if (p.batch_sumsq != nullptr) {
        // Newton-Schulz on an un-normalised input: the matrix norm enters as a per-matrix factor of the whole output
        const float inv = 1.f / (sqrtf(p.batch_sumsq[b]) + 1e-7f);
        const float f = p.sumsq_pow == 2 ? inv * inv : inv;
        alpha *= f;
        beta *= f;
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, ST_WAIT_TMEM_FULL, tile)) { ok = false; break; }
      tc_fence_after();
      if constexpr (EPI == EPI_QKV_NORM_ROPE) {
        // one head (two chunks) at a time: the norm needs all 64 values of the row before either chunk can be written
#pragma unroll
        for (int cc = 0; cc < CH; cc += 2) {
          const int c = c_begin + cc;
          const int n0 = tn * BN + c * 32;
          if (n0 < p.N) {                         // warp-uniform; N is a multiple of 64 (checked on the host)
            uint32_t ra[32], rb[32];
            PGB_TMEM_LD32(taddr + c * 32, ra);
            PGB_TMEM_LD32(taddr + c * 32 + 32, rb);
            PGB_TMEM_WAIT_LD32(ra);
            PGB_TMEM_WAIT_LD32(rb);
            epilogue_qkv_head_staged(p, b, m_base, lane, n0, ra, rb, slots);
          }
        }
      } else {
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) {
        const int c = c_begin + cc;
        const int n0 = tn * BN + c * 32;
        uint8_t* slot = slots + (cc & 1) * STG_WARP_BYTES;
        if (n0 < p.N) {                           // warp-uniform
          uint32_t rr[32];
          PGB_TMEM_LD32(taddr + c * 32, rr);
          if constexpr (HAS_AUX) {
            if (aux_async) {                      // two groups are pending; this chunk's is the older one
              cp_async_wait<1>();
              __syncwarp();
            }
          }
          PGB_TMEM_WAIT_LD32(rr);
          if constexpr (BF16_OUT) {
            if (staged_ok && n0 + 32 <= p.N && (aux_async || !HAS_AUX)) epilogue_chunk_staged<EPI>(p, alpha, beta, b, m_base, lane, n0, rr, slot, slot);
            else if (m < p.M) epilogue_chunk<EPI>(p, alpha, beta, b, m, n0, rr);
          } else {
            if (m < p.M) epilogue_chunk<EPI>(p, alpha, beta, b, m, n0, rr);
          }
        }
        if constexpr (HAS_AUX) {
          if (aux_async) {
            __syncwarp();                         // every lane is done with this slot
            if (cc + 2 < CH) issue_aux(b, tm, tn, cc + 2, slot);
            else if (next < total_tiles) issue_aux(nb, ntm, ntn, cc + 2 - CH, slot);
            else cp_async_commit();
          }
        }
      }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side --------------------------------------------------------------------------------------------------
static int g_num_sms = 0;

static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

static CUtensorMap operand_map(const void* ptr, bool kmajor, int rows, int K, long long ld, long long batch_stride, int batch,
                               int tile_rows) {
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  if (kmajor) {         // memory [batch][rows][K]
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)rows; dims[2] = (uint64_t)batch;
    box[0] = BK; box[1] = (uint32_t)tile_rows; box[2] = 1;
  } else {              // memory [batch][K][rows]
    dims[0] = (uint64_t)rows; dims[1] = (uint64_t)K; dims[2] = (uint64_t)batch;
    box[0] = 64; box[1] = BK; box[2] = 1;
  }
  strides[0] = (uint64_t)ld * 2;
  strides[1] = (uint64_t)(batch > 1 ? batch_stride : (long long)dims[1] * ld) * 2;
  return make_tmap_bf16(ptr, 3, dims, strides, box);
}

template <int BN, bool AK, bool BKM, int EPI>
static void launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mx, const GemmKernelParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<BN, AK, BKM, EPI>;
  static bool configured[64] = {};          // the attribute is a per-device property of the kernel
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(ma, mb, mx, p);
}

template <int BN, int EPI>
static void launch_major(const GemmArgs& a, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mx, const GemmKernelParams& p, int grid,
                         cudaStream_t stream) {
  if (a.a_kmajor && a.b_kmajor) launch_variant<BN, true, true, EPI>(ma, mb, mx, p, grid, stream);
  else if (a.a_kmajor && !a.b_kmajor) launch_variant<BN, true, false, EPI>(ma, mb, mx, p, grid, stream);
  else if (!a.a_kmajor && a.b_kmajor) launch_variant<BN, false, true, EPI>(ma, mb, mx, p, grid, stream);
  else launch_variant<BN, false, false, EPI>(ma, mb, mx, p, grid, stream);
}

template <int BN>
static void launch_epi(const GemmArgs& a, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mx, const GemmKernelParams& p, int grid,
                       cudaStream_t stream) {
  switch (a.epi) {
    case EPI_BF16: launch_major<BN, EPI_BF16>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_F32: launch_major<BN, EPI_F32>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_F32_ATOMIC: launch_major<BN, EPI_F32_ATOMIC>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_AXPBY_BF16: launch_major<BN, EPI_AXPBY_BF16>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_RESID_BF16: launch_major<BN, EPI_RESID_BF16>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_ACT_SQ: launch_major<BN, EPI_ACT_SQ>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_MUL_ACTGRAD: launch_major<BN, EPI_MUL_ACTGRAD>(a, ma, mb, mx, p, grid, stream); break;
    case EPI_QKV_NORM_ROPE:
      if (!(a.a_kmajor && a.b_kmajor)) throw std::runtime_error("gemm: the QKV epilogue takes row-major activations and [N][K] weights");
      launch_variant<BN, true, true, EPI_QKV_NORM_ROPE>(ma, mb, mx, p, grid, stream);
      break;
    default: throw std::runtime_error("gemm: unknown epilogue");
  }
}

void gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) throw std::runtime_error("gemm: empty problem");
  if ((a.lda % 8) || (a.ldb % 8)) throw std::runtime_error("gemm: leading dimensions must be multiples of 8 elements");
  const int bn = (a.N > 128) ? 256 : 128;
  GemmKernelParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + bn - 1) / bn;
  p.kb_total = (a.K + BK - 1) / BK;
  int splits = a.splits;
  if (splits <= 0) {
    splits = 1;
    if (a.epi == EPI_F32_ATOMIC) {
      // Fill the machine when the output is small and K is long, in whole waves: with `base` output tiles, base * splits
      // work items run in ceil(items / SMs) rounds, so 2 * SMs + a few items would cost a third round for nothing.
      // Two rounds are preferred (the second tile's main loop hides the first one's epilogue), then one, then three.
      const int base = p.tiles_m * p.tiles_n * a.batch, sms = num_sms();
      const int max_splits = std::max(1, p.kb_total / 8);
      double best_eff = 0.0;
      for (int waves : {2, 1, 3}) {
        const int sp = std::min(max_splits, std::max(1, waves * sms / base));
        const int items = base * sp;
        const double eff = (double)items / ((double)((items + sms - 1) / sms) * sms);
        if (eff > best_eff + 0.02) {
          best_eff = eff;
          splits = sp;
        }
      }
    }
  }
  if (splits > 1 && a.epi != EPI_F32_ATOMIC) throw std::runtime_error("gemm: split-K needs the atomic fp32 epilogue");
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  p.ldd = a.ldd; p.stride_d = a.stride_d;
  p.ld_aux = a.ld_aux; p.stride_aux = a.stride_aux;
  p.D = a.D; p.D2 = a.D2; p.aux = a.aux; p.colscale = a.colscale;
  p.alpha = a.alpha; p.beta = a.beta; p.slope = a.slope;
  p.status = a.status;
  p.wait_flag = a.wait_flag;
  p.wait_value = a.wait_value;
  p.batch_sumsq = a.batch_sumsq;
  p.sumsq_pow = a.sumsq_pow;
  for (int k = 0; k < 2; ++k) {
    p.seg_rows[k] = a.seg_rows[k];
    p.seg_D[k] = a.seg_D[k];
  }
  if ((a.seg_rows[0] > 0 || a.seg_rows[1] > 0) && !(a.epi == EPI_F32 || a.epi == EPI_F32_ATOMIC))
    throw std::runtime_error("gemm: row segments need an fp32 epilogue");
  p.rope_cos = a.rope_cos;
  p.rope_sin = a.rope_sin;
  p.head_gain = a.head_gain;
  p.q_heads = a.q_heads;
  p.qk_heads = a.q_heads + a.kv_heads;
  p.rope_half = a.rope_dims / 2;
  p.seq_len = a.seq_len;
  p.norm_eps = a.norm_eps;
  if (a.epi == EPI_QKV_NORM_ROPE) {
    const bool rope_ok = a.rope_dims == 0 || ((a.rope_dims == 16 || a.rope_dims == 32 || a.rope_dims == 64) && a.rope_cos && a.rope_sin &&
                                              (reinterpret_cast<uintptr_t>(a.rope_cos) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.rope_sin) & 15) == 0);
    if (a.batch != 1 || a.D2 == nullptr || a.N != (a.q_heads + 2 * a.kv_heads) * 64 || a.seq_len <= 0 || !rope_ok || (a.ldd % 8) ||
        (reinterpret_cast<uintptr_t>(a.D) & 15) || (reinterpret_cast<uintptr_t>(a.D2) & 15))
      throw std::runtime_error("gemm: the QKV epilogue needs heads of 64, rope_dims in {0,16,32,64}, 16-byte aligned outputs of one row pitch and a sequence length");
  }
  const CUtensorMap ma = operand_map(a.A, a.a_kmajor, a.M, a.K, a.lda, a.stride_a, a.batch, BM);
  const CUtensorMap mb = operand_map(a.B, a.b_kmajor, a.N, a.K, a.ldb, a.stride_b, a.batch, bn);
  const int total = p.tiles_m * p.tiles_n * p.splits * a.batch;
  const int grid = std::min(total, num_sms());
  // L2 prefetch of the epilogue's second operand ([batch][M][N] bf16, row pitch ld_aux) one tile ahead of its readers
  const bool has_aux = a.aux != nullptr && (a.epi == EPI_AXPBY_BF16 || a.epi == EPI_MUL_ACTGRAD);
  p.aux_l2_prefetch = (has_aux && a.ld_aux % 8 == 0 && (a.batch == 1 || a.stride_aux % 8 == 0) &&
                       (reinterpret_cast<uintptr_t>(a.aux) & 15) == 0 && total > grid) ? 1 : 0;
  const CUtensorMap mx = p.aux_l2_prefetch ? operand_map(a.aux, true, a.M, a.N, a.ld_aux, a.stride_aux, a.batch, BM) : ma;
  if (bn == 256) launch_epi<256>(a, ma, mb, mx, p, grid, stream);
  else launch_epi<128>(a, ma, mb, mx, p, grid, stream);
}

}  // namespace pgb
