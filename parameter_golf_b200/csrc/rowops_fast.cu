// Occupancy- and coalescing-tuned versions of the two row kernels that dominated the step profile:
//   * RMSNorm-backward + residual-mix / skip backward, specialised on which terms exist so the plain
//     norm backward carries no accumulators (2 CTAs/SM instead of 1);
//   * per-head RMSNorm + partial RoPE (+ q gain) forward/backward for head_dim 64 with 8 lanes per head
//     vector (one 16-byte load per lane, fully coalesced) instead of one thread per vector.
#include "common.cuh"
#include "pgb.h"

namespace pgb {

namespace {
struct V8 {
  float v[8];
};
__device__ __forceinline__ V8 ldv(const __nv_bfloat16* p) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  V8 r;
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; r.v[4] = c.x; r.v[5] = c.y; r.v[6] = d.x; r.v[7] = d.y;
  return r;
}
__device__ __forceinline__ void stv(__nv_bfloat16* p, const V8& r) {
  *reinterpret_cast<uint4*>(p) =
      make_uint4(pack_bf16x2(r.v[0], r.v[1]), pack_bf16x2(r.v[2], r.v[3]), pack_bf16x2(r.v[4], r.v[5]), pack_bf16x2(r.v[6], r.v[7]));
}
__device__ __forceinline__ V8 ldf(const float* p) {
  V8 r;
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w; r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  return r;
}
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ uint4 ldraw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ V8 cvt8(const uint4& q) {
  V8 r;
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; r.v[4] = c.x; r.v[5] = c.y; r.v[6] = d.x; r.v[7] = d.y;
  return r;
}
}  // namespace

constexpr int RT = 256, RW = 8;

template <int NV>
__device__ __forceinline__ void flush_cols2(float (&acc)[NV][8], float* dst, int d, float* sm) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) sm[warp * (NV * 256) + (j * 32 + lane) * 8 + e] = acc[j][e];
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += RT) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < RW; ++w) s += sm[w * (NV * 256) + c];
    atomicAdd(dst + c, s);
  }
}

template <int NV, bool MIX, bool SKIP>
__global__ void __launch_bounds__(RT, (NV <= 2) ? 2 : 1)
mix_norm_bwd2_kernel(const __nv_bfloat16* __restrict__ d_h, const __nv_bfloat16* __restrict__ d_res, const __nv_bfloat16* __restrict__ x_in,
                     const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ skip,
                     const float* __restrict__ sw, const float* __restrict__ mix, const __nv_bfloat16* __restrict__ add_grad,
                     __nv_bfloat16* __restrict__ d_x, __nv_bfloat16* __restrict__ d_x0, __nv_bfloat16* __restrict__ d_skip, float* __restrict__ d_mix,
                     float* __restrict__ d_sw, int skip_to_dx, int rows, int d, float s, float eps) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float am0[MIX ? NV : 1][8], am1[MIX ? NV : 1][8], asw[SKIP ? NV : 1][8];
  if constexpr (MIX) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) am0[j][e] = am1[j][e] = 0.f;
  }
  if constexpr (SKIP) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) asw[j][e] = 0.f;
  }
  for (int row = blockIdx.x * RW + warp; row < rows; row += gridDim.x * RW) {
    const size_t base = (size_t)row * d;
    V8 xi[NV], dy[NV];
    // every operand of the row is requested before the first reduction, so one DRAM round trip covers them all
    uint4 q_res[NV], q_x0[MIX ? NV : 1], q_x[MIX ? NV : 1], q_acc0[MIX ? NV : 1], q_skip[SKIP ? NV : 1], q_ag[NV];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        const uint4 r_xi = ldraw(x_in + base + c), r_dy = ldraw(d_h + base + c);
        if (d_res) q_res[j] = ldraw(d_res + base + c);
        if constexpr (MIX) {
          q_x0[j] = ldraw(x0 + base + c);
          q_x[j] = ldraw(x + base + c);
          q_acc0[j] = ldraw(d_x0 + base + c);
        }
        if constexpr (SKIP) q_skip[j] = ldraw(skip + base + c);
        if (add_grad) q_ag[j] = ldraw(add_grad + base + c);
        xi[j] = cvt8(r_xi);
        dy[j] = cvt8(r_dy);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ss += xi[j].v[e] * xi[j].v[e];
          dot += xi[j].v[e] * dy[j].v[e];
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float ms = ss / d + eps;
    const float k1 = s * rsqrtf(ms), k2 = dot / (ms * d);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        V8 g;
#pragma unroll
        for (int e = 0; e < 8; ++e) g.v[e] = k1 * (dy[j].v[e] - xi[j].v[e] * k2);
        if (d_res) {
          const V8 r = cvt8(q_res[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) g.v[e] += r.v[e];
        }
        if constexpr (MIX) {
          V8 m0 = ldf(mix + c), m1 = ldf(mix + d + c), b = cvt8(q_x0[j]), a = cvt8(q_x[j]);
          V8 k, w;
          if constexpr (SKIP) {
            k = cvt8(q_skip[j]);
            w = ldf(sw + c);
#pragma unroll
            for (int e = 0; e < 8; ++e) a.v[e] = bfr(a.v[e] + w.v[e] * k.v[e]);
          }
          V8 acc0 = cvt8(q_acc0[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            am0[j][e] += g.v[e] * a.v[e];
            am1[j][e] += g.v[e] * b.v[e];
            acc0.v[e] += m1.v[e] * g.v[e];
            g.v[e] *= m0.v[e];
          }
          stv(d_x0 + base + c, acc0);
          if constexpr (SKIP) {
            V8 ds;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              asw[j][e] += g.v[e] * k.v[e];
              ds.v[e] = w.v[e] * g.v[e];
            }
            if (skip_to_dx) {
#pragma unroll
              for (int e = 0; e < 8; ++e) g.v[e] += ds.v[e];
            } else {
              stv(d_skip + base + c, ds);
            }
          }
        }
        if (add_grad) {
          const V8 ag = cvt8(q_ag[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) g.v[e] += ag.v[e];
        }
        stv(d_x + base + c, g);
      }
    }
  }
  if constexpr (MIX) {
    flush_cols2<NV>(am0, d_mix, d, sm);
    flush_cols2<NV>(am1, d_mix + d, d, sm);
  }
  if constexpr (SKIP) flush_cols2<NV>(asw, d_sw, d, sm);
}

template <int NV>
static void launch_mnb(const void* d_h, const void* d_res, const void* x_in, const void* x, const void* x0, const void* skip, const float* sw,
                       const float* mix, const void* add_grad, void* d_x, void* d_x0, void* d_skip, float* d_mix, float* d_sw, int skip_to_dx, int rows,
                       int d, float s, float eps, cudaStream_t st) {
  const int grid = std::max(1, std::min((rows + RW - 1) / RW, 148 * 6));
  const size_t smem = (size_t)RW * NV * 256 * sizeof(float);
#define PGB_MNB(MIXF, SKIPF)                                                                                                              \
  {                                                                                                                                       \
    auto kern = mix_norm_bwd2_kernel<NV, MIXF, SKIPF>;                                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                             \
    kern<<<grid, RT, (MIXF) ? smem : 0, st>>>((const __nv_bfloat16*)d_h, (const __nv_bfloat16*)d_res, (const __nv_bfloat16*)x_in,          \
                                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, (const __nv_bfloat16*)skip, sw, mix,      \
                                              (const __nv_bfloat16*)add_grad, (__nv_bfloat16*)d_x, (__nv_bfloat16*)d_x0,                  \
                                              (__nv_bfloat16*)d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps);                          \
  }
  if (!mix) PGB_MNB(false, false)
  else if (!skip) PGB_MNB(true, false)
  else PGB_MNB(true, true)
#undef PGB_MNB
}

void mix_norm_bwd_v2(const void* d_h, const void* d_res, const void* x_in, const void* x, const void* x0, const void* skip, const float* sw,
                     const float* mix, const void* add_grad, void* d_x, void* d_x0, void* d_skip, float* d_mix, float* d_sw, int skip_to_dx, int rows,
                     int d, float s, float eps, cudaStream_t st) {
  if (d % 8) throw std::runtime_error("row width must be a multiple of 8");
  switch ((d + 255) / 256) {
    case 1: launch_mnb<1>(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st); break;
    case 2: launch_mnb<2>(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st); break;
    case 3: launch_mnb<3>(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st); break;
    case 4: launch_mnb<4>(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st); break;
    case 5: case 6: launch_mnb<6>(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st); break;
    default: throw std::runtime_error("row width above 1536 is not supported");
  }
}

// ---- QK norm + RoPE, head_dim 64, 8 lanes per head vector --------------------------------------------------------------
// rotate: lanes with sub < hp hold x1 (first half of the rotary dims), lanes hp <= sub < 2hp hold x2; hp = rope_dims/16.
__device__ __forceinline__ void rope8(V8& n, int sub, int hp, int pos, int half, const float* cosT, const float* sinT, bool inverse) {
  const int lane = threadIdx.x & 31;
  const bool in_rope = sub < 2 * hp;
  const bool first = sub < hp;
  const int partner = in_rope ? (first ? lane + hp : lane - hp) : lane;
  const int ibase = pos * half + (first ? sub : sub - hp) * 8;          // half is a multiple of 8: 32-byte aligned table rows
  float cs[8], sn[8];
  if (in_rope) {
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cosT + ibase)), c1 = __ldg(reinterpret_cast<const float4*>(cosT + ibase) + 1);
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sinT + ibase)), s1 = __ldg(reinterpret_cast<const float4*>(sinT + ibase) + 1);
    cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
  }
  const float sgn = (first != inverse) ? 1.f : -1.f;       // first half: +sin (forward) ; second half: -sin; the inverse rotation flips both
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float other = __shfl_sync(0xffffffffu, n.v[e], partner);
    if (in_rope) n.v[e] = n.v[e] * cs[e] + sgn * other * sn[e];
  }
}

__global__ void __launch_bounds__(256) qk_norm_rope_fwd64_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                                 const float* __restrict__ cosT, const float* __restrict__ sinT,
                                                                 const float* __restrict__ gain, int nvec, int ld, int H, int Hkv, int rope_dims,
                                                                 int seq_len, float eps) {
  const int sub = threadIdx.x & 7;
  const int nh = H + Hkv, half = rope_dims / 2, hp = half / 8;
  // 32-bit index arithmetic throughout: the vector count (rows x heads) fits, and a 64-bit divide per vector costs
  // more instructions than the rest of the loop body
  const int vstride = (int)gridDim.x * (blockDim.x / 8);
  const int nvec_pad = (nvec + 3) / 4 * 4;                 // whole warps stay converged for the shuffles
  for (int v = (int)blockIdx.x * (blockDim.x / 8) + (threadIdx.x >> 3); v < nvec_pad; v += vstride) {
    const bool live = v < nvec;
    const int vv = live ? v : nvec - 1;
    const int row = (int)((unsigned)vv / (unsigned)nh), head = vv - row * nh;
    const size_t off = (size_t)row * ld + head * 64 + sub * 8;
    V8 a = ldv(src + off);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a.v[e] * a.v[e];
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    const float inv = rsqrtf(ss / 64.f + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) a.v[e] *= inv;
    if (hp > 0) rope8(a, sub, hp, (int)((unsigned)row % (unsigned)seq_len), half, cosT, sinT, false);
    const float g = (head < H && gain) ? gain[head] : 1.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) a.v[e] *= g;                // one rounding, at the store
    if (live) stv(dst + off, a);
  }
}

__global__ void __launch_bounds__(256) qk_norm_rope_bwd64_kernel(const __nv_bfloat16* __restrict__ d_post, const __nv_bfloat16* __restrict__ pre,
                                                                 __nv_bfloat16* __restrict__ d_pre, const float* __restrict__ cosT,
                                                                 const float* __restrict__ sinT, const float* __restrict__ gain, float* __restrict__ d_gain,
                                                                 int nvec, int ld, int H, int Hkv, int rope_dims, int seq_len, float eps) {
  __shared__ float sg[64];
  for (int i = threadIdx.x; i < 64; i += blockDim.x) sg[i] = 0.f;
  __syncthreads();
  const int sub = threadIdx.x & 7;
  const int nh = H + Hkv, half = rope_dims / 2, hp = half / 8;
  const int vstride = (int)gridDim.x * (blockDim.x / 8);
  const int nvec_pad = (nvec + 3) / 4 * 4;
  for (int v = (int)blockIdx.x * (blockDim.x / 8) + (threadIdx.x >> 3); v < nvec_pad; v += vstride) {
    const bool live = v < nvec;
    const int vv = live ? v : nvec - 1;
    const int row = (int)((unsigned)vv / (unsigned)nh), head = vv - row * nh;
    const int pos = (int)((unsigned)row % (unsigned)seq_len);
    const size_t off = (size_t)row * ld + head * 64 + sub * 8;
    const V8 x = ldv(pre + off);
    V8 dy = ldv(d_post + off);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x.v[e] * x.v[e];
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    const float ms = ss / 64.f + eps;
    const float inv = rsqrtf(ms);
    const float g = (head < H && gain) ? gain[head] : 1.f;
    // post = g * R(inv * x) with R the rotation: d_gain = <dy, R(inv x)> = inv * <R^T dy, x>, and the same inner product
    // (times g) is the norm backward's, so one inverse rotation and one reduction serve both
    if (hp > 0) rope8(dy, sub, hp, pos, half, cosT, sinT, true);
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) dot += x.v[e] * dy.v[e];
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    dot += __shfl_xor_sync(0xffffffffu, dot, 4);
    if (d_gain != nullptr && live && sub == 0 && head < H) atomicAdd(&sg[head], dot * inv);
    const float k2 = g * dot / (ms * 64.f), gi = g * inv;
    V8 o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = gi * dy.v[e] - inv * x.v[e] * k2;
    if (live) stv(d_pre + off, o);
  }
  __syncthreads();
  if (d_gain)
    for (int i = threadIdx.x; i < H && i < 64; i += blockDim.x)
      if (sg[i] != 0.f) atomicAdd(d_gain + i, sg[i]);
}

bool qk_norm_rope_fast_ok(int H, int hd, int rope_dims) { return hd == 64 && H <= 64 && (rope_dims / 2) % 8 == 0 && rope_dims <= 64; }

void qk_norm_rope_fwd64(const void* src, void* dst, const float* cosT, const float* sinT, const float* gain, int rows, int ld, int H, int Hkv,
                        int rope_dims, int seq_len, float eps, cudaStream_t st) {
  if ((long long)rows * (H + Hkv) > 0x7fffff00ll) throw std::runtime_error("qk_norm_rope: too many head vectors for 32-bit indexing");
  const int nvec = rows * (H + Hkv);
  const int grid = std::max(1, std::min((nvec + 31) / 32, 148 * 16));
  qk_norm_rope_fwd64_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, cosT, sinT, gain, nvec, ld, H, Hkv, rope_dims, seq_len,
                                                  eps);
}

void qk_norm_rope_bwd64(const void* d_post, const void* pre, void* d_pre, const float* cosT, const float* sinT, const float* gain, float* d_gain,
                        int rows, int ld, int H, int Hkv, int rope_dims, int seq_len, float eps, cudaStream_t st) {
  if ((long long)rows * (H + Hkv) > 0x7fffff00ll) throw std::runtime_error("qk_norm_rope: too many head vectors for 32-bit indexing");
  const int nvec = rows * (H + Hkv);
  const int grid = std::max(1, std::min((nvec + 31) / 32, 148 * 8));
  qk_norm_rope_bwd64_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)d_post, (const __nv_bfloat16*)pre, (__nv_bfloat16*)d_pre, cosT, sinT, gain,
                                                  d_gain, nvec, ld, H, Hkv, rope_dims, seq_len, eps);
}

// ---- XSA forward / backward, head_dim 64, 8 lanes per (token, KV head) ------------------------------------------------------
// z_h = y_h - (<y_h, v> / (|v|^2 + eps)) v for the `group` query heads h that share one value head. A lane holds 8 of the 64
// features (one 16-byte load, 128 contiguous bytes per head vector), the three inner products are 8-lane shuffles, and no
// thread keeps a whole head vector in registers (the one-thread-per-vector form needed ~170 registers and ran at 3 CTAs/SM).
__device__ __forceinline__ float sum8(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

__global__ void __launch_bounds__(256) xsa_fwd64_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ v,
                                                        __nv_bfloat16* __restrict__ z, int nvec, int Hkv, int group, int ld_y, int ld_v, float eps) {
  const int sub = threadIdx.x & 7;
  const int vstride = (int)gridDim.x * (blockDim.x / 8);
  const int nvec_pad = (nvec + 3) / 4 * 4;                 // whole warps stay converged for the shuffles
  for (int i = (int)blockIdx.x * (blockDim.x / 8) + (threadIdx.x >> 3); i < nvec_pad; i += vstride) {
    const bool live = i < nvec;
    const int ii = live ? i : nvec - 1;
    const int row = (int)((unsigned)ii / (unsigned)Hkv), kh = ii - row * Hkv;
    const V8 vv = ldv(v + (size_t)row * ld_v + kh * 64 + sub * 8);
    float n = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) n += vv.v[e] * vv.v[e];
    n = sum8(n) + eps;
    for (int g = 0; g < group; ++g) {
      const size_t off = (size_t)row * ld_y + (kh * group + g) * 64 + sub * 8;
      V8 a = ldv(y + off);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += a.v[e] * vv.v[e];
      const float coef = sum8(dot) / n;
#pragma unroll
      for (int e = 0; e < 8; ++e) a.v[e] -= coef * vv.v[e];
      if (live) stv(z + off, a);
    }
  }
}

// dy_h = dz_h - (<dz_h,v>/n) v ;  dv (+)= sum_h [ -c_h dz_h - (<dz_h,v>/n) y_h + 2 c_h (<dz_h,v>/n) v ],  c_h = <y_h,v>/n
__global__ void __launch_bounds__(256) xsa_bwd64_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ y,
                                                        const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ dy,
                                                        __nv_bfloat16* __restrict__ dv, int accumulate_dv, int nvec, int Hkv, int group, int ld_y,
                                                        int ld_v, int ld_dv, float eps, float* __restrict__ dsum, int seq_len) {
  const int sub = threadIdx.x & 7;
  const int vstride = (int)gridDim.x * (blockDim.x / 8);
  const int nvec_pad = (nvec + 3) / 4 * 4;
  for (int i = (int)blockIdx.x * (blockDim.x / 8) + (threadIdx.x >> 3); i < nvec_pad; i += vstride) {
    const bool live = i < nvec;
    const int ii = live ? i : nvec - 1;
    const int row = (int)((unsigned)ii / (unsigned)Hkv), kh = ii - row * Hkv;
    const V8 vv = ldv(v + (size_t)row * ld_v + kh * 64 + sub * 8);
    __nv_bfloat16* dvp = dv + (size_t)row * ld_dv + kh * 64 + sub * 8;
    V8 acc;
    if (accumulate_dv) {
      acc = ldv(dvp);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc.v[e] = 0.f;
    }
    float n = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) n += vv.v[e] * vv.v[e];
    n = sum8(n) + eps;
    for (int g = 0; g < group; ++g) {
      const size_t off = (size_t)row * ld_y + (kh * group + g) * 64 + sub * 8;
      const V8 a = ldv(y + off), b = ldv(dz + off);
      float yv = 0.f, gv = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        yv += a.v[e] * vv.v[e];
        gv += b.v[e] * vv.v[e];
      }
      const float ch = sum8(yv) / n, gn = sum8(gv) / n;
      V8 o;
      float dd = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o.v[e] = b.v[e] - gn * vv.v[e];
        acc.v[e] += -ch * b.v[e] - gn * a.v[e] + 2.f * ch * gn * vv.v[e];
        dd += __bfloat162float(__float2bfloat16_rn(o.v[e])) * a.v[e];       // with dy as the attention backward will read it
      }
      if (live) stv(dy + off, o);
      if (dsum != nullptr) {
        // -rowsum(dy * y) per (token, head): the attention backward's per-query term, here for free
        dd = sum8(dd);
        if (live && sub == 0) {
          const int bb = row / seq_len, ss = row - bb * seq_len;
          dsum[((size_t)bb * (Hkv * group) + kh * group + g) * seq_len + ss] = -dd;
        }
      }
    }
    if (live) stv(dvp, acc);
  }
}

void xsa_fwd64(const void* y, const void* v, void* z, int rows, int Hkv, int group, int ld_y, int ld_v, float eps, cudaStream_t st) {
  if ((long long)rows * Hkv > 0x7fffff00ll) throw std::runtime_error("xsa: too many head vectors for 32-bit indexing");
  const int nvec = rows * Hkv;
  const int grid = std::max(1, std::min((nvec + 31) / 32, 148 * 16));
  xsa_fwd64_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)v, (__nv_bfloat16*)z, nvec, Hkv, group, ld_y, ld_v, eps);
}

void xsa_bwd64(const void* dz, const void* y, const void* v, void* dy, void* dv, int accumulate_dv, int rows, int Hkv, int group, int ld_y, int ld_v,
               int ld_dv, float eps, cudaStream_t st, float* dsum, int seq_len) {
  if (dsum && (seq_len <= 0 || rows % seq_len)) throw std::runtime_error("xsa: the rows must be whole sequences when the attention term is requested");
  if ((long long)rows * Hkv > 0x7fffff00ll) throw std::runtime_error("xsa: too many head vectors for 32-bit indexing");
  const int nvec = rows * Hkv;
  const int grid = std::max(1, std::min((nvec + 31) / 32, 148 * 16));
  xsa_bwd64_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dz, (const __nv_bfloat16*)y, (const __nv_bfloat16*)v, (__nv_bfloat16*)dy,
                                         (__nv_bfloat16*)dv, accumulate_dv, nvec, Hkv, group, ld_y, ld_v, ld_dv, eps, dsum, seq_len);
}

}  // namespace pgb
