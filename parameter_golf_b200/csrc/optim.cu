// Optimizer and weight-preparation kernels (fp32 master state, bf16 compute copies).
//
// Hyper-parameters that change every step live in a small device array `hp` so that a captured CUDA
// graph of the step can be replayed with new values (one tiny host-to-device copy per step):
//   hp[0] lr_scale   hp[1] muon_momentum   hp[2] adam bias-correction 1   hp[3] adam bias-correction 2
//   hp[4] grad scale applied before use (1/accum * clip factor is formed on the device, see clip_factor_kernel)
// Replaces the K3 family and the per-step shadow refresh of the reference
// (parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:416-547, 4481-4575; pg-optim/src/gpu.rs:218-613).
#include "common.cuh"
#include "pgb.h"

namespace pgb {

// ---- weight cast: fp32 master rows -> bf16 compute rows, optional per-row scale and int6 fake-quant ---------------
// dst[r, c] = bf16( rowscale[r * scale_stride] * fq(src[r, c]) ), fq(w) = clamp(round(w/s), -32, 31) * s, s = max(rowmax/31, 1/31).
// One warp per row.
__global__ void __launch_bounds__(256) cast_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, const float* __restrict__ rowscale,
                                                        int scale_stride, int scale_mod, int rows, int cols, long long ld_dst, int qat) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const float* s = src + (size_t)row * cols;
    __nv_bfloat16* o = dst + (size_t)row * ld_dst;
    float qs = 0.f;
    if (qat) {
      float mx = 0.f;
      for (int c = lane * 4; c < cols; c += 128) {
        float4 a = *reinterpret_cast<const float4*>(s + c);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
      }
      mx = warp_max(mx);
      qs = fmaxf(mx / 31.f, 1.f / 31.f);
    }
    const float rs = rowscale ? rowscale[(size_t)(row % scale_mod) * scale_stride] : 1.f;
    for (int c = lane * 4; c < cols; c += 128) {
      float4 a = *reinterpret_cast<const float4*>(s + c);
      if (qat) {
        a.x = fminf(fmaxf(rintf(a.x / qs), -32.f), 31.f) * qs;
        a.y = fminf(fmaxf(rintf(a.y / qs), -32.f), 31.f) * qs;
        a.z = fminf(fmaxf(rintf(a.z / qs), -32.f), 31.f) * qs;
        a.w = fminf(fmaxf(rintf(a.w / qs), -32.f), 31.f) * qs;
      }
      uint2 p = make_uint2(pack_bf16x2(a.x * rs, a.y * rs), pack_bf16x2(a.z * rs, a.w * rs));
      *reinterpret_cast<uint2*>(o + c) = p;
    }
  }
}

// Fold the gradient of a row-scaled weight:  W_eff = scale[r] * Wq  =>  dW += scale[r] * G,  dscale[r] += sum_c Wq[r,c] * G[r,c].
// Wq is the un-scaled weight as the forward saw it: either the fp32 master (optionally fake-quantised here) or the
// un-scaled bf16 compute copy (already fake-quantised when QAT is on; this is what non-owner ranks of a sharded bank have).
template <typename WT>
__device__ __forceinline__ float4 load_w4(const WT* p);
template <>
__device__ __forceinline__ float4 load_w4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load_w4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 q = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename WT>
__global__ void __launch_bounds__(256) fold_scaled_grad_kernel(const float* __restrict__ G, const WT* __restrict__ W, const float* __restrict__ rowscale,
                                                               int scale_stride, int scale_mod, float* __restrict__ dW, float* __restrict__ dscale,
                                                               int rows, int cols, int qat) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const float* g = G + (size_t)row * cols;
    const WT* w = W + (size_t)row * cols;
    float* o = dW + (size_t)row * cols;
    float qs = 0.f;
    if (qat) {
      float mx = 0.f;
      for (int c = lane * 4; c < cols; c += 128) {
        float4 a = load_w4<WT>(w + c);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
      }
      mx = warp_max(mx);
      qs = fmaxf(mx / 31.f, 1.f / 31.f);
    }
    const size_t sidx = (size_t)(row % scale_mod) * scale_stride;
    const float rs = rowscale[sidx];
    float dot = 0.f;
    for (int c = lane * 4; c < cols; c += 128) {
      float4 a = load_w4<WT>(w + c);
      float4 gg = *reinterpret_cast<const float4*>(g + c);
      if (qat) {
        a.x = fminf(fmaxf(rintf(a.x / qs), -32.f), 31.f) * qs;
        a.y = fminf(fmaxf(rintf(a.y / qs), -32.f), 31.f) * qs;
        a.z = fminf(fmaxf(rintf(a.z / qs), -32.f), 31.f) * qs;
        a.w = fminf(fmaxf(rintf(a.w / qs), -32.f), 31.f) * qs;
      }
      dot += a.x * gg.x + a.y * gg.y + a.z * gg.z + a.w * gg.w;
      float4 d = *reinterpret_cast<float4*>(o + c);
      d.x += rs * gg.x; d.y += rs * gg.y; d.z += rs * gg.z; d.w += rs * gg.w;
      *reinterpret_cast<float4*>(o + c) = d;
    }
    dot = warp_sum(dot);
    if (lane == 0) atomicAdd(dscale + sidx, dot);
  }
}

// ---- global-norm clipping ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ x, long long n, float scale, float* __restrict__ out) {
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      float4 a = *reinterpret_cast<const float4*>(x + i);
      s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    } else {
      for (long long j = i; j < n; ++j) s += x[j] * x[j];
    }
  }
  s = warp_sum(s);
  __shared__ float ws[8];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += ws[w];
    atomicAdd(out, t * scale * scale);
  }
}

// dst[i] += sum_s part[s * split_stride + i], s ascending: the fixed-order second half of a deterministic split-K product
// (each partial was written by exactly one CTA with a fixed K order, so the result does not depend on scheduling).
__global__ void __launch_bounds__(256) sum_splits_add_kernel(const float* __restrict__ part, int splits, long long split_stride,
                                                             float* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    float4 acc = *reinterpret_cast<const float4*>(dst + i);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(part + (size_t)s * split_stride + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(dst + i) = acc;
  }
}

// hp[4] = base_scale * min(1, max_norm / (sqrt(sumsq) * base_scale + 1e-6));  stats[1] = norm (for logging); stats[0] reset.
__global__ void clip_factor_kernel(float* __restrict__ stats, float* __restrict__ hp, float base_scale, float max_norm) {
  const float norm = sqrtf(stats[0]) * base_scale;
  float f = 1.f;
  if (max_norm > 0.f && norm > max_norm) f = max_norm / (norm + 1e-6f);
  hp[4] = base_scale * f;
  stats[1] = norm;
  stats[0] = 0.f;
}

// ---- Muon ------------------------------------------------------------------------------------------------------------------
// buf = mu*buf + g*gs;  u = g*gs + mu*buf (Nesterov);  U (bf16) = u;  sumsq[matrix] += |u|^2.   grid.y = matrix index.
__global__ void __launch_bounds__(256) muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf, __nv_bfloat16* __restrict__ U,
                                                            float* __restrict__ sumsq, const float* __restrict__ hp, long long per_matrix, int nesterov) {
  const int mat = blockIdx.y;
  const float mu = hp[1], gs = hp[4];
  const float* gp = g + (size_t)mat * per_matrix;
  float* bp = buf + (size_t)mat * per_matrix;
  __nv_bfloat16* up = U + (size_t)mat * per_matrix;
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < per_matrix; i += stride) {
    float4 a = *reinterpret_cast<const float4*>(gp + i);
    float4 b = *reinterpret_cast<float4*>(bp + i);
    a.x *= gs; a.y *= gs; a.z *= gs; a.w *= gs;
    b.x = mu * b.x + a.x; b.y = mu * b.y + a.y; b.z = mu * b.z + a.z; b.w = mu * b.w + a.w;
    *reinterpret_cast<float4*>(bp + i) = b;
    float4 u = nesterov ? make_float4(a.x + mu * b.x, a.y + mu * b.y, a.z + mu * b.z, a.w + mu * b.w) : b;
    s += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    *reinterpret_cast<uint2*>(up + i) = make_uint2(pack_bf16x2(u.x, u.y), pack_bf16x2(u.z, u.w));
  }
  s = warp_sum(s);
  __shared__ float ws[8];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += ws[w];
    atomicAdd(sumsq + mat, t);
  }
}

// X = U / (sqrt(sumsq[matrix]) + eps)   (bf16 -> bf16)
__global__ void __launch_bounds__(256) muon_normalize_kernel(const __nv_bfloat16* __restrict__ U, __nv_bfloat16* __restrict__ X,
                                                             const float* __restrict__ sumsq, long long per_matrix, float eps) {
  const int mat = blockIdx.y;
  const float inv = 1.f / (sqrtf(sumsq[mat]) + eps);
  const __nv_bfloat16* up = U + (size_t)mat * per_matrix;
  __nv_bfloat16* xp = X + (size_t)mat * per_matrix;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < per_matrix; i += stride) {
    uint4 q = *reinterpret_cast<const uint4*>(up + i);
    float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
    *reinterpret_cast<uint4*>(xp + i) = make_uint4(pack_bf16x2(a.x * inv, a.y * inv), pack_bf16x2(b.x * inv, b.y * inv),
                                                  pack_bf16x2(c.x * inv, c.y * inv), pack_bf16x2(d.x * inv, d.y * inv));
  }
}

// p = (1 - lr*wd) * p - lr*scale * X;  optional EMA: ema = decay*ema + (1-decay)*p.    lr = base_lr * hp[0]
__global__ void __launch_bounds__(256) muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ X, float* __restrict__ ema,
                                                         const float* __restrict__ hp, long long n, float base_lr, float wd, float scale, float decay) {
  const float lr = base_lr * hp[0];
  const float keep = 1.f - lr * wd, step = lr * scale;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    float4 a = *reinterpret_cast<float4*>(p + i);
    uint2 q = *reinterpret_cast<const uint2*>(X + i);
    float2 x0 = unpack_bf16x2(q.x), x1 = unpack_bf16x2(q.y);
    a.x = keep * a.x - step * x0.x; a.y = keep * a.y - step * x0.y; a.z = keep * a.z - step * x1.x; a.w = keep * a.w - step * x1.y;
    *reinterpret_cast<float4*>(p + i) = a;
    if (ema) {
      float4 e = *reinterpret_cast<float4*>(ema + i);
      e.x = decay * e.x + (1.f - decay) * a.x; e.y = decay * e.y + (1.f - decay) * a.y;
      e.z = decay * e.z + (1.f - decay) * a.z; e.w = decay * e.w + (1.f - decay) * a.w;
      *reinterpret_cast<float4*>(ema + i) = e;
    }
  }
}

// ---- AdamW over one flat group -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                                    float* __restrict__ ema, const float* __restrict__ hp, long long n, float base_lr, float b1, float b2,
                                                    float eps, float wd, float decay) {
  const float lr = base_lr * hp[0], c1 = hp[2], c2 = hp[3], gs = hp[4];
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = i0; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i] * gs;
    const float mm = b1 * m[i] + (1.f - b1) * gr;
    const float vv = b2 * v[i] + (1.f - b2) * gr * gr;
    m[i] = mm;
    v[i] = vv;
    float pp = p[i] * (1.f - lr * wd);
    pp -= lr * (mm / c1) / (sqrtf(vv / c2) + eps);
    p[i] = pp;
    if (ema) ema[i] = decay * ema[i] + (1.f - decay) * pp;
  }
}

// plain SGD with momentum on a flat buffer (test-time training):  mom = mu*mom + g*gs;  p -= lr*mom
__global__ void __launch_bounds__(256) sgd_momentum_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ mom,
                                                           const float* __restrict__ hp, long long n, float lr, float mu) {
  const float gs = hp[4];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float mm = mu * mom[i] + g[i] * gs;
    mom[i] = mm;
    p[i] -= lr * mm;
  }
}

// ---- launchers ----------------------------------------------------------------------------------------------------------------------
static int ew_grid(long long n, int per_thread) {
  long long b = (n / per_thread + 255) / 256;
  return (int)std::max<long long>(1, std::min<long long>(b, 148 * 16));
}

void cast_rows(const float* src, void* dst, const float* rowscale, int scale_stride, int scale_mod, int rows, int cols, long long ld_dst, int qat,
               cudaStream_t st) {
  if (cols % 4) throw std::runtime_error("cast_rows: cols must be a multiple of 4");
  cast_rows_kernel<<<std::min((rows + 7) / 8, 148 * 8), 256, 0, st>>>(src, (__nv_bfloat16*)dst, rowscale, scale_stride, std::max(scale_mod, 1), rows,
                                                                     cols, ld_dst, qat);
}

void fold_scaled_grad(const float* G, const float* W, const float* rowscale, int scale_stride, int scale_mod, float* dW, float* dscale, int rows,
                      int cols, int qat, cudaStream_t st) {
  if (cols % 4) throw std::runtime_error("fold_scaled_grad: cols must be a multiple of 4");
  fold_scaled_grad_kernel<float><<<std::min((rows + 7) / 8, 148 * 8), 256, 0, st>>>(G, W, rowscale, scale_stride, std::max(scale_mod, 1), dW, dscale,
                                                                                   rows, cols, qat);
}

void fold_scaled_grad_bf16(const float* G, const void* W, const float* rowscale, int scale_stride, int scale_mod, float* dW, float* dscale, int rows,
                           int cols, cudaStream_t st) {
  if (cols % 4) throw std::runtime_error("fold_scaled_grad: cols must be a multiple of 4");
  fold_scaled_grad_kernel<__nv_bfloat16><<<std::min((rows + 7) / 8, 148 * 8), 256, 0, st>>>(G, (const __nv_bfloat16*)W, rowscale, scale_stride,
                                                                                           std::max(scale_mod, 1), dW, dscale, rows, cols, 0);
}

void sumsq(const float* x, long long n, float scale, float* out, cudaStream_t st) { sumsq_kernel<<<ew_grid(n, 4), 256, 0, st>>>(x, n, scale, out); }

void sum_splits_add(const float* part, int splits, long long split_stride, float* dst, long long n, cudaStream_t st) {
  if ((n % 4) || (split_stride % 4)) throw std::runtime_error("sum_splits_add: sizes must be multiples of 4");
  if (n == 0 || splits <= 0) return;
  sum_splits_add_kernel<<<ew_grid(n, 4), 256, 0, st>>>(part, splits, split_stride, dst, n);
}

void clip_factor(float* stats, float* hp, float base_scale, float max_norm, cudaStream_t st) {
  clip_factor_kernel<<<1, 1, 0, st>>>(stats, hp, base_scale, max_norm);
}

void muon_momentum(const float* g, float* buf, void* U, float* sumsq_out, const float* hp, int matrices, long long per_matrix, int nesterov,
                   cudaStream_t st) {
  if (per_matrix % 8) throw std::runtime_error("muon: matrix size must be a multiple of 8");
  dim3 grid(ew_grid(per_matrix, 4) > 64 ? 64 : ew_grid(per_matrix, 4), matrices);
  muon_momentum_kernel<<<grid, 256, 0, st>>>(g, buf, (__nv_bfloat16*)U, sumsq_out, hp, per_matrix, nesterov);
}

void muon_normalize(const void* U, void* X, const float* sumsq_in, int matrices, long long per_matrix, float eps, cudaStream_t st) {
  dim3 grid(ew_grid(per_matrix, 8) > 64 ? 64 : ew_grid(per_matrix, 8), matrices);
  muon_normalize_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)U, (__nv_bfloat16*)X, sumsq_in, per_matrix, eps);
}

void muon_apply(float* p, const void* X, float* ema, const float* hp, long long n, float base_lr, float wd, float scale, float decay, cudaStream_t st) {
  if (n % 4) throw std::runtime_error("muon_apply: size must be a multiple of 4");
  muon_apply_kernel<<<ew_grid(n, 4), 256, 0, st>>>(p, (const __nv_bfloat16*)X, ema, hp, n, base_lr, wd, scale, decay);
}

void adamw(float* p, const float* g, float* m, float* v, float* ema, const float* hp, long long n, float base_lr, float b1, float b2, float eps,
           float wd, float decay, cudaStream_t st) {
  adamw_kernel<<<ew_grid(n, 1), 256, 0, st>>>(p, g, m, v, ema, hp, n, base_lr, b1, b2, eps, wd, decay);
}

void sgd_momentum(float* p, const float* g, float* mom, const float* hp, long long n, float lr, float mu, cudaStream_t st) {
  sgd_momentum_kernel<<<ew_grid(n, 1), 256, 0, st>>>(p, g, mom, hp, n, lr, mu);
}

}  // namespace pgb
