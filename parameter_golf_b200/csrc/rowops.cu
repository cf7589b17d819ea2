// Bandwidth-bound row kernels of the model (bf16 in/out, fp32 arithmetic). One warp owns one row of
// `d` features at a time and every lane keeps the same feature columns for all of its rows, so
// per-feature gradient sums (gate, mix, skip weights) are accumulated in registers and flushed with a
// handful of atomics per CTA. These replace the K4/K5/K7/K8/K10/K14 families of the reference's NVRTC
// module (parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:549-2377, 2429-3610, 5635-5894), each
// of which was a separate fp32 pass there.
#include "common.cuh"
#include "pgb.h"

namespace pgb {

constexpr int ROW_THREADS = 256;
constexpr int ROW_WARPS = ROW_THREADS / 32;

struct F8 {
  float v[8];
};

__device__ __forceinline__ F8 ld8(const __nv_bfloat16* p) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  F8 r;
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; r.v[4] = c.x; r.v[5] = c.y; r.v[6] = d.x; r.v[7] = d.y;
  return r;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const F8& r) {
  *reinterpret_cast<uint4*>(p) =
      make_uint4(pack_bf16x2(r.v[0], r.v[1]), pack_bf16x2(r.v[2], r.v[3]), pack_bf16x2(r.v[4], r.v[5]), pack_bf16x2(r.v[6], r.v[7]));
}
__device__ __forceinline__ F8 ld8f(const float* p) {
  F8 r;
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w; r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  return r;
}
__device__ __forceinline__ float bfround(float x) { return __bfloat162float(__float2bfloat16(x)); }

// Flush per-lane column accumulators: CTA-level reduction through shared memory, then one atomic per column.
template <int NV>
__device__ __forceinline__ void flush_cols(float (&acc)[NV][8], float* dst, int d, float* sm /* [ROW_WARPS][NV*256] */) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) sm[warp * (NV * 256) + (j * 32 + lane) * 8 + e] = acc[j][e];
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += ROW_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ROW_WARPS; ++w) s += sm[w * (NV * 256) + c];
    atomicAdd(dst + c, s);
  }
}

// -------------------------------------------------------------------------------------------------------------
// mix + RMSNorm forward:  xe = x (+ sw*skip);  x_in = bf16(mix0*xe + mix1*x0);  h = bf16(rmsnorm(x_in) * s)
template <int NV>
__global__ void __launch_bounds__(ROW_THREADS) mix_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                                                                   const __nv_bfloat16* __restrict__ skip, const float* __restrict__ sw,
                                                                   const float* __restrict__ mix, __nv_bfloat16* __restrict__ x_in,
                                                                   __nv_bfloat16* __restrict__ h, int rows, int d, float s, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * d;
    F8 xi[NV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 a = ld8(x + base + c);
        if (skip) {
          F8 k = ld8(skip + base + c), w = ld8f(sw + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) a.v[e] = bfround(a.v[e] + w.v[e] * k.v[e]);
        }
        if (mix) {
          F8 b = ld8(x0 + base + c), m0 = ld8f(mix + c), m1 = ld8f(mix + d + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) a.v[e] = bfround(m0.v[e] * a.v[e] + m1.v[e] * b.v[e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += a.v[e] * a.v[e];
        xi[j] = a;
        if (x_in) st8(x_in + base + c, a);
      }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / d + eps) * s;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 o;
#pragma unroll
        for (int e = 0; e < 8; ++e) o.v[e] = xi[j].v[e] * inv;
        st8(h + base + c, o);
      }
    }
  }
}

// RMSNorm backward (+ residual-path gradient) and mix / skip backward:
//   g_in = d_res + rmsnorm_bwd(d_h; x_in, s)          gradient w.r.t. x_in
//   d_x0 += mix1 * g_in;  g_xe = mix0 * g_in;  d_mix += sum_rows(g_in * {xe, x0})
//   d_x = g_xe (+ add_grad) (+ sw * g_xe when skip_to_dx);  d_skip = sw * g_xe;  d_sw += sum_rows(g_xe * skip)
// With mix == nullptr it is a plain "norm backward + add": d_x = d_res + rmsnorm_bwd(d_h; x_in, s).
template <int NV>
__global__ void __launch_bounds__(ROW_THREADS) mix_norm_bwd_kernel(const __nv_bfloat16* __restrict__ d_h, const __nv_bfloat16* __restrict__ d_res,
                                                                   const __nv_bfloat16* __restrict__ x_in, const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ skip,
                                                                   const float* __restrict__ sw, const float* __restrict__ mix,
                                                                   const __nv_bfloat16* __restrict__ add_grad, __nv_bfloat16* __restrict__ d_x,
                                                                   __nv_bfloat16* __restrict__ d_x0, __nv_bfloat16* __restrict__ d_skip,
                                                                   float* __restrict__ d_mix, float* __restrict__ d_sw, int skip_to_dx, int rows, int d,
                                                                   float s, float eps) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float am0[NV][8], am1[NV][8], asw[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) am0[j][e] = am1[j][e] = asw[j][e] = 0.f;

  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * d;
    F8 xi[NV], dy[NV];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        xi[j] = ld8(x_in + base + c);
        dy[j] = ld8(d_h + base + c);
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
    const float inv = rsqrtf(ms);
    const float k1 = s * inv, k2 = dot / (ms * d);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 g;
#pragma unroll
        for (int e = 0; e < 8; ++e) g.v[e] = k1 * (dy[j].v[e] - xi[j].v[e] * k2);
        if (d_res) {
          F8 r = ld8(d_res + base + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) g.v[e] += r.v[e];
        }
        if (mix) {
          F8 m0 = ld8f(mix + c), m1 = ld8f(mix + d + c), b = ld8(x0 + base + c), a = ld8(x + base + c);
          F8 k;
          if (skip) {
            k = ld8(skip + base + c);
            F8 w = ld8f(sw + c);
#pragma unroll
            for (int e = 0; e < 8; ++e) a.v[e] = bfround(a.v[e] + w.v[e] * k.v[e]);
          }
          F8 acc0 = ld8(d_x0 + base + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            am0[j][e] += g.v[e] * a.v[e];
            am1[j][e] += g.v[e] * b.v[e];
            acc0.v[e] += m1.v[e] * g.v[e];
            g.v[e] *= m0.v[e];
          }
          st8(d_x0 + base + c, acc0);
          if (skip) {
            F8 w = ld8f(sw + c), ds;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              asw[j][e] += g.v[e] * k.v[e];
              ds.v[e] = w.v[e] * g.v[e];
            }
            if (skip_to_dx) {
#pragma unroll
              for (int e = 0; e < 8; ++e) g.v[e] += ds.v[e];
            } else {
              st8(d_skip + base + c, ds);
            }
          }
        }
        if (add_grad) {
          F8 ag = ld8(add_grad + base + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) g.v[e] += ag.v[e];
        }
        st8(d_x + base + c, g);
      }
    }
  }
  if (mix) {
    flush_cols<NV>(am0, d_mix, d, sm);
    flush_cols<NV>(am1, d_mix + d, d, sm);
    if (skip) flush_cols<NV>(asw, d_sw, d, sm);
  }
}

// -------------------------------------------------------------------------------------------------------------
// Embedding front: out = smear(rmsnorm(xe)) with the previous row's norm recomputed (no extra pass).
//   n_t = rmsnorm(xe_t);  out_t = (1-g)*n_t + g*n_{t-1};  n_{-1} = 0 at sequence starts and where ids[t] == boundary.
template <int NV>
__global__ void __launch_bounds__(ROW_THREADS) norm_smear_fwd_kernel(const __nv_bfloat16* __restrict__ xe, const float* __restrict__ gate,
                                                                     const int* __restrict__ ids, __nv_bfloat16* __restrict__ out, int rows, int d,
                                                                     int seq_len, int boundary, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * d;
    const bool has_prev = gate && (row % seq_len != 0) && !(boundary >= 0 && ids[row] == boundary);
    F8 a[NV], b[NV];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        a[j] = ld8(xe + base + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) sa += a[j].v[e] * a[j].v[e];
        if (has_prev) {
          b[j] = ld8(xe + base - d + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) sb += b[j].v[e] * b[j].v[e];
        }
      }
    }
    sa = warp_sum(sa);
    sb = warp_sum(sb);
    const float ia = rsqrtf(sa / d + eps), ib = has_prev ? rsqrtf(sb / d + eps) : 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 o;
        if (gate) {
          F8 g = ld8f(gate + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float sg = 1.f / (1.f + __expf(-g.v[e]));
            const float na = bfround(a[j].v[e] * ia), nb = has_prev ? bfround(b[j].v[e] * ib) : 0.f;
            o.v[e] = (1.f - sg) * na + sg * nb;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o.v[e] = a[j].v[e] * ia;
        }
        st8(out + base + c, o);
      }
    }
  }
}

// Backward of the front: given g = dL/d out, dn_t = (1-s)*g_t + s*g_{t+1} (when row t+1 uses row t), then RMSNorm backward;
// d_gate += sum_t g_t * (n_{t-1} - n_t) * s*(1-s).
template <int NV>
__global__ void __launch_bounds__(ROW_THREADS) norm_smear_bwd_kernel(const __nv_bfloat16* __restrict__ g_out, const __nv_bfloat16* __restrict__ xe,
                                                                     const float* __restrict__ gate, const int* __restrict__ ids,
                                                                     __nv_bfloat16* __restrict__ d_xe, float* __restrict__ d_gate, int rows, int d,
                                                                     int seq_len, int boundary, float eps) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float ag[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) ag[j][e] = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * d;
    const bool has_prev = gate && (row % seq_len != 0) && !(boundary >= 0 && ids[row] == boundary);
    const bool has_next = gate && (row + 1 < rows) && ((row + 1) % seq_len != 0) && !(boundary >= 0 && ids[row + 1] == boundary);
    F8 a[NV], b[NV];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        a[j] = ld8(xe + base + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) sa += a[j].v[e] * a[j].v[e];
        if (has_prev) {
          b[j] = ld8(xe + base - d + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) sb += b[j].v[e] * b[j].v[e];
        }
      }
    }
    sa = warp_sum(sa);
    sb = warp_sum(sb);
    const float msa = sa / d + eps;
    const float ia = rsqrtf(msa), ib = has_prev ? rsqrtf(sb / d + eps) : 0.f;
    F8 dn[NV];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 g = ld8(g_out + base + c);
        if (gate) {
          F8 gt = ld8f(gate + c), gn;
          if (has_next) gn = ld8(g_out + base + d + c);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float sg = 1.f / (1.f + __expf(-gt.v[e]));
            const float na = bfround(a[j].v[e] * ia), nb = has_prev ? bfround(b[j].v[e] * ib) : 0.f;
            ag[j][e] += g.v[e] * (nb - na) * sg * (1.f - sg);
            dn[j].v[e] = (1.f - sg) * g.v[e] + (has_next ? sg * gn.v[e] : 0.f);
          }
        } else {
          dn[j] = g;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) dot += a[j].v[e] * dn[j].v[e];
      }
    }
    dot = warp_sum(dot);
    const float k2 = dot / (msa * d);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < d) {
        F8 o;
#pragma unroll
        for (int e = 0; e < 8; ++e) o.v[e] = ia * (dn[j].v[e] - a[j].v[e] * k2);
        st8(d_xe + base + c, o);
      }
    }
  }
  if (gate) flush_cols<NV>(ag, d_gate, d, sm);
}

// -------------------------------------------------------------------------------------------------------------
// Per-head RMSNorm + partial RoPE (+ q gain) on the packed QKV activations. One thread per (token, head) for
// heads 0 .. H+Hkv-1 (q heads then k heads); v is left untouched. `src` and `dst` rows have `ld` elements.
template <int HD>
__global__ void qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, const float* __restrict__ cosT,
                                        const float* __restrict__ sinT, const float* __restrict__ gain, int rows, int ld, int H, int Hkv, int hd,
                                        int rope_dims, int seq_len, float eps) {
  if (HD > 0) hd = HD;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int nh = H + Hkv;
  if (idx >= (long long)rows * nh) return;
  const int row = (int)(idx / nh), head = (int)(idx % nh);
  const __nv_bfloat16* s = src + (size_t)row * ld + head * hd;
  __nv_bfloat16* o = dst + (size_t)row * ld + head * hd;
  const int pos = row % seq_len;
  const int half = rope_dims / 2;
  float v[HD > 0 ? HD : 256];
  float ss = 0.f;
  for (int c = 0; c < hd; c += 8) {
    F8 a = ld8(s + c);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[c + e] = a.v[e];
      ss += a.v[e] * a.v[e];
    }
  }
  const float inv = rsqrtf(ss / hd + eps);
  const float g = (head < H && gain) ? gain[head] : 1.f;
  for (int c = 0; c < hd; ++c) v[c] = bfround(v[c] * inv);
  for (int i = 0; i < half; ++i) {
    const float cs = cosT[pos * half + i], sn = sinT[pos * half + i];
    const float x1 = v[i], x2 = v[i + half];
    v[i] = x1 * cs + x2 * sn;
    v[i + half] = -x1 * sn + x2 * cs;
  }
  for (int c = 0; c < hd; c += 8) {
    F8 r;
#pragma unroll
    for (int e = 0; e < 8; ++e) r.v[e] = bfround(v[c + e]) * g;
    st8(o + c, r);
  }
}

// Backward: dq (w.r.t. the post-gain q) -> gradient w.r.t. the raw projection; d_gain[h] += sum <dq, q_rot>.
template <int HD>
__global__ void qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ d_post, const __nv_bfloat16* __restrict__ pre,
                                        __nv_bfloat16* __restrict__ d_pre, const float* __restrict__ cosT, const float* __restrict__ sinT,
                                        const float* __restrict__ gain, float* __restrict__ d_gain, int rows, int ld, int H, int Hkv, int hd,
                                        int rope_dims, int seq_len, float eps) {
  if (HD > 0) hd = HD;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int nh = H + Hkv;
  const bool live = idx < (long long)rows * nh;
  // `head` is identical for threads idx and idx + k*nh; a warp covers 32 consecutive idx, so the gain
  // gradient is reduced through shared memory per head.
  extern __shared__ float sg[];   // [H]
  for (int i = threadIdx.x; i < H; i += blockDim.x) sg[i] = 0.f;
  __syncthreads();
  if (live) {
    const int row = (int)(idx / nh), head = (int)(idx % nh);
    const __nv_bfloat16* s = pre + (size_t)row * ld + head * hd;
    const __nv_bfloat16* dg = d_post + (size_t)row * ld + head * hd;
    __nv_bfloat16* o = d_pre + (size_t)row * ld + head * hd;
    const int pos = row % seq_len;
    const int half = rope_dims / 2;
    float x[HD > 0 ? HD : 256], dy[HD > 0 ? HD : 256];
    float ss = 0.f;
    for (int c = 0; c < hd; c += 8) {
      F8 a = ld8(s + c), b = ld8(dg + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[c + e] = a.v[e];
        dy[c + e] = b.v[e];
        ss += a.v[e] * a.v[e];
      }
    }
    const float ms = ss / hd + eps;
    const float inv = rsqrtf(ms);
    const float g = (head < H && gain) ? gain[head] : 1.f;
    if (head < H && d_gain) {
      // q_rot = rope(norm(x)); d_gain = <dy, q_rot>
      float acc = 0.f;
      for (int c = 0; c < hd; ++c) {
        float n = bfround(x[c] * inv);
        float r;
        if (c < half) {
          const float n2 = bfround(x[c + half] * inv);
          r = n * cosT[pos * half + c] + n2 * sinT[pos * half + c];
        } else if (c < 2 * half) {
          const float n1 = bfround(x[c - half] * inv);
          r = -n1 * sinT[pos * half + c - half] + n * cosT[pos * half + c - half];
        } else {
          r = n;
        }
        acc += dy[c] * bfround(r);
      }
      atomicAdd(&sg[head], acc);
    }
    // undo gain, undo rotation (transpose), then RMSNorm backward
    for (int c = 0; c < hd; ++c) dy[c] *= g;
    for (int i = 0; i < half; ++i) {
      const float cs = cosT[pos * half + i], sn = sinT[pos * half + i];
      const float d1 = dy[i], d2 = dy[i + half];
      dy[i] = d1 * cs - d2 * sn;
      dy[i + half] = d1 * sn + d2 * cs;
    }
    float dot = 0.f;
    for (int c = 0; c < hd; ++c) dot += x[c] * dy[c];
    const float k2 = dot / (ms * hd);
    for (int c = 0; c < hd; c += 8) {
      F8 r;
#pragma unroll
      for (int e = 0; e < 8; ++e) r.v[e] = inv * (dy[c + e] - x[c + e] * k2);
      st8(o + c, r);
    }
  }
  __syncthreads();
  if (d_gain)
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      if (sg[i] != 0.f) atomicAdd(d_gain + i, sg[i]);
}

// -------------------------------------------------------------------------------------------------------------
// XSA: z_h = y_h - (<y_h, v> / (|v|^2 + eps)) v for the `group` query heads that share one value head.
// One thread per (token, kv head). y/z rows have ld_y elements, v rows ld_v.
template <int HD>
__global__ void xsa_fwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ z, int rows,
                               int Hkv, int group, int hd, int ld_y, int ld_v, float eps) {
  if (HD > 0) hd = HD;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * Hkv) return;
  const int row = (int)(idx / Hkv), kh = (int)(idx % Hkv);
  const __nv_bfloat16* vp = v + (size_t)row * ld_v + kh * hd;
  float vv[HD > 0 ? HD : 256];
  float n = eps;
  for (int c = 0; c < hd; c += 8) {
    F8 a = ld8(vp + c);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      vv[c + e] = a.v[e];
      n += a.v[e] * a.v[e];
    }
  }
  for (int g = 0; g < group; ++g) {
    const int h = kh * group + g;
    const __nv_bfloat16* yp = y + (size_t)row * ld_y + h * hd;
    __nv_bfloat16* zp = z + (size_t)row * ld_y + h * hd;
    float dot = 0.f;
    for (int c = 0; c < hd; c += 8) {
      F8 a = ld8(yp + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += a.v[e] * vv[c + e];
    }
    const float coef = dot / n;
    for (int c = 0; c < hd; c += 8) {
      F8 a = ld8(yp + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) a.v[e] -= coef * vv[c + e];
      st8(zp + c, a);
    }
  }
}

// dy_h = dz_h - (<dz_h,v>/n) v ;  dv (+)= sum_h [ -c_h dz_h - (<dz_h,v>/n) y_h + 2 c_h (<dz_h,v>/n) v ]
template <int HD>
__global__ void xsa_bwd_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ v,
                               __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dv, int accumulate_dv, int rows, int Hkv, int group, int hd,
                               int ld_y, int ld_v, int ld_dv, float eps) {
  if (HD > 0) hd = HD;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * Hkv) return;
  const int row = (int)(idx / Hkv), kh = (int)(idx % Hkv);
  const __nv_bfloat16* vp = v + (size_t)row * ld_v + kh * hd;
  __nv_bfloat16* dvp = dv + (size_t)row * ld_dv + kh * hd;
  float vv[HD > 0 ? HD : 256], acc[HD > 0 ? HD : 256];
  float n = eps;
  for (int c = 0; c < hd; c += 8) {
    F8 a = ld8(vp + c);
    F8 b;
    if (accumulate_dv) b = ld8(dvp + c);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      vv[c + e] = a.v[e];
      n += a.v[e] * a.v[e];
      acc[c + e] = accumulate_dv ? b.v[e] : 0.f;
    }
  }
  for (int g = 0; g < group; ++g) {
    const int h = kh * group + g;
    const __nv_bfloat16* yp = y + (size_t)row * ld_y + h * hd;
    const __nv_bfloat16* gp = dz + (size_t)row * ld_y + h * hd;
    __nv_bfloat16* op = dy + (size_t)row * ld_y + h * hd;
    float yv = 0.f, gv = 0.f;
    for (int c = 0; c < hd; c += 8) {
      F8 a = ld8(yp + c), b = ld8(gp + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        yv += a.v[e] * vv[c + e];
        gv += b.v[e] * vv[c + e];
      }
    }
    const float ch = yv / n, gn = gv / n;
    for (int c = 0; c < hd; c += 8) {
      F8 a = ld8(yp + c), b = ld8(gp + c), o;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o.v[e] = b.v[e] - gn * vv[c + e];
        acc[c + e] += -ch * b.v[e] - gn * a.v[e] + 2.f * ch * gn * vv[c + e];
      }
      st8(op + c, o);
    }
  }
  for (int c = 0; c < hd; c += 8) {
    F8 o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = acc[c + e];
    st8(dvp + c, o);
  }
}

// tanh(x) = 1 - 2 / (exp(2x) + 1) on the hardware exponential and reciprocal: absolute error ~1e-7, which the cap (30)
// turns into ~4e-6 on a capped logit. Used by the wide-vocabulary kernel, which evaluates tanh twice per logit (1.82 ->
// 1.57 ms at 98,304 x 8192); the one-warp-per-row kernel keeps the library tanhf: with the fast form its loss+gradient
// variant measured slower (0.47 vs 0.36 ms). Saturates cleanly: exp overflow gives 2 / inf = 0.
__device__ __forceinline__ float tanh_fast(float x) {
  const float e = __expf(2.f * x);
  return 1.f - __fdividef(2.f, e + 1.f);
}

// -------------------------------------------------------------------------------------------------------------
// Soft-capped cross-entropy over bf16 logits [rows, V]: c = cap*tanh(z/cap), nll = lse(c) - c[target];
// optionally dz = gscale * (softmax(c) - onehot) * (1 - tanh^2) written over the logits (or to `dlogits`).
// One warp per row; V <= 32*64.
__global__ void __launch_bounds__(ROW_THREADS) softcap_ce_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                                                 float* __restrict__ nll, __nv_bfloat16* __restrict__ dlogits,
                                                                 float* __restrict__ loss_sum, int rows, int V, float cap, float gscale,
                                                                 const float* __restrict__ tok_w, const float* __restrict__ w_total, int norm_rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ float wsum[ROW_WARPS];
  float local = 0.f;
  // Per-token loss weights (complementary training): the loss becomes sum(w l) / sum(w). `loss_sum` and the gradient
  // are rescaled by norm_rows / sum(w) so that callers keep dividing by the row count; `norm_rows` is the number of rows
  // the weights were summed over (more than `rows` when the batch is processed in chunks of rows).
  const float wnorm = (tok_w && w_total) ? (float)norm_rows / fmaxf(*w_total, 1e-12f) : 1.f;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const __nv_bfloat16* z = logits + (size_t)row * V;
    const int tgt = targets[row];
    float c[64];
    float mx = -1e30f;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int col = lane * 8 + it * 256, cnt = it * 8;
      if (col < V) {
        F8 a = ld8(z + col);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          c[cnt + e] = cap * tanhf(a.v[e] / cap);
          mx = fmaxf(mx, c[cnt + e]);
        }
      }
    }
    mx = warp_max(mx);
    float se = 0.f, ct = 0.f;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int col = lane * 8 + it * 256, cnt = it * 8;
      if (col < V) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          se += __expf(c[cnt + e] - mx);
          if (col + e == tgt) ct = c[cnt + e];
        }
      }
    }
    se = warp_sum(se);
    ct = warp_sum(ct);
    const float lse = mx + __logf(se);
    const float l = lse - ct;
    const float tw = tok_w ? tok_w[row] * wnorm : 1.f;
    if (lane == 0) {
      if (nll) nll[row] = l;
      local += l * tw;
    }
    if (dlogits) {
      __nv_bfloat16* dz = dlogits + (size_t)row * V;
      const float gs = gscale * tw;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int col = lane * 8 + it * 256, cnt = it * 8;
        if (col < V) {
          F8 o;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float p = __expf(c[cnt + e] - lse);
            const float th = c[cnt + e] / cap;
            o.v[e] = gs * (p - (col + e == tgt ? 1.f : 0.f)) * (1.f - th * th);
          }
          st8(dz + col, o);
        }
      }
    }
  }
  if (loss_sum) {
    if (lane == 0) wsum[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < ROW_WARPS; ++w) s += wsum[w];
      atomicAdd(loss_sum, s);
    }
  }
}

// Wide-vocabulary form of the kernel above (V > 2048, e.g. the 8192-token vocabularies): one CTA per row, the row is
// streamed twice from L2 instead of being held in registers. Pass 1 keeps a running (max, sum of exponentials) per thread
// and merges them across the CTA; pass 2 recomputes the capped logits and writes the gradient. Counterpart of the
// reference's tiled output cross-entropy (pg-kernels/src/gpu_kernels.rs:4241-4386, online max/sum across vocabulary tiles).
__global__ void __launch_bounds__(256) softcap_ce_wide_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                                              float* __restrict__ nll, __nv_bfloat16* __restrict__ dlogits,
                                                              float* __restrict__ loss_sum, int rows, int V, float cap, float gscale,
                                                              const float* __restrict__ tok_w, const float* __restrict__ w_total, int norm_rows) {
  __shared__ float s_mx[8], s_se[8], s_ct[8], s_bcast[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float wnorm = (tok_w && w_total) ? (float)norm_rows / fmaxf(*w_total, 1e-12f) : 1.f;
  const float inv_cap = 1.f / cap;
  float local = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* z = logits + (size_t)row * V;
    const int tgt = targets[row];
    float mx = -1e30f, se = 0.f, ct = 0.f;
    for (int col = threadIdx.x * 8; col < V; col += 256 * 8) {
      F8 a = ld8(z + col);
      float c[8], m8 = -1e30f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        c[e] = cap * tanh_fast(a.v[e] * inv_cap);
        m8 = fmaxf(m8, c[e]);
        if (col + e == tgt) ct = c[e];
      }
      if (m8 > mx) {
        se *= __expf(mx - m8);
        mx = m8;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) se += __expf(c[e] - mx);
    }
    // merge (max, sum) pairs: first inside the warp, then across the 8 warps
    const float wm = warp_max(mx);
    se = warp_sum(se * __expf(mx - wm));
    ct = warp_sum(ct);
    if (lane == 0) { s_mx[warp] = wm; s_se[warp] = se; s_ct[warp] = ct; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = s_mx[0], C = 0.f;
      for (int w = 1; w < 8; ++w) M = fmaxf(M, s_mx[w]);
      float S = 0.f;
      for (int w = 0; w < 8; ++w) { S += s_se[w] * __expf(s_mx[w] - M); C += s_ct[w]; }
      const float lse = M + __logf(S);
      s_bcast[0] = lse;
      s_bcast[1] = lse - C;
    }
    __syncthreads();
    const float lse = s_bcast[0], l = s_bcast[1];
    const float tw = tok_w ? tok_w[row] * wnorm : 1.f;
    if (threadIdx.x == 0) {
      if (nll) nll[row] = l;
      local += l * tw;
    }
    if (dlogits) {
      __nv_bfloat16* dz = dlogits + (size_t)row * V;
      const float gs = gscale * tw;
      for (int col = threadIdx.x * 8; col < V; col += 256 * 8) {
        F8 a = ld8(z + col);
        F8 o;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float th = tanh_fast(a.v[e] * inv_cap);
          const float p = __expf(cap * th - lse);
          o.v[e] = gs * (p - (col + e == tgt ? 1.f : 0.f)) * (1.f - th * th);
        }
        st8(dz + col, o);
      }
    }
    __syncthreads();            // s_bcast is rewritten by the next row
  }
  if (loss_sum && threadIdx.x == 0) atomicAdd(loss_sum, local);
}

// Weight of every (previous token, target) pair from a [V, V] table, and the sum of the weights (complementary training,
// parameter-golf-rs/crates/pg-kernels/src/complementary.rs:204-224). `w_total` must be zero on entry.
__global__ void __launch_bounds__(256) pair_weights_kernel(const int* __restrict__ prev, const int* __restrict__ curr, const float* __restrict__ table,
                                                           float* __restrict__ w, float* __restrict__ w_total, int rows, int V) {
  __shared__ float part[8];
  float local = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x) {
    const int a = prev[i], b = curr[i];
    const float x = ((unsigned)a < (unsigned)V && (unsigned)b < (unsigned)V) ? __ldg(table + (size_t)a * V + b) : 1.f;
    w[i] = x;
    local += x;
  }
  local = warp_sum(local);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int k = 0; k < 8; ++k) s += part[k];
    atomicAdd(w_total, s);
  }
}

// -------------------------------------------------------------------------------------------------------------
// Embedding gathers: e[t] = table[ids[t]] (bf16 rows of width d); bigram bucket = ((36313*cur) ^ (27191*prev)) % (B-1),
// sentinel bucket B-1 at sequence starts.
// A token id outside the table (a shard written with another tokenizer, a corrupted span) must not become an address: the
// row is written as zeros and the status word records the row, so the host can stop the run with a message.
__global__ void embed_gather_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out, int rows,
                                    int d, int table_rows, int bigram_buckets, int seq_len, int* __restrict__ status) {
  const int vec = d / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * vec) return;
  const int row = (int)(i / vec), c = (int)(i % vec) * 8;
  int id;
  if (bigram_buckets > 0) {
    if (row % seq_len == 0) id = bigram_buckets - 1;
    else id = (int)(((36313u * (uint32_t)ids[row]) ^ (27191u * (uint32_t)ids[row - 1])) % (uint32_t)(bigram_buckets - 1));
  } else {
    id = ids[row];
  }
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if ((unsigned)id < (unsigned)table_rows) v = *reinterpret_cast<const uint4*>(table + (size_t)id * d + c);
  else if (c == 0) report(status, ST_BAD_INDEX, row);
  *reinterpret_cast<uint4*>(out + (size_t)row * d + c) = v;
}

// Scatter-add of row gradients into an embedding-table gradient: each CTA owns a slice of `SLICE` columns and
// a range of rows, accumulates into a [table_rows][SLICE] fp32 tile in shared memory and flushes it once.
template <int SLICE>
__global__ void __launch_bounds__(256) embed_scatter_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ g, float* __restrict__ dtable,
                                                            int rows, int d, int table_rows, int bigram_buckets, int seq_len, int rows_per_cta) {
  extern __shared__ float tile[];
  const int c0 = blockIdx.x * SLICE;
  const int r0 = blockIdx.y * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  for (int i = threadIdx.x; i < table_rows * SLICE; i += blockDim.x) tile[i] = 0.f;
  __syncthreads();
  constexpr int LPR = SLICE / 8;                    // lanes per row
  for (int row = r0 + threadIdx.x / LPR; row < r1; row += blockDim.x / LPR) {
    const int sub = (threadIdx.x % LPR) * 8;
    int id;
    if (bigram_buckets > 0) {
      if (row % seq_len == 0) id = bigram_buckets - 1;
      else id = (int)(((36313u * (uint32_t)ids[row]) ^ (27191u * (uint32_t)ids[row - 1])) % (uint32_t)(bigram_buckets - 1));
    } else {
      id = ids[row];
    }
    if ((unsigned)id >= (unsigned)table_rows) continue;       // no table row to add to (the forward gather has flagged it)
    if (c0 + sub < d) {
      F8 a = ld8(g + (size_t)row * d + c0 + sub);
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(&tile[id * SLICE + sub + e], a.v[e]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < table_rows * SLICE; i += blockDim.x) {
    const int r = i / SLICE, c = i % SLICE;
    const float v = tile[i];
    if (v != 0.f && c0 + c < d) atomicAdd(dtable + (size_t)r * d + c0 + c, v);
  }
}

// Tables too tall for the shared-memory tile (8192-row vocabularies): one warp per gradient row, fp32 atomics straight into
// the table gradient. With thousands of table rows the atomics rarely collide.
__global__ void __launch_bounds__(256) embed_scatter_atomic_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ g,
                                                                   float* __restrict__ dtable, int rows, int d, int table_rows, int bigram_buckets,
                                                                   int seq_len) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    int id;
    if (bigram_buckets > 0) {
      if (row % seq_len == 0) id = bigram_buckets - 1;
      else id = (int)(((36313u * (uint32_t)ids[row]) ^ (27191u * (uint32_t)ids[row - 1])) % (uint32_t)(bigram_buckets - 1));
    } else {
      id = ids[row];
    }
    if ((unsigned)id >= (unsigned)table_rows) continue;       // warp-uniform: no table row to add to
    float* dst = dtable + (size_t)id * d;
    for (int col = lane * 8; col < d; col += 256) {
      F8 a = ld8(g + (size_t)row * d + col);
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(dst + col + e, a.v[e]);
    }
  }
}

// ---- launchers ---------------------------------------------------------------------------------------------------
static int row_grid(int rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return std::max(1, std::min((rows + ROW_WARPS - 1) / ROW_WARPS, sms * 8));
}

#define PGB_NV_DISPATCH(d, CALL)                                        \
  do {                                                                  \
    const int nv__ = ((d) + 255) / 256;                                 \
    if ((d) % 8) throw std::runtime_error("row width must be a multiple of 8"); \
    switch (nv__) {                                                     \
      case 1: { constexpr int NV = 1; CALL; } break;                    \
      case 2: { constexpr int NV = 2; CALL; } break;                    \
      case 3: { constexpr int NV = 3; CALL; } break;                    \
      case 4: { constexpr int NV = 4; CALL; } break;                    \
      case 5: case 6: { constexpr int NV = 6; CALL; } break;            \
      default: throw std::runtime_error("row width above 1536 is not supported"); \
    }                                                                   \
  } while (0)

void mix_norm_fwd(const void* x, const void* x0, const void* skip, const float* sw, const float* mix, void* x_in, void* h, int rows, int d, float s,
                  float eps, cudaStream_t st) {
  PGB_NV_DISPATCH(d, (mix_norm_fwd_kernel<NV><<<row_grid(rows), ROW_THREADS, 0, st>>>(
                         (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, (const __nv_bfloat16*)skip, sw, mix, (__nv_bfloat16*)x_in,
                         (__nv_bfloat16*)h, rows, d, s, eps)));
}

void mix_norm_bwd(const void* d_h, const void* d_res, const void* x_in, const void* x, const void* x0, const void* skip, const float* sw,
                  const float* mix, const void* add_grad, void* d_x, void* d_x0, void* d_skip, float* d_mix, float* d_sw, int skip_to_dx, int rows,
                  int d, float s, float eps, cudaStream_t st) {
  if (d <= 1536) {      // specialised variants (no accumulators when there is no mix/skip term, two CTAs per SM)
    mix_norm_bwd_v2(d_h, d_res, x_in, x, x0, skip, sw, mix, add_grad, d_x, d_x0, d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps, st);
    return;
  }
  const int grid = std::min(row_grid(rows), 148 * 4);
  PGB_NV_DISPATCH(d, (mix_norm_bwd_kernel<NV><<<grid, ROW_THREADS, ROW_WARPS * NV * 256 * sizeof(float), st>>>(
                         (const __nv_bfloat16*)d_h, (const __nv_bfloat16*)d_res, (const __nv_bfloat16*)x_in, (const __nv_bfloat16*)x,
                         (const __nv_bfloat16*)x0, (const __nv_bfloat16*)skip, sw, mix, (const __nv_bfloat16*)add_grad, (__nv_bfloat16*)d_x,
                         (__nv_bfloat16*)d_x0, (__nv_bfloat16*)d_skip, d_mix, d_sw, skip_to_dx, rows, d, s, eps)));
}

void norm_smear_fwd(const void* xe, const float* gate, const int* ids, void* out, int rows, int d, int seq_len, int boundary, float eps,
                    cudaStream_t st) {
  PGB_NV_DISPATCH(d, (norm_smear_fwd_kernel<NV><<<row_grid(rows), ROW_THREADS, 0, st>>>((const __nv_bfloat16*)xe, gate, ids, (__nv_bfloat16*)out,
                                                                                        rows, d, seq_len, boundary, eps)));
}

void norm_smear_bwd(const void* g_out, const void* xe, const float* gate, const int* ids, void* d_xe, float* d_gate, int rows, int d, int seq_len,
                    int boundary, float eps, cudaStream_t st) {
  const int grid = std::min(row_grid(rows), 148 * 4);
  PGB_NV_DISPATCH(d, (norm_smear_bwd_kernel<NV><<<grid, ROW_THREADS, ROW_WARPS * NV * 256 * sizeof(float), st>>>(
                         (const __nv_bfloat16*)g_out, (const __nv_bfloat16*)xe, gate, ids, (__nv_bfloat16*)d_xe, d_gate, rows, d, seq_len, boundary,
                         eps)));
}

void qk_norm_rope_fwd(const void* src, void* dst, const float* cosT, const float* sinT, const float* gain, int rows, int ld, int H, int Hkv, int hd,
                      int rope_dims, int seq_len, float eps, cudaStream_t st) {
  if (hd > 256 || hd % 8) throw std::runtime_error("head_dim must be a multiple of 8 and <= 256");
  if (qk_norm_rope_fast_ok(H, hd, rope_dims)) {
    qk_norm_rope_fwd64(src, dst, cosT, sinT, gain, rows, ld, H, Hkv, rope_dims, seq_len, eps, st);
    return;
  }
  const long long n = (long long)rows * (H + Hkv);
  auto kern = hd == 64 ? qk_norm_rope_fwd_kernel<64> : qk_norm_rope_fwd_kernel<0>;
  kern<<<(unsigned)((n + 127) / 128), 128, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, cosT, sinT, gain, rows, ld, H,
                                                                       Hkv, hd, rope_dims, seq_len, eps);
}

void qk_norm_rope_bwd(const void* d_post, const void* pre, void* d_pre, const float* cosT, const float* sinT, const float* gain, float* d_gain,
                      int rows, int ld, int H, int Hkv, int hd, int rope_dims, int seq_len, float eps, cudaStream_t st) {
  if (hd > 256 || hd % 8) throw std::runtime_error("head_dim must be a multiple of 8 and <= 256");
  if (qk_norm_rope_fast_ok(H, hd, rope_dims)) {
    qk_norm_rope_bwd64(d_post, pre, d_pre, cosT, sinT, gain, d_gain, rows, ld, H, Hkv, rope_dims, seq_len, eps, st);
    return;
  }
  const long long n = (long long)rows * (H + Hkv);
  auto kern = hd == 64 ? qk_norm_rope_bwd_kernel<64> : qk_norm_rope_bwd_kernel<0>;
  kern<<<(unsigned)((n + 127) / 128), 128, H * sizeof(float), st>>>(
      (const __nv_bfloat16*)d_post, (const __nv_bfloat16*)pre, (__nv_bfloat16*)d_pre, cosT, sinT, gain, d_gain, rows, ld, H, Hkv, hd, rope_dims,
      seq_len, eps);
}

void xsa_fwd(const void* y, const void* v, void* z, int rows, int Hkv, int group, int hd, int ld_y, int ld_v, float eps, cudaStream_t st) {
  if (hd == 64 && ld_y % 8 == 0 && ld_v % 8 == 0) {
    xsa_fwd64(y, v, z, rows, Hkv, group, ld_y, ld_v, eps, st);
    return;
  }
  const long long n = (long long)rows * Hkv;
  auto kern = hd == 64 ? xsa_fwd_kernel<64> : xsa_fwd_kernel<0>;
  kern<<<(unsigned)((n + 127) / 128), 128, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)v, (__nv_bfloat16*)z, rows, Hkv, group,
                                                              hd, ld_y, ld_v, eps);
}

void xsa_bwd(const void* dz, const void* y, const void* v, void* dy, void* dv, int accumulate_dv, int rows, int Hkv, int group, int hd, int ld_y,
             int ld_v, int ld_dv, float eps, cudaStream_t st, float* dsum, int seq_len) {
  if (hd == 64 && ld_y % 8 == 0 && ld_v % 8 == 0 && ld_dv % 8 == 0) {
    xsa_bwd64(dz, y, v, dy, dv, accumulate_dv, rows, Hkv, group, ld_y, ld_v, ld_dv, eps, st, dsum, seq_len);
    return;
  }
  if (dsum) throw std::runtime_error("xsa: the attention term is only produced by the head_dim 64 kernel");
  const long long n = (long long)rows * Hkv;
  auto kern = hd == 64 ? xsa_bwd_kernel<64> : xsa_bwd_kernel<0>;
  kern<<<(unsigned)((n + 127) / 128), 128, 0, st>>>((const __nv_bfloat16*)dz, (const __nv_bfloat16*)y, (const __nv_bfloat16*)v,
                                                              (__nv_bfloat16*)dy, (__nv_bfloat16*)dv, accumulate_dv, rows, Hkv, group, hd, ld_y, ld_v,
                                                              ld_dv, eps);
}

void softcap_ce(const void* logits, const int* targets, float* nll, void* dlogits, float* loss_sum, int rows, int V, float cap, float gscale,
                cudaStream_t st, const float* tok_w, const float* w_total, int norm_rows) {
  if (V % 8) throw std::runtime_error("vocab must be a multiple of 8 for the fused CE kernel");
  if (norm_rows <= 0) norm_rows = rows;
  if (V > 2048) {             // the row no longer fits the registers of one warp: one CTA per row, two passes
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    softcap_ce_wide_kernel<<<std::max(1, std::min(rows, sms * 8)), 256, 0, st>>>((const __nv_bfloat16*)logits, targets, nll, (__nv_bfloat16*)dlogits,
                                                                                 loss_sum, rows, V, cap, gscale, tok_w, w_total, norm_rows);
    return;
  }
  softcap_ce_kernel<<<row_grid(rows), ROW_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets, nll, (__nv_bfloat16*)dlogits, loss_sum, rows, V,
                                                            cap, gscale, tok_w, w_total, norm_rows);
}

void pair_weights(const int* prev, const int* curr, const float* table, float* w, float* w_total, int rows, int V, cudaStream_t st) {
  cudaMemsetAsync(w_total, 0, sizeof(float), st);
  const int grid = std::max(1, std::min(148 * 4, (rows + 255) / 256));
  pair_weights_kernel<<<grid, 256, 0, st>>>(prev, curr, table, w, w_total, rows, V);
}

void embed_gather(const int* ids, const void* table, void* out, int rows, int d, int table_rows, int bigram_buckets, int seq_len, cudaStream_t st,
                  int* status) {
  const long long n = (long long)rows * (d / 8);
  embed_gather_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, rows, d, table_rows,
                                                                   bigram_buckets, seq_len, status);
}

void embed_scatter_add(const int* ids, const void* g, float* dtable, int rows, int d, int table_rows, int bigram_buckets, int seq_len,
                       cudaStream_t st) {
  // slice width so that table_rows * slice * 4 bytes fits in ~200 KB of shared memory
  int slice = 32;
  while (slice > 8 && (size_t)table_rows * slice * 4 > 200 * 1024) slice /= 2;
  if ((size_t)table_rows * slice * 4 > 200 * 1024) {
    embed_scatter_atomic_kernel<<<std::max(1, std::min((rows + 7) / 8, 148 * 8)), 256, 0, st>>>(ids, (const __nv_bfloat16*)g, dtable, rows, d,
                                                                                               table_rows, bigram_buckets, seq_len);
    return;
  }
  const int cslices = (d + slice - 1) / slice;
  const int ychunks = std::max(1, std::min(148 * 2 / cslices, (rows + 2047) / 2048));
  const int rows_per = (rows + ychunks - 1) / ychunks;
  const size_t smem = (size_t)table_rows * slice * 4;
  dim3 grid(cslices, ychunks);
  auto launch = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 256, smem, st>>>(ids, (const __nv_bfloat16*)g, dtable, rows, d, table_rows, bigram_buckets, seq_len, rows_per);
  };
  if (slice == 32) launch(embed_scatter_kernel<32>);
  else if (slice == 16) launch(embed_scatter_kernel<16>);
  else launch(embed_scatter_kernel<8>);
}

}  // namespace pgb
