// Per-head attention output gates: out_h = y_h * g_h with g_h = mult * sigmoid(scale * <W_h, x[:w]> + bias_h), where x is the
// block's normed input (first `w` features of its row) and h a query head. One kernel pair covers both gates of the
// model: the attention-output gate (mult 2, scale 1, bias) and the sparse attention gate (mult 1, scale s, no bias).
// Same math as the reference's attn_out_gate_* / sparse_attn_gate_* kernels
// (parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:4973-5076, :5078-5123, :5282-5413), restated for bf16
// activations and with the weight-gradient reduction done per CTA in shared memory before one atomic per (head, k).
#include "common.cuh"
#include "pgb.h"

namespace pgb {

namespace {

constexpr int GATE_THREADS = 128;
constexpr int GATE_MAX_W = 64;

struct G8 { float v[8]; };
__device__ __forceinline__ G8 g_ld8(const __nv_bfloat16* p) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  return G8{{a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y}};
}
__device__ __forceinline__ void g_st8(__nv_bfloat16* p, const G8& f) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f.v[0], f.v[1]), pack_bf16x2(f.v[2], f.v[3]), pack_bf16x2(f.v[4], f.v[5]),
                                            pack_bf16x2(f.v[6], f.v[7]));
}

// One thread per (token, head). x rows have ld_x elements, y/out rows H*hd.
__global__ void head_gate_fwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x, const float* __restrict__ W,
                                     const float* __restrict__ bias, __nv_bfloat16* __restrict__ out, float* __restrict__ gate, int rows, int H,
                                     int hd, int w, int ld_x, float scale, float mult) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * H) return;
  const int row = (int)(idx / H), h = (int)(idx % H);
  const __nv_bfloat16* xp = x + (size_t)row * ld_x;
  const float* wp = W + (size_t)h * w;
  float pre = 0.f;
  for (int k = 0; k < w; ++k) pre += __bfloat162float(xp[k]) * wp[k];
  const float u = scale * pre + (bias ? bias[h] : 0.f);
  const float g = mult / (1.f + __expf(-u));
  gate[idx] = g;
  const __nv_bfloat16* yp = y + (size_t)row * H * hd + h * hd;
  __nv_bfloat16* op = out + (size_t)row * H * hd + h * hd;
  for (int c = 0; c < hd; c += 8) {
    G8 a = g_ld8(yp + c);
#pragma unroll
    for (int e = 0; e < 8; ++e) a.v[e] *= g;
    g_st8(op + c, a);
  }
}

// d_out is overwritten in place by the gradient with respect to y. The gradient of the gate's pre-activation goes to
// the weights (CTA-level reduction, then atomics), to the bias, and to the first w features of d_x (added when
// `accumulate_dx`, stored otherwise). blockDim.x = tokens_per_block * H.
__global__ void head_gate_bwd_kernel(__nv_bfloat16* __restrict__ d_out, const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                     const float* __restrict__ W, const float* __restrict__ gate, float* __restrict__ dW, float* __restrict__ dbias,
                                     __nv_bfloat16* __restrict__ d_x, int accumulate_dx, int rows, int H, int hd, int w, int ld_x, int ld_dx,
                                     float scale, float mult) {
  extern __shared__ float sm[];
  const int tpb = blockDim.x / H;                 // tokens per block
  float* s_dpre = sm;                             // [tpb][H]
  float* s_x = sm + tpb * H;                      // [tpb][w]
  const int tok = threadIdx.x / H, h = threadIdx.x % H;
  const int row = blockIdx.x * tpb + tok;
  float dpre = 0.f;
  if (row < rows) {
    const float g = gate[(size_t)row * H + h];
    __nv_bfloat16* gp = d_out + (size_t)row * H * hd + h * hd;
    const __nv_bfloat16* yp = y + (size_t)row * H * hd + h * hd;
    float dg = 0.f;
    for (int c = 0; c < hd; c += 8) {
      G8 a = g_ld8(gp + c);
      const G8 b = g_ld8(yp + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dg += a.v[e] * b.v[e];
        a.v[e] *= g;
      }
      g_st8(gp + c, a);
    }
    dpre = dg * g * (1.f - g / mult);            // d/du of mult * sigmoid(u)
  }
  s_dpre[tok * H + h] = dpre;
  for (int i = threadIdx.x; i < tpb * w; i += blockDim.x) {
    const int t = i / w, k = i % w, r = blockIdx.x * tpb + t;
    s_x[i] = r < rows ? __bfloat162float(x[(size_t)r * ld_x + k]) : 0.f;
  }
  __syncthreads();
  // weights and bias: sum over the block's tokens, one atomic per (head, k)
  for (int i = threadIdx.x; i < H * w; i += blockDim.x) {
    const int hh = i / w, k = i % w;
    float acc = 0.f;
    for (int t = 0; t < tpb; ++t) acc += s_dpre[t * H + hh] * s_x[t * w + k];
    if (acc != 0.f) atomicAdd(dW + i, scale * acc);
  }
  if (dbias != nullptr)
    for (int hh = threadIdx.x; hh < H; hh += blockDim.x) {
      float acc = 0.f;
      for (int t = 0; t < tpb; ++t) acc += s_dpre[t * H + hh];
      if (acc != 0.f) atomicAdd(dbias + hh, acc);
    }
  // input features: sum over heads, one owner per (token, k)
  for (int i = threadIdx.x; i < tpb * w; i += blockDim.x) {
    const int t = i / w, k = i % w, r = blockIdx.x * tpb + t;
    if (r >= rows) continue;
    float acc = 0.f;
    for (int hh = 0; hh < H; ++hh) acc += s_dpre[t * H + hh] * W[(size_t)hh * w + k];
    acc *= scale;
    __nv_bfloat16* dp = d_x + (size_t)r * ld_dx + k;
    if (accumulate_dx) acc += __bfloat162float(*dp);
    *dp = __float2bfloat16(acc);
  }
}

}  // namespace

void head_gate_fwd(const void* y, const void* x, const float* W, const float* bias, void* out, float* gate, int rows, int H, int hd, int w, int ld_x,
                   float scale, float mult, cudaStream_t st) {
  if (hd % 8) throw std::runtime_error("head_gate: head_dim must be a multiple of 8");
  const long long n = (long long)rows * H;
  head_gate_fwd_kernel<<<(unsigned)((n + GATE_THREADS - 1) / GATE_THREADS), GATE_THREADS, 0, st>>>(
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)x, W, bias, (__nv_bfloat16*)out, gate, rows, H, hd, w, ld_x, scale, mult);
}

void head_gate_bwd(void* d_out, const void* y, const void* x, const float* W, const float* gate, float* dW, float* dbias, void* d_x, int accumulate_dx,
                   int rows, int H, int hd, int w, int ld_x, int ld_dx, float scale, float mult, cudaStream_t st) {
  if (hd % 8) throw std::runtime_error("head_gate: head_dim must be a multiple of 8");
  if (H > GATE_THREADS || w > GATE_MAX_W) throw std::runtime_error("head_gate: at most 128 heads and a gate width of 64");
  const int tpb = std::max(1, GATE_THREADS / H);
  const int threads = tpb * H;
  const size_t smem = (size_t)(tpb * H + tpb * w) * sizeof(float);
  head_gate_bwd_kernel<<<(unsigned)((rows + tpb - 1) / tpb), threads, smem, st>>>(
      (__nv_bfloat16*)d_out, (const __nv_bfloat16*)y, (const __nv_bfloat16*)x, W, gate, dW, dbias, (__nv_bfloat16*)d_x, accumulate_dx, rows, H, hd,
      w, ld_x, ld_dx, scale, mult);
}

}  // namespace pgb
