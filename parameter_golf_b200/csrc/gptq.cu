// GPTQ row kernel: column-by-column quantisation with Hessian error feedback, one warp per weight row.
//
// Inputs are what the host prepared once per matrix: the column-permuted weights Wp [rows, cols] (activation order),
// the upper Cholesky factor U [cols, cols] of the inverse permuted Hessian, and one fixed scale per row (one clip
// candidate; the caller loops over candidates and keeps the best per row).  Rows are independent, so the only serial
// dimension is the column index; the row lives in shared memory and the current 128-column block in registers
// (4 per lane), column values are broadcast with shuffles, the rank-1 feedback inside the block reads U from a shared
// 128x128 tile and the feedback to the columns right of the block is a 128-term dot product per column.
// The arithmetic inside a block is written with explicitly rounded operations (no fused multiply-add) so that the
// codes match the float32 reference except where the two summation orders of the trailing update differ.
//
// Reference behaviour: the full-Hessian GPTQ of records/track_10min_16mb/2026-03-25_ValCalib_GPTQ_XSA_BigramHash3072/
// train_gpt.py:1171-1224 (block size 128, act-order, per-row clip candidates).
#include <cuda_runtime.h>
#include <stdint.h>

#include "pgb.h"

namespace pgb {

namespace {
constexpr int GQ_WARPS = 8;
constexpr int GQ_BLOCK = 128;

__device__ __forceinline__ float round_half_away(float x) { return copysignf(floorf(fabsf(x) + 0.5f), x); }

__global__ void __launch_bounds__(GQ_WARPS * 32)
gptq_rows_kernel(const float* __restrict__ Wp, const float* __restrict__ U, const float* __restrict__ scales, int8_t* __restrict__ Q, int rows,
                 int cols, float qmin, float qmax) {
  extern __shared__ float sm[];
  float* sU = sm;                                   // [128][128] diagonal tile of U
  float* sW = sU + GQ_BLOCK * GQ_BLOCK;             // [warps][cols] working rows
  float* sE = sW + GQ_WARPS * cols;                 // [warps][128] scaled errors of the current block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * GQ_WARPS + warp;
  const bool active = row < rows;
  float* w_row = sW + warp * cols;
  float* e_row = sE + warp * GQ_BLOCK;
  if (active)
    for (int c = lane; c < cols; c += 32) w_row[c] = Wp[(size_t)row * cols + c];
  const float s = active ? scales[row] : 1.f;
  for (int i1 = 0; i1 < cols; i1 += GQ_BLOCK) {
    const int nb = min(GQ_BLOCK, cols - i1);
    __syncthreads();
    for (int idx = threadIdx.x; idx < GQ_BLOCK * GQ_BLOCK; idx += blockDim.x) {
      const int j = idx >> 7, c = idx & 127;
      sU[idx] = (j < nb && c < nb) ? U[(size_t)(i1 + j) * cols + i1 + c] : 0.f;
    }
    __syncthreads();
    if (!active) continue;
    float reg[4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int c = ii * 32 + lane;
      reg[ii] = c < nb ? w_row[i1 + c] : 0.f;
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      for (int jj = 0; jj < 32; ++jj) {
        const int j = ii * 32 + jj;
        if (j >= nb) break;                                            // uniform across the warp
        const float w = __shfl_sync(0xffffffffu, reg[ii], jj);
        const float q = fminf(fmaxf(round_half_away(__fdiv_rn(w, s)), qmin), qmax);
        const float err = __fdiv_rn(__fsub_rn(w, __fmul_rn(q, s)), sU[j * GQ_BLOCK + j]);
        if (lane == jj) {
          Q[(size_t)row * cols + i1 + j] = (int8_t)q;
          e_row[j] = err;
        }
        const float* u_row = sU + j * GQ_BLOCK;
#pragma unroll
        for (int i2 = 0; i2 < 4; ++i2) {
          if (i2 >= ii) {
            const int c = i2 * 32 + lane;
            if (c >= j) reg[i2] = __fsub_rn(reg[i2], __fmul_rn(err, u_row[c]));
          }
        }
      }
    }
    __syncwarp();
    // feedback to every column right of the block: w[c] -= sum_j err[j] * U[i1 + j][c]
    for (int c = i1 + nb + lane; c < cols; c += 32) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float* u = U + (size_t)i1 * cols + c;
      int j = 0;
      for (; j + 4 <= nb; j += 4) {
        a0 = fmaf(e_row[j], u[(size_t)j * cols], a0);
        a1 = fmaf(e_row[j + 1], u[(size_t)(j + 1) * cols], a1);
        a2 = fmaf(e_row[j + 2], u[(size_t)(j + 2) * cols], a2);
        a3 = fmaf(e_row[j + 3], u[(size_t)(j + 3) * cols], a3);
      }
      for (; j < nb; ++j) a0 = fmaf(e_row[j], u[(size_t)j * cols], a0);
      w_row[c] -= (a0 + a1) + (a2 + a3);
    }
    __syncwarp();
  }
}
}  // namespace

void gptq_rows(const float* Wp, const float* U, const float* scales, int8_t* Q, int rows, int cols, int bits, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return;
  if (bits < 2 || bits > 8) throw std::runtime_error("gptq_rows: bits must be in 2..8");
  const size_t smem = ((size_t)GQ_BLOCK * GQ_BLOCK + (size_t)GQ_WARPS * cols + GQ_WARPS * GQ_BLOCK) * sizeof(float);
  if (smem > 227 * 1024) throw std::runtime_error("gptq_rows: rows of more than " + std::to_string((227 * 1024 / 4 - GQ_BLOCK * GQ_BLOCK - GQ_WARPS * GQ_BLOCK) / GQ_WARPS) + " columns do not fit in shared memory");
  static size_t configured[64] = {};        // largest size set so far, per device (the attribute is a per-device property)
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || smem > configured[dev]) {
    cudaFuncSetAttribute(gptq_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (dev >= 0 && dev < 64) configured[dev] = smem;
  }
  const float qmax = (float)((1 << (bits - 1)) - 1), qmin = -(float)(1 << (bits - 1));
  gptq_rows_kernel<<<(rows + GQ_WARPS - 1) / GQ_WARPS, GQ_WARPS * 32, smem, st>>>(Wp, U, scales, Q, rows, cols, qmin, qmax);
}

}  // namespace pgb
