// Host API of the sm_100a kernel library (raw pointers + stream; no framework types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <stdexcept>

namespace pgb {

// ---- GEMM ---------------------------------------------------------------------------------------------
enum GemmEpilogue : int {
  EPI_BF16 = 0,         // D = bf16(alpha * acc)
  EPI_F32 = 1,          // D = alpha * acc                      (fp32)
  EPI_F32_ATOMIC = 2,   // D += alpha * acc                     (fp32, red.add; split-K allowed)
  EPI_AXPBY_BF16 = 3,   // D = bf16(alpha * acc + beta * aux)   (aux bf16, same shape)
  EPI_RESID_BF16 = 4,   // D = bf16(aux + colscale[n] * acc)    (residual add with per-feature scale)
  EPI_ACT_SQ = 5,       // D = bf16(acc), D2 = bf16(leaky_relu(acc, slope)^2)
  EPI_MUL_ACTGRAD = 6,  // D = bf16(acc * d/dh leaky_relu(h, slope)^2), h = aux
};

struct GemmArgs {
  const void* A = nullptr;   // bf16
  const void* B = nullptr;   // bf16
  void* D = nullptr;
  void* D2 = nullptr;
  const void* aux = nullptr;
  const float* colscale = nullptr;
  int M = 0, N = 0, K = 0, batch = 1;
  bool a_kmajor = true;      // true: A stored [M][K]; false: A stored [K][M]
  bool b_kmajor = true;      // true: B stored [N][K]; false: B stored [K][N]
  long long lda = 0, ldb = 0, ldd = 0, ld_aux = 0;                    // row strides in elements
  long long stride_a = 0, stride_b = 0, stride_d = 0, stride_aux = 0; // batch strides in elements
  int epi = EPI_BF16;
  int splits = 0;            // 0 = automatic
  float alpha = 1.f, beta = 0.f, slope = 0.f;
  int* status = nullptr;     // device status word (4 ints) or null
};

void gemm_bf16(const GemmArgs& args, cudaStream_t stream);

}  // namespace pgb
