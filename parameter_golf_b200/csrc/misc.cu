// Small utility kernels: token-span expansion and an L2 flush.
#include "common.cuh"
#include "pgb.h"

namespace pgb {

// span: uint16[n+1] as uploaded from the shard (2 bytes per token over PCIe instead of 2 x 8);
// ids[i] = span[i], targets[i] = span[i+1]   (parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:2414 has the same role).
__global__ void expand_span_kernel(const uint16_t* __restrict__ span, int* __restrict__ ids, int* __restrict__ targets, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    ids[i] = span[i];
    targets[i] = span[i + 1];
  }
}

void expand_span_u16(const void* span, int* ids, int* targets, int n, cudaStream_t st) {
  expand_span_kernel<<<(n + 255) / 256, 256, 0, st>>>((const uint16_t*)span, ids, targets, n);
}

}  // namespace pgb
