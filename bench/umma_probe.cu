// Throughput probe for tcgen05.mma instruction shapes: one CTA per SM issues a long run of independent-accumulator-free
// (same accumulator) MMAs from one thread and measures cycles per instruction with clock64. Operands are whatever is
// in shared / tensor memory; only timing matters.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I parameter_golf_b200/csrc bench/umma_probe.cu -o /tmp/umma_probe && /tmp/umma_probe
#include <cstdio>
#include "common.cuh"
using namespace pgb;

template <int N, bool TS, bool B_MN>
__global__ void probe(long long* out, int iters) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, B_MN ? 1 : 0);
    const uint32_t sa = smem_u32(smem), sb = smem_u32(smem + 32768);
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const int k = i & 3;
      const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
      if (TS) umma_ts(tm + 256, tm + k * 8, db, idesc, 1u);
      else umma_ss(tm + 256, make_smem_desc(sa + k * 32, 16, 1024), db, idesc, 1u);
    }
    umma_commit(&bar);
    volatile int abort_flag = 0;
    mbar_wait(&bar, 0, &abort_flag, nullptr, 0, 0);
    long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

// Round trip: MMA thread issues `nmma` MMAs + commit -> 128 consumer threads wake on the mbarrier, (optionally) load `ldcols`
// TMEM columns, arrive on a second mbarrier -> MMA thread wakes. Cycles per round trip.
template <int LDCOLS>
__global__ void pingpong(long long* out, int iters, int nmma) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t barA, barB;
  __shared__ uint32_t slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) { mbar_init(&barA, 1); mbar_init(&barB, 128); abort_flag_s = 0; fence_barrier_init(); }
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t sa = smem_u32(smem), sb = smem_u32(smem + 32768);
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      for (int k = 0; k < nmma; ++k) umma_ss(tm, make_smem_desc(sa + (k & 3) * 32, 16, 1024), make_smem_desc(sb + (k & 3) * 32, 16, 1024), idesc, 1u);
      umma_commit(&barA);
      mbar_wait(&barB, i & 1, abort_flag, nullptr, 0, 0);
      tc_fence_after();
    }
    long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  } else if (warp >= 1 && warp <= 4) {
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t sink = 0;
    for (int i = 0; i < iters; ++i) {
      mbar_wait(&barA, i & 1, abort_flag, nullptr, 0, 0);
      tc_fence_after();
      if (LDCOLS > 0) {
        uint32_t r[32];
        for (int c = 0; c < LDCOLS; c += 32) { PGB_TMEM_LD32(tm + lane_off + c, r); }
        tmem_wait_ld();
        sink += r[0] + r[31];
      }
      tc_fence_before();
      mbar_arrive(&barB);
    }
    if (sink == 0x12345) out[1] = sink;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

template <int LDCOLS>
void run_pp(const char* name, long long* d, int nmma) {
  const int iters = 2000;
  cudaFuncSetAttribute(pingpong<LDCOLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  pingpong<LDCOLS><<<148, 160, 100 * 1024>>>(d, iters, nmma);
  cudaDeviceSynchronize();
  pingpong<LDCOLS><<<148, 160, 100 * 1024>>>(d, iters, nmma);
  cudaError_t e = cudaDeviceSynchronize();
  long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  printf("%-44s %7.1f clk/round trip (%s)\n", name, (double)h / iters, cudaGetErrorString(e));
}

template <int N, bool TS, bool B_MN>
void run(const char* name, long long* d) {
  const int iters = 4096;
  cudaFuncSetAttribute(probe<N, TS, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  probe<N, TS, B_MN><<<148, 128, 100 * 1024>>>(d, iters);
  cudaDeviceSynchronize();
  probe<N, TS, B_MN><<<148, 128, 100 * 1024>>>(d, iters);
  cudaError_t e = cudaDeviceSynchronize();
  long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  const double cyc = (double)h / iters;
  printf("%-28s %7.1f clk/instr  %7.0f FLOP/clk/SM  (%s)\n", name, cyc, 2.0 * 128 * N * 16 / cyc, cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 8);
  run<256, false, false>("SS M128 N256 K-major B", d);
  run<128, false, false>("SS M128 N128 K-major B", d);
  run<64, false, false>("SS M128 N64  K-major B", d);
  run<64, false, true>("SS M128 N64  MN-major B", d);
  run<128, true, true>("TS M128 N128 MN-major B", d);
  run<64, true, true>("TS M128 N64  MN-major B", d);
  run<64, true, false>("TS M128 N64  K-major B", d);
  run_pp<0>("round trip, 1 MMA (64 clk), no TMEM load", d, 1);
  run_pp<0>("round trip, 4 MMA (256 clk), no TMEM load", d, 4);
  run_pp<128>("round trip, 4 MMA, load 128 columns", d, 4);
  run_pp<32>("round trip, 4 MMA, load 32 columns", d, 4);
  return 0;
}
