// Attention backward without any allocation: the per-row scratch (rowsum(dO * O), written by the dQ kernel and read
// by the dK/dV kernel) lives in a file-scope device array instead of a caller- or allocator-provided buffer.
//
// Nothing on this path calls cudaMalloc/cudaFree, a stream-ordered allocator or a tensor library: the host side only
// encodes tensor maps on the stack and launches the two kernels of attn_bwd.cu.  The one-off work is the set-up
// (symbol address look-up, which makes the runtime load this module on the device; the first launch also sets the
// kernels' dynamic shared-memory attribute); it happens once per device and should happen before any stream capture
// begins.
#include <cuda_runtime.h>

#include <stdio.h>

#include <exception>

#include "pgb.h"
#include "pgb_noalloc.h"

namespace {

// 4 MiB per device: covers e.g. 64 sequences x 8 heads x 2048 tokens.
static __device__ __align__(256) float g_attn_bwd_scratch[PGB_ATTN_BWD_NOALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};      // device address of the array above, per device ordinal
thread_local char g_err[256] = "";

int fail(int code, const char* what, const char* detail) {
  snprintf(g_err, sizeof(g_err), "%s%s%s", what, detail[0] ? ": " : "", detail);
  return code;
}

}  // namespace

extern "C" int pgb_attn_bwd_noalloc_setup(void) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(3, "cudaGetDevice", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(3, "device ordinal out of range", "");
  if (g_scratch_ptr[dev]) return 0;
  float* ptr = nullptr;
  e = cudaGetSymbolAddress((void**)&ptr, g_attn_bwd_scratch);
  if (e != cudaSuccess || ptr == nullptr) return fail(3, "cudaGetSymbolAddress(attention backward scratch)", cudaGetErrorString(e));
  g_scratch_ptr[dev] = ptr;
  return 0;
}

extern "C" int pgb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk,
                                    void* dv, long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq,
                                    long long lddk, long long lddv, int B, int S, int H, int Hkv, int hd, int accumulate_dv, int* status,
                                    void* stream) {
  if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return fail(2, "bad shape", "B, S, H, Hkv must be positive and Hkv must divide H");
  if (hd != 64 || S % 128 != 0) return fail(2, "bad shape", "head_dim must be 64 and seq_len a multiple of 128");
  const long long rows = (long long)B * H * S;
  if (rows > PGB_ATTN_BWD_NOALLOC_MAX_ROWS) {
    char d[160];
    snprintf(d, sizeof(d), "B*H*S = %lld exceeds the built-in scratch of %lld rows; use the entry point that takes a caller-provided dsum", rows,
             (long long)PGB_ATTN_BWD_NOALLOC_MAX_ROWS);
    return fail(1, "problem too large for the no-allocation entry point", d);
  }
  const int rc = pgb_attn_bwd_noalloc_setup();
  if (rc) return rc;
  int dev = 0;
  const cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess || dev < 0 || dev >= kMaxDevices || g_scratch_ptr[dev] == nullptr) return fail(3, "cudaGetDevice", cudaGetErrorString(ge));
  try {
    pgb::attn_bwd(q, k, v, o, d_o, lse, g_scratch_ptr[dev], dq, dk, dv, ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv, B, S, H, Hkv, hd, accumulate_dv,
                  status, (cudaStream_t)stream);
  } catch (const std::exception& ex) {
    return fail(2, "attention backward rejected the arguments", ex.what());
  }
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(3, "kernel launch", cudaGetErrorString(e));
  return 0;
}

extern "C" const char* pgb_noalloc_last_error(void) { return g_err; }
