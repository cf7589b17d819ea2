// Symmetric memory over CUDA IPC: every rank cudaMalloc's the same-sized buffer, publishes its IPC handle,
// opens the others' and ends with a table of `world` device pointers (own entry = local pointer).
// The exchange itself happens in Python over the process group (control plane only).
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <string>

#include "pgb.h"

namespace pgb {

static void ck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void* symm_alloc(size_t bytes) {
  void* p = nullptr;
  ck(cudaMalloc(&p, bytes), "cudaMalloc (symmetric buffer)");
  ck(cudaMemset(p, 0, bytes), "cudaMemset (symmetric buffer)");
  return p;
}

std::string symm_export(void* p) {
  cudaIpcMemHandle_t h;
  ck(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void* symm_import(const std::string& handle) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  ck(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return p;
}

void symm_close(void* p) { cudaIpcCloseMemHandle(p); }
void symm_free(void* p) { cudaFree(p); }

}  // namespace pgb
