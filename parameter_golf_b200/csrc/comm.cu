// Collectives over NVLink/NVSwitch peer memory, fused with the work that follows them. No NCCL here.
//
// Every rank allocates the same buffers and exchanges IPC handles once (symm.cpp); kernels receive a table of
// the `world` peer base pointers and use plain peer loads/stores (no TMA on peer memory, no multicast).
// Cross-rank ordering uses 32-bit epoch flags in a symmetric signal pad written with st.release.sys and
// polled with ld.acquire.sys; every poll loop is bounded (PGB_WAIT_LIMIT_NS) and reports to the status word.
//
//   reduce_peers_kernel    out[i] = scale * sum_r peer_r[off + i]  (+ sum of squares of the result):
//                          with out == my own slice it is the reduce-scatter of the bank gradients fused with the
//                          1/world scale and the global-norm partial (sites N3 + K3 of the reference,
//                          parameter-golf-rs/crates/pg-train/src/lib.rs:3400-3446, 3491-3608); with a separate
//                          `out` it is the one-shot all-reduce of the small replicated gradients (site N2).
//   push_cast_rows_kernel  updated fp32 master rows -> bf16 compute rows (row scale, int6 fake-quant) written into
//                          EVERY rank's weight buffer: the parameter all-gather (site N6) fused with the shadow
//                          refresh; a per-layer ready counter is bumped on every rank afterwards and the next
//                          forward's QKV GEMM polls it before its first TMA load (gemm.cu).
//   scalar_allreduce_kernel  sum of one float per rank through the signal pad (site N5); doubles as the barrier
//                          that tells every rank its gradients have been consumed.
#include "common.cuh"
#include "pgb.h"

namespace pgb {

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) { asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

__device__ __forceinline__ bool wait_flag_ge(const int* p, int want, int* status, int detail) {
  if (ld_acquire_sys(p) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(p) < want) {
    if (globaltimer_ns() - t0 > PGB_WAIT_LIMIT_NS) {
      report(status, ST_WAIT_FLAG, detail);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// One block of `world` threads (<= 32): thread r raises my flag on rank r, then waits for rank r's flag here.
// sig_tbl[r] = base of rank r's signal pad; slot = first of `world` consecutive ints used by this barrier.
__global__ void barrier_kernel(int* const* __restrict__ sig_tbl, int my_rank, int world, int slot, int epoch, int* status) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(sig_tbl[r] + slot + my_rank, epoch);
    wait_flag_ge(sig_tbl[my_rank] + slot + r, epoch, status, r);
  }
}

// out[i] = scale * sum_r src_tbl[r][off + i], i in [0, n); stats[0] += sq_weight * sum(out^2). n, off multiples of 4.
// WORLD > 0 fixes the rank count at compile time: all peers' 16-byte loads of one element group are issued before the
// first add, so a thread keeps WORLD NVLink requests in flight instead of one.
// `wait_flag` (optional): a local counter that every rank bumps once its part of these gradients is final (release at
// system scope after the producing kernels); each block polls it, bounded, before its first peer load, so the kernel can
// be queued on a side stream while the backward pass that produces the gradients is still running.
template <int WORLD>
__global__ void __launch_bounds__(256) reduce_peers_kernel(const float* const* __restrict__ src_tbl, int world_rt, long long off, long long n,
                                                           float* __restrict__ out, float scale, float* __restrict__ stats, float sq_weight,
                                                           const int* __restrict__ wait_flag, int wait_value, int* status) {
  if (wait_flag != nullptr) {
    __shared__ int ready;
    if (threadIdx.x == 0) ready = wait_flag_ge(wait_flag, wait_value, status, wait_value) ? 1 : 0;
    __syncthreads();
    if (!ready) return;
  }
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  if constexpr (WORLD > 0) {
    const float* src[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) src[r] = src_tbl[r] + off;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
      float4 v[WORLD];
#pragma unroll
      for (int r = 0; r < WORLD; ++r) v[r] = *reinterpret_cast<const float4*>(src[r] + i);
      float4 acc = v[0];
#pragma unroll
      for (int r = 1; r < WORLD; ++r) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      *reinterpret_cast<float4*>(out + i) = acc;
      s += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  } else {
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world_rt; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(src_tbl[r] + off + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      *reinterpret_cast<float4*>(out + i) = acc;
      s += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  if (stats) {
    s = warp_sum(s);
    __shared__ float ws[8];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += ws[w];
      atomicAdd(stats, t * sq_weight);
    }
  }
}

// Each rank contributes stats[0]; every rank ends with the sum in stats[0]. val_tbl[r] = rank r's float pad (>= world floats at val_slot).
__global__ void scalar_allreduce_kernel(float* const* __restrict__ val_tbl, int* const* __restrict__ sig_tbl, int my_rank, int world, int val_slot,
                                        int sig_slot, int epoch, float* __restrict__ stats, int* status) {
  __shared__ float part[32];
  const int r = threadIdx.x;
  if (r < world) {
    const float mine = stats[0];
    val_tbl[r][val_slot + my_rank] = mine;
    __threadfence_system();
    st_release_sys(sig_tbl[r] + sig_slot + my_rank, epoch);
    const bool ok = wait_flag_ge(sig_tbl[my_rank] + sig_slot + r, epoch, status, r);
    part[r] = ok ? *reinterpret_cast<volatile float*>(val_tbl[my_rank] + val_slot + r) : 0.f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < world; ++i) t += part[i];      // fixed order: bit-identical on every rank
    stats[0] = t;
  }
}

// Row cast with fan-out: dst_tbl[r] + dst_off is the destination matrix on rank r (row stride ld_dst).
__global__ void __launch_bounds__(256) push_cast_rows_kernel(const float* __restrict__ src, __nv_bfloat16* const* __restrict__ dst_tbl, int world,
                                                             long long dst_off, const float* __restrict__ rowscale, int scale_stride, int scale_mod,
                                                             int rows, int cols, long long ld_dst, int qat) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const float* s = src + (size_t)row * cols;
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
      const uint2 p = make_uint2(pack_bf16x2(a.x * rs, a.y * rs), pack_bf16x2(a.z * rs, a.w * rs));
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(dst_tbl[r] + dst_off + (size_t)row * ld_dst + c) = p;
    }
  }
}

// The same for a run of consecutive bank slots in ONE launch.  desc[s] = {destination element offset of slot s,
// offset of its un-scaled twin or -1, address of its first row scale or 0, index of its ready counter}; slot s starts
// at src + s * rows * cols.  Slots with a row scale write both the scaled rows and the un-scaled twin.
__global__ void __launch_bounds__(256) push_cast_slots_kernel(const float* __restrict__ src, __nv_bfloat16* const* __restrict__ dst_tbl, int world,
                                                              const long long* __restrict__ desc, int n_slots, int rows, int cols, long long ld_dst,
                                                              int qat) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)n_slots * rows;
  for (long long item = (long long)blockIdx.x * 8 + warp; item < total; item += (long long)gridDim.x * 8) {
    const int slot = (int)(item / rows), row = (int)(item - (long long)slot * rows);
    const long long dst_off = desc[slot * 4], dst_plain = desc[slot * 4 + 1];
    const float* rowscale = reinterpret_cast<const float*>(desc[slot * 4 + 2]);
    const float* s = src + ((size_t)slot * rows + row) * cols;
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
    const float rs = rowscale ? rowscale[row] : 1.f;
    for (int c = lane * 4; c < cols; c += 128) {
      float4 a = *reinterpret_cast<const float4*>(s + c);
      if (qat) {
        a.x = fminf(fmaxf(rintf(a.x / qs), -32.f), 31.f) * qs;
        a.y = fminf(fmaxf(rintf(a.y / qs), -32.f), 31.f) * qs;
        a.z = fminf(fmaxf(rintf(a.z / qs), -32.f), 31.f) * qs;
        a.w = fminf(fmaxf(rintf(a.w / qs), -32.f), 31.f) * qs;
      }
      const uint2 p = make_uint2(pack_bf16x2(a.x * rs, a.y * rs), pack_bf16x2(a.z * rs, a.w * rs));
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(dst_tbl[r] + dst_off + (size_t)row * ld_dst + c) = p;
      if (dst_plain >= 0) {
        const uint2 q = make_uint2(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w));
        for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(dst_tbl[r] + dst_plain + (size_t)row * ld_dst + c) = q;
      }
    }
  }
}

// One increment per (rank, slot) on the ready counter that desc names for the slot.
__global__ void flag_add_slots_kernel(int* const* __restrict__ sig_tbl, int world, const long long* __restrict__ desc, int n_slots, int value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < world * n_slots) {
    __threadfence_system();
    red_release_sys_add(sig_tbl[i / n_slots] + (int)desc[(i % n_slots) * 4 + 3], value);
  }
}

// Fan-out copy: dst_tbl[r][off + i] = src[i] for every rank r != my_rank (second half of a two-shot all-reduce).
__global__ void __launch_bounds__(256) push_copy_kernel(const float* __restrict__ src, float* const* __restrict__ dst_tbl, int world, int my_rank,
                                                        long long off, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(src + i);
    for (int r = 0; r < world; ++r)
      if (r != my_rank) *reinterpret_cast<float4*>(dst_tbl[r] + off + i) = v;
  }
}

// After a push on this stream: bump counter `slot` on every rank (release at system scope).
__global__ void flag_add_kernel(int* const* __restrict__ sig_tbl, int world, int slot, int count, int value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < world * count) {
    __threadfence_system();
    red_release_sys_add(sig_tbl[i / count] + slot + (i % count), value);
  }
}

// Bounded wait on a local flag, as its own launch; the host reads the status word afterwards.
__global__ void wait_flag_kernel(const int* flag, int want, int* status) { wait_flag_ge(flag, want, status, want); }

// ---- launchers ----------------------------------------------------------------------------------------------------------
void comm_barrier(int* const* sig_tbl, int my_rank, int world, int slot, int epoch, int* status, cudaStream_t st) {
  barrier_kernel<<<1, 32, 0, st>>>(sig_tbl, my_rank, world, slot, epoch, status);
}
void comm_reduce_peers(const float* const* src_tbl, int world, long long off, long long n, float* out, float scale, float* stats, float sq_weight,
                       const int* wait_flag, int wait_value, int* status, cudaStream_t st) {
  if ((off % 4) || (n % 4)) throw std::runtime_error("reduce_peers: offset and count must be multiples of 4");
  if (n == 0) return;
  const int grid = (int)std::max<long long>(1, std::min<long long>((n / 4 + 255) / 256, 148 * 8));
  switch (world) {
    case 2: reduce_peers_kernel<2><<<grid, 256, 0, st>>>(src_tbl, world, off, n, out, scale, stats, sq_weight, wait_flag, wait_value, status); break;
    case 4: reduce_peers_kernel<4><<<grid, 256, 0, st>>>(src_tbl, world, off, n, out, scale, stats, sq_weight, wait_flag, wait_value, status); break;
    case 8: reduce_peers_kernel<8><<<grid, 256, 0, st>>>(src_tbl, world, off, n, out, scale, stats, sq_weight, wait_flag, wait_value, status); break;
    default: reduce_peers_kernel<0><<<grid, 256, 0, st>>>(src_tbl, world, off, n, out, scale, stats, sq_weight, wait_flag, wait_value, status); break;
  }
}
void comm_scalar_allreduce(float* const* val_tbl, int* const* sig_tbl, int my_rank, int world, int val_slot, int sig_slot, int epoch, float* stats,
                           int* status, cudaStream_t st) {
  scalar_allreduce_kernel<<<1, 32, 0, st>>>(val_tbl, sig_tbl, my_rank, world, val_slot, sig_slot, epoch, stats, status);
}
void comm_push_cast_rows(const float* src, void* const* dst_tbl, int world, long long dst_off, const float* rowscale, int scale_stride, int scale_mod,
                         int rows, int cols, long long ld_dst, int qat, cudaStream_t st) {
  if (cols % 4) throw std::runtime_error("push_cast_rows: cols must be a multiple of 4");
  push_cast_rows_kernel<<<std::min((rows + 7) / 8, 148 * 8), 256, 0, st>>>(src, (__nv_bfloat16* const*)dst_tbl, world, dst_off, rowscale, scale_stride,
                                                                          std::max(scale_mod, 1), rows, cols, ld_dst, qat);
}
void comm_push_cast_slots(const float* src, void* const* dst_tbl, int world, const long long* desc, int n_slots, int rows, int cols, long long ld_dst,
                          int qat, cudaStream_t st) {
  if (cols % 4) throw std::runtime_error("push_cast_slots: cols must be a multiple of 4");
  if (n_slots <= 0) return;
  const long long blocks = ((long long)n_slots * rows + 7) / 8;
  push_cast_slots_kernel<<<(int)std::min<long long>(blocks, 148 * 8), 256, 0, st>>>(src, (__nv_bfloat16* const*)dst_tbl, world, desc, n_slots, rows, cols,
                                                                                   ld_dst, qat);
}
void comm_flag_add_slots(int* const* sig_tbl, int world, const long long* desc, int n_slots, int value, cudaStream_t st) {
  if (n_slots <= 0) return;
  flag_add_slots_kernel<<<(world * n_slots + 63) / 64, 64, 0, st>>>(sig_tbl, world, desc, n_slots, value);
}
void comm_push_copy(const float* src, float* const* dst_tbl, int world, int my_rank, long long off, long long n, cudaStream_t st) {
  if ((off % 4) || (n % 4)) throw std::runtime_error("push_copy: offset and count must be multiples of 4");
  if (n == 0) return;
  const int grid = (int)std::max<long long>(1, std::min<long long>((n / 4 + 255) / 256, 148 * 4));
  push_copy_kernel<<<grid, 256, 0, st>>>(src, dst_tbl, world, my_rank, off, n);
}
void comm_flag_add(int* const* sig_tbl, int world, int slot, int count, int value, cudaStream_t st) {
  flag_add_kernel<<<(world * count + 63) / 64, 64, 0, st>>>(sig_tbl, world, slot, count, value);
}
void comm_wait_flag(const int* flag, int want, int* status, cudaStream_t st) { wait_flag_kernel<<<1, 1, 0, st>>>(flag, want, status); }

}  // namespace pgb
