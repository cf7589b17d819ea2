// C entry points that never allocate (attn_bwd_noalloc.cu).  No counterpart in the reference: its attention
// backward is a library call that takes whatever workspace the caching allocator hands it.
//
// Who needs this: callers that may not allocate while they run -- a replayed or in-capture launch sequence whose
// buffers are fixed, a step that runs with the caching allocator's pool full, a host thread that must not take the
// allocator lock -- and callers that are not Python at all and only hold raw device pointers.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest B * H * S (one fp32 scratch word per query row and head) the built-in scratch covers.
#define PGB_ATTN_BWD_NOALLOC_MAX_ROWS (1ll << 20)

// Set-up for the current device: looks up the scratch array's device address (which makes the runtime load the module
// there).  Runs implicitly inside the first pgb_attn_bwd_noalloc() on a device, whose first launch also sets the
// kernels' dynamic shared-memory attribute; so make the first call (or at least this one) before any stream capture
// begins.  Returns 0, or non-zero with pgb_noalloc_last_error().
int pgb_attn_bwd_noalloc_setup(void);

// Causal grouped-query attention backward (head_dim 64, bf16), same arguments and results as pgb::attn_bwd minus the
// caller-provided `dsum` scratch, which lives in a file-scope device array here.
//   q/k/v/o/d_o/dq/dk/dv: bf16 [B*S, heads*64] views, row strides ld* in elements; lse: fp32 [B,H,S] as written by
//   the forward kernel; status: device int[4] status word or null; stream: a cudaStream_t.
// Returns 0 when the launches were queued, non-zero otherwise (nothing launched; text in pgb_noalloc_last_error()):
//   1 = B*H*S exceeds PGB_ATTN_BWD_NOALLOC_MAX_ROWS, 2 = bad shape, 3 = CUDA error during set-up or launch.
// The scratch is ONE array per device shared by every call: it keeps whatever the previous call left in it (nothing
// in it has to start at zero -- every word the second kernel reads was written by the first kernel of the same
// call), and two calls that overlap in time on one device (different streams, different threads) race on it.
int pgb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                         long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk, long long lddv,
                         int B, int S, int H, int Hkv, int hd, int accumulate_dv, int* status, void* stream);

// Text of the calling thread's last non-zero return (static storage; valid until that thread's next failing call).
const char* pgb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
