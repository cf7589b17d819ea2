// Host API of the sm_100a kernel library (raw pointers + stream; no framework types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <stdexcept>
#include <string>

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
  EPI_QKV_NORM_ROPE = 7,  // D = bf16(acc) and, for the query and key heads (64 columns each), D2 = gain_h * rope(rms_norm(D)):
                          // the QKV projection with per-head RMSNorm, partial RoPE and the query gain in its output stage
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
  const int* wait_flag = nullptr;   // optional readiness counter for B (see comm.cu); polled with a bounded wait
  int wait_value = 0;
  int seg_rows[2] = {0, 0};  // fp32 epilogues: output rows >= seg_rows[k] go to seg_D[k] (row index rebased), same ldd
  float* seg_D[2] = {nullptr, nullptr};
  // optional per-batch normalisation: the output of batch b is scaled by (1 / (sqrt(batch_sumsq[b]) + 1e-7)) ^ sumsq_pow
  // (alpha and beta both), so a Newton-Schulz iteration can start from an un-normalised matrix
  const float* batch_sumsq = nullptr;
  int sumsq_pow = 1;
  // EPI_QKV_NORM_ROPE: columns are [q_heads | kv_heads | kv_heads] heads of 64; cos/sin tables [seq_len][rope_dims / 2];
  // row m is position m % seq_len; head_gain (q_heads floats) may be null; rope_dims in {0, 16, 32, 64}
  const float* rope_cos = nullptr;
  const float* rope_sin = nullptr;
  const float* head_gain = nullptr;
  int q_heads = 0, kv_heads = 0, rope_dims = 0, seq_len = 0;
  float norm_eps = 0.f;
};

void gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// ---- row kernels (rowops.cu); activations bf16, parameters fp32 ------------------------------------------------
void mix_norm_fwd(const void* x, const void* x0, const void* skip, const float* sw, const float* mix, void* x_in, void* h, int rows, int d, float s,
                  float eps, cudaStream_t st);
void mix_norm_bwd(const void* d_h, const void* d_res, const void* x_in, const void* x, const void* x0, const void* skip, const float* sw,
                  const float* mix, const void* add_grad, void* d_x, void* d_x0, void* d_skip, float* d_mix, float* d_sw, int skip_to_dx, int rows,
                  int d, float s, float eps, cudaStream_t st);
void norm_smear_fwd(const void* xe, const float* gate, const int* ids, void* out, int rows, int d, int seq_len, int boundary, float eps,
                    cudaStream_t st);
void norm_smear_bwd(const void* g_out, const void* xe, const float* gate, const int* ids, void* d_xe, float* d_gate, int rows, int d, int seq_len,
                    int boundary, float eps, cudaStream_t st);
void qk_norm_rope_fwd(const void* src, void* dst, const float* cosT, const float* sinT, const float* gain, int rows, int ld, int H, int Hkv, int hd,
                      int rope_dims, int seq_len, float eps, cudaStream_t st);
void qk_norm_rope_bwd(const void* d_post, const void* pre, void* d_pre, const float* cosT, const float* sinT, const float* gain, float* d_gain,
                      int rows, int ld, int H, int Hkv, int hd, int rope_dims, int seq_len, float eps, cudaStream_t st);
void xsa_fwd(const void* y, const void* v, void* z, int rows, int Hkv, int group, int hd, int ld_y, int ld_v, float eps, cudaStream_t st);
// dsum (optional, head_dim 64 only): fp32 [B, H, S] with -rowsum(dy * y), the per-query term the attention backward needs, so
// that its own pass over dy and y can be skipped; seq_len gives the [B, S] split of the rows.
void xsa_bwd(const void* dz, const void* y, const void* v, void* dy, void* dv, int accumulate_dv, int rows, int Hkv, int group, int hd, int ld_y,
             int ld_v, int ld_dv, float eps, cudaStream_t st, float* dsum = nullptr, int seq_len = 0);
// Per-head output gates (gates.cu): out_h = y_h * mult * sigmoid(scale * <W_h, x[:w]> + bias_h); `gate` [rows, H] keeps the factors
// for the backward, which rewrites d_out in place into the gradient of y and adds the input-feature part into d_x[:, :w].
void head_gate_fwd(const void* y, const void* x, const float* W, const float* bias, void* out, float* gate, int rows, int H, int hd, int w, int ld_x,
                   float scale, float mult, cudaStream_t st);
void head_gate_bwd(void* d_out, const void* y, const void* x, const float* W, const float* gate, float* dW, float* dbias, void* d_x, int accumulate_dx,
                   int rows, int H, int hd, int w, int ld_x, int ld_dx, float scale, float mult, cudaStream_t st);
// tok_w / w_total (both or neither): per-row loss weights and their sum, as written by `pair_weights`; norm_rows: the number
// of rows the sum covers when this call sees only a chunk of them (0: the same `rows`)
void softcap_ce(const void* logits, const int* targets, float* nll, void* dlogits, float* loss_sum, int rows, int V, float cap, float gscale,
                cudaStream_t st, const float* tok_w = nullptr, const float* w_total = nullptr, int norm_rows = 0);
// w[i] = table[prev[i] * V + curr[i]], *w_total = sum_i w[i] (zeroed here first)
void pair_weights(const int* prev, const int* curr, const float* table, float* w, float* w_total, int rows, int V, cudaStream_t st);
// ids outside [0, table_rows) give a zero row and ST_BAD_INDEX in the status word instead of an address
void embed_gather(const int* ids, const void* table, void* out, int rows, int d, int table_rows, int bigram_buckets, int seq_len, cudaStream_t st,
                  int* status = nullptr);
void embed_scatter_add(const int* ids, const void* g, float* dtable, int rows, int d, int table_rows, int bigram_buckets, int seq_len,
                       cudaStream_t st);

// tuned variants (rowops_fast.cu), called by the launchers above when their preconditions hold
void mix_norm_bwd_v2(const void* d_h, const void* d_res, const void* x_in, const void* x, const void* x0, const void* skip, const float* sw,
                     const float* mix, const void* add_grad, void* d_x, void* d_x0, void* d_skip, float* d_mix, float* d_sw, int skip_to_dx, int rows,
                     int d, float s, float eps, cudaStream_t st);
bool qk_norm_rope_fast_ok(int H, int hd, int rope_dims);
void qk_norm_rope_fwd64(const void* src, void* dst, const float* cosT, const float* sinT, const float* gain, int rows, int ld, int H, int Hkv,
                        int rope_dims, int seq_len, float eps, cudaStream_t st);
void qk_norm_rope_bwd64(const void* d_post, const void* pre, void* d_pre, const float* cosT, const float* sinT, const float* gain, float* d_gain,
                        int rows, int ld, int H, int Hkv, int rope_dims, int seq_len, float eps, cudaStream_t st);

void xsa_fwd64(const void* y, const void* v, void* z, int rows, int Hkv, int group, int ld_y, int ld_v, float eps, cudaStream_t st);
void xsa_bwd64(const void* dz, const void* y, const void* v, void* dy, void* dv, int accumulate_dv, int rows, int Hkv, int group, int ld_y, int ld_v,
               int ld_dv, float eps, cudaStream_t st, float* dsum = nullptr, int seq_len = 0);

// ---- optimizer / weight preparation (optim.cu) --------------------------------------------------------------------------
// hp: device fp32[8] = {lr_scale, muon_momentum, adam_bias_corr1, adam_bias_corr2, grad_scale, ...}
void cast_rows(const float* src, void* dst, const float* rowscale, int scale_stride, int scale_mod, int rows, int cols, long long ld_dst, int qat,
               cudaStream_t st);
void fold_scaled_grad(const float* G, const float* W, const float* rowscale, int scale_stride, int scale_mod, float* dW, float* dscale, int rows,
                      int cols, int qat, cudaStream_t st);
void fold_scaled_grad_bf16(const float* G, const void* W, const float* rowscale, int scale_stride, int scale_mod, float* dW, float* dscale, int rows,
                           int cols, cudaStream_t st);
void sumsq(const float* x, long long n, float scale, float* out, cudaStream_t st);
void sum_splits_add(const float* part, int splits, long long split_stride, float* dst, long long n, cudaStream_t st);
void clip_factor(float* stats, float* hp, float base_scale, float max_norm, cudaStream_t st);
void muon_momentum(const float* g, float* buf, void* U, float* sumsq_out, const float* hp, int matrices, long long per_matrix, int nesterov,
                   cudaStream_t st);
void muon_normalize(const void* U, void* X, const float* sumsq_in, int matrices, long long per_matrix, float eps, cudaStream_t st);
void muon_apply(float* p, const void* X, float* ema, const float* hp, long long n, float base_lr, float wd, float scale, float decay, cudaStream_t st);
void adamw(float* p, const float* g, float* m, float* v, float* ema, const float* hp, long long n, float base_lr, float b1, float b2, float eps,
           float wd, float decay, cudaStream_t st);
void sgd_momentum(float* p, const float* g, float* mom, const float* hp, long long n, float lr, float mu, cudaStream_t st);

// ---- peer-memory collectives (comm.cu) and symmetric memory (symm.cpp) --------------------------------------------------
void comm_barrier(int* const* sig_tbl, int my_rank, int world, int slot, int epoch, int* status, cudaStream_t st);
void comm_reduce_peers(const float* const* src_tbl, int world, long long off, long long n, float* out, float scale, float* stats, float sq_weight,
                       const int* wait_flag, int wait_value, int* status, cudaStream_t st);
void comm_scalar_allreduce(float* const* val_tbl, int* const* sig_tbl, int my_rank, int world, int val_slot, int sig_slot, int epoch, float* stats,
                           int* status, cudaStream_t st);
void comm_push_cast_rows(const float* src, void* const* dst_tbl, int world, long long dst_off, const float* rowscale, int scale_stride, int scale_mod,
                         int rows, int cols, long long ld_dst, int qat, cudaStream_t st);
// A run of consecutive bank slots in one launch; desc = int64 [n_slots][4] on the device:
// {destination offset, offset of the un-scaled twin or -1, address of the slot's row scales or 0, ready-counter index}.
void comm_push_cast_slots(const float* src, void* const* dst_tbl, int world, const long long* desc, int n_slots, int rows, int cols, long long ld_dst,
                          int qat, cudaStream_t st);
void comm_flag_add_slots(int* const* sig_tbl, int world, const long long* desc, int n_slots, int value, cudaStream_t st);
void comm_push_copy(const float* src, float* const* dst_tbl, int world, int my_rank, long long off, long long n, cudaStream_t st);
void comm_flag_add(int* const* sig_tbl, int world, int slot, int count, int value, cudaStream_t st);
void comm_wait_flag(const int* flag, int want, int* status, cudaStream_t st);
void* symm_alloc(size_t bytes);
std::string symm_export(void* p);
void* symm_import(const std::string& handle);
void symm_close(void* p);
void symm_free(void* p);

// ---- misc (misc.cu) ------------------------------------------------------------------------------------------------------
void expand_span_u16(const void* span, int* ids, int* targets, int n, cudaStream_t st);

// ---- post-training quantisation (gptq.cu) --------------------------------------------------------------------------------
// GPTQ with fixed per-row scales: Wp [rows, cols] fp32 (columns already in activation order), U [cols, cols] upper
// Cholesky factor of the inverse Hessian, Q int8 codes out. Column blocks of 128.
void gptq_rows(const float* Wp, const float* U, const float* scales, int8_t* Q, int rows, int cols, int bits, cudaStream_t st);

// ---- attention (attn_fwd.cu, attn_bwd.cu): causal, grouped KV heads, head_dim 64, bf16 ----------------------------------
// q/k/v/y are [B*S, heads*hd] views with row strides ld* (elements); lse is fp32 [B, H, S] and holds the NEGATED
// base-2 log-sum-exp of the scaled scores (the form the backward kernels feed straight into their FMAs).
// z (optional): second output with the exclusive-self-attention projection applied, z_h = y_h - (<y_h, v> / (|v|^2 + eps)) v
void attn_fwd(const void* q, const void* k, const void* v, void* y, float* lse, long long ldq, long long ldk, long long ldv, long long ldy, int B,
              int S, int H, int Hkv, int hd, int* status, cudaStream_t st, void* z = nullptr, long long ldz = 0, float xsa_eps = 0.f);
// dsum: fp32 [B, H, S] scratch-free side output (rowsum(dO * O)), written by the dQ kernel and read by the dK/dV kernel.
void attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, float* dsum, void* dq, void* dk, void* dv,
              long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk, long long lddv, int B, int S,
              int H, int Hkv, int hd, int accumulate_dv, int* status, cudaStream_t st);
// Single-pass form (attn_bwd_fused.cu): scores computed once per tile pair, dQ summed with fp32 `red.add` into `dq_acc`
// (attn_bwd_fused_scratch_floats(B, S, H) floats, ZERO on entry, left zero on return), then scaled and cast into `dq`.
// dsum is written by a small pre-kernel. dQ is reproducible to fp32 rounding only; attn_bwd is bit-reproducible.
size_t attn_bwd_fused_scratch_floats(int B, int S, int H);
void attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, float* dsum, float* dq_acc, void* dq,
                    void* dk, void* dv, long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk,
                    long long lddv, int B, int S, int H, int Hkv, int hd, int accumulate_dv, int* status, cudaStream_t st, int dsum_ready = 0);

}  // namespace pgb
