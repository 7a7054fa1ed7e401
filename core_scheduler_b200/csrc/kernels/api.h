// SPDX-License-Identifier: Apache-2.0
// Host-side launch interface of the hand-written sm_100a kernels. Plain C++ (no torch
// headers) so the .cu files compile in seconds and the C++ ops call them with raw pointers.
// Every launcher enqueues on `stream` and returns a cudaError_t value as int (0 = success).
// bf16 buffers are passed as `void*` (element type __nv_bfloat16).
#pragma once
#include <cstddef>
#include <cstdint>

namespace cs::kernels {
using stream_t = void *;  // cudaStream_t

// Number of kernels of this library launched by this process so far (all streams).
int64_t launch_count();
void count_launch(int n);
// Adds n to the launch counter and returns cudaGetLastError() as int.
int finish_launch(int n = 1);

// ---- optimizer -------------------------------------------------------------------------
struct AdamWArgs {
  void *param;          // master values, dtype given by param_dtype
  const void *grad;     // dtype given by grad_dtype
  void *exp_avg;        // same dtype as param
  void *exp_avg_sq;     // same dtype as param
  void *max_exp_avg_sq; // nullptr unless amsgrad
  void *lp;             // optional bf16 working copy written with the new value (nullptr = none)
  int64_t n;
  int param_dtype;      // 0 = fp32, 1 = bf16, 2 = fp16
  int grad_dtype;       // 0 = fp32, 1 = bf16, 2 = fp16
  float lr, beta1, beta2, eps, weight_decay;
  float inv_bias_correction1, inv_bias_correction2;
  float grad_scale;     // gradient is multiplied by this before use (1/world, loss scale, ...)
  const float *clip_coef;  // optional device scalar multiplied into the gradient (clip factor)
};
int adamw_step(stream_t stream, const AdamWArgs &args);

// ---- elementwise / normalisation ---------------------------------------------------------
// y = gelu(x) (exact erf form); bf16 in/out.
int gelu_forward(stream_t stream, const void *x, void *y, int64_t n);
// dx = dy * gelu'(x)
int gelu_backward(stream_t stream, const void *dy, const void *x, void *dx, int64_t n);
// out = a + b (bf16)
int add_bf16(stream_t stream, const void *a, const void *b, void *out, int64_t n);
// out(bf16) = acc(fp32) (+ residual(bf16) when given); n % 8 == 0.
int add_f32_residual_to_bf16(stream_t stream, const float *acc, const void *residual, void *out, int64_t n);
// dst(bf16) = src(fp32); optionally also writes the [cols, rows] transpose of a row-major
// [rows, cols] matrix (dst_t may be nullptr).
int cast_fp32_to_bf16(stream_t stream, const float *src, void *dst, int64_t n);
int transpose_cast_to_bf16(stream_t stream, const void *src, int src_dtype, void *dst_t, int64_t rows, int64_t cols);

// Interleaves three bf16 tensors (q, k, v gradients) into one packed [B,T,3,H,D] tensor in a
// single pass (D % 8 == 0). Sources are contiguous [B,H,T,D] (src_bthd = 0) or [B,T,H,D] (1).
int pack_qkv(stream_t stream, const void *q, const void *k, const void *v, void *packed, int64_t B, int64_t H, int64_t T,
             int64_t D, int src_bthd);

// LayerNorm over the last dimension d (d % 8 == 0, d <= 8192). x,y bf16; gamma/beta fp32 or
// bf16 (param_dtype as above); mean/rstd fp32 [rows].
int layernorm_forward(stream_t stream, const void *x, const void *gamma, const void *beta, int param_dtype, void *y,
                      float *mean, float *rstd, int64_t rows, int64_t d, float eps);
// Single pass: dx (+ grad_residual when given) and per-CTA partial dgamma/dbeta reduced by a
// second tiny kernel. `scratch` holds 2 * layernorm_backward_scratch_rows() * d floats.
// dgamma/dbeta are fp32; accumulate != 0 adds to their current contents.
int64_t layernorm_backward_scratch_rows();
int layernorm_backward(stream_t stream, const void *dy, const void *x, const void *gamma, int param_dtype,
                       const float *mean, const float *rstd, const void *grad_residual, void *dx, float *dgamma,
                       float *dbeta, int accumulate, float *scratch, int64_t rows, int64_t d);

// out[r, :] = wte[idx[r], :] (+ wpe[r % seq_len, :]) as bf16. Table dtype per table_dtype.
int embedding_forward(stream_t stream, const int64_t *idx, const void *wte, const void *wpe, int table_dtype,
                      void *out, int64_t rows, int64_t seq_len, int64_t d, int64_t vocab);
// dwte[idx[r], :] += dy[r, :] (fp32 atomics, rows with idx == padding_idx skipped);
// dwpe[t, :] (+)= sum_b dy[b*T + t, :]. Either table may be nullptr. The caller zeroes dwte
// when it must not accumulate; dwpe honours accumulate_wpe.
int embedding_backward(stream_t stream, const int64_t *idx, const void *dy, float *dwte, float *dwpe,
                       int accumulate_wpe, int64_t rows, int64_t seq_len, int64_t d, int64_t vocab,
                       int64_t padding_idx);

// ---- tcgen05 GEMM -------------------------------------------------------------------------
// D[M,N] = op(A) * op(B)^T with bf16 operands and fp32 accumulation in tensor memory.
//   layout kTN : A is [M,K] row-major (K contiguous), B is [N,K] row-major.        (forward / dgrad)
//   layout kNT : A is [K,M] row-major (M contiguous), B is [K,N] row-major.        (weight gradient)
//   layout kTM : A is [M,K] row-major (K contiguous), B is [K,N] row-major.        (input gradient dY * W)
// Leading dimensions are in elements and must be multiples of 8; base pointers 16-byte aligned.
enum GemmLayout : int { kTN = 0, kNT = 1, kTM = 2 };
enum GemmEpilogue : int {
  kEpiStoreBf16 = 0,     // D(bf16) = acc (+ bias[n])
  kEpiResidualBf16 = 1,  // D(bf16) = acc (+ bias[n]) + aux[m,n]
  kEpiGeluDual = 2,      // D(bf16) = acc (+ bias[n]); D2(bf16) = gelu(D)
  kEpiDGelu = 3,         // D(bf16) = acc * gelu'(aux[m,n])
  kEpiStoreF32 = 4,      // D(fp32) = acc
  kEpiAccumF32 = 5,      // D(fp32) += acc
  kEpiCrossEntropy = 6,  // D(bf16) = acc; per-(row, n-tile) softmax partials to `stats`
};
struct GemmArgs {
  const void *a;
  const void *b;
  void *d;
  void *d2;          // second output (kEpiGeluDual)
  const void *aux;   // residual / pre-activation, same shape & leading dim as d
  const void *bias;  // bf16 [N] or nullptr
  float *stats;      // kEpiCrossEntropy: [M, gemm_ce_stat_tiles(N), 2] (max, sum-exp) partials
  int64_t m, n, k;
  int64_t lda, ldb, ldd;
  int layout;
  int epilogue;
  int64_t n_valid;   // kEpiCrossEntropy: columns >= n_valid are excluded from the softmax
  // Fused collectives over peer memory (tensor parallelism); peer_count > 1 enables one of:
  //   a_peers: all-gather -> GEMM. Row block j of A ([m / peer_count, k], leading dim lda) is read
  //            by TMA straight from a_peers[j] (a peer's symmetric memory); no gathered copy exists.
  //   d_peers: GEMM -> reduce-scatter. Row block j of D goes to d_peers[j] ([m / peer_count, n], leading dim
  //            ldd) on its owner: reduce-added in fp32 (epilogue kEpiAccumF32), or stored as bf16 into the slot
  //            the owner keeps for this rank (epilogue kEpiStoreBf16; the owner sums its slots afterwards).
  //            Tiles are visited starting with the next rank's block, this rank's own block last.
  //   ready_flags: GEMM beside an all-gather that is still in flight. A is local memory that the ranks fill in
  //            row chunks; word [owner * 8 + chunk] of ready_flags reaches ready_epoch (acquire load) once the
  //            chunk has landed. Tiles are visited in arrival order.
  // m / peer_count must be a multiple of 256 (and of 256 * ready_chunks).
  int peer_count;
  int peer_rank;
  const void *a_peers[8];
  void *d_peers[8];
  const uint32_t *ready_flags;
  uint32_t ready_epoch;
  int ready_chunks;
};
// Returns 0 on success, -1 when the shape/alignment is not supported (caller falls back).
int gemm_bf16(stream_t stream, const GemmArgs &args);
// Number of (max, sum-exp) partials per row that kEpiCrossEntropy writes for N columns.
int64_t gemm_ce_stat_tiles(int64_t n);
// Copies / clears the status word of the GEMM kernel (synchronises the device).
struct DeviceStatus;
int gemm_status(DeviceStatus *out);
int gemm_status_reset();

// ---- tcgen05 causal attention (forward) -----------------------------------------------------------
// qkv: packed bf16 [B, T, 3, H, D] (D == 64, T % 128 == 0); out: bf16 [B, T, H*D]; lse: fp32
// [B, H, T] = log-sum-exp of the scaled scores. causal != 0 masks the keys after each query.
// Returns -1 when the shape is not covered.
int attention_forward_packed(stream_t stream, const void *qkv, void *out, float *lse, int64_t B, int64_t T, int64_t H, int64_t D,
                             float scale, int causal = 1);
struct DeviceStatus;
// Backward of the same attention: dqkv [B, T, 3, H, 64] from qkv, the forward output `out`, its
// gradient `dout` [B, T, H*64] and `lse`; `delta` is a [3, B, H, T] fp32 workspace (plane 0 receives
// rowsum(dout * out)). Same shape limits.
int attention_backward_packed(stream_t stream, const void *qkv, const void *out, const void *dout, const float *lse, float *delta,
                              void *dqkv, int64_t B, int64_t T, int64_t H, int64_t D, float scale, int causal = 1);
int attention_status(DeviceStatus *out);

// ---- fused cross-entropy helpers -----------------------------------------------------------
// Reduces the per-tile partials to lse[row], computes loss_row = lse - logit[target] and the
// mean over non-ignored rows into loss[0] (fp32); count[0] receives the number of valid rows.
int cross_entropy_finalize(stream_t stream, const float *stats, int64_t n_tiles, const void *logits, int64_t ld,
                           const int64_t *target, float *lse, float *loss, float *count, int64_t rows,
                           int64_t ignore_index);
// logits <- (softmax(logits) - onehot(target)) * grad_scale / count, in place (bf16); padded
// columns (>= n_valid) and ignored rows become 0.
// With a vocabulary slice (tensor parallel) `col_offset` is the class of column 0: targets and n_valid are then
// global class numbers, lse the log-sum-exp over the whole vocabulary.
int cross_entropy_backward_inplace(stream_t stream, void *logits, int64_t ld, const float *lse,
                                   const int64_t *target, const float *count, float grad_scale, int64_t rows,
                                   int64_t n, int64_t n_valid, int64_t ignore_index, int64_t col_offset = 0);
// Per-row statistics of one vocabulary slice (classes [col_offset, col_offset + ld)): out[row] = (log-sum-exp over
// the slice's valid columns from the GEMM's per-tile partials, or -inf when it has none; the target's logit when the
// target class falls into the slice's first n_valid_local columns, else 0).
int cross_entropy_slice_stats(stream_t stream, const float *stats, int64_t n_tiles, const void *logits, int64_t ld,
                              const int64_t *target, int64_t col_offset, int64_t n_valid_local, float *out, int64_t rows);

// ---- gradient norm ---------------------------------------------------------------------------
// sumsq[0] += sum(x^2) over n elements (fp32 or bf16 input); caller zeroes sumsq first.
int sum_squares(stream_t stream, const void *x, int dtype, int64_t n, float *sumsq);
// coef[0] = min(1, max_norm / (sqrt(sumsq[0]) + 1e-6)); norm_out[0] = sqrt(sumsq[0])
int clip_coefficient(stream_t stream, const float *sumsq, float max_norm, float *coef, float *norm_out);
// x *= coef[0]
int scale_by_device_scalar(stream_t stream, void *x, int dtype, int64_t n, const float *coef);

// Device status words written by kernels whose bounded waits expired (0 = fine).
struct DeviceStatus {
  int code;      // 0 ok, 1 = mbarrier wait timed out, 2 = peer flag wait timed out
  int kernel_id;
  int block;
  int detail;
};

// First out-of-range index seen by a kernel of the diagnostic build (-DCS_BOUNDS_CHECK); see
// bounds_check.h. `code` 0 = nothing recorded. In the normal build the report is always empty.
struct BoundsReport {
  int code;
  int kernel_id;
  int block;
  int thread;
  long long index;
  long long limit;
};
bool bounds_check_enabled();
// Copies the report (merged over the kernel translation units; synchronises the device) and
// optionally clears it.
int bounds_report(BoundsReport *out, bool reset);
}  // namespace cs::kernels
