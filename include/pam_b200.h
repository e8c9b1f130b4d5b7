/*
 * pam_b200 — C ABI of the B200 (sm_100a) kernels for piecewise affine multiplication (PAM).
 *
 * This is the drop-in boundary for the native layer of epfml/pam: each entry point replaces one
 * of the functions the reference binds from pam/cuda_kernels.cu (its pybind table, lines
 * 932-947), or fuses a chain of them that the reference runs from Python.  Conventions:
 *
 *   - every pointer is a DEVICE pointer to fp32 data on the device that is current for the
 *     calling thread; nothing here allocates, frees or synchronises (scratch is passed in);
 *   - sizes and strides are int64 element counts; `stream` is a cudaStream_t passed as void*;
 *   - `offset` is the reference's float offset (1.0f = none); the integer added to the bit
 *     pattern is bits(offset) - 0x3f800000, exactly as pam/cuda_kernels.cu:168 derives it;
 *   - the return value is PAMK_OK or a negative PAMK_ERR_* code; on PAMK_ERR_CUDA
 *     pamk_last_cuda_error() returns the cudaError_t of the failed launch;
 *   - results follow the reference bit for bit for every per-element operation; sums
 *     (matrix products, row reductions) add the same terms, matrix products in the same
 *     k order unless split-K is requested (see pamk_matmul).
 */
#ifndef PAM_B200_H
#define PAM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PAMK_OK 0
#define PAMK_ERR_ARG (-1)          /* null pointer, negative size, unknown enum value      */
#define PAMK_ERR_SIZE (-2)         /* a dimension exceeds what the kernel indexes           */
#define PAMK_ERR_LAYOUT (-3)       /* neither of a matrix's two strides is 1                */
#define PAMK_ERR_WORKSPACE (-4)    /* scratch buffer missing, misaligned or too small       */
#define PAMK_ERR_CUDA (-5)         /* a CUDA call failed; see pamk_last_cuda_error()        */

const char* pamk_status_string(int status);
int pamk_last_cuda_error(void);
/* ABI version of this header (bumped when a signature changes). */
int pamk_abi_version(void);
/* Number of kernels this library has launched in this process so far (all threads). */
long long pamk_launch_count(void);

/* ---- operand descriptors for the elementwise entry points ---------------------------------
 * The reference broadcasts in Python and materialises the expanded operand
 * (pam/cuda_bindings.py:60-63, pam/cuda_kernels.cu:163-164).  Here the broadcast is described
 * instead: an operand is (ptr, kind); with `n` output elements viewed as [n / inner, inner],
 *   PAMK_FULL    ptr[i]              one value per output element
 *   PAMK_SCALAR  ptr[0]              a 0-d device tensor
 *   PAMK_ROW     ptr[i % inner]      a vector along the last dimension (e.g. LayerNorm weight)
 *   PAMK_COL     ptr[i / inner]      one value per row (e.g. a row-wise denominator)
 *   PAMK_IMM     the float passed beside the pointer (a Python number); ptr is ignored
 */
#define PAMK_FULL 0
#define PAMK_SCALAR 1
#define PAMK_ROW 2
#define PAMK_COL 3
#define PAMK_IMM 4

/* out[i] = pam(a, b)            replaces pam_fwd  — elementwise_pam_caller, cuda_kernels.cu:155-183 */
int pamk_pam_fwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream);
/* out[i] = pad(a, b)            replaces pad_fwd  — elementwise_pad_caller, cuda_kernels.cu:251-279 */
int pamk_pad_fwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream);
/* out[i] = pam_bwd(a, b, dc): exact d pam(a,b)/da * dc
 *                               replaces pam_bwd — elementwise_pam_bwd_caller, cuda_kernels.cu:200-232 */
int pamk_pam_bwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 const float* dc, int dc_kind, float dc_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream);
/* out[i] = pad_bwd(a, b, dc): exact d pad(a,b)/db * dc
 *                               replaces pad_bwd — elementwise_pad_bwd_caller, cuda_kernels.cu:296-328 */
int pamk_pad_bwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 const float* dc, int dc_kind, float dc_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream);
/* y = base^x                    replaces pa_exp_fwd — elementwise_pa_exp_caller, cuda_kernels.cu:348-373 */
int pamk_pa_exp_fwd(const float* x, float* y, int64_t n, float base, float offset, void* stream);
/* exact backward of base^x      replaces pa_exp_bwd — cuda_kernels.cu:395-423 */
int pamk_pa_exp_bwd(const float* x, const float* dy, float* dx, int64_t n, float base, float offset,
                    void* stream);
/* y = log_base(x)               replaces pa_log_fwd — cuda_kernels.cu:443-468 */
int pamk_pa_log_fwd(const float* x, float* y, int64_t n, float base, float offset, void* stream);
/* exact backward of log_base(x) replaces pa_log_bwd — cuda_kernels.cu:488-516 */
int pamk_pa_log_bwd(const float* x, const float* dy, float* dx, int64_t n, float base, float offset,
                    void* stream);

/* ---- matrix products ------------------------------------------------------------------------
 * C[z][i][j] = sum_k MUL(A[z][i][k], B[z][k][j]),  C contiguous [batch, M, N].
 * Operands are addressed by element strides (batch, row, column); for each operand one of the
 * two matrix strides must be 1 — the reference's row-/column-major flags
 * (pam/cuda_bindings.py:106-115) are exactly these two cases.  batch == 1 is the 2-D product.
 *
 * Replaces pam_matmul_fwd / pam_bmm_fwd (mul_kind PAMK_MUL_PAM) and standard_matmul /
 * standard_bmm (PAMK_MUL_STANDARD): matmul_caller, cuda_kernels.cu:648-723.
 *
 * split_k: 1  = every output is summed by one thread strictly in k order, as the reference does;
 *               results are then bit-identical to the reference's.
 *          >1 = K is cut into that many contiguous ranges summed independently and then added in
 *               range order (deterministic, but a different association than the reference);
 *               needs `workspace` of pamk_matmul_workspace_bytes(...) bytes, 256-byte aligned.
 *          0  = let the library choose; it only splits when `workspace` is large enough.
 */
#define PAMK_MUL_PAM 0
#define PAMK_MUL_STANDARD 1
int pamk_matmul(int mul_kind, const float* A, const float* B, float* C,
                int64_t batch, int64_t M, int64_t N, int64_t K,
                int64_t sAb, int64_t sAm, int64_t sAk,
                int64_t sBb, int64_t sBk, int64_t sBn,
                float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream);
/* pamk_matmul with an optional bias: C[z][i][j] = (sum_k ...) + bias[j], the bias added with an
 * ordinary fp32 add after the complete sum, i.e. the same value as the reference's
 * `matmul(X, W.T) + bias` (pam/pam_ops.py:107-115) without the extra pass over the output.
 * bias = NULL is pamk_matmul. */
int pamk_matmul_bias(int mul_kind, const float* A, const float* B, const float* bias, float* C,
                     int64_t batch, int64_t M, int64_t N, int64_t K,
                     int64_t sAb, int64_t sAm, int64_t sAk,
                     int64_t sBb, int64_t sBk, int64_t sBn,
                     float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream);
/* PAM product over a two-level batch with strided operands and a strided output, for attention
 * products that read q, k, v straight out of the fused projection's output and write the context
 * back in token-major layout (timm vision_transformer.py:72-93 folds and copies these with
 * flatten / transpose / reshape before and after pam.bmm).  Batch z = o * batch_inner + i:
 *   C[o*sCo + i*sCi + m*sCm + n] = sum_k pam(A[o*sAo + i*sAi + m*sAm + k*sAk], B[o*sBo + i*sBi + k*sBk + n*sBn])
 * with the columns of C contiguous (sCm >= N).  Each operand needs sAm == 1 or sAk == 1 (sBn or sBk)
 * as for pamk_matmul.  has_post_scale != 0: every finished sum is PAM-multiplied by post_scale
 * (the `* self.scale` after the score product, as the operator dictionary's mul does it) before it
 * is stored.  Products, order of summation and the choice of split_k = 0 are those of pamk_matmul
 * on the same shapes, so the values equal the copy-then-bmm route bit for bit. */
int pamk_matmul_strided(const float* A, const float* B, float* C,
                        int64_t batch_outer, int64_t batch_inner, int64_t M, int64_t N, int64_t K,
                        int64_t sAo, int64_t sAi, int64_t sAm, int64_t sAk,
                        int64_t sBo, int64_t sBi, int64_t sBk, int64_t sBn,
                        int64_t sCo, int64_t sCi, int64_t sCm,
                        float offset, int has_post_scale, float post_scale,
                        int split_k, void* workspace, size_t workspace_bytes, void* stream);
/* Scratch needed by pamk_matmul for a given split_k (0 for split_k <= 1). */
size_t pamk_matmul_workspace_bytes(int64_t batch, int64_t M, int64_t N, int split_k);
/* The split the library would choose for split_k = 0 given unlimited workspace. */
int pamk_matmul_auto_split(int64_t batch, int64_t M, int64_t N, int64_t K);

/* Split-K PAM product for callers that cannot allocate.  It has no counterpart in the reference.
 *
 * pamk_matmul with split_k > 1 needs a scratch buffer for the partial sums, which the caller has
 * to allocate.  Some callers cannot: code running inside a CUDA stream capture or a real-time loop
 * where cudaMalloc is forbidden, a plugin whose host gives it fixed input / output buffers and no
 * allocator, or a process that has handed all device memory to another pool.  This variant takes
 * the same operands and computes the same result (bit for bit the same as pamk_matmul with the
 * same split_k), but keeps the partial sums in a fixed 32 MiB array inside the library, so it
 * never calls cudaMalloc, cudaFree or any allocating routine.
 *
 *   - limit: split_k * batch * M * N floats must fit in pamk_matmul_static_scratch_bytes();
 *     larger problems are refused with PAMK_ERR_SIZE (nothing is launched); split_k must be >= 1;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call outside any stream capture;
 *   - every call on a device shares the one array.  Nothing in it has to start at zero: each call
 *     overwrites every partial sum it later reads, so stale contents from an earlier call are never
 *     seen.  Two calls that overlap on the GPU (different streams, or two host threads) would race
 *     on the array: serialise them. */
size_t pamk_matmul_static_scratch_bytes(void);
int pamk_matmul_static_scratch(const float* A, const float* B, float* C,
                               int64_t batch, int64_t M, int64_t N, int64_t K,
                               int64_t sAb, int64_t sAm, int64_t sAk,
                               int64_t sBb, int64_t sBk, int64_t sBn,
                               float offset, int split_k, void* stream);

/* Exact-gradient product: out[z][i][j] = sum_k pam_bwd(D[z][i][j], other, delta) with
 * (other, delta) = (R[k][j], L[i][k]) if delta_l else (L[i][k], R[k][j]).
 * Replaces pam_matmul_bwd / pam_bmm_bwd: pam_matmul_bwd_caller, cuda_kernels.cu:834-927.
 * split_k, workspace, workspace_bytes: as for pamk_matmul (1 = the reference's summation order;
 * a weight gradient, whose K is the token count, needs a split to fill the GPU); scratch size from
 * pamk_matmul_workspace_bytes, automatic choice from pamk_matmul_bwd_auto_split. */
int pamk_matmul_bwd(const float* L, const float* R, const float* D, float* out,
                    int64_t batch, int64_t M, int64_t N, int64_t K,
                    int64_t sLb, int64_t sLm, int64_t sLk,
                    int64_t sRb, int64_t sRk, int64_t sRn,
                    int64_t sDb, int64_t sDm, int64_t sDn,
                    int delta_l, float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream);
int pamk_matmul_bwd_auto_split(int64_t batch, int64_t M, int64_t N, int64_t K);

/* Column sums of a contiguous row-major [rows x cols] matrix, out[c] = sum_r X[r][c], ordinary
 * fp32 adds in a fixed order (deterministic): the bias gradient of a linear layer, which the
 * reference leaves to autograd's sum over the token dimension.  `workspace`: 16-byte aligned,
 * pamk_column_sum_workspace_bytes(rows, cols) bytes. */
size_t pamk_column_sum_workspace_bytes(int64_t rows, int64_t cols);
int pamk_column_sum(const float* X, float* out, int64_t rows, int64_t cols, void* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- fused layer normalisation (pam_ln) -----------------------------------------------------------
 * Replaces the chain of launches that pam/pam_ops.py:350-378 (layer_norm) issues through
 * pam/cuda_bindings.py — pam_fwd/pad_fwd/pa_log_fwd/pa_exp_fwd forward and their gradient kernels
 * backward — with one kernel each way, rounding where the chain rounds:
 *   mu = pad(sum x, n); c = x - mu; var = pad(sum pam(c,c), n); denom = pow(var + eps, 0.5);
 *   y = pam(pad(c, denom), weight) + bias.
 * x, y, dy, dx are [rows, width] contiguous; weight / bias / dweight / dbias are [width] or NULL.
 * width <= pamk_layer_norm_max_width().  Row sums are warp-shuffle trees, so y and the gradients
 * agree with the reference up to the association of those fp32 sums.
 * The backward needs scratch (per-CTA column sums for dweight / dbias) when either is requested:
 * pamk_layer_norm_bwd_workspace_bytes(rows, width) bytes, 16-byte aligned.
 * approx_bwd selects the reference's approximate (PAM-product) or exact (slope) gradient rules. */
int pamk_layer_norm_max_width(void);
int pamk_layer_norm_fwd(const float* x, const float* weight, const float* bias, float* y,
                        int64_t rows, int64_t width, float eps, float offset, void* stream);
size_t pamk_layer_norm_bwd_workspace_bytes(int64_t rows, int64_t width);
int pamk_layer_norm_bwd(const float* x, const float* weight, const float* dy, float* dx,
                        float* dweight, float* dbias, int64_t rows, int64_t width, float eps, float offset,
                        int approx_bwd, void* workspace, size_t workspace_bytes, void* stream);

/* The approximate backward pass (approx_bwd) without recomputing the forward chain:
 * pamk_layer_norm_fwd_save is pamk_layer_norm_fwd that also writes, per row, the
 * pamk_layer_norm_stats_per_row() scalars of the forward chain (mean, variance + eps, its square root
 * and the exact thresholds of the division by it) into stats ([rows, 8] floats, 16-byte aligned), and
 * pamk_layer_norm_bwd_saved computes from x, dy and stats what pamk_layer_norm_bwd(..., approx_bwd = 1)
 * computes from x and dy: dx bit for bit; dweight / dbias the same per-row terms, summed over the rows in
 * another order (a warp walks two rows per pass instead of four). */
int pamk_layer_norm_stats_per_row(void);
int pamk_layer_norm_fwd_save(const float* x, const float* weight, const float* bias, float* y, float* stats,
                             int64_t rows, int64_t width, float eps, float offset, void* stream);
int pamk_layer_norm_bwd_saved(const float* x, const float* weight, const float* dy, const float* stats, float* dx,
                              float* dweight, float* dbias, int64_t rows, int64_t width, float offset,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ---- fused softmax / logsumexp over the last dimension ----------------------------------------------
 * Replace the launch chains of pam_ops.softmax (pam/pam_ops.py:305-328) and pam_ops.logsumexp
 * (:331-342) and of their autograd:
 *   s = pam(x, log2 e) (-inf stays -inf);  shift = floor(max of s over the WHOLE tensor);
 *   e = exp2_op(s - shift) (0 where x = -inf);  softmax = pad(e, row sum of e);
 *   logsumexp = pad(shift + log2_op(row sum of e), log2 e)   [that log2 always with offset 1].
 * x, y, dy, dx are [rows, len] contiguous (logsumexp: y and dy are [rows]); len <=
 * pamk_softmax_max_len().  Every call first reduces the whole-tensor maximum into `workspace`
 * (pamk_softmax_workspace_bytes(rows, len) bytes, 16-byte aligned), also in the backward calls,
 * which recompute the forward chain from x. */
int pamk_softmax_max_len(void);
size_t pamk_softmax_workspace_bytes(int64_t rows, int64_t len);
int pamk_softmax_fwd(const float* x, float* y, int64_t rows, int64_t len, float offset,
                     void* workspace, size_t workspace_bytes, void* stream);
int pamk_softmax_bwd(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                     int approx_bwd, void* workspace, size_t workspace_bytes, void* stream);
/* The approximate backward pass (approx_bwd) without recomputing the forward chain: pamk_softmax_fwd_save
 * is pamk_softmax_fwd that also writes the exponentials e = exp2_op(s - shift) ([rows, len]; -0.0f
 * where x was -inf, so that masked entries stay distinguishable from exponentials that underflowed), and
 * pamk_softmax_bwd_saved computes from e and dy what pamk_softmax_bwd(..., approx_bwd = 1) computes from
 * x and dy, bit for bit (optionally followed by the PAM multiplication by post_scale of
 * pamk_softmax_bwd_scaled): no maximum pass, no workspace, 12 B/element. */
int pamk_softmax_fwd_save(const float* x, float* y, float* e, int64_t rows, int64_t len, float offset,
                          void* workspace, size_t workspace_bytes, void* stream);
int pamk_softmax_bwd_saved(const float* e, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                           int has_post_scale, float post_scale, void* stream);
/* pamk_softmax_bwd followed by a PAM multiplication of dx by post_scale, in the same pass: the
 * gradient of softmax(pam(scores, scale)) with respect to the scores when the scaling's backward
 * is the approximate form pam(d, scale) (pam/cuda_bindings.py:39-50 with approx_bwd). */
int pamk_softmax_bwd_scaled(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                            int approx_bwd, float post_scale, void* workspace, size_t workspace_bytes, void* stream);
int pamk_logsumexp_fwd(const float* x, float* y, int64_t rows, int64_t len, float offset,
                       void* workspace, size_t workspace_bytes, void* stream);
int pamk_logsumexp_bwd(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                       int approx_bwd, void* workspace, size_t workspace_bytes, void* stream);

/* ---- PAM loss kernels ----------------------------------------------------------------------------------
 * Label-smoothed negative log-likelihood straight from the logits: the PAM log-softmax
 * (lprobs = x - logsumexp(x), pam/pam_ops.py:344-347) fused with the gather and the row sum of fairseq's
 * label_smoothed_nll_loss (fairseq/criterions/label_smoothed_cross_entropy.py:36-54).
 *   forward:  rows_out[r] = { logsumexp(x_r), -lprobs[r, target_r], -(sum_j lprobs[r, j]) }  ([rows, 3]);
 *             the last two are 0 for rows whose target is ignore_index (when has_ignore);
 *   backward: dlogits for grads = { d(loss)/d(sum of the nll column), d(loss)/d(sum of the smooth column) }
 *             (two fp32 values on the device, so that no host read is needed): -(d smooth) - (d nll at the
 *             target) plus the logsumexp gradient chain.
 * The scalar combination loss = pam(1 - eps - eps_i, nll) + pam(eps_i, smooth) stays with the caller.
 * logits [rows, len] contiguous, target [rows] int64, len <= pamk_softmax_max_len(); workspace as for
 * pamk_softmax_fwd. */
int pamk_ls_loss_fwd(const float* logits, const long long* target, float* rows_out, int64_t rows, int64_t len,
                     int has_ignore, long long ignore_index, float offset,
                     void* workspace, size_t workspace_bytes, void* stream);
int pamk_ls_loss_bwd(const float* logits, const long long* target, const float* grads, float* dlogits,
                     int64_t rows, int64_t len, int has_ignore, long long ignore_index, float offset, int approx_bwd,
                     void* workspace, size_t workspace_bytes, void* stream);
/* Gradient of pam_opt.cross_entropy (pam/pam_opt.py:27-51) in one launch:
 *   d = pam_softmax(x) - target distribution (hot_prob at the target, cold_prob elsewhere);
 *   d = pam(d, class_weight[target]) if class_weight; rows with target == ignore_index times 0;
 *   d = pad(d, mean_rows) if mean_rows > 0 (reduction = "mean"); dlogits = pam(d, *grad_out).
 * grad_out points to one fp32 value on the device (the incoming gradient of the scalar loss). */
int pamk_cross_entropy_bwd(const float* logits, const long long* target, const float* class_weight, const float* grad_out,
                           float* dlogits, int64_t rows, int64_t len, float hot_prob, float cold_prob, float mean_rows,
                           int has_ignore, long long ignore_index, float offset,
                           void* workspace, size_t workspace_bytes, void* stream);

/* ---- fused PAM Adam ------------------------------------------------------------------------------
 * Replaces the per-tensor launch chain of the reference's PAM Adam
 * (submodules/fairseq/fairseq/optim/adam.py:226-252 over pam.mul / pam.div / pam.pow):
 *   m = pam(m, beta1) + pam(g, 1-beta1);  v = pam(v, beta2) + pam(pam(g, g), 1-beta2);
 *   p -= pam(p, decay) [if decay != 0];   p -= pam(pad(m, pow(v, 0.5) + eps), step_size)
 * in place, for `count` tensors in one call.  p, g, m, v, n are HOST arrays of `count` entries:
 * device pointers to the fp32 parameter, gradient, exp_avg, exp_avg_sq, and their element counts.
 * The scalars are the reference's Python doubles rounded to fp32 once (as pam/utils.py:13 does):
 * decay = weight_decay * lr, step_size = lr * sqrt(1 - beta2^t) / (1 - beta1^t).
 * Results are bit-identical to the reference's chain (purely per-element arithmetic). */
int pamk_adam_step(float* const* p, const float* const* g, float* const* m, float* const* v,
                   const int64_t* n, int count,
                   float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                   float eps, float decay, float step_size, float offset, void* stream);

/* ---- roofline measurement --------------------------------------------------------------------
 * No counterpart in the reference.  Runs register-only chains of the instructions a PAM
 * multiply-accumulate is made of and reports how many chain steps ran in how many milliseconds;
 * variant 0 fp32 add, 1 int32 add, 2 int add + fp add (1:1), 3 int multiply-add + fp add,
 * 4 alternating int add / multiply-add + fp add, 5 fp32 fma, 6 the checked loop's mix
 * (add, multiply, compare, predicated add), 7 packed fp32 add (add.rn.f32x2), 8 two int adds +
 * one packed fp add, 9 int add + int multiply-add + one packed fp add, 10 fp64 add,
 * 11 and 12 mixes that form part of the products on the fp64 pipe (the low word of
 * (2^52 + a) + b is a + b).  Variants 7-12 exist to show that no other instruction mix beats
 * variant 2 on this GPU.  `scratch` is one device int.  This call
 * synchronises (CUDA events on `stream`). */
int pamk_issue_rate(int variant, int iters, int ctas_per_sm, int* scratch, float* elapsed_ms,
                    double* chain_steps, void* stream);

#ifdef __cplusplus
}
#endif
#endif
