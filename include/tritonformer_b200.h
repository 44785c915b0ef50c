/*
 * tritonformer_b200 -- C ABI of the sm_100a kernel library behind the
 * tritonformer autograd Functions.
 *
 * Every entry point
 *   - takes plain device pointers, 64-bit sizes/strides (in ELEMENTS), a dtype
 *     code, and the CUDA stream (as void*) to launch on;
 *   - is asynchronous and stream ordered, never synchronises the host, never
 *     allocates or frees device memory (scratch buffers are passed in), never
 *     writes to an input;
 *   - returns 0 on success or a negative tfb_status; the text of the last
 *     failure on the calling thread is available from tfb_last_error().
 *
 * The comment above each declaration names the piece of the reference
 * (fattorib/tritonformer, paths relative to that project) it stands in for.
 */
#ifndef TRITONFORMER_B200_H
#define TRITONFORMER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes */
#define TFB_F16 0
#define TFB_BF16 1
#define TFB_F32 2

/* status codes */
#define TFB_OK 0
#define TFB_ERR_ARG (-1)      /* bad shape / stride / alignment / dtype      */
#define TFB_ERR_UNSUPPORTED (-2)
#define TFB_ERR_LAUNCH (-3)   /* CUDA reported an error at launch            */
#define TFB_ERR_DRIVER (-4)   /* tensor-map encoding / driver entry missing  */

/* Library ABI version (bumped when a signature changes). */
int tfb_version(void);
/* Text of the last error raised on the calling thread ("" if none). */
const char* tfb_last_error(void);
/* Number of kernels this library has launched in the calling process. */
int64_t tfb_launch_count(void);
/* Device-side status word of the library on the calling thread's CURRENT device (one word per GPU,
 * shared by every kernel of the library): 0, or the code of the first bounded wait that expired
 * (0x2xxx attention backward, 0x5xxx attention forward, 0x1xxx / 0x3xxx GEMM, 0x7e00 the test probe)
 * or 0x7100 for a token id outside the embedding table.  While it is non-zero the tcgen05 kernels
 * (GEMM, attention) return at once without writing their outputs; the other kernels still run.
 * Synchronises the device; call it where the host synchronises anyway (the loss read-back).
 * reset != 0 clears the word; the caller must then also zero its GEMM workspaces, whose arrival
 * counters an abandoned split product can leave non-zero.                                     */
int tfb_device_status(int reset);

/* Which device an entry point works on: the calling thread's current device.  It must be the device
 * that owns the stream and every buffer of the call (a launch on another device's stream fails with
 * TFB_ERR_LAUNCH); per-device set-up (shared-memory limits, the fixed scratch of
 * tfb_layernorm_bwd_static, the status word) is keyed by it.  Entry points are re-entrant; forward
 * and backward may come from different host threads as long as each has that device current.      */
/* ------------------------------------------------------------------ LayerNorm
 * Replaces layernorm_fwd + layernorm_fwd_kernel (tritonformer/kernels/layernorm.py:9-87).
 * y = alpha * (x - mean) * rstd + beta over the last dim; additionally stores the
 * per-row mean and rstd (fp32) so the backward does not recompute them.
 * x, y: (rows, d) with row strides x_ld / y_ld, unit inner stride.           */
int tfb_layernorm_fwd(const void* x, const void* alpha, const void* beta, void* y,
                      float* mean, float* rstd, int64_t rows, int64_t d,
                      int64_t x_ld, int64_t y_ld, float eps, int dtype, void* stream);

/* Number of fp32 partial rows the backward needs: scratch = n * 2 * d floats. */
int64_t tfb_layernorm_bwd_partials(int64_t rows, int64_t d);

/* Replaces dx_layernorm + layernorm_da_db + _unbroadcast
 * (tritonformer/kernels/layernorm.py:91-259, kernels/reductions.py:25-63): one pass
 * over (dy, x) writes dx and fp32 partial column sums; a second small kernel folds the
 * partials into dalpha / dbeta (dtype `dtype`, shape (d,)).                    */
int tfb_layernorm_bwd(const void* dy, const void* x, const void* alpha,
                      const float* mean, const float* rstd, void* dx,
                      void* dalpha, void* dbeta, float* partials, int64_t n_partials,
                      int64_t rows, int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dx_ld,
                      int dtype, void* stream);

/* The same backward with the gradient of a residual branch folded in (no counterpart in the
 * reference, where autograd adds the two with a separate kernel): dx = dLayerNorm(dy) + dres, for
 * the pre-LN pattern h -> (LayerNorm(h), h).  dres may be NULL.                              */
int tfb_layernorm_bwd_res(const void* dy, const void* x, const void* alpha,
                          const float* mean, const float* rstd, const void* dres, void* dx,
                          void* dalpha, void* dbeta, float* partials, int64_t n_partials,
                          int64_t rows, int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dres_ld,
                          int64_t dx_ld, int dtype, void* stream);

/* The same again, optionally ADDING the column sums to what dalpha / dbeta already hold
 * (accumulate != 0): gradient accumulation into existing .grad buffers without a separate add
 * (no counterpart in the reference, where autograd adds).                                   */
int tfb_layernorm_bwd_acc(const void* dy, const void* x, const void* alpha,
                          const float* mean, const float* rstd, const void* dres, void* dx,
                          void* dalpha, void* dbeta, float* partials, int64_t n_partials,
                          int64_t rows, int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dres_ld,
                          int64_t dx_ld, int accumulate, int dtype, void* stream);

/* LayerNorm backward for callers that cannot supply scratch memory (no counterpart in the
 * reference, which allocates freely through torch): same results as tfb_layernorm_bwd, but the
 * fp32 partial sums live in a fixed array inside the library image (about 9.7 MB, held by every
 * GPU that loads the library) and the call allocates nothing.  Limit: d <= 4096; wider rows are
 * rejected with TFB_ERR_UNSUPPORTED.  The first call on a device looks up the array's device
 * address (with that device current); make that first call outside any stream capture.  The
 * address is remembered per device for the life of the process: after cudaDeviceReset() it is
 * stale and the entry must not be used again in that process.  All calls share the one array:
 * two calls whose kernels overlap on the GPU (different streams) race on it, so keep them
 * stream-ordered.                                                                           */
int tfb_layernorm_bwd_static(const void* dy, const void* x, const void* alpha,
                             const float* mean, const float* rstd, void* dx,
                             void* dalpha, void* dbeta,
                             int64_t rows, int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dx_ld,
                             int dtype, void* stream);

/* -------------------------------------------------------------------- Softmax
 * Replaces softmax_fwd / softmax_bwd (tritonformer/kernels/softmax.py:7-111).
 * Row softmax over the last dim; the backward writes a fresh tensor (the reference
 * overwrites grad_out).  dtype may be F16, BF16 or F32.                        */
int tfb_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols,
                    int64_t x_ld, int64_t y_ld, int dtype, void* stream);
int tfb_softmax_bwd(const void* dy, const void* y, void* dx, int64_t rows, int64_t cols,
                    int64_t dy_ld, int64_t y_ld, int64_t dx_ld, int dtype, void* stream);

/* -------------------------------------------------------------- Cross-entropy
 * Replaces cross_entropy_fwd / cross_entropy_bwd (tritonformer/kernels/crossentropy.py:7-127)
 * and the multiply that follows in tritonformer/crossentropy.py:24.
 * fwd: loss[i] = logsumexp(logits[i,:]) - logits[i,label[i]] (dtype `dtype`), lse[i] fp32;
 *      loss_f32 (may be NULL) receives the same per-row loss unrounded.
 * bwd: dlogits[i,j] = (exp(logits[i,j]-lse[i]) - [j==label[i]]) * grad[i].
 * `grad` has element stride grad_stride (0 broadcasts one value).
 * A label outside [0, vocab) makes its row contribute zero loss and zero gradient.   */
int tfb_cross_entropy_fwd(const void* logits, const int64_t* labels, void* loss, float* loss_f32,
                          float* lse, int64_t rows, int64_t vocab, int64_t logits_ld, int dtype,
                          void* stream);
int tfb_cross_entropy_bwd(const void* logits, const int64_t* labels, const float* lse,
                          const void* grad, int64_t grad_stride, void* dlogits,
                          int64_t rows, int64_t vocab, int64_t logits_ld, int64_t dlogits_ld,
                          int dtype, void* stream);

/* ---------------------------------------------------------- ReLU grad / bias grad
 * Replaces mask_grad (tritonformer/kernels/activation.py:7-44) without mutating the
 * incoming gradient: dz = act > 0 ? dy : 0 for n contiguous elements.          */
int tfb_relu_bwd(const void* dy, const void* act, void* dz, int64_t n, int dtype, void* stream);

/* fp32 partial rows needed by tfb_colsum: scratch = n * cols floats.           */
int64_t tfb_colsum_partials(int64_t rows, int64_t cols);
/* Replaces unbroadcast_leading + _unbroadcast (tritonformer/kernels/reductions.py:25-122):
 * out[j] = sum_i x[i,j], accumulated in fp32.                                  */
int tfb_colsum(const void* x, void* out, float* partials, int64_t n_partials,
               int64_t rows, int64_t cols, int64_t x_ld, int dtype, void* stream);

/* ------------------------------------------------------------------- embeddings
 * Replaces the two torch.nn.Embedding lookups and their sum at the head of
 * Transformer.forward (transformer.py:259-272, 311-321) and their gradients.
 *   out[b,t,:] = tok[ids[b,t],:] (+ pos[t,:] when pos is not NULL), summed in fp32.
 * ids is a contiguous (batch, seq) int64 array; tok is (vocab, d), pos (pos_rows, d) with
 * pos_rows >= seq (checked), out (batch, seq, d), all contiguous.  A token id outside
 * [0, vocab) gives a zero row and the sticky code 0x7100 in tfb_device_status().  */
int tfb_embedding_fwd(const int64_t* ids, const void* tok, const void* pos, void* out,
                      int64_t batch, int64_t seq, int64_t d, int64_t vocab, int64_t pos_rows,
                      int dtype, void* stream);
/* Bytes of scratch tfb_embedding_bwd needs (two int32 tables over the vocabulary
 * plus one fp32 row per position).                                             */
int64_t tfb_embedding_bwd_scratch_bytes(int64_t batch, int64_t seq, int64_t d, int64_t vocab);
/* ADDS the gradients to what dtok (vocab, d; NULL for a frozen table: nothing is indexed or
 * written for it) and dpos (pos_rows >= seq, d; may be NULL) hold:
 *   dtok[v,:] += sum over positions holding v of dout[b,t,:],  dpos[t,:] += sum_b dout[b,t,:]
 * with fp32 sums and one rounding per touched row; untouched rows are not written.
 * Tokens held by several positions are summed with fp32 atomics, so the order of
 * that sum (not its operands) may differ between runs.  scratch needs no
 * initialisation and is 16-byte aligned.                                       */
int tfb_embedding_bwd(const int64_t* ids, const void* dout, void* dtok, void* dpos,
                      void* scratch, int64_t scratch_bytes, int64_t batch, int64_t seq,
                      int64_t d, int64_t vocab, int64_t pos_rows, int dtype, void* stream);

/* ------------------------------------------------------------------------ GEMM
 * Replaces mm / gemm / bmm + torch.sum (tritonformer/kernels/gemm.py:81-616,
 * tritonformer/linear.py:15-102).
 *   C[m,n] = act( sum_k A(m,k) * B(k,n) + bias[n] ) (+ C[m,n] if accumulate)
 * A(m,k) lives at a[m*a_sm + k*a_sk], B(k,n) at b[k*b_sk + n*b_sn] (element strides,
 * one of each pair must be 1); C is row-major with leading dimension ldc.
 * fp16/bf16 operands, fp32 accumulation over the whole contraction, one rounding.
 * The weight gradient is this same call with the contraction over all B*T rows.
 * bias may be NULL; relu != 0 applies max(.,0) after the bias.
 * Shapes whose operand rows are 16-byte aligned run on the tcgen05/TMA kernel; the
 * rest run on a generic-stride tensor-core kernel.  `path` (may be NULL) receives
 * 1 for the tcgen05 kernel, 0 for the generic one.                              */
int tfb_gemm(const void* a, const void* b, void* c, const void* bias,
             int64_t M, int64_t N, int64_t K,
             int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc,
             int relu, int accumulate, int dtype, void* stream, int* path);

/* The same product with the epilogue fusions the model uses (no counterpart in the reference, which
 * runs these as separate kernels: the residual add of transformer.py:245,250, mask_grad of
 * kernels/activation.py:7-44, the gradient accumulation of autograd):
 *   C[m,n] = mask( act( sum_k A(m,k) B(k,n) + bias[n] ) + addend[m,n] )
 * addend (may be NULL; may be C itself to accumulate) has leading dimension ld_addend; mask (may be
 * NULL) zeroes the result wherever mask[m,n] <= 0 (pass a saved ReLU output to get the ReLU
 * gradient).  workspace (may be NULL) is scratch of at least tfb_gemm_workspace_bytes() bytes, 16-byte
 * aligned, whose first 8192 bytes are ZERO on entry; they are zero again when the kernel has finished,
 * so one buffer cleared once serves every call on a stream (calls that share a workspace must be
 * stream-ordered).  With a workspace, when the output tiles do not fill whole waves of SMs, the
 * contraction of some tiles is shared between SMs ("stream-K": fp32 partial tiles, summed in a fixed
 * order, so the result does not depend on timing).                                                 */
int64_t tfb_gemm_workspace_bytes(void);
int tfb_gemm_fused(const void* a, const void* b, void* c, const void* bias,
                   const void* addend, int64_t ld_addend, const void* mask, int64_t ld_mask,
                   int64_t M, int64_t N, int64_t K,
                   int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc,
                   int relu, int dtype, void* workspace, int64_t workspace_bytes,
                   void* stream, int* path);

/* ------------------------------------------------------------------- Attention
 * Replaces flash_wrapper_fwd / flash_wrapper_fwd_attn_bias
 * (tritonformer/kernels/attention.py:9-217, kernels/biased_attention.py:9-245).
 * q,k,v,o: (B,H,T,hd) with element strides {b,h,t} each and unit stride on hd.
 * Causal. Optional additive bias, one of:
 *   slopes != NULL : ALiBi, bias(i,j) = -slope[h]*(i-j), slopes fp32 (H,).  With
 *                    alibi_round = 1 (fp16) or 2 (bf16) each entry is rebuilt the way the
 *                    reference table is (transformer.py:55-75): distance and slope rounded
 *                    to that type and multiplied in it; 0 = exact fp32 product.
 *   bias != NULL   : dense (H,T,T) table of dtype `dtype`, element strides bias_sh, bias_si,
 *                    unit stride on j (entries above the diagonal are ignored).
 * lse: (B,H,T) fp32 contiguous = natural-log-sum-exp of the scaled, biased scores.  */
int tfb_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                      int64_t B, int64_t H, int64_t T, int64_t hd,
                      const int64_t* q_strides, const int64_t* k_strides,
                      const int64_t* v_strides, const int64_t* o_strides,
                      const float* slopes, int alibi_round,
                      const void* bias, int64_t bias_sh, int64_t bias_si,
                      int dtype, void* stream, int* path);

/* Bytes of scratch tfb_attention_bwd needs (fp32 delta (B,H,T) plus, on the tcgen05
 * path, an fp32 dQ accumulator (B,H,T,hd)).                                     */
int64_t tfb_attention_bwd_scratch_bytes(int64_t B, int64_t H, int64_t T, int64_t hd);

/* Replaces flash_wrapper_bwd / flash_wrapper_bwd_attn_bias
 * (tritonformer/kernels/attention.py:221-607, kernels/biased_attention.py:249-660).
 * Every tensor carries its own {b,h,t} strides.                                 */
int tfb_attention_bwd(const void* q, const void* k, const void* v, const void* o,
                      const void* d_o, const float* lse,
                      void* dq, void* dk, void* dv,
                      int64_t B, int64_t H, int64_t T, int64_t hd,
                      const int64_t* q_strides, const int64_t* k_strides,
                      const int64_t* v_strides, const int64_t* o_strides,
                      const int64_t* do_strides, const int64_t* dq_strides,
                      const int64_t* dk_strides, const int64_t* dv_strides,
                      const float* slopes, int alibi_round,
                      const void* bias, int64_t bias_sh, int64_t bias_si,
                      void* scratch, int64_t scratch_bytes,
                      int dtype, void* stream, int* path);

/* ------------------------------------------------------------------- optimizer step
 * No counterpart in the reference, which ships no optimizer (its README trains with one, README.md:89-113):
 * the step that follows forward+backward in a training loop, on the flat 16-bit gradient buckets the
 * weight-gradient products write into.  Everything is decided on the device; nothing reads back to the host.
 *
 * tfb_grad_check: sets *found_inf to 1 if any of the n gradients is inf or nan (leaves it alone otherwise).   */
int tfb_grad_check(const void* grad, int64_t n, int dtype, int* found_inf, void* stream);
/* tfb_adamw_step: AdamW on n elements with fp32 master weights (torch.optim.AdamW's arithmetic, operation by
 * operation): g = grad * *inv_scale; master *= 1 - lr*weight_decay; exp_avg, exp_avg_sq updated; master -=
 * lr / (1 - beta1^t) * exp_avg / (sqrt(exp_avg_sq) / sqrt(1 - beta2^t) + eps) with t = *steps_taken + 1;
 * param = master rounded to the 16-bit dtype.  Does nothing at all while *found_inf != 0 (step skipped).
 * inv_scale, found_inf, steps_taken are device pointers and may be NULL (1, 0, 0).  beta1 > 0.5.  The
 * hyper-parameters are doubles, like the Python floats of torch.optim.AdamW, and rounded to fp32 once.       */
int tfb_adamw_step(const void* grad, void* param, float* master, float* exp_avg, float* exp_avg_sq,
                   int64_t n, int dtype, const float* inv_scale, const int* found_inf,
                   const float* steps_taken, double lr, double beta1, double beta2, double eps,
                   double weight_decay, void* stream);
/* tfb_loss_scale_update: after the step kernels of every bucket.  state4 (device) = {loss scale, 1 / scale,
 * good steps since the scale last changed, optimizer steps taken}.  If *found_inf: scale *= backoff, the
 * good-step count restarts; else the step counter advances and after `interval` good steps scale *= growth
 * (torch.amp.GradScaler.update's rule).  Clears *found_inf.                                                 */
int tfb_loss_scale_update(float* state4, int* found_inf, float growth, float backoff, int interval,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITONFORMER_B200_H */
