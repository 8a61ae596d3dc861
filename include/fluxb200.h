/*
 * fluxb200.h — C ABI of libfluxb200.so: the forward + backward hot path of Flux.jl's own layers
 * as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * Flux has no FFI of its own: its layers call NNlib / BLAS / Optimisers / NCCL.jl through Julia
 * dispatch on the array type.  Each entry point below names the reference call site it replaces
 * (file:line inside the Flux.jl source tree); a Julia package extension binds them with `ccall`
 * for arrays of a new device type.
 *
 * Conventions
 *  - every function returns an int32 status (FB_OK == 0, negative on error), never aborts, throws
 *    or exits; fb_last_error() returns the message of the calling thread's last failure;
 *  - pointers are raw device pointers unless the name ends in `_host`; sizes are int64; enums are
 *    int32; scalars are passed by value;
 *  - arrays are dense and column-major exactly as Julia stores them: a Julia `W[out,in]` is read by
 *    the kernels as row-major `[in][out]`, `x[in,N]` as `[N][in]`, WHCN images as `[N][C][H*W]`;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Calls enqueue work
 *    and return; only fb_sync, fb_memcpy_d2h and the fb_comm_* bootstrap calls block;
 *  - the caller owns all tensors, including the saved-for-backward buffers (statistics, gates,
 *    log-sum-exp); the library owns only a per-context scratch arena that grows on demand.
 */
#ifndef FLUXB200_H
#define FLUXB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_VERSION 100

/* status codes */
#define FB_OK 0
#define FB_ERR_INVALID_ARG (-1)
#define FB_ERR_SHAPE (-2)
#define FB_ERR_ALLOC (-3)
#define FB_ERR_CUDA (-4)
#define FB_ERR_NCCL (-5)
#define FB_ERR_TIMEOUT (-6)
#define FB_ERR_UNSUPPORTED (-7)

/* activation enum (NNlib activations that Flux layers are constructed with) */
#define FB_ACT_IDENTITY 0
#define FB_ACT_RELU 1
#define FB_ACT_TANH 2
#define FB_ACT_SIGMOID 3
#define FB_ACT_GELU_TANH 4
#define FB_ACT_GELU_ERF 5

/* matmul precision for Float32 data */
#define FB_PREC_DEFAULT 0 /* 3xTF32 on the tensor cores when the shape allows, else fp32 FMA */
#define FB_PREC_FP32_SIMT 1 /* always the fp32 FMA kernel */
#define FB_PREC_3XTF32 2  /* tcgen05 tensor cores, error-compensated TF32 (fp32-level accuracy) */
#define FB_PREC_TF32 3    /* tcgen05 tensor cores, single TF32 pass */
#define FB_PREC_3XTF32_PAIR 4 /* 3xTF32 on 256 x 256 tiles computed by CTA pairs (cta_group::2) where M, N >= 256 */

/* reduction op for collectives (DistributedUtils.avg is FB_OP_AVG) */
#define FB_OP_SUM 0
#define FB_OP_AVG 1

typedef struct fb_ctx fb_ctx;
typedef struct fb_comm fb_comm;

/* ---------------------------------------------------------------- context, memory, errors -- */

/* Library version (FB_VERSION of the build). No reference counterpart. */
int32_t fb_version(void);

/* Number of kernels this library has launched in the calling process (diagnostic counter). No reference
 * counterpart. */
int64_t fb_kernel_launches(void);

/* Creates the per-(thread, device) context: selects `device`, creates the scratch arena.
 * Replaces what CUDA.jl's task-local state gives FluxCUDAExt (ext/FluxCUDAExt.jl:1-13). */
int32_t fb_ctx_create(int32_t device, fb_ctx** out);
int32_t fb_ctx_destroy(fb_ctx* ctx);
/* The persistent GEMM launches one CTA per SM; a communication kernel (NCCL) that holds a few SMs when the GEMM
 * starts would make part of that grid wait until the communication ends.  With n SMs reserved the GEMM grid is
 * sized for sm_count - n, so both run side by side.  0 (the default) uses every SM.  Host-side setting, read at
 * launch (a captured graph keeps the grid it was captured with).  No counterpart in the reference. */
int32_t fb_ctx_set_reserved_sms(fb_ctx* ctx, int32_t n);


/* Message of the last error raised on the calling thread ("" if none). */
const char* fb_last_error(void);

/* Device memory for the B200 array type: allocation, release, copies and fill.
 * Replaces Adapt.adapt_storage / `gpu` / `cpu` movement (src/functor.jl:85, 116). */
int32_t fb_malloc(fb_ctx* ctx, int64_t bytes, void** out);
int32_t fb_free(fb_ctx* ctx, void* ptr);
int32_t fb_memcpy_h2d(fb_ctx* ctx, void* stream, void* dst, const void* src_host, int64_t bytes);
int32_t fb_memcpy_d2h(fb_ctx* ctx, void* stream, void* dst_host, const void* src, int64_t bytes);
int32_t fb_memcpy_d2d(fb_ctx* ctx, void* stream, void* dst, const void* src, int64_t bytes);
int32_t fb_memset(fb_ctx* ctx, void* stream, void* dst, int32_t byte_value, int64_t bytes);
int32_t fb_sync(fb_ctx* ctx, void* stream);

/* Device-side error word set by kernels whose bounded waits ran out (0 = none).  While it is set the
 * tensor-core kernels return without computing.  Reading it synchronises the stream and clears it. */
int32_t fb_device_error(fb_ctx* ctx, void* stream, int32_t* out_host);

/* Launches a one-block kernel whose only act is a bounded wait (at most `polls` <= 4096 polls) on a barrier
 * that nothing signals: the wait runs out, code 9001 lands in the device error word, the kernel returns.  It lets
 * a caller exercise its handling of that word (report, clear, carry on) without any real kernel misbehaving.
 * Test aid; no counterpart in the reference. */
int32_t fb_selftest_bounded_wait(fb_ctx* ctx, void* stream, int32_t polls);

/* ------------------------------------------------------------------------------- matmul -- */

/* C = op(A) * op(B) (+ C when accumulate != 0), column-major BLAS convention, Float32.
 * transa/transb: 0 = 'N', 1 = 'T'.  Replaces `a.weight * xT` (src/layers/basic.jl:199) and the
 * `*` calls of the recurrent cells (src/layers/recurrent.jl:414, 616-617) for the new array type. */
int32_t fb_gemm_f32(fb_ctx* ctx, void* stream, int32_t transa, int32_t transb, int64_t m, int64_t n,
                    int64_t k, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                    int64_t ldc, int32_t accumulate, int32_t precision);

/* ------------------------------------------------------------------------------- Dense -- */

/* y[out,n] = act.(W[out,in] * x[in,n] .+ b) in one fused kernel.  `b` may be NULL (bias=false).
 * `z` (optional, may be NULL) receives the pre-activation, needed by fb_dense_bwd for the gelu
 * activations.  Replaces (a::Dense)(x) = NNlib.bias_act!(sigma, a.weight * xT, a.bias)
 * (src/layers/basic.jl:196-200). */
int32_t fb_dense_fwd(fb_ctx* ctx, void* stream, int32_t act, int32_t precision, const float* W,
                     const float* b, const float* x, float* y, float* z, int64_t out_dim,
                     int64_t in_dim, int64_t n);

/* Reverse of fb_dense_fwd (the Zygote pullback of basic.jl:199; external rrules of `*` and
 * NNlib.bias_act!): delta = dy .* act'(.), dW = delta * x', db = sum_n delta, dx = W' * delta.
 * `y` is the forward output (used by relu/tanh/sigmoid), `z` the saved pre-activation (gelu; may be
 * NULL otherwise).  `delta` is caller scratch of out*n floats (may be NULL for FB_ACT_IDENTITY).
 * db and dx may be NULL to skip them. */
int32_t fb_dense_bwd(fb_ctx* ctx, void* stream, int32_t act, int32_t precision, const float* W,
                     const float* x, const float* y, const float* z, const float* dy, float* delta,
                     float* dW, float* db, float* dx, int64_t out_dim, int64_t in_dim, int64_t n);

/* The same three calls for BFloat16 storage (raw bf16 bit patterns in uint16), the opt-in low-precision path of
 * Flux.bf16 / Flux._to_bf16 (src/functor.jl:137-183, 274): operands, bias, outputs and gradients are bf16, products
 * are accumulated in Float32 on the tensor cores (tcgen05.mma.kind::f16).  Pointers must be 16-byte aligned and
 * leading dimensions multiples of 8 (FB_ERR_UNSUPPORTED otherwise).  fb_gemm_bf16 writes C as Float32 when
 * c_is_f32 != 0. */
int32_t fb_gemm_bf16(fb_ctx* ctx, void* stream, int32_t transa, int32_t transb, int64_t m, int64_t n, int64_t k,
                     const uint16_t* A, int64_t lda, const uint16_t* B, int64_t ldb, void* C, int64_t ldc,
                     int32_t accumulate, int32_t c_is_f32);
/* y += alpha * x on bf16 arrays (tangent accumulation of a bf16 model; one rounding per element). */
int32_t fb_axpy_bf16(fb_ctx* ctx, void* stream, float alpha, const uint16_t* x, uint16_t* y, int64_t count);
int32_t fb_dense_fwd_bf16(fb_ctx* ctx, void* stream, int32_t act, const uint16_t* W, const uint16_t* b,
                          const uint16_t* x, uint16_t* y, uint16_t* z, int64_t out_dim, int64_t in_dim, int64_t n);
int32_t fb_dense_bwd_bf16(fb_ctx* ctx, void* stream, int32_t act, const uint16_t* W, const uint16_t* x,
                          const uint16_t* y, const uint16_t* z, const uint16_t* dy, uint16_t* delta, uint16_t* dW,
                          uint16_t* db, uint16_t* dx, int64_t out_dim, int64_t in_dim, int64_t n);

/* ---------------------------------------------------------------------------- LayerNorm -- */

/* y[d,n] = act.(gamma .* (x - mean) * rstd .+ beta), statistics over the first (flattened) d
 * elements of every column, biased variance, eps added to the variance.  gamma/beta may be NULL
 * (affine=false).  mean/rstd (n floats each) are saved for the backward pass.
 * Replaces (a::LayerNorm)(x) = a.diag(NNlib.normalise(x; dims, eps)) (src/layers/normalise.jl:203-210,
 * Scale: src/layers/basic.jl:284-287). */
int32_t fb_layernorm_fwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma,
                         const float* beta, float* y, float* mean, float* rstd, int64_t d, int64_t n,
                         float eps, int32_t act);

/* Reverse of fb_layernorm_fwd (external NNlib rrules): dx, dgamma[d], dbeta[d] (the last two may be
 * NULL when gamma is NULL). */
int32_t fb_layernorm_bwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma,
                         const float* beta, const float* mean, const float* rstd, const float* dy,
                         float* dx, float* dgamma, float* dbeta, int64_t d, int64_t n, int32_t act);

/* fb_layernorm_bwd for callers that may not allocate device memory (a process whose memory budget is fixed at
 * start-up, code inside a stream capture, runtime threads that must not risk the implicit synchronisation of
 * cudaMalloc / cudaFree).  No counterpart in the reference; same arguments and results as fb_layernorm_bwd minus the
 * context.  The dgamma / dbeta partials live in a fixed 16 MiB device array inside the library image (held by every
 * GPU that loads the library until the process exits), so: d <= 2 Mi features when dgamma / dbeta are requested
 * (FB_ERR_UNSUPPORTED otherwise); the call allocates and frees nothing; all calls share the array, so two calls
 * that overlap on the GPU (different streams) race - serialise them.  The first call on each device also resolves
 * the array's device address (cudaGetSymbolAddress, with that device current); make that first call before any
 * stream capture begins.  Uses the current device.  Having no context, the call has no device error word either:
 * it only launches kernels that wait on nothing (rows held in registers), so there is no timeout to report. */
int32_t fb_layernorm_bwd_noalloc(void* stream, const float* x, const float* gamma, const float* beta,
                                 const float* mean, const float* rstd, const float* dy, float* dx,
                                 float* dgamma, float* dbeta, int64_t d, int64_t n, int32_t act);

/* ---------------------------------------------------------------------------- BatchNorm -- */

/* Training-mode BatchNorm on x viewed as [n][c][s] (s = product of the dims before the channel dim):
 * per-channel batch mean and biased variance, y = act.(gamma*(x-mu)*rstd+beta); running statistics are
 * updated in place (mu <- (1-m) mu + m mu_B, var <- (1-m) var + m var_B * cnt/(cnt-1)) when
 * track_stats != 0.  save_mean/save_rstd (c floats) are saved for the backward pass.  cnt == 1 is
 * rejected with FB_ERR_SHAPE.  Replaces (BN::BatchNorm)(x) in training
 * (src/layers/normalise.jl:292-304 -> NNlib.batchnorm, then BN.lambda.(y)). */
int32_t fb_batchnorm_fwd_train(fb_ctx* ctx, void* stream, const float* x, const float* gamma,
                               const float* beta, float* running_mean, float* running_var, float* y,
                               float* save_mean, float* save_rstd, int64_t s, int64_t c, int64_t n,
                               float eps, float momentum, int32_t act, int32_t track_stats);

/* Inference-mode BatchNorm: normalises with the running statistics (normalise.jl:292-304 with
 * training == false).  running_mean/running_var NULL means track_stats=false: batch statistics are
 * used as in training, without an update. */
int32_t fb_batchnorm_fwd_infer(fb_ctx* ctx, void* stream, const float* x, const float* gamma,
                               const float* beta, const float* running_mean, const float* running_var,
                               float* y, int64_t s, int64_t c, int64_t n, float eps, int32_t act);

/* Reverse of fb_batchnorm_fwd_train (external NNlib rrule): dx, dgamma[c], dbeta[c]. */
int32_t fb_batchnorm_bwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma,
                         const float* beta, const float* save_mean, const float* save_rstd,
                         const float* dy, float* dx, float* dgamma, float* dbeta, int64_t s, int64_t c,
                         int64_t n, int32_t act);

/* ------------------------------------------------------------------- GroupNorm / InstanceNorm -- */

/* GroupNorm on x viewed as [n][c][s]: every (sample, group of c/groups channels) is normalised with its own mean and
 * biased variance over (c/groups)*s values, then y = act.(gamma[ch] * xhat + beta[ch]) per channel.  gamma/beta may be
 * NULL (affine=false).  mean/rstd hold n*groups floats, saved for the backward pass.  groups must divide c.
 * Replaces (gn::GroupNorm)(x) = gn.lambda.(NNlib.groupnorm(gamma, beta, x, G; eps)) (src/layers/normalise.jl:486-489).
 * With groups == c this is InstanceNorm's training-mode arithmetic (normalise.jl:388-393 -> NNlib.instancenorm). */
int32_t fb_groupnorm_fwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma, const float* beta,
                         float* y, float* mean, float* rstd, int64_t s, int64_t c, int64_t n, int64_t groups,
                         float eps, int32_t act);
/* Reverse of fb_groupnorm_fwd (external NNlib rrule): dx, dgamma[c], dbeta[c] (the last two may be NULL). */
int32_t fb_groupnorm_bwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma, const float* beta,
                         const float* mean, const float* rstd, const float* dy, float* dx, float* dgamma,
                         float* dbeta, int64_t s, int64_t c, int64_t n, int64_t groups, int32_t act);
/* InstanceNorm with track_stats=true: running_mean <- (1-m) running_mean + m * mean over samples of the per-instance
 * means, running_var likewise from the per-instance biased variances times s/(s-1), from the mean/rstd (n*c floats)
 * that fb_groupnorm_fwd saved with groups == c (rule pinned by test/layers/normalisation.jl:262-275).  Inference with
 * tracked statistics is fb_batchnorm_fwd_infer. */
int32_t fb_instancenorm_update_stats(fb_ctx* ctx, void* stream, const float* mean, const float* rstd,
                                     float* running_mean, float* running_var, int64_t s, int64_t c, int64_t n,
                                     float eps, float momentum);

/* ------------------------------------------------------------------------ Embedding / Dropout -- */

/* y[:, i] = W[:, idx[i]] for 1-based int32 indices (NNlib.gather), zero columns where idx[i] == padding_idx
 * (padding_idx 0 = none).  An index outside 1:vocab records code 5001 in the device error word (the reference throws
 * a BoundsError) and yields a zero column.  Replaces (m::Embedding)(x) (src/layers/basic.jl:794-800). */
int32_t fb_embedding_fwd(fb_ctx* ctx, void* stream, const float* W, const int32_t* idx, float* y, int64_t out_dim,
                         int64_t vocab, int64_t n, int32_t padding_idx);
/* Reverse of fb_embedding_fwd: dW[out, vocab] is zeroed and receives the scatter-add of dy's columns (the rrule of
 * NNlib.gather); the padding column stays zero. */
int32_t fb_embedding_bwd(fb_ctx* ctx, void* stream, const float* dy, const int32_t* idx, float* dW, int64_t out_dim,
                         int64_t vocab, int64_t n, int32_t padding_idx);
/* y[i] = x[i] / (1 - p) where the mask keeps element i, else 0 (NNlib.dropout, called at src/layers/normalise.jl:83).
 * The mask is a pure function of (seed, offset + i): Philox4x32-10 keyed by `seed`, counter offset + i/4, word i%4,
 * keep iff (word >> 8) * 2^-24 >= p.  Calling it again with the same seed and offset on the cotangent is the
 * backward pass.  The reference draws from a Julia RNG whose stream cannot be reproduced; only the distribution
 * matches. */
int32_t fb_dropout(fb_ctx* ctx, void* stream, const float* x, float* y, int64_t count, float p, uint64_t seed,
                   uint64_t offset);

/* ----------------------------------------------------------------------- losses / helpers -- */

/* loss = mean_n( -sum_c y[c,n] * logsoftmax(yhat)[c,n] ) with one-hot y given as 1-based int32 labels;
 * dyhat (optional) = dloss * (softmax - onehot)/n in the same pass.  `loss` is one device float.
 * Replaces Flux.logitcrossentropy (src/losses/functions.jl:270-273) for one-hot targets. */
int32_t fb_logitcrossentropy_labels(fb_ctx* ctx, void* stream, const float* yhat,
                                    const int32_t* labels, float* loss, float* dyhat, int64_t c,
                                    int64_t n, float dloss);

/* Same for a dense target y[c,n] (label smoothing, soft targets). */
int32_t fb_logitcrossentropy_dense(fb_ctx* ctx, void* stream, const float* yhat, const float* y,
                                   float* loss, float* dyhat, int64_t c, int64_t n, float dloss);

/* out[0] = sum(abs2, x) (Base.sum(abs2, y) in the benchmark losses). */
int32_t fb_sumsq(fb_ctx* ctx, void* stream, const float* x, int64_t count, float* out);
/* out[0] = sum(x) (Base.sum on the new array type; its cotangent is a fill, done with fb_fill). */
int32_t fb_sum(fb_ctx* ctx, void* stream, const float* x, int64_t count, float* out);
/* x[i] = value for all i (Base.fill!, the cotangent of sum). */
int32_t fb_fill(fb_ctx* ctx, void* stream, float* x, float value, int64_t count);
/* out_dev[0] = the GPU's nanosecond timer when the stream reaches this point: a time mark that can be placed
 * inside a captured graph (on any stream) to see how compute and communication interleave.  Measurement aid, no
 * counterpart in the reference. */
int32_t fb_timestamp(fb_ctx* ctx, void* stream, uint64_t* out_dev);
/* y = alpha * x (the cotangent 2y of sum(abs2, y); Optimisers' eta scaling). */
int32_t fb_scale(fb_ctx* ctx, void* stream, const float* x, float alpha, float* y, int64_t count);
/* y += alpha * x (tangent accumulation `+` of Zygote; `x .-= dx` of Optimisers.update!). */
int32_t fb_axpy(fb_ctx* ctx, void* stream, float alpha, const float* x, float* y, int64_t count);
/* Float32 -> BFloat16 bits, round-to-nearest-even in the integer domain, NaN -> 0x7fc0; bit-exact
 * with Flux._to_bf16 (src/functor.jl:161-166). */
int32_t fb_cast_f32_bf16(fb_ctx* ctx, void* stream, const float* x, uint16_t* y, int64_t count);
int32_t fb_cast_bf16_f32(fb_ctx* ctx, void* stream, const uint16_t* x, float* y, int64_t count);
/* y[i] = Float32(BFloat16(x[i])): the value a bf16 model holds, kept in a Float32 container (in place when y == x).
 * The opt-in bf16 path (Flux.bf16, src/functor.jl:274) keeps bf16-valued operands in Float32 storage: products of
 * such values are exact on the single-pass TF32 tensor path and accumulate in Float32, which is the arithmetic of a
 * bf16 tensor-core GEMM; results are rounded back with this call. */
int32_t fb_round_bf16(fb_ctx* ctx, void* stream, const float* x, float* y, int64_t count);

/* ------------------------------------------------------------------------------- Adam -- */

/* One Adam update of `ntensors` parameter leaves in one launch per 32 leaves:
 * m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2; w -= m/(1-b1t) / (sqrt(v/(1-b2t)) + eps) * eta.
 * b1t/b2t are the running powers beta^t *before* this step (the caller multiplies them afterwards,
 * as the rule's state does).  The pointer tables are host arrays of device pointers.
 * Replaces Optimisers.update! with the Adam rule (src/train.jl:425; arithmetic as in
 * src/optimise/optimisers.jl:171-184). grad_scale multiplies g first (1.0 normally). */
int32_t fb_adam_step(fb_ctx* ctx, void* stream, int32_t ntensors, float* const* w_host,
                     const float* const* g_host, float* const* m_host, float* const* v_host,
                     const int64_t* counts_host, float eta, float beta1, float beta2, float eps,
                     float b1t, float b2t, float grad_scale);

/* The same update with its step state on the device, for a train step replayed from a CUDA graph (the
 * device-specific one-launch `trainstep!` hook, src/train.jl:335-339): bt_dev[2] holds the running powers
 * (beta1^t, beta2^t); guard_dev (optional) is a device scalar - the loss - whose non-finite value skips the update,
 * as `_eager_step!` does (src/train.jl:377).  fb_adam_advance multiplies the powers by (beta1, beta2) under the
 * same guard. */
int32_t fb_adam_step_dev(fb_ctx* ctx, void* stream, int32_t ntensors, float* const* w_host,
                         const float* const* g_host, float* const* m_host, float* const* v_host,
                         const int64_t* counts_host, float eta, float beta1, float beta2, float eps,
                         const float* bt_dev, const float* guard_dev, float grad_scale);
/* The same update for ONE contiguous block, as a kernel shaped to run on an SM beside a resident GEMM CTA (128 threads
 * of at most 32 registers): the sharded optimiser's update on the communication stream (no counterpart in the
 * reference; public_api.jl:291-294 updates every leaf on every rank). */
int32_t fb_adam_block_dev(fb_ctx* ctx, void* stream, float* w, const float* g, float* m, float* v, int64_t count, float eta,
                          float beta1, float beta2, float eps, const float* bt_dev, const float* guard_dev, float grad_scale);
int32_t fb_adam_advance(fb_ctx* ctx, void* stream, float* bt_dev, float beta1, float beta2,
                        const float* guard_dev);

/* ------------------------------------------------------------------------- Recurrence -- */

/* Bytes of the saved-for-backward buffer of fb_lstm_fwd / fb_gru_fwd. */
int64_t fb_lstm_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);
int64_t fb_gru_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);

/* Recurrence(LSTMCell)(x): x[in,T,B] -> out[H,T,B], final h[H,B], c[H,B]; zero initial state when
 * h0/c0 are NULL, else h0/c0 are [H,B].  Gate rows of Wi[4H,in], Wh[4H,H], b[4H] are i,f,g,o.
 * The input projection runs as one GEMM over all T*B columns; the time loop is one persistent kernel.
 * `cache` (fb_lstm_cache_bytes) may be NULL when no backward pass follows.
 * Replaces scan(cell, x, state) (src/layers/recurrent.jl:1-8) over LSTMCell (:411-419). */
int32_t fb_lstm_fwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* b,
                    const float* x, const float* h0, const float* c0, float* out, float* hT, float* cT,
                    void* cache, int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);

/* Reverse of fb_lstm_fwd (Zygote's BPTT over recurrent.jl:1-8): dout[H,T,B] (+ optional dhT, dcT)
 * -> dWi, dWh, db (may be NULL), dx (may be NULL).  h0/c0 are the initial
 * state given to the forward call (NULL = zeros).  The cache is consumed (overwritten). */
int32_t fb_lstm_bwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* x,
                    const float* h0, const float* c0, const float* out, const void* cache,
                    const float* dout, const float* dhT, const float* dcT, float* dWi, float* dWh, float* db, float* dx, int64_t in_dim,
                    int64_t hidden, int64_t seq_len, int64_t batch);

/* Recurrence(GRUCell)(x) (src/layers/recurrent.jl:614-628; rows r,z,h~; r multiplies Wh3*h). */
int32_t fb_gru_fwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* b,
                   const float* x, const float* h0, float* out, float* hT, void* cache, int64_t in_dim,
                   int64_t hidden, int64_t seq_len, int64_t batch);
int32_t fb_gru_bwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* x,
                   const float* h0, const float* out, const void* cache, const float* dout, const float* dhT, float* dWi,
                   float* dWh, float* db, float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len,
                   int64_t batch);

/* Recurrence(RNNCell)(x): h' = act.(Wi x + Wh h + b) (src/layers/recurrent.jl:193-198) over x[in,T,B] -> out[H,T,B],
 * final state hT[H,B] (optional); act is identity, relu, tanh or sigmoid.  The input projection is one GEMM over all
 * steps; every step is one GEMM with a fused accumulate + activation epilogue. */
int64_t fb_rnn_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);
int32_t fb_rnn_fwd(fb_ctx* ctx, void* stream, int32_t act, const float* Wi, const float* Wh, const float* b,
                   const float* x, const float* h0, float* out, float* hT, int64_t in_dim, int64_t hidden,
                   int64_t seq_len, int64_t batch);
/* Reverse (BPTT) of fb_rnn_fwd; `cache` is scratch of fb_rnn_cache_bytes. db and dx may be NULL. */
int32_t fb_rnn_bwd(fb_ctx* ctx, void* stream, int32_t act, const float* Wi, const float* Wh, const float* x,
                   const float* h0, const float* out, void* cache, const float* dout, const float* dhT, float* dWi,
                   float* dWh, float* db, float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);

/* Recurrence(GRUv3Cell)(x) (src/layers/recurrent.jl:795-809): r, z from the first two row blocks of Wi / Wh[3H,H],
 * htilde = tanh(gx3 + Wh_h (r .* h) + b3) with the separate matrix Wh_h[H,H], h' = (1-z) htilde + z h.  The third row
 * block of Wh is never read by the cell, so its gradient is zero.  `cache` (fb_gruv3_cache_bytes) is filled by the
 * forward pass and consumed by the backward pass; it may be NULL when no backward pass follows. */
int64_t fb_gruv3_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch);
int32_t fb_gruv3_fwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* b, const float* Wh_h,
                     const float* x, const float* h0, float* out, float* hT, void* cache, int64_t in_dim,
                     int64_t hidden, int64_t seq_len, int64_t batch);
int32_t fb_gruv3_bwd(fb_ctx* ctx, void* stream, const float* Wi, const float* Wh, const float* Wh_h, const float* x,
                     const float* h0, const float* out, void* cache, const float* dout, const float* dhT, float* dWi,
                     float* dWh, float* db, float* dWh_h, float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len,
                     int64_t batch);

/* -------------------------------------------------------------------------- Attention -- */

/* NNlib.dot_product_attention(q, k, v; nheads, mask) without materialising the score tensor:
 * q[E,Lq,B], k[E,Lk,B], v[Ev,Lk,B] -> o[Ev,Lq,B]; head h is the contiguous feature block
 * h*d..(h+1)*d-1; scores k'q/sqrt(d); softmax over the kv axis; causal != 0 keeps key j for query i
 * iff j <= i.  `mask` (optional uint8 [Lk,Lq], nonzero = keep) is applied as well.  lse[Lq,h,B]
 * (log-sum-exp per query, caller buffer) is saved for the backward pass.
 * Replaces the call at src/layers/attention.jl:128. */
int32_t fb_attn_fwd(fb_ctx* ctx, void* stream, const float* q, const float* k, const float* v,
                    const uint8_t* mask, float* o, float* lse, int64_t e_dim, int64_t ev_dim,
                    int64_t lq, int64_t lk, int64_t batch, int32_t nheads, int32_t causal);

/* Reverse of fb_attn_fwd (external NNlib rrule): probabilities are recomputed from lse. */
int32_t fb_attn_bwd(fb_ctx* ctx, void* stream, const float* q, const float* k, const float* v,
                    const uint8_t* mask, const float* o, const float* lse, const float* dout, float* dq,
                    float* dk, float* dv, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk,
                    int64_t batch, int32_t nheads, int32_t causal);

/* The attention weights alpha[Lk,Lq,h,B], the second return value of dot_product_attention
 * (src/layers/attention.jl:128-132), materialised on demand from q, k and lse. */
int32_t fb_attn_scores(fb_ctx* ctx, void* stream, const float* q, const float* k, const uint8_t* mask,
                       const float* lse, float* alpha, int64_t e_dim, int64_t lq, int64_t lk,
                       int64_t batch, int32_t nheads, int32_t causal);

/* The same three calls with the remaining arguments of NNlib.dot_product_attention(q, k, v, bias; nheads, mask, fdrop)
 * (src/layers/attention.jl:120-128):
 *  - bias (optional): added to the scaled scores before the mask and the softmax.  It is read at
 *    bias[j + lk * i + bias_stride_h * h + bias_stride_b * b] for key j, query i: a [lk, lq] bias shared by all heads
 *    and batch entries has both strides 0, a full [lk, lq, h, B] bias has strides lk*lq and lk*lq*h.  The bias gets no
 *    gradient (it is a constant of the layer call, attention.jl:40-44).
 *  - p_drop, seed, offset: dropout on the attention weights (the layer's `attn_drop`, attention.jl:91): weight
 *    (i, j) of head h, batch entry b is kept iff element ((b * nheads + h) * lq + i) * lk + j of the mask stream of
 *    fb_dropout(seed, offset) is kept, and scaled by 1 / (1 - p_drop).  fb_attn_scores_ex returns the weights after
 *    dropout, as the reference does.
 *  - dalpha (fb_attn_bwd_ex, optional [lk, lq, h, B]): a cotangent of the returned attention weights, for losses
 *    that read them (test/layers/attention.jl:56-61).
 * With any of these present the general (FMA) kernels run; without them the calls are the ones above. */
int32_t fb_attn_fwd_ex(fb_ctx* ctx, void* stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                       const float* bias, int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed,
                       uint64_t offset, float* o, float* lse, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk,
                       int64_t batch, int32_t nheads, int32_t causal);
int32_t fb_attn_bwd_ex(fb_ctx* ctx, void* stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                       const float* bias, int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed,
                       uint64_t offset, const float* o, const float* lse, const float* dout, const float* dalpha,
                       float* dq, float* dk, float* dv, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk,
                       int64_t batch, int32_t nheads, int32_t causal);
int32_t fb_attn_scores_ex(fb_ctx* ctx, void* stream, const float* q, const float* k, const uint8_t* mask,
                          const float* bias, int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed,
                          uint64_t offset, const float* lse, float* alpha, int64_t e_dim, int64_t lq, int64_t lk,
                          int64_t batch, int32_t nheads, int32_t causal);

/* ------------------------------------------------------------------- DistributedUtils -- */

/* NCCL unique id (128 bytes) created on one rank and handed to the others by the caller's bootstrap
 * (MPI broadcast in ext/FluxMPINCCLExt/FluxMPINCCLExt.jl:19-30; a store or file elsewhere). */
#define FB_UNIQUE_ID_BYTES 128
int32_t fb_comm_get_unique_id(void* id_host);
/* Joins the communicator (NCCL.Communicator, FluxMPINCCLExt.jl:26-29). Blocks until all ranks join. */
int32_t fb_comm_init_rank(fb_ctx* ctx, const void* id_host, int32_t nranks, int32_t rank, fb_comm** out);
int32_t fb_comm_destroy(fb_comm* comm);
/* DistributedUtils.local_rank / total_workers (src/distributed/public_api.jl:82-93). */
int32_t fb_comm_rank(const fb_comm* comm);
int32_t fb_comm_size(const fb_comm* comm);
/* DistributedUtils.allreduce! on a Float32 device buffer, in place when send == recv
 * (NCCL.Allreduce!, FluxMPINCCLExt.jl:61-78); FB_OP_AVG is DistributedUtils.avg. */
int32_t fb_allreduce(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t op);
/* The two halves of an all-reduce, for an optimiser whose state is sharded over the workers: every rank receives
 * the reduced block `rank` of `send` (recv_count elements; send holds nranks * recv_count), updates its share of the
 * parameters, and fb_allgather puts the blocks together again (recv holds nranks * send_count; in place when
 * send == recv + rank * send_count).  No counterpart in the reference, whose DistributedOptimizer all-reduces and
 * updates everything on every rank (src/distributed/public_api.jl:286-294); results are the same. */
int32_t fb_reduce_scatter(fb_comm* comm, void* stream, const float* send, float* recv, int64_t recv_count, int32_t op);
int32_t fb_allgather(fb_comm* comm, void* stream, const float* send, float* recv, int64_t send_count);
/* DistributedUtils.bcast! (NCCL.Broadcast!, FluxMPINCCLExt.jl:38-53). */
int32_t fb_bcast(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t root);
/* DistributedUtils.reduce! (NCCL.Reduce!, FluxMPINCCLExt.jl:86-102). */
int32_t fb_reduce(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t op, int32_t root);

/* Gradient exchange over peer memory (single node, NVLink / NVSwitch), for the sharded optimiser: reduce-scatter and
 * all-gather as small kernels that store into buffers the other ranks have mapped into this process; they are shaped
 * to run on an SM beside a resident GEMM CTA, which NCCL's kernels are not.  No counterpart in the reference (which
 * calls NCCL.Allreduce! per leaf, ext/FluxMPINCCLExt/FluxMPINCCLExt.jl:61-66); results equal a mean all-reduce
 * followed by the same update on every rank.
 *  - fb_peer_alloc allocates `bytes` of zeroed device memory and returns a FB_PEER_HANDLE_BYTES handle that the
 *    caller hands to the other processes (any host channel); fb_peer_open maps a peer's handle into this process.
 *  - fb_peer_push_blocks: for every peer p, blk floats at src + p * src_stride are copied to peer_dst_host[p] (the
 *    entry of this rank is ignored).  Reduce-scatter: src = my bucket, src_stride = blk, peer_dst_host[p] = slot
 *    [me] of the bucket's staging area in peer p's memory.  All-gather: src = my updated block, src_stride = 0,
 *    peer_dst_host[p] = the block's place in peer p's parameter buffer.
 *  - fb_reduce_slots: out = scale * (slots[0] + slots[1] + ... ) in that order; out may be one of the slots.
 *  - fb_peer_barrier: a barrier between the ranks as one warp on `stream`.  peer_flags_host[r] = rank r's array of
 *    nranks 32-bit epoch words (zero at the start, allocated with fb_peer_alloc and mapped by the others); epoch_dev =
 *    a zeroed device word of this rank that counts the barriers passed (the launch is therefore replayable from a
 *    CUDA graph).  Every rank must enqueue the same sequence of barriers.  What a rank stored before its barrier
 *    (into its own or a peer's memory) is visible to a kernel another rank enqueues behind its own.  A rank that waits
 *    longer than timeout_ms for a peer stores 9101 in the device error word (fb_device_error) and lets its stream
 *    continue: nothing hangs. */
#define FB_PEER_HANDLE_BYTES 64
int32_t fb_peer_alloc(fb_ctx* ctx, int64_t bytes, void** ptr_out, void* handle_host);
int32_t fb_peer_open(fb_ctx* ctx, const void* handle_host, void** ptr_out);
int32_t fb_peer_close(fb_ctx* ctx, void* ptr);
int32_t fb_peer_free(fb_ctx* ctx, void* ptr);
int32_t fb_peer_barrier(fb_ctx* ctx, void* stream, uint32_t* const* peer_flags_host, int32_t nranks, int32_t rank,
                        uint32_t* epoch_dev, int64_t timeout_ms);
int32_t fb_peer_push_blocks(fb_ctx* ctx, void* stream, const float* src, int64_t src_stride, float* const* peer_dst_host,
                            int32_t nranks, int32_t rank, int64_t blk);
int32_t fb_reduce_slots(fb_ctx* ctx, void* stream, int32_t nslots, const float* const* slots_host, float* out,
                        int64_t count, float scale);

/* Bucketed, overlapped gradient averaging for DistributedOptimizer (src/distributed/public_api.jl:286-300, which
 * all-reduces leaf by leaf with no overlap).  `flat` is one gradient buffer of `total` floats cut into `nbuckets`
 * buckets ending at bucket_ends_host[i] (increasing, the last one == total); every gradient leaf is registered as a
 * slice lying inside one bucket.  Per step: fb_bucket_begin_step; the reverse sweep calls fb_bucket_mark_ready for
 * a leaf once the kernels that write its gradient are enqueued on `compute_stream`; when a bucket's last leaf is
 * ready its mean all-reduce starts on the communication stream (the given one, or a high-priority stream the set
 * creates when comm_stream is NULL) while the compute stream continues; fb_bucket_wait starts whatever has not
 * started and makes `compute_stream` wait for all of it.  With one worker nothing is communicated.  Host-side
 * bookkeeping only: call from the thread that enqueues the step. */
typedef struct fb_bucket_set fb_bucket_set;
int32_t fb_bucket_create(fb_ctx* ctx, fb_comm* comm, float* flat, int64_t total, int32_t nbuckets,
                         const int64_t* bucket_ends_host, void* comm_stream, fb_bucket_set** out);
int32_t fb_bucket_destroy(fb_bucket_set* set);
int32_t fb_bucket_register(fb_bucket_set* set, int64_t offset, int64_t count, int32_t* leaf_id);
int32_t fb_bucket_begin_step(fb_bucket_set* set);
int32_t fb_bucket_mark_ready(fb_bucket_set* set, int32_t leaf_id, void* compute_stream);
int32_t fb_bucket_wait(fb_bucket_set* set, void* compute_stream);
/* Non-zero when NCCL reported an asynchronous error on this communicator (polled by the host between
 * steps; a dead rank otherwise hangs the next collective, as it does in the reference). */
int32_t fb_comm_async_error(fb_comm* comm, int32_t* out_host);

#ifdef __cplusplus
}
#endif
#endif /* FLUXB200_H */
