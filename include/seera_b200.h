/* seera_b200.h - C ABI of the B200-native Seera training engine.
 *
 * Drop-in boundary for the reference's GPU engine: every entry of the reference's
 * `seera_cuda` namespace (engine_cuda/include/seera_engine_cuda.hpp:9-123) and every
 * memory/transfer lambda of its Python binding (engine_cuda/src/cuda_bindings.cpp:23-170)
 * has a function here with the same name (prefixed `seera_`), the same argument order and
 * the same meaning.  Plain pointers and sizes only; all tensor pointers are device
 * addresses of dense, C-contiguous buffers (fp32 unless stated; activations NCHW).
 *
 * Differences from the reference that a caller can observe:
 *   - every function returns an int status: 0 = ok, otherwise a SEERA_E_* code;
 *     seera_last_error() gives the text.  The reference returns void and drops errors.
 *   - calls ENQUEUE work on the engine's stream and return; results are complete after
 *     seera_synchronize() or any seera_to_host_* call.  The reference blocks in every call.
 *   - max-pool writes cuda_maxpool_fwd's mask as the window-local argmax index kh*KW+kw of
 *     the first strict maximum (the reference CPU engine's rule, engine/src/pool_ops.cpp:21-38)
 *     in the first N*C*OH*OW ints of the caller's N*C*H*W-int buffer; cuda_maxpool_bwd reads
 *     that encoding.  When OH*OW > H*W (stride-1 pooling with padding) the buffer is too small
 *     and the call fails with SEERA_E_ARG.
 *   - argmax/argmin return the FIRST extremal index (NumPy's rule); the reference GPU kernel
 *     returns the last (engine_cuda/src/reductionKernels.cu:81,104).
 *
 * Not thread-safe: one host thread drives one device, as in the reference.
 */
#ifndef SEERA_B200_H
#define SEERA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    SEERA_OK = 0,
    SEERA_E_CUDA = 1,     /* a CUDA runtime call failed (sticky)            */
    SEERA_E_ARG = 2,      /* bad size / shape / null pointer                */
    SEERA_E_OOM = 3,      /* device allocation failed                       */
    SEERA_E_DEVICE = 4,   /* a kernel reported a status word != 0           */
    SEERA_E_LIMIT = 5     /* size beyond a documented maximum               */
};

/* ---- runtime ------------------------------------------------------------------ */
int         seera_init(int device);                 /* selects the device, creates the stream; idempotent for the same device, SEERA_E_ARG for another (one device per process) */
int         seera_synchronize(void);                /* waits for the engine's stream                     */
int         seera_set_stream(void *cuda_stream);    /* adopt an external cudaStream_t (NULL = own stream) */
void       *seera_get_stream(void);
const char *seera_last_error(void);
int         seera_last_status(void);                /* last non-zero status since seera_clear_status()   */
void        seera_clear_status(void);
uint64_t    seera_launch_count(void);               /* kernels launched by this library so far           */
int         seera_device_sm_count(void);
/* CUDA events on the engine's stream, for callers that time the hot path without another CUDA binding. */
void       *seera_event_create(void);
int         seera_event_record(void *event);
float       seera_event_elapsed_ms(void *start, void *stop);   /* waits for `stop`; < 0 on error */
int         seera_event_destroy(void *event);
/* Launch profile: while enabled, every GEMM / convolution launch of this library and every bandwidth-bound pass
 * (optimizer, activation backward, pooling, loss heads, operand copies) is bracketed by events on the engine's
 * stream.  Enabling starts an empty table.  seera_profile_read() waits for the events and returns the
 * contractions' count, summed device time and summed algorithmic FLOPs (2*M*N*K each), then clears the table.
 * seera_profile_read_kinds() gives the same three figures split by kind (index 0 forward products, 1 data
 * gradients dX / dA, 2 weight gradients dW / dB) and leaves the table alone.  seera_profile_report() writes one
 * line per tag, "tag<TAB>kind<TAB>launches<TAB>ms<TAB>work<NEWLINE>" (kind 0-2: work = FLOPs; kind 3: work =
 * algorithmic bytes of a bandwidth-bound pass), and leaves the table alone.  Nothing is recorded during a
 * stream capture.  No counterpart in the reference. */
int         seera_profile_enable(int on);
int         seera_profile_read(uint64_t *launches, double *ms, double *flops);
int         seera_profile_read_kinds(uint64_t *launches3, double *ms3, double *flops3);
int         seera_profile_report(char *buf, size_t size);
/* Precision of the GEMM / convolution contractions:
 *   0 fp32 CUDA-core tiles (bit-for-bit fp32 products, default for the fp32 configurations)
 *   1 bf16 operands, fp32 accumulate on the tensor cores (one pass)
 *   2 bf16x3: a_hi*b_hi + a_hi*b_lo + a_lo*b_hi on the tensor cores (16 mantissa bits per operand, ~5e-6)
 *   3 bf16x6: three-way split hi+lo+lo2, six products (24 mantissa bits per operand, fp32-class); on the
 *     TMA-fed kernels; the kernel that gathers in its producer warps runs mode 3 as mode 2
 *   4 fp16x3: two-way split into fp16 copies (11 + 11 mantissa bits), three products - the accuracy of mode 3
 *     (the dropped lo*lo term is 2^-22 of a product) at the cost of mode 2.  fp16 has a 5-bit exponent, so the
 *     copies carry a power-of-two factor by class of tensor, taken out again exactly in the epilogue:
 *     activations x 2^4 (saturate at 4094), weights x 2^8 (at 255.9), gradients x 2^12 (at 15.99); magnitudes
 *     down to 2^-7 / 2^-11 / 2^-15 keep all 22 bits, smaller ones an absolute error of 2^-29 / 2^-33 / 2^-37.
 *     Conversion saturates, it never produces infinities.  Data outside these ranges belongs in modes 2 / 3.
 *     Kernels that convert inside their producer warps (short patches, the gather fallback) run mode 4 as mode 2.
 *   5 fp16: ONE fp16 copy per operand with the scales of mode 4, one product (11 mantissa bits per operand, 2^-12
 *     rounding: eight times finer than mode 1).  It is the first copy of a mode-4 set, so a forward pass in mode 4
 *     followed by a backward pass in mode 5 converts nothing twice.  Meant for backward products: they take no
 *     decisions, so their rounding (2e-4 per contraction) stays a rounding.  Producer-warp kernels run it as mode 2. */
int         seera_set_precision(int mode);
int         seera_get_precision(void);
/* Engine options by name.
 *   "dense_tma" (default 1): in precision modes 1-3 the Dense GEMMs convert their operands to bf16 shadows once
 *       and feed the tensor cores by TMA; 0 selects the kernel that converts inside its producer warps.
 *   "conv_tma" (default 1): the same choice for the convolution family (TMA im2col).
 *   "sm_reserve" (default 0): the persistent kernels size their grids for that many SMs fewer than the device has.
 *       They hold one CTA with ~214 KB of shared memory per SM for their whole duration, so a kernel of another
 *       stream (a collective that should overlap them) otherwise finds no SM until they end.
 *   "pool_short_patch" (default 0): let seera_conv2d_bias_act_pool_fwd_s also serve short-patch convolutions
 *       (C*R*S <= 64).  Correct, but that kernel is bound by its epilogue warps and runs slower with the pool folded in
 *       than followed by a separate pool.
 *   "pair_tiles" (default 0; also SEERA_PAIR_TILES): run the TMA-fed GEMMs as clusters of two CTAs on 256-row tiles
 *       (tcgen05 cta_group::2: each CTA stages its own 128 rows of A and half of B's columns, the even CTA issues the
 *       MMAs for both, completion of both CTAs' plain tensor copies is counted on its barrier; no multicast load).
 *       It cuts the operand bytes per CTA and k-step by a quarter to a third.  Bit-for-bit the same results; measured
 *       3-8 % SLOWER on every configuration here (C3 dgrad 51.3 -> 53.2 us, wgrad 41.2 -> 51.1 us), because these
 *       kernels are bound by the MMA issue rate at accumulator widths of 64-128 columns, not by the operand stream.
 *   "wgrad_single" (default 1): in precision mode 4 a weight gradient (conv dW, Dense dB) is formed from the FIRST fp16
 *       copy of each operand alone - one product instead of three.  Its 2^-12 rounding stays inside that one tensor
 *       (nothing downstream in the backward pass reads dW); measured on the VGG configuration it moves no dW error
 *       by more than 3e-5.  Data gradients keep all three products: their rounding would compound layer by layer.
 *   "skinny_gemm" (default 1): in precision modes 1-5 a Dense product of at most 16 output columns (a classifier head: the
 *       forward, dA and dB of seera_cuda_matmul[_bwd] and of the fused Dense entries) runs as plain fp32 on the CUDA cores,
 *       one small launch each, reading the fp32 operands in place: no conversion passes, no pipeline fill for a tile that is
 *       mostly padding.  Results are fp32-exact (operands are not rounded to 16 bits) and bit-reproducible; the Dense entries
 *       keep no 16-bit copies for such a layer.  0 sends these products to the tensor cores like any other.
 *   "tc_wait_ms" (1..60000, default 2000; also SEERA_TC_WAIT_MS): budget of every wait inside the TMA-fed tensor-core
 *       kernel, in milliseconds at ~2 GHz.  A wait that runs out makes the kernel record its code in the status word
 *       (seera_tc_device_status), let the copies already in flight land (bounded), free its TMEM and return.
 *   "tc_test_skip_load" (k-step index, -1 off): TEST HOOK for that path.  The next TMA-fed launch's first CTA leaves out
 *       the loads of that k-step, so the MMA issuer's wait for the stage runs out.  Nothing faults, traps or spins
 *       without a bound; the result of that one launch is garbage and the status word reads 2.  Clears itself.
 *   "tile_n_cap2" / "tile_n_cap3" (64, 128 or 256; defaults 128 / 128): widest accumulator tile used with two /
 *       three bf16 copies per operand; wider tiles raise the arithmetic per byte loaded but leave fewer stages. */
int         seera_set_option(const char *name, int value);
/* Status word of the tensor-core kernels: 0 when every bounded wait inside them completed, otherwise
 * the code of the first wait that ran out (1 producer, 2 MMA issuer, 3 epilogue); reading clears it.
 * Synchronises the stream.  -1 if it could not be read. */
int         seera_tc_device_status(void);

/* ---- memory (cuda_bindings.cpp:23-66) ----------------------------------------------- */
void *seera_cuda_malloc(size_t n_bytes);            /* :23  pooled, stream-ordered; NULL on failure */
void *seera_cuda_malloc_f32(int n_elements);        /* :37 (and cuda_malloc_f16 :30, same size)     */
void *seera_cuda_malloc_i32(int n_elements);        /* :44 */
void *seera_cuda_malloc_i16(int n_elements);        /* :51 */
int   seera_cuda_free(void *ptr);                   /* :58  returns the block to the pool           */
int   seera_cuda_memcopy_devicetodevice(void *dst, const void *src, int num_elem); /* :61 counts FLOAT elements */
int   seera_cuda_memset(void *ptr, int value, size_t n_bytes);                     /* :65 */
int   seera_pool_trim(void);                        /* releases cached blocks to the driver         */
size_t seera_pool_bytes_reserved(void);
/* Stream capture of a whole step into a CUDA graph.  Between graph_begin and graph_end every call of this
 * library is recorded instead of executed; blocks the recorded work allocates stay reserved for the graph
 * (they are written again by every replay) until graph_destroy.  Run the step eagerly at least once first.
 * No call that reads back to the host (seera_to_host, seera_synchronize) may be made while capturing. */
int   seera_graph_begin(void);
void *seera_graph_end(void);                        /* NULL on failure */
int   seera_graph_launch(void *graph);
int   seera_graph_destroy(void *graph);
int   seera_is_capturing(void);
void *seera_host_alloc_pinned(size_t n_bytes);      /* page-locked staging for callers that time H2D */
int   seera_host_free_pinned(void *p);

/* ---- transfers (cuda_bindings.cpp:73-170) ------------------------------------------------ */
void *seera_to_device(const void *host, size_t n_bytes);              /* :98,:155,:164 allocate + upload */
int   seera_upload(void *dev, const void *host, size_t n_bytes);      /* upload into an existing buffer  */
/* A second stream for transfers that overlap the compute stream (next batch in, previous loss out, while a step
 * runs).  Host memory must be page-locked (seera_host_alloc_pinned).  The two fences order "everything queued so
 * far" on one stream before everything queued later on the other.  Not usable while a graph is being captured.
 * No counterpart in the reference, which copies synchronously on the default stream (cuda_bindings.cpp:98-170). */
/* Batch normalisation on the device for x[N, C, S] (S = H*W; 1 for the 1-D layer).  The reference computes this layer
 * on the host even in its GPU path (Seera_init.py:870-921, Seera_Engine.py:381-415, engine/src/batchnorm_ops.cpp:12-138);
 * same arithmetic: per-channel mean, biased variance from the differences to that mean, std_inv = 1/sqrt(var + eps),
 * y = gamma * x_hat + beta; training != 0 also moves running_mean / running_var by `momentum`, training == 0
 * normalises with them.  mean_out and std_inv_out (C floats each) are what the backward needs; x_hat is recomputed
 * there from x.  Backward: dgamma = sum dy * x_hat, dbeta = sum dy,
 * dx = (1/M) * std_inv * (M * dxh - sum dxh - x_hat * sum dxh * x_hat) with dxh = dy * gamma, M = N * S. */
int   seera_batchnorm_fwd(const float *x, const float *gamma, const float *beta, float *running_mean, float *running_var, float *y,
                          float *mean_out, float *std_inv_out, int N, int C, int S, float momentum, float eps, int training);
int   seera_batchnorm_bwd(const float *dy, const float *x, const float *mean, const float *std_inv, const float *gamma, float *dx,
                          float *dgamma, float *dbeta, int N, int C, int S);
/* The same over the shards of ALL ranks of the data-parallel communicator (seera_dp_init; with one rank or none they are the
 * calls above).  Forward: every rank's per-channel moments (count, mean, sum of squared differences) travel in one small sum over
 * the ranks and are merged in rank order, so every rank normalises with the statistics of the joined batch and moves its running
 * statistics by them.  Backward: the two sums of the dx formula and the element count are summed over the ranks first; dgamma /
 * dbeta stay the rank's own sums, which the gradient exchange averages like every other parameter gradient.  A sharded step
 * then equals the step on the joined batch.  The collectives run on the compute stream and can be recorded into a graph.
 * No counterpart in the reference (it has neither a device BatchNorm nor a multi-GPU path). */
int   seera_batchnorm_fwd_sync(const float *x, const float *gamma, const float *beta, float *running_mean, float *running_var, float *y,
                               float *mean_out, float *std_inv_out, int N, int C, int S, float momentum, float eps, int training);
int   seera_batchnorm_bwd_sync(const float *dy, const float *x, const float *mean, const float *std_inv, const float *gamma, float *dx,
                               float *dgamma, float *dbeta, int N, int C, int S);
/* Concatenation of two tensors along axis 1 ([N, n1] and [N, n2] rows, n = C*H*W of each sample) and the backward
 * split of the joined gradient, one launch each.  Replaces the per-sample cudaMemcpy loops of cuten.concatenate2D /
 * concatenate1D and their backward forms (cuTen.py:688-796, used by Seera_init.py:764-779, Seera_Engine.py:418-429). */
int   seera_concat_fwd(const float *a, const float *b, float *out, int N, int n1, int n2);
int   seera_concat_bwd(const float *dout, float *da, float *db, int N, int n1, int n2);
/* One-hot rows on the device: out[i, c] = (labels[i] == c) as float, n x classes.  Lets a training loop upload 4 bytes
 * of label per sample instead of a one-hot row (Sequential.fit of the reference takes host one-hot arrays and uploads
 * them batch by batch, Seera.py:748-755). */
int   seera_onehot_f32(const int *labels, float *out, int n, int classes);
/* Measurement aid: occupies the compute stream for about `microseconds` (0..100000) with a one-thread kernel, so that
 * work enqueued right after it queues up and runs back to back (used before a per-kernel event pass). */
int   seera_stream_delay(int microseconds);
int   seera_copy_upload(void *dev, const void *pinned_host, size_t n_bytes);
int   seera_copy_download(void *pinned_host, const void *dev, size_t n_bytes);
int   seera_copy_wait_compute(void);     /* later copy-stream work waits for the compute stream's current tail */
int   seera_compute_wait_copy(void);     /* later compute-stream work waits for the copy stream's current tail */
int   seera_copy_synchronize(void);      /* host waits for the copy stream                                    */
int   seera_to_host(void *host, const void *dev, size_t n_bytes);     /* :107,:123,:139 download + sync  */

/* ---- unary ops: out = f(x), grad = f'(x)   (seera_engine_cuda.hpp:9-25) -------------------- */
int seera_cuda_relu_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_sigmoid_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_tanh_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_log_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_exp_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_abs_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_sqrt_fwd(const float *x, float *out, float *grad, int size);
int seera_cuda_pow_fwd(const float *x, float exponent, float *out, float *grad, int size);
int seera_cuda_clip_fwd(const float *x, float lo, float hi, float *out, float *grad, int size);

/* ---- softmax over the last axis (seera_engine_cuda.hpp:27-29) ------------------------------ */
int seera_cuda_softmax_fwd(const float *x, float *out, int N, int C);
int seera_cuda_softmax_vjp(const float *s, const float *dout, float *dx, int N, int C);

/* ---- GEMM (seera_engine_cuda.hpp:40-44) ------------------------------------------------------
 * cuda_matmul:      C[b,M,N] = A[b,M,K] * B[K,N]           (B shared by all batches)
 * cuda_matmul_bwd:  dA[b,M,K] = dC[b,M,N] * B^T ;  dB[K,N] = sum_b A[b]^T * dC[b]            */
int seera_cuda_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch);
int seera_cuda_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB,
                          int M, int N, int K, int Nbatch);
int seera_cuda_transpose_2d(const float *in, float *out, int rows, int cols);
int seera_cuda_transpose_3d(const float *in, float *out, int Nbatch, int M, int K);

/* ---- Conv2D (seera_engine_cuda.hpp:31-38)  X[N,C,H,W], W[F,C,R,S], Y[N,F,OH,OW] --------------
 * note the argument order: fwd takes pad before stride, bwd takes stride before pad.          */
int seera_cuda_conv2d_fwd(const float *image, const float *kernel, float *out,
                          int batchN, int C, int H, int W, int F, int R, int S,
                          int pad_h, int pad_w, int stride_h, int stride_w);
int seera_cuda_conv2d_bwd(const float *W, const float *X, const float *dY, float *dX, float *dW,
                          int batch, int C, int H, int W_in, int F, int R, int S,
                          int strideh, int stridew, int padh, int padw);

/* ---- ConvTranspose2D (seera_engine_cuda.hpp:45-53)  X[N,Cin,H,W], W[Cin,Cout,KH,KW] ----------
 * Hout = (H-1)*stride - 2*pad + KH                                                             */
int seera_cuda_conv2DTranpose_fwd(const float *X, const float *W, float *out, int batch,
                                  int Cin, int Hin, int Win, int Cout, int KH, int KW,
                                  int strideh, int stridew, int padh, int padw);
int seera_cuda_conv2DTranspose_bwd(const float *W, const float *X, const float *dY, float *dX, float *dW,
                                   int batch, int Cin, int Hin, int Win, int Cout, int KH, int KW,
                                   int strideh, int stridew, int padh, int padw);

/* ---- pooling (seera_engine_cuda.hpp:55-71) ---------------------------------------------------- */
int seera_cuda_maxpool_fwd(const float *image, float *out, int *mask, int batchN, int C, int H, int W,
                           int R, int S, int pad_h, int pad_w, int stride_h, int stride_w);
int seera_cuda_maxpool_bwd(const float *dout, const int *mask, float *dX, int batchN, int C, int H, int W,
                           int R, int S, int pad_h, int pad_w, int stride_h, int stride_w);
int seera_cuda_unpooling_fwd(const float *inp, float *out, int batchN, int C, int H, int W, int sh, int sw);
int seera_cuda_unpooling_bwd(const float *dout, float *dx, int batchN, int C, int H, int W, int sh, int sw);

/* ---- single-axis reductions (seera_engine_cuda.hpp:72-95); dimarr is a HOST array of ndims ints -- */
int seera_cuda_sum_fwd(const float *A, float *out, int ndims, int dim, const int *dimarr);
int seera_cuda_mean_fwd(const float *A, float *out, int ndims, int dim, const int *dimarr);
int seera_cuda_max_fwd(const float *A, float *out, int ndims, int dim, const int *dimarr);
int seera_cuda_min_fwd(const float *A, float *out, int ndims, int dim, const int *dimarr);
int seera_cuda_argmax_fwd(const float *A, int *out, int ndims, int dim, const int *dimarr);
int seera_cuda_argmin_fwd(const float *A, int *out, int ndims, int dim, const int *dimarr);
int seera_cuda_sum_bwd(const float *dOut, float *dA, int ndims, int dim, const int *dimarr);
int seera_cuda_mean_bwd(const float *dOut, float *dA, int ndims, int dim, const int *dimarr);
int seera_cuda_max_bwd(const float *dOut, const float *fwdInput, const float *fwdOutput, float *dA,
                       int ndims, int dim, const int *dimarr);   /* adds into dA (caller zero-fills) */
int seera_cuda_min_bwd(const float *dOut, const float *fwdInput, const float *fwdOutput, float *dA,
                       int ndims, int dim, const int *dimarr);

/* ---- in-place scalar ops and fills (seera_engine_cuda.hpp:97-108) ------------------------------- */
int seera_cuda_scaler_multiply_f(float *arr, float k, int total_elements);
int seera_cuda_scaler_add_f(float *arr, float k, int total_elements);
int seera_cuda_scaler_power_f(float *arr, float k, int total_elements);
int seera_cuda_ones_f(float *arr, int total_elements);
int seera_cuda_zeros_f(float *arr, int total_elements);

/* ---- flat binary ops (seera_engine_cuda.hpp:110-116) --------------------------------------------- */
int seera_cuda_elemadd_gputogpu(const float *A, const float *B, float *C, int size);
int seera_cuda_elemmult_gputogpu(const float *A, const float *B, float *C, int size);
int seera_cuda_elemsub_gputogpu(const float *A, const float *B, float *C, int size);
int seera_cuda_elemdiv_gputogpu(const float *A, const float *B, float *C, int size);

/* ---- NumPy-rule broadcast of two <=4-D tensors (seera_engine_cuda.hpp:119-127) -------------------- */
int seera_broadcast_add_4d(const float *A, const float *B, float *C, int aN, int aC, int aH, int aW,
                           int bN, int bC, int bH, int bW);
int seera_broadcast_mul_4d(const float *A, const float *B, float *C, int aN, int aC, int aH, int aW,
                           int bN, int bC, int bH, int bW);

/* =====================================================================================================
 * Additive entry points.  The reference composes these steps from several calls above (bias add +
 * activation, activation gradient, bias gradient, the optimizers); here each is one pass over HBM.
 * ===================================================================================================== */
enum { SEERA_ACT_NONE = 0, SEERA_ACT_RELU = 1, SEERA_ACT_SIGMOID = 2, SEERA_ACT_TANH = 3 };

/* y = act(z + bias[channel]); element i belongs to channel (i / inner) % channels.
 * Replaces broadcast_add_4d + cuda_*_fwd (Seera.py:136-137, :255-258). In place allowed (y == z). */
int seera_bias_act_fwd(const float *z, const float *bias, float *y, int size, int channels, int inner, int act);
/* Forward products with the bias and activation applied before the one store of the output:
 *   C   = act(A[M,K] * B[K,N] + bias[n])                       (Dense.forward, Seera.py:133-138)
 *   out = act(conv2d(image, kernel) + bias[f])                 (Conv2D.forward, Seera.py:235-259)
 *   out = act(conv2DTranspose(X, W) + bias[cout])              (ConvTranspose2D.forward, Seera.py:398-423)
 * Arguments as cuda_matmul / cuda_conv2d_fwd / cuda_conv2DTranpose_fwd plus bias (may be NULL) and a SEERA_ACT_*
 * code.  Same values as the product followed by seera_bias_act_fwd in place. */
int seera_matmul_bias_act_fwd(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int act);
int seera_conv2d_bias_act_fwd(const float *image, const float *kernel, const float *bias, float *out, int batchN, int C, int H, int W,
                              int F, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w, int act);
int seera_conv2DTranspose_bias_act_fwd(const float *X, const float *W, const float *bias, float *out, int batch, int Cin, int Hin,
                                       int Win, int Cout, int KH, int KW, int strideh, int stridew, int padh, int padw, int act);
/* Channels-last bf16 copies of one NCHW activation tensor, as the tensor-core convolutions read them.  A forward call
 * can hand the copies of its input to the matching backward call instead of producing them twice.  Opaque; owned
 * by the caller once returned; release with seera_shadow_free (stream-ordered, NULL allowed).
 * No counterpart in the reference, whose convolutions re-run im2col in every call
 * (engine_cuda/src/convolution.cu:15-453). */
typedef struct seera_shadow seera_shadow_t;
void seera_shadow_free(seera_shadow_t *s);
/* The same for Dense layers: row-major 16-bit copies of one [rows, cols] matrix (a layer's input, its weight matrix, or
 * its output).  Opaque; owned by the caller once returned; release with seera_rows_free (stream-ordered, NULL allowed).
 * No counterpart in the reference, whose cuda_matmul_bwd transposes both operands through HBM on every call
 * (engine_cuda/src/GEMM.cu:164-225). */
typedef struct seera_rows seera_rows_t;
void seera_rows_free(seera_rows_t *r);
/* seera_conv2d_bias_act_fwd with kept copies: x_in (may be NULL) are copies of `image` from an earlier call;
 * *x_keep (x_keep may be NULL) receives the copies this call produced, or NULL when it produced none (x_in was
 * used, or the shape does not run on copies: exact-fp32 mode, short patches, unsupported geometry). */
int seera_conv2d_bias_act_fwd_s(const float *image, const float *kernel, const float *bias, float *out, int batchN, int C, int H,
                                int W, int F, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w, int act,
                                seera_shadow_t *x_in, seera_shadow_t **x_keep);
/* cuda_maxpool_fwd for a 2x2 window, stride 2, no padding, even H and W, which also returns the channels-last
 * copies of its OUTPUT in *out_shadow for the convolution that consumes it (pass them as x_in).  Same values
 * and mask as cuda_maxpool_fwd.  *out_shadow is NULL when no copies were made (exact-fp32 mode). */
int seera_maxpool2x2_fwd_s(const float *X, float *out, int *mask, int N, int C, int H, int W, seera_shadow_t **out_shadow);
/* Convolution + bias + activation + the 2x2 / stride-2 max-pool of the result in ONE launch: the tensor-core epilogue
 * reduces each window with warp shuffles and stores only `pooled` [N,F,OH/2,OW/2], the pool's `mask` (as
 * cuda_maxpool_fwd) and, when pooled_copies is non-NULL, the channels-last copies of `pooled` for the next convolution.
 * The full-resolution layer output never reaches HBM; seera_conv2d_act_bwd accepts y == NULL when it is given gp, the
 * mask and y_pooled.  Values and mask equal seera_conv2d_bias_act_fwd followed by cuda_maxpool_fwd bit for bit.
 * Available when seera_conv2d_pool_fusable(...) returns 1 (tensor-core modes; even OH and OW; OW in {2,4,8,16}; with
 * the option "pool_short_patch" also short patches C*R*S <= 64 with at most 128 filters); otherwise SEERA_E_LIMIT.  Replaces Conv2D.forward +
 * MaxPool2D.forward of the reference (Seera.py:235-259, :471-480). */
int seera_conv2d_pool_fusable(int batchN, int C, int H, int W, int F, int R, int S, int stride_h, int stride_w, int pad_h, int pad_w);
int seera_conv2d_bias_act_pool_fwd_s(const float *image, const float *kernel, const float *bias, float *pooled, int *mask, int batchN,
                                     int C, int H, int W, int F, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w, int act,
                                     seera_shadow_t *x_in, seera_shadow_t **x_keep, seera_shadow_t **pooled_copies);
/* Backward of y = act(conv2d(X, W) + bias) in one call (Conv2D backward: Seera_Engine.py:571-583 activation,
 * :43-65 bias, :67-115 convolution; with gp also MaxPool2D backward, :117-131).  The gradient arrives either
 * as g = dL/dy [N,F,OH,OW] or as gp = dL/d(maxpool2x2(y)) [N,F,OH/2,OW/2] with that pool's mask from
 * cuda_maxpool_fwd (window 2x2, stride 2, no padding); exactly one of g / gp is non-NULL.  Produces dX (may be
 * NULL), dW and dbias (may be NULL).  dz = dy * act'(y) goes straight into the bf16 copies the tensor-core
 * kernels read and is never stored in fp32; shapes those kernels do not serve run as the separate entries.
 * y_pooled (with gp; may be NULL): that pool's output.  It equals y at each window's argmax, the only pixel of the
 * window with a non-zero dz, so the activation slope is taken from it and y (four times larger) is not read.
 * x_shadow: kept copies of X from the forward call, or NULL. */
int seera_conv2d_act_bwd(const float *W, const float *X, const float *y, const float *g, const float *gp, const int *pool_mask,
                         const float *y_pooled, float *dX, float *dW, float *dbias, int batch, int C, int H, int W_in, int F, int R, int S,
                         int strideh, int stridew, int padh, int padw, int act, seera_shadow_t *x_shadow);
/* dz = dy * act'(y), with the derivative written in terms of the OUTPUT y (relu: y > 0; sigmoid:
 * y(1-y); tanh: 1-y^2), and dbias[c] = sum of dz over that channel.  Replaces cuda_elemmult with the
 * stored local gradient plus broadcast_mul_4d + three cuda_sum_fwd (Seera_Engine.py:571-583, :43-65). */
int seera_act_bias_bwd(const float *dy, const float *y, float *dz, float *dbias,
                       int size, int channels, int inner, int act);
/* A Dense layer as two calls that convert nothing twice (tensor-core modes; in mode 0 they compose the plain entries).
 * Forward: C = act(A B + bias) (Seera.py:133-138).  `a_in` (may be NULL): copies of A made by the layer before;
 * `*a_keep`, `*w_keep` (may be NULL pointers): the copies of A and of B this call made, for the backward call;
 * `*c_copies` (may be a NULL pointer): copies of C written by the same epilogue that stores C, for the next Dense layer.
 * Backward of that layer (replaces Seera_Engine.py:571-583 + GEMM.cu:164-225): dz = g * act'(y) is formed straight into
 * 16-bit copies together with dbias (no fp32 dz, no separate conversion of it), then dA = dz B^T and dB = A^T dz read
 * those and the kept copies.  dA, dB or dbias may be NULL.  In the fp16 modes the gradient copies use the dynamic
 * factor of the current backward pass (seera_grad_scale_update on the loss gradient). */
int seera_matmul_bias_act_fwd_s(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int act,
                                seera_rows_t *a_in, seera_rows_t **a_keep, seera_rows_t **w_keep, seera_rows_t **c_copies);
int seera_matmul_act_bwd(const float *A, const float *B, const float *y, const float *g, float *dA, float *dB,
                         float *dbias, int M, int N, int K, int act, seera_rows_t *a_keep, seera_rows_t *w_keep);
/* seera_act_bias_bwd for callers that must not allocate.  No counterpart in the reference.
 * Some hosts of this library cannot let a call reach cudaMalloc: code that runs between fixed memory budgets
 * (an inference server or a plugin that was handed its device memory up front), code on a latency path where a
 * pool miss would stall on the driver's allocator, and code that has already begun recording work it will
 * replay.  The regular entry takes its partial-sum scratch from the pool; this one uses a fixed 256 KiB device
 * array built into the library (present on every GPU that loads it, until exit) and never calls cudaMalloc,
 * cudaFree or the pool.  Same arguments and results as seera_act_bias_bwd, with these limits:
 *   - channels <= 65536 (the array holds one partial sum per channel and split); more -> SEERA_E_LIMIT.
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call before any stream capture begins.
 *   - all calls share the one array: two calls whose kernels overlap on the GPU (different streams or
 *     processes sharing a context) race on it.  Calls on this library's single stream are ordered and safe.
 *   - the array keeps the last call's partial sums; every element a call reads it has written first. */
int seera_act_bias_bwd_noalloc(const float *dy, const float *y, float *dz, float *dbias,
                               int size, int channels, int inner, int act);
/* Softmax + categorical cross-entropy: the reference's chain softmax -> clip(eps, 1-eps) -> log ->
 * (-y * .) -> sum(-1) -> mean (Seera.py:955-969) and its backward (Seera_Engine.py:352-379, :571-583)
 * evaluated row by row.  Writes p = softmax(z), loss_rows[n] = -sum_c y*log(clip(p)),
 * *loss_mean = inv_count * sum_n loss_rows[n] (summed in index order), and
 * dz = d(inv_count * sum_n loss_rows[n]) / dz.  inv_count is 1/N for a single process and
 * 1/(global batch) when the batch is sharded over ranks. */
int seera_softmax_cce_fwd_bwd(const float *z, const float *onehot, float *p, float *loss_rows,
                              float *loss_mean, float *dz, int N, int C, float eps, float inv_count);
/* Mean-squared error (Seera.py:943-945): *loss_mean = inv_count * sum (p-y)^2 (deterministic two-stage
 * sum; `partials` is caller scratch of seera_mse_partials(size) floats), dp = 2 (p-y) * inv_count. */
int seera_mse_partials(int size);
int seera_mse_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp,
                      int size, float inv_count);
/* Mean absolute error (Seera.py:947-949; the gradient of |d| is sign(d) with 0 at 0, as abs_fwd of
 * engine/src/activation_ops.cpp:50-56) and binary cross-entropy -y log(p+eps) - (1-y) log(1-p+eps)
 * (Seera.py:951-953), same calling convention and scratch as seera_mse_fwd_bwd. */
int seera_mae_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp,
                      int size, float inv_count);
int seera_bce_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp,
                      int size, float inv_count, float eps);

/* Dynamic factor of the fp16 gradient copies of precision modes 4 and 5.  Gradients have no fixed magnitude - they
 * shrink by orders of magnitude as training converges - so a loss head calls this on the gradient it hands to the
 * backward pass (n floats at g): two small launches find its largest |entry| and set a power-of-two factor, kept in
 * device memory, under which that entry lands in [128, 256) after the static 2^12 of the gradient class.  Every
 * gradient copy made until the next call uses it and every product's epilogue takes it out again (exactly).
 * Stream-ordered and capturable; in the other modes the factor is never read.  Without any call it is 1.
 * The entries that are handed an fp32 gradient tensor (seera_cuda_matmul_bwd, seera_cuda_conv2d_bwd,
 * seera_cuda_conv2DTranspose_bwd) call it on that tensor themselves; a caller of the fused layer-backward entries
 * (seera_conv2d_act_bwd with a pooled gradient) calls it once per backward pass on the loss gradient.
 * No counterpart in the reference. */
int seera_grad_scale_update(const float *g, long long n);

/* Adam (Seera.py:1069-1084) and SGD with momentum (Seera.py:1006-1008) in one pass, in place.
 * The caller passes the fp32-rounded scalars omb1 = 1-beta1, omb2 = 1-beta2, c1 = 1-beta1^t,
 * c2 = 1-beta2^t; g is multiplied by grad_scale first (1/world for data-parallel averaging). */
int seera_adam_step(float *w, const float *g, float *m, float *v, int n, float lr, float beta1, float omb1,
                    float beta2, float omb2, float eps, float c1, float c2, float grad_scale);
int seera_sgd_step(float *w, const float *g, float *vel, int n, float lr, float momentum, float grad_scale);
/* The same updates with the scalars read from DEVICE memory at run time, so a captured graph can be replayed
 * with a new step count: hyper = {lr, beta1, 1-beta1, beta2, 1-beta2, eps, 1-beta1^t, 1-beta2^t, grad_scale}
 * for Adam, {lr, momentum, grad_scale} for SGD. */
int seera_adam_step_dev(float *w, const float *g, float *m, float *v, int n, const float *hyper);
int seera_sgd_step_dev(float *w, const float *g, float *vel, int n, const float *hyper);

/* ---- data parallel: the gradient exchange of a batch sharded over the GPUs of one node -----------------------------
 * No counterpart in the reference (single GPU only).  One process per GPU; every rank holds the same weights and
 * trains its shard; the weight-gradient arena is summed over the ranks with NCCL over NVLink / NVSwitch and the
 * optimizer divides by the world size (grad_scale).  NCCL is opened with dlopen by seera_dp_init: a single-GPU
 * caller never loads it.
 *   seera_dp_unique_id   rank 0 makes the communicator id (seera_dp_unique_id_bytes() bytes) and hands it to the
 *                        other ranks by any means (a file, a socket, the launcher's store)
 *   seera_dp_init        joins the communicator on the device chosen by seera_init; collective over the ranks
 *   seera_dp_alloc/free  device memory the collectives use in place (ncclMemAlloc, registered with the
 *                        communicator: no staging copy, in-switch reduction where NVSwitch offers it); zeroed
 *   seera_dp_allreduce   in-place sum (op 0), max (1) or min (2) of n floats on the COMPUTE stream
 *   seera_dp_broadcast   in-place broadcast from `root` on the compute stream
 *   seera_dp_reduce_range  in-place sum of floats [begin, end) of `arena` on the engine's COMMUNICATION stream,
 *                        ordered after everything the compute stream holds so far; returns at once, so the
 *                        backward kernels of earlier layers overlap the exchange
 *   seera_dp_join        the compute stream waits for every range enqueued since the last join
 *   seera_dp_side_begin / _end   between the two, every launch of this library goes to the communication stream, behind the
 *                        sums enqueued there and behind what the compute stream held at the call; meant for the optimizer's
 *                        update of a bucket right behind that bucket's sum (entries that take pool scratch must not run
 *                        there).  seera_dp_join covers these launches too and ends a window left open.
 *                        (reduce_range and join are event edges: a step recorded with seera_graph_begin/end
 *                        carries its collectives inside the one graph)
 *   seera_dp_poll        NCCL's asynchronous error state as a status
 *   seera_dp_wait_host   host-side wait for both streams with a deadline in milliseconds (< 0: none); on expiry
 *                        or on an NCCL error the communicator is aborted and an error status returned - a peer
 *                        that left becomes a status code on the host, never a wait inside a kernel
 *   seera_dp_abort       drops the communicator without talking to the peers (one of them is known to be gone)
 *   seera_dp_finalize    destroys the communicator and frees seera_dp_alloc blocks still held */
int   seera_dp_unique_id_bytes(void);
int   seera_dp_unique_id(void *out, int size);
int   seera_dp_init(int rank, int world, const void *unique_id, int size);
int   seera_dp_rank(void);
int   seera_dp_world(void);
int   seera_dp_nccl_version(void);
void *seera_dp_alloc(size_t bytes);
int   seera_dp_free(void *p);
int   seera_dp_allreduce(float *buf, long long n, int op);
int   seera_dp_broadcast(float *buf, long long n, int root);
int   seera_dp_reduce_range(float *arena, long long begin, long long end);
int   seera_dp_join(void);
int   seera_dp_side_begin(void);
int   seera_dp_side_end(void);
int   seera_dp_poll(void);
int   seera_dp_wait_host(int timeout_ms);
int   seera_dp_abort(void);
int   seera_dp_finalize(void);

#ifdef __cplusplus
}
#endif
#endif /* SEERA_B200_H */
