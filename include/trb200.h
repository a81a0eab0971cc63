/*
 * trb200.h -- C ABI of the B200 (sm_100a) kernels for the Renaissance training
 * backward hot path: Conv+BN+ReLU block backward, fused softmax-cross-entropy,
 * and the small kernels either side of the gradient all-reduce.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".
 *   - Activations are NHWC, filters are KRSC, both compact (the reference's
 *     DTensor strides for every shape whose channel count is a multiple of 8,
 *     include/renaissance/tensor/distributed_tensor.h:173-207).  Half tensors
 *     are IEEE binary16.
 *   - `stream` / `event` arguments are a cudaStream_t / cudaEvent_t passed as
 *     void*; NULL stream = the legacy default stream.
 *   - Functions only enqueue work.  They never synchronise, never allocate and
 *     never free: scratch memory is a caller-owned workspace whose size the
 *     matching *_workspace_bytes() function returns (the reference's
 *     DeviceContext::ensure_workspace_grow contract,
 *     src/backend/device_context.cpp:379-428), so they can be called inside
 *     stream capture.
 *   - Return value: 0 on success, a negative trb200_status otherwise; the text
 *     of the last failure on the calling thread is trb200_last_error().  The C
 *     side never throws.  The reference's convention is exceptions
 *     (TR_DEVICE_ERROR, include/renaissance/core/tr_exception.h:271); the
 *     plugin adapter turns a non-zero return into one.
 */
#ifndef TRB200_H_
#define TRB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum trb200_status {
    TRB200_OK = 0,
    TRB200_ERR_INVALID_ARGUMENT = -1,  /* null pointer, bad size, misaligned pointer */
    TRB200_ERR_UNSUPPORTED = -2,       /* shape outside what the kernels cover */
    TRB200_ERR_WORKSPACE = -3,         /* workspace missing or too small */
    TRB200_ERR_CUDA = -4,              /* a CUDA runtime / driver call failed */
    TRB200_ERR_DEVICE_TIMEOUT = -5     /* a bounded device-side wait gave up */
} trb200_status;

/* Text of the last error on this thread ("" if none).  Host pointer, valid until
 * the next failing call on the same thread. */
const char* trb200_last_error(void);

/* Library version, major*10000 + minor*100 + patch. */
int trb200_version(void);

/* Number of kernels this library has launched in this process so far. */
uint64_t trb200_kernel_launch_count(void);

/* Compute capability (major*10 + minor) of the current device, or a negative
 * trb200_status.  The tensor-core kernels need 100. */
int trb200_device_arch(void);

/* ------------------------------------------------------------------------- */
/* Convolution geometry shared by the conv entry points.                      */
/* ------------------------------------------------------------------------- */
/* Storage type of the 16-bit tensors (activations, filters, their gradients).
 * Arithmetic is float for both.  Half is the reference's AMP type (DType::FP16);
 * bfloat16 is what its ResNet-50 configuration names and the reference has no
 * backend for. */
#define TRB200_DTYPE_F16 0
#define TRB200_DTYPE_BF16 1

typedef struct trb200_conv_desc {
    int32_t n, h, w, c;          /* input activation X  [n,h,w,c]            */
    int32_t k, r, s;             /* filters W           [k,r,s,c]            */
    int32_t pad_h, pad_w;
    int32_t stride_h, stride_w;
    int32_t dtype;               /* TRB200_DTYPE_*; 0 (half) when zero-initialised */
} trb200_conv_desc;              /* output Y / dY is [n,oh,ow,k], oh = (h+2*pad_h-r)/stride_h+1 */

/* ------------------------------------------------------------------------- */
/* BN + ReLU backward of the fused block.                                     */
/* Replaces the cuDNN-FE graph MUL(dY, mask) -> batchnorm_backward built by   */
/* build_cbr_bn_bwd_fused_graph, src/backend/ops/dtensor/cbr_op.cpp:1259-1353 */
/* (executed at cbr_op.cpp:1371-1429).                                        */
/*   dy_m   = dY * mask                      (mask: 1 bit / element, LSB first, */
/*                                            flat NHWC index)                */
/*   dbeta  = sum_m dy_m        dgamma = sum_m dy_m * (x - mean) * inv_std    */
/*   dconv  = gamma*inv_std*(dy_m - dbeta/m - xhat*dgamma/m)   -> half        */
/* m = n*h*w rows, c channels, c % 8 == 0.  dconv may be NULL (sums only) and */
/* may alias neither input.  Sums are fixed-order (bitwise reproducible).     */
/* mask_bits may be NULL: a BN with no ReLU behind it (a residual block's     */
/* shortcut BN), i.e. the plain batch-norm backward, bn_op.cpp:119-168.       */
/* ------------------------------------------------------------------------- */
size_t trb200_bnrelu_bwd_workspace_bytes(int64_t m, int32_t c);
int trb200_bnrelu_bwd(const void* dy, const void* mask_bits, const void* x,
                      const float* gamma, const float* saved_mean, const float* saved_inv_std,
                      void* dconv, float* dgamma, float* dbeta,
                      int64_t m, int32_t c,
                      void* workspace, size_t workspace_bytes, void* stream);
/* The same with the storage type of dy, x and dconv given (TRB200_DTYPE_*). */
int trb200_bnrelu_bwd_dtype(const void* dy, const void* mask_bits, const void* x,
                            const float* gamma, const float* saved_mean, const float* saved_inv_std,
                            void* dconv, float* dgamma, float* dbeta,
                            int64_t m, int32_t c, int32_t dtype,
                            void* workspace, size_t workspace_bytes, void* stream);

/* The same operator for callers that cannot allocate device memory (a runtime
 * whose memory plan is frozen, a plugin running inside someone else's capture, a
 * process that gave the whole GPU to its own arena).  It has no counterpart in the
 * reference.  Instead of a workspace it uses a fixed 4 MiB array inside the library
 * image (held by every GPU that loads the library until the process exits) and it
 * calls no cudaMalloc, cudaFree or other allocating routine.
 *   - Limit: c <= 4096 (and c % 8 == 0); anything larger is rejected with
 *     TRB200_ERR_UNSUPPORTED.  m is not limited.
 *   - Narrower than trb200_bnrelu_bwd in two ways: half tensors only (there is no
 *     dtype argument, bfloat16 callers use trb200_bnrelu_bwd_dtype with a workspace),
 *     and mask_bits is required (NULL is rejected with TRB200_ERR_INVALID_ARGUMENT;
 *     the BN without a ReLU behind it is served by the workspace entry point only).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before
 *     any stream capture begins.
 *   - All calls on a device share the array: calls whose kernels can overlap on the
 *     GPU (different streams without ordering) race and give wrong sums.  Calls on
 *     one stream, or ordered by events, are fine; nothing has to be cleared between
 *     calls. */
int trb200_bnrelu_bwd_static(const void* dy, const void* mask_bits, const void* x,
                             const float* gamma, const float* saved_mean, const float* saved_inv_std,
                             void* dconv, float* dgamma, float* dbeta,
                             int64_t m, int32_t c, void* stream);

/* ------------------------------------------------------------------------- */
/* Convolution weight gradient, dW[k,r,s,c] = sum dY[n,oh,ow,k] * X[...]      */
/* 16-bit in (d->dtype), float accumulate, 16-bit out, fixed-order split      */
/* reduction.  3x3 pad 1 and 1x1 pad 0 at stride 1 or 2 with c and k          */
/* multiples of 64 (k = 64, 128 or a multiple of 256), and half 3x3 stride 1  */
/* with c = 4, run on the tcgen05 kernels (stride 2 through tensor maps that   */
/* step two pixels); every other geometry on the direct kernels.              */
/* Replaces build_cbr_conv_amp_wgrad_graph + execute,                         */
/* src/backend/ops/dtensor/cbr_op.cpp:763-840, 1431-1468.                     */
/* ------------------------------------------------------------------------- */
size_t trb200_conv_wgrad_workspace_bytes(const trb200_conv_desc* d);
int trb200_conv_wgrad(const trb200_conv_desc* d, const void* dy, const void* x, void* dw,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Convolution data gradient, dX[n,ih,iw,c] = sum dY[...] * W[k,r,s,c]        */
/* 16-bit in (d->dtype), float accumulate, 16-bit out.  dx must not alias dy  */
/* or w (it may be the buffer that held X: the reference writes dX in place   */
/* over X).  Tensor-core coverage as for the weight gradient, with c = 64,    */
/* 128 or a multiple of 256.                                                  */
/* Replaces build_cbr_conv_amp_dgrad_graph + execute,                         */
/* src/backend/ops/dtensor/cbr_op.cpp:842-917, 1470-1508.                     */
/* ------------------------------------------------------------------------- */
size_t trb200_conv_dgrad_workspace_bytes(const trb200_conv_desc* d);
int trb200_conv_dgrad(const trb200_conv_desc* d, const void* dy, const void* w, void* dx,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Forward convolution Y = X (*) W, 16-bit in (d->dtype), float accumulate, 16-bit
 * out, on the same tensor-core kernel as dgrad (3x3 pad 1 or 1x1 pad 0 at stride 1
 * or 2, k = 64, 128 or a multiple of 256, c % 64 == 0, or half 3x3 stride 1 with
 * c == 4; anything else returns TRB200_ERR_UNSUPPORTED).
 * With c == 4 (the padded first layer) the workspace receives the 3x3
 * neighbourhoods of every pixel, n*h*w*128 bytes: any activation-sized buffer that
 * is free at that point will do (the block's relu-output buffer, say).
 * Counterpart of the conv_fprop part of the reference's forward block,
 * src/backend/ops/dtensor/cbr_op.cpp:622-718 (statistics not included). */
size_t trb200_conv_fprop_workspace_bytes(const trb200_conv_desc* d);
int trb200_conv_fprop(const trb200_conv_desc* d, const void* x, const void* w, void* y,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Forward convolution with the batch statistics taken in its epilogue, followed by
 * bn_finalize: the reference's conv_fprop + genstats graph and its bn_finalize graph
 * (cbr_op.cpp:622-718, 430-528) in two launches, without a separate pass over the
 * conv output.  Outputs and optional pointers as in trb200_bn_stats_finalize; the
 * statistics are those of the stored (half) output.  Shapes: what the tensor-core
 * kernels run at stride 1, and 3x3 pad 1 / 1x1 pad 0 at stride 2 with c a multiple
 * of 64 and k = 64, 128 or a multiple of 256. */
size_t trb200_conv_fprop_bn_stats_workspace_bytes(const trb200_conv_desc* d);
int trb200_conv_fprop_bn_stats(const trb200_conv_desc* d, const void* x, const void* w, void* y,
                               const float* gamma, const float* beta, float eps, float momentum,
                               float* ch_sum, float* ch_sqsum, float* saved_mean, float* saved_inv_std,
                               float* eq_scale, float* eq_bias, float* running_mean, float* running_var,
                               void* workspace, size_t workspace_bytes, void* stream);

/* Diagnostics.  backend 0 = automatic (tensor cores where the shape allows),
 * 1 = direct CUDA-core kernels only (used by tests to cross-check the two). */
int trb200_set_conv_backend(int backend);

/* Synchronous: reads the device-side status word.  TRB200_OK, or
 * TRB200_ERR_DEVICE_TIMEOUT if a kernel's bounded wait gave up since the last
 * call (the word is cleared).  Call it after synchronising, never in capture. */
int trb200_device_status(void);

/* Self-test of the bounded waits (failure detection without a fault): launches a
 * two-warp kernel in which warp 0 waits, with the library's own wait routine and a
 * limit of `limit_ns` (1 us .. 100 ms), on an mbarrier that nothing arrives on, and
 * warp 1 waits on it with the kernels' normal one-second limit.  Warp 0 gives up
 * after the limit, records a status code and raises the block's abort flag; warp 1
 * sees the flag and leaves too.  out4 (device, 4 ints) = {warp 0 got the barrier (0
 * expected), ns it waited, warp 1 got the barrier (0 expected), ns it waited}.
 * Afterwards trb200_device_status() returns TRB200_ERR_DEVICE_TIMEOUT once and the
 * context is as usable as before.  This is the path every tcgen05 kernel of the
 * library takes when a copy or an MMA it waits for never completes; it has no
 * counterpart in the reference (which waits inside cuDNN). */
int trb200_selftest_wait_timeout(uint64_t limit_ns, int32_t* out4, void* stream);

/* Which implementation the two conv entry points would pick for this shape:
 * 1 = tcgen05/TMEM implicit GEMM fed by TMA, 0 = direct CUDA-core kernel.
 * `which`: 0 = wgrad, 1 = dgrad, 2 = fprop. */
int trb200_conv_uses_tensor_cores(const trb200_conv_desc* d, int which);

/* ------------------------------------------------------------------------- */
/* Whole block backward = launch_cbr_amp_bwd_cuda / _first_layer_cuda,        */
/* src/backend/ops/dtensor/cbr_op.cpp:1359-1522 and 1528-1651: BN+ReLU        */
/* backward on stream_bn, then wgrad on stream_wgrad, then dgrad on           */
/* stream_dgrad (after wgrad: dX overwrites X), then a join back onto         */
/* stream_bn.  The three events are recorded after the respective stage (the  */
/* caller's MultiStreamCaptureState::last_done_event of each stream); on      */
/* return `ev_bn` has been re-recorded on stream_bn after the join.  All      */
/* three streams may be the same stream and the events may be NULL then.      */
/* dx == NULL selects the first-layer variant (no dgrad).                     */
/* ------------------------------------------------------------------------- */
typedef struct trb200_cbr_bwd_args {
    trb200_conv_desc conv;
    const void* dy;            /* in  [0] upstream gradient, half [n,oh,ow,k]        */
    const void* w;             /* in  [1] filters, half KRSC                        */
    const float* gamma;        /* in  [2] BN weight [k]                             */
    const float* saved_mean;   /* in  [3]                                           */
    const float* saved_inv_std;/* in  [4]                                           */
    const void* mask_bits;     /* in  [5] ReLU mask, bit-packed                     */
    const void* x;             /* in  [6] block input, half [n,h,w,c]               */
    void* dx;                  /* out [0] = buffer of x (in place) or NULL          */
    void* dw;                  /* out [1] half KRSC                                 */
    float* dgamma;             /* out [2]                                           */
    float* dbeta;              /* out [3]                                           */
    void* conv_out;            /* out [4] conv output saved by the forward: read by
                                  the BN stage                                       */
    void* bn_scratch;          /* out [5] activation-sized scratch: receives dconv  */
    void* workspace;
    size_t workspace_bytes;
    void* stream_bn;           /* COMP_1 */
    void* stream_wgrad;        /* COMP_3 */
    void* stream_dgrad;        /* COMP_2 */
    void* ev_bn;
    void* ev_wgrad;
    void* ev_dgrad;
    const void* pool_argmax;   /* optional: the block is followed by a 2x2 max pool and `dy` is the
                                  gradient of the POOLED output [n,oh/2,ow/2,k]; this is the pool's
                                  argmax tensor (trb200_maxpool2x2_fwd layout).  NULL = dy is the
                                  gradient of the block's own output, as in the reference. */
    void* ev_time[4];          /* optional (all NULL = off; never while capturing): timing events recorded
                                  before the BN stage on stream_bn and after the BN, wgrad and dgrad stages
                                  on their streams (the last one stays unrecorded in the first-layer
                                  variant), so that a caller can read each stage's device time. */
} trb200_cbr_bwd_args;

size_t trb200_cbr_bwd_workspace_bytes(const trb200_conv_desc* d, int first_layer);
int trb200_cbr_bwd(const trb200_cbr_bwd_args* a);

/* ------------------------------------------------------------------------- */
/* Softmax + cross entropy with label smoothing, AMP variant.                 */
/* `scaling`, `label_smoothing`, `inv_scaling` are device scalars as in the   */
/* reference (DTensor scalars).  Row strides are in elements.                 */
/* ------------------------------------------------------------------------- */

/* Forward node = softmax_ce_fwd_kernel<true> + softmax_ce_reduce_kernel,
 * src/backend/ops/dtensor/softmax_ce_op.cu:63-177, 372-429, 504-532 (launcher
 * softmax_ce_op.cpp:409-455): probs (fp32), loss_partial[b] (already times
 * 1/batch), *loss = fixed-order sum of the partials (not multiplied by the loss
 * scale), *inv_scaling = 1/batch.  probs may be NULL. */
int trb200_softmax_ce_fwd(const void* logits, int64_t logits_stride, const int32_t* labels,
                          const float* label_smoothing,
                          float* probs, int64_t probs_stride,
                          float* loss_partial, float* loss, float* inv_scaling,
                          int32_t batch, int32_t classes, void* stream);

/* Backward node = softmax_ce_bwd_kernel<true>, softmax_ce_op.cu:438-468, 613-627
 * (launcher softmax_ce_op.cpp:591-627):
 * d_logits = half((p - ls/C - [c==y](1-ls)) * scaling * inv_scaling). */
int trb200_softmax_ce_bwd(const float* probs, int64_t probs_stride, const int32_t* labels,
                          const float* scaling, const float* inv_scaling,
                          const float* label_smoothing,
                          void* dlogits, int64_t dlogits_stride,
                          int32_t batch, int32_t classes, void* stream);

/* Both nodes in one pass over the logits: reads each logit once, writes
 * d_logits (and probs if not NULL), loss partials, loss and inv_scaling.  The
 * arithmetic is that of the two nodes above.
 * When probs is NULL and the rows are whole 16-byte vectors of at most 32768
 * classes, the row kernel also finishes the loss (last block to end adds
 * per-block sums in block order; bitwise reproducible on a given GPU) using a
 * completion counter kept in the library.  A counter belongs to the (device,
 * stream) of the call, so calls on one stream, which run in order, never share
 * one while in flight; the 65th distinct (device, stream) pair gets none and
 * its loss is finished by the separate reduction launch instead.  A captured
 * call keeps the counter of the stream it was captured on: do not replay such
 * a graph while eager calls on that same capture stream are in flight.
 * A label outside [0, classes) matches no class (the reference reads through
 * it unchecked): nothing is read or written through it, its probability counts
 * as 0 in the loss and its row of d_logits gets no -(1 - ls) entry.  The same
 * holds for trb200_softmax_ce_fwd / _bwd. */
int trb200_softmax_ce_fused(const void* logits, int64_t logits_stride, const int32_t* labels,
                            const float* scaling, const float* label_smoothing,
                            float* probs, int64_t probs_stride,
                            void* dlogits, int64_t dlogits_stride,
                            float* loss_partial, float* loss, float* inv_scaling,
                            int32_t batch, int32_t classes, void* stream);

/* The fused call without probs for logits and d_logits of either 16-bit type
 * (TRB200_DTYPE_*).  bfloat16: rows of whole 16-byte vectors and at most 2048
 * classes (a 1000-class head), anything else returns TRB200_ERR_UNSUPPORTED;
 * half: as trb200_softmax_ce_fused with probs = NULL. */
int trb200_softmax_ce_fused_dtype(const void* logits, int64_t logits_stride, const int32_t* labels,
                                  const float* scaling, const float* label_smoothing,
                                  void* dlogits, int64_t dlogits_stride,
                                  float* loss_partial, float* loss, float* inv_scaling,
                                  int32_t batch, int32_t classes, int32_t dtype, void* stream);

/* ------------------------------------------------------------------------- */
/* Classifier: fully connected layers of the AMP step.                        */
/* FC_AMP_FWD / FC_AMP_BWD, src/backend/ops/dtensor/fc_op.cpp:259-480 (cuBLAS  */
/* GEMMs + the bias kernels of fc_op.cu:20-101), with the ReLU                 */
/* (relu_op.cu:101-126) and dropout (dropout_op.cu:50-274) that follow an FC   */
/* layer folded into the bias pass.  The GEMMs run on this library's own       */
/* tcgen05 kernel for batch-sized GEMMs, which reads x, w and dy in place;     */
/* in_features and out_features must be multiples of 8.  x [batch][in],        */
/* w [out][in], y [batch][out]: half, compact; bias and db float, as in the    */
/* reference.                                                                  */
/* ------------------------------------------------------------------------- */

/* y = x W^T (+ bias, rounded to half as fc_fwd_bias_add_amp_kernel does), then, if
 * asked, ReLU and inverted dropout: an element is dropped with probability
 * dropout_p, kept ones are scaled by 1 / (1 - dropout_p).  The random bits come
 * from Philox4x32-10 keyed by `seed`, with `offset` as the call's counter (give
 * every step and layer its own) and the element index: nothing is stored.
 * bias may be NULL (no bias).  The GEMM is split over in_features; workspace (of
 * trb200_fc_amp_workspace_bytes(), 16-byte aligned; the same size serves the
 * layer's backward) holds its float partial sums, which the bias pass adds in
 * split order. */
size_t trb200_fc_amp_workspace_bytes(int32_t batch, int32_t in_features, int32_t out_features);
int trb200_fc_amp_fwd(const void* x, const void* w, const float* bias, void* y,
                      int32_t batch, int32_t in_features, int32_t out_features,
                      int32_t relu, float dropout_p, uint64_t seed, uint64_t offset,
                      void* workspace, size_t workspace_bytes, void* stream);

/* The same with x, w and y in d-type `dtype` (TRB200_DTYPE_F16 or TRB200_DTYPE_BF16): the classifier of a bfloat16
 * network (BASELINE configuration 4; the reference has no counterpart). */
int trb200_fc_amp_fwd_dtype(const void* x, const void* w, const float* bias, void* y,
                            int32_t batch, int32_t in_features, int32_t out_features,
                            int32_t relu, float dropout_p, uint64_t seed, uint64_t offset, int32_t dtype,
                            void* workspace, size_t workspace_bytes, void* stream);

/* dz = act > 0 ? da * scale : 0 for n half elements, where `act` is the OUTPUT of
 * trb200_fc_amp_fwd with relu and/or dropout (zero exactly where the ReLU or the
 * dropout zeroed it) and scale = 1 / (1 - dropout_p).  dz may be da. */
int trb200_fc_act_bwd(const void* da, const void* act, void* dz, int64_t n, float scale, void* stream);

/* db[o] = sum_b dy[b][o] (float, rows added in a fixed order; NULL: not computed),
 * dW = dy^T x ([out][in]; half, or float when dw_float != 0: the reference's
 * FC_AMP_BWD writes float dW, fc_op.cpp:349-480), dx = dy W (half; NULL: not computed).  `act` (may
 * be NULL) is the layer's INPUT as the previous layer's trb200_fc_amp_fwd wrote it
 * with relu / dropout: dx then also carries that activation's backward,
 * dx = act > 0 ? dx * act_scale : 0 (trb200_fc_act_bwd folded in).  The three run
 * on `stream` in that order.  When the data gradient has few output tiles its GEMM
 * is split over out_features and needs the workspace of
 * trb200_fc_amp_workspace_bytes() for float partial sums (added in split order). */
int trb200_fc_amp_bwd(const void* dy, const void* w, const void* x, void* dx, void* dw, int32_t dw_float,
                      float* db, const void* act, float act_scale,
                      int32_t batch, int32_t in_features, int32_t out_features,
                      void* workspace, size_t workspace_bytes, void* stream);
/* ... with dy, w, x, dx, act (and dW unless dw_float) in d-type `dtype`. */
int trb200_fc_amp_bwd_dtype(const void* dy, const void* w, const void* x, void* dx, void* dw, int32_t dw_float,
                            float* db, const void* act, float act_scale,
                            int32_t batch, int32_t in_features, int32_t out_features, int32_t dtype,
                            void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Kernels either side of the gradient all-reduce (the collective itself is   */
/* NCCL, issued by the host side).                                            */
/* ------------------------------------------------------------------------- */

/* data[i] *= factor, tr_scale_fp32_kernel, src/backend/ops/range/infra_kernels.cu:82-96
 * (the 1/world step of launch_allreduce_cuda_impl, allreduce_op.cpp:87-95). */
int trb200_scale_f32(float* data, int64_t n, float factor, void* stream);

/* dst[i] = float(src[i]) * factor: RANGE_CAST_FP16_TO_FP32
 * (src/backend/ops/range/cast_op.cu:18-37) with the all-reduce's mean folded in. */
int trb200_cast_f16_to_f32(const void* src, float* dst, int64_t n, float factor, void* stream);

/* ------------------------------------------------------------------------- */
/* Element-wise pieces of a residual block (ResNet bottleneck) around the      */
/* block kernels.  n elements, n % 8 == 0; 16-bit tensors of `dtype`           */
/* (TRB200_DTYPE_*); masks are bit-packed like the block's ReLU mask.          */
/* ------------------------------------------------------------------------- */

/* out = a + b rounded to the 16-bit type: the join of two branches (forward)
 * or of their gradients (backward).  AXPY with alpha = 1, axpy_op.cu:30-58, on
 * 16-bit data.  out may be a or b. */
int trb200_add16(const void* a, const void* b, void* out, int64_t n, int32_t dtype, void* stream);

/* t = a + b rounded to the 16-bit type; out = max(t, 0); mask bit = t > 0: that
 * AXPY followed by relu_fwd_amp_mask_kernel, relu_op.cu:101-114.  out may be a
 * or b. */
int trb200_add_relu_mask(const void* a, const void* b, void* out, void* mask_bits, int64_t n, int32_t dtype,
                         void* stream);

/* dx = mask bit ? dy : 0, relu_bwd_amp_kernel, relu_op.cu:116-126 (either 16-bit
 * type).  dx may be dy.  The result is the gradient both branches of the join
 * receive: the shortcut takes it as it is, the main branch's last BN takes it
 * through trb200_bnrelu_bwd_dtype with mask_bits = NULL. */
int trb200_relu_mask_bwd(const void* dy, const void* mask_bits, void* dx, int64_t n, void* stream);

/* Max pooling with a k x k window, any stride and padding (ResNet: 3x3, stride 2,
 * pad 1), NHWC tensors of `dtype`, c % 8 == 0.  argmax: one byte per output
 * element = kh*k + kw of the first maximum (0xff for a window that lies outside
 * the image): maxpool_amp_fwd_mask_kernel, maxpool_op.cu:83-133.  Backward: every
 * input pixel gathers the dy of the windows whose argmax points at it, in float, in
 * (oh, ow) order (no atomics): maxpool_bwd_deterministic_kernel, maxpool_op.cu:155-217.
 * h, w are the input extents; the output is [n, (h+2*pad-k)/stride+1, ..., c]. */
int trb200_maxpool_fwd(const void* x, void* y, void* argmax, int32_t n, int32_t h, int32_t w, int32_t c,
                       int32_t k, int32_t stride, int32_t pad, int32_t dtype, void* stream);
int trb200_maxpool_bwd(const void* dy, const void* argmax, void* dx, int32_t n, int32_t h, int32_t w, int32_t c,
                       int32_t k, int32_t stride, int32_t pad, int32_t dtype, void* stream);

/* Global average pooling [n,h,w,c] -> [n,c] and its backward: y = sum * 1/(h*w)
 * with the sum in float over (h, w) in order, gap_op.cpp:137-155; dx = dy * 1/(h*w),
 * gap_bwd_amp_compact_kernel, gap_op.cu:92-112. */
int trb200_avgpool_global_fwd(const void* x, void* y, int32_t n, int32_t h, int32_t w, int32_t c, int32_t dtype,
                              void* stream);
int trb200_avgpool_global_bwd(const void* dy, void* dx, int32_t n, int32_t h, int32_t w, int32_t c, int32_t dtype,
                              void* stream);

/* ------------------------------------------------------------------------- */
/* Forward side of the block that produces the backward's inputs, and the     */
/* steps after the all-reduce (the callers either side of the hot path).      */
/* ------------------------------------------------------------------------- */

/* Per-channel sum and sum of squares of the (half) conv output, then
 * bn_finalize: saved_mean, saved_inv_std = 1/sqrt(biased var + eps), eq_scale =
 * gamma*inv_std, eq_bias = beta - mean*eq_scale, running stats (unbiased var)
 * updated in place when not NULL.  ch_sum / ch_sqsum may be NULL.  Counterparts:
 * genstats and build_cbr_bn_finalize_graph, cbr_op.cpp:622-718 and 430-528. */
size_t trb200_bn_stats_workspace_bytes(int64_t m, int32_t c);
int trb200_bn_stats_finalize(const void* conv_out, const float* gamma, const float* beta, float eps,
                             float momentum, float* ch_sum, float* ch_sqsum, float* saved_mean,
                             float* saved_inv_std, float* eq_scale, float* eq_bias,
                             float* running_mean, float* running_var, int64_t m, int32_t c,
                             void* workspace, size_t workspace_bytes, void* stream);

/* trb200_bn_stats_finalize for conv outputs of either 16-bit type (TRB200_DTYPE_*). */
int trb200_bn_stats_finalize_dtype(const void* conv_out, const float* gamma, const float* beta, float eps,
                                   float momentum, float* ch_sum, float* ch_sqsum, float* saved_mean,
                                   float* saved_inv_std, float* eq_scale, float* eq_bias,
                                   float* running_mean, float* running_var, int64_t m, int32_t c, int32_t dtype,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* The apply stage for either 16-bit type, with the ReLU (relu != 0: as
 * trb200_bn_apply_relu_mask below) or without it (out = t, mask_bits unused and may
 * be NULL: the BN in front of a residual join and the BN of its shortcut). */
int trb200_bn_apply_dtype(const void* conv_out, const float* eq_scale, const float* eq_bias, void* out,
                          void* mask_bits, int64_t m, int32_t c, int32_t relu, int32_t dtype, void* stream);

/* relu_out = max(t, 0), mask bit = (t > 0) with t = half(half(x*eq_scale) + eq_bias):
 * build_cbr_bn_relu_graph, cbr_op.cpp:534-616 (MUL, ADD with HALF intermediates,
 * RELU_FWD, CMP_GT -> BOOLEAN).  Mask layout as in trb200_bnrelu_bwd. */
int trb200_bn_apply_relu_mask(const void* conv_out, const float* eq_scale, const float* eq_bias,
                              void* relu_out, void* mask_bits, int64_t m, int32_t c, void* stream);

/* 2x2 stride-2 max pooling on NHWC half, argmax byte = kh*2 + kw with the first
 * maximum winning, and its backward (gradient routed to the argmax position,
 * zeros elsewhere): maxpool_amp_fwd_mask_kernel / maxpool_bwd_deterministic_kernel,
 * src/backend/ops/dtensor/maxpool_op.cu:23-217.  h, w even, c % 8 == 0. */
int trb200_maxpool2x2_fwd(const void* x, void* y, void* argmax, int32_t n, int32_t h, int32_t w,
                          int32_t c, void* stream);
int trb200_maxpool2x2_bwd(const void* dy, const void* argmax, void* dx, int32_t n, int32_t h, int32_t w,
                          int32_t c, void* stream);

/* A block followed by a 2x2 max pool, with the pool fused into the block's HBM-bound
 * kernels so that the full-resolution ReLU output (forward) and its gradient
 * (backward) are never written to or read from HBM.
 *   forward : = trb200_bn_apply_relu_mask + trb200_maxpool2x2_fwd, bit for bit; relu_out
 *             may be NULL (nothing downstream of a pooled block reads it).
 *   backward: = trb200_maxpool2x2_bwd + trb200_bnrelu_bwd (dy_pooled is [n,h/2,w/2,c]).
 * h, w are the block's output extents (even), c % 8 == 0. */
int trb200_bn_apply_relu_mask_pool(const void* conv_out, const float* eq_scale, const float* eq_bias,
                                   void* relu_out, void* mask_bits, void* pool_out, void* argmax,
                                   int32_t n, int32_t h, int32_t w, int32_t c, void* stream);
size_t trb200_bnrelu_pool_bwd_workspace_bytes(int32_t n, int32_t h, int32_t w, int32_t c);
int trb200_bnrelu_pool_bwd(const void* dy_pooled, const void* argmax, const void* mask_bits, const void* x,
                           const float* gamma, const float* saved_mean, const float* saved_inv_std,
                           void* dconv, float* dgamma, float* dbeta, int32_t n, int32_t h, int32_t w,
                           int32_t c, void* workspace, size_t workspace_bytes, void* stream);

/* *flag = 1 if any of the n floats is NaN or Inf (flag is never cleared here):
 * check_nan_kernel, src/backend/ops/range/check_op.cu:15-79. */
int trb200_check_nonfinite(const float* grads, int64_t n, int32_t* flag, void* stream);

/* SGD with momentum over a flat float range, loss scale undone on the fly, and
 * the half working copy refreshed in the same sweep (weights_half may be NULL):
 *   m = beta*m + g/scaling ; w = w*(1 - lr*wd) - lr*m ; w16 = half(w)
 * Skipped entirely when *skip_flag != 0 (the non-finite guard).  `scaling` is a
 * device scalar (NULL = 1).  Counterparts: momentum kernel,
 * src/backend/ops/range/optimizer_op.cu:40-60 (CPU form optimizer_op.cpp:306-313),
 * and RANGE_CAST_FP32_TO_FP16, cast_op.cu:18-37. */
int trb200_sgd_momentum(float* weights, const float* grads, float* momentum, void* weights_half,
                        int64_t n, float lr, float weight_decay, float beta, const float* scaling,
                        const int32_t* skip_flag, void* stream);

/* The same sweep with Nesterov momentum (update_nesterov_kernel, optimizer_op.cu:68-93):
 *   m = beta*m + g/scaling ; w = w*(1 - lr*wd) - lr*(beta*m + g/scaling) */
int trb200_sgd_nesterov(float* weights, const float* grads, float* momentum, void* weights_half,
                        int64_t n, float lr, float weight_decay, float beta, const float* scaling,
                        const int32_t* skip_flag, void* stream);

/* ... and without momentum (update_sgd_kernel, optimizer_op.cu:22-38):
 *   w = w*(1 - lr*wd) - lr*g/scaling */
int trb200_sgd_plain(float* weights, const float* grads, void* weights_half, int64_t n, float lr,
                     float weight_decay, const float* scaling, const int32_t* skip_flag, void* stream);

/* RANGE_CHECK_NAN with clipping (check_nan_and_clip_kernel, check_op.cu:54-79): a NaN
 * raises *flag and stays as it is (the optimizer then skips the step); every other
 * value, infinities included, is clamped to [-clip, clip] in place. */
int trb200_check_nan_and_clip(float* grads, int64_t n, float clip, int32_t* flag, void* stream);

/* RANGE_GRAD_SCALING (grad_scaling_kernel, grad_scaling_op.cu:15-22): after a step
 * whose check raised the flag the loss scale is halved, never below 1:
 *   if (*has_nan) *scaling = max(*scaling / 2, 1).
 * clear_flag != 0 also resets *has_nan afterwards, ready for the next step's check
 * (the reference's flag is reset by its host loop). */
int trb200_grad_scaling(int32_t* has_nan, float* scaling, int32_t clear_flag, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRB200_H_ */
