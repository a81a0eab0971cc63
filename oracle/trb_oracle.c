/*
 * trb_oracle.c -- CPU restatement of the Renaissance training-backward hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed CPU
 * baseline.  Nothing in the product path (the CUDA library or its host-side
 * plugin) links, loads or calls it.
 *
 * Every function restates the arithmetic of a reference CPU operator (unfused
 * FP32 ops) or, where the reference only has a GPU path (the fused AMP
 * Conv+BN+ReLU block and the GPU softmax-CE kernels), the arithmetic that the
 * reference asks its libraries for.  Citations are to the reference project's
 * own paths.
 *
 *   conv fwd (naive)     src/backend/ops/dtensor/conv_op.cpp:664-729
 *   conv bwd (naive)     src/backend/ops/dtensor/conv_op.cpp:744-850
 *   BN fwd / bwd         src/backend/ops/dtensor/bn_op.cpp:55-116, 119-168
 *   ReLU fwd / bwd       src/backend/ops/dtensor/relu_op.cpp:348-419
 *   softmax-CE CPU       src/backend/ops/dtensor/softmax_ce_op.cpp:114-156, 237-256
 *   softmax-CE GPU order src/backend/ops/dtensor/softmax_ce_op.cu:63-177, 372-468
 *   FC fwd / bwd         src/backend/ops/dtensor/fc_op.cpp:802-898
 *   SGD                  src/backend/ops/range/optimizer_op.cpp:297-304
 *   CBR fwd pieces       src/backend/ops/dtensor/cbr_op.cpp:430-616
 *   CBR bwd pieces       src/backend/ops/dtensor/cbr_op.cpp:1259-1353, 763-917
 *   mask bit order       tests/op/cbr_amp_test_utils.hpp:115-145
 *
 * Parity pin: the functions are checked against golden vectors produced by
 * PyTorch CPU autograd with the recipes of the reference's own test generators
 * (tests/op/test_conv_fwd_bwd.py, tests/op/test_bn_fwd_bwd_legacy.py,
 * tests/correction/test_softmax_ce.py); the reference stores no golden numbers
 * of its own.  The label-smoothing branch of softmax-CE and the bit-packed mask
 * have no reference-side golden at all and are pinned only to the formulas in
 * the cited source lines.
 *
 * Layouts: activations NHWC, weights KRSC, all compact.  "h16" arguments are
 * IEEE binary16 stored as uint16_t.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

typedef _Float16 h16;

/* ------------------------------------------------------------------------- */
/* helpers                                                                    */
/* ------------------------------------------------------------------------- */

/* Minimal fork-join parallel-for on pthreads (this image has no OpenMP
 * runtime).  Work items are split into contiguous blocks, one per thread, so
 * every output element is still produced by exactly one thread in a fixed
 * order and results do not depend on the thread count. */
static int g_threads = 0;

int orc_num_threads(void) {
    if (g_threads <= 0) {
        long n = sysconf(_SC_NPROCESSORS_ONLN);
        g_threads = n > 0 ? (int)n : 1;
    }
    return g_threads;
}

void orc_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*orc_body)(int64_t begin, int64_t end, void* ctx);
typedef struct { orc_body fn; void* ctx; int64_t begin, end; } orc_job;

static void* orc_job_main(void* p) {
    orc_job* j = (orc_job*)p;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}

static void orc_parallel_for(int64_t n, orc_body fn, void* ctx) {
    int t = orc_num_threads();
    if (t > n) t = (int)n;
    if (t <= 1) { fn(0, n, ctx); return; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)t);
    orc_job* jobs = (orc_job*)malloc(sizeof(orc_job) * (size_t)t);
    for (int i = 0; i < t; ++i) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].begin = n * i / t; jobs[i].end = n * (i + 1) / t;
        if (pthread_create(&th[i], NULL, orc_job_main, &jobs[i]) != 0) {
            jobs[i].fn(jobs[i].begin, jobs[i].end, ctx);
            th[i] = 0;
        }
    }
    for (int i = 0; i < t; ++i) if (th[i]) pthread_join(th[i], NULL);
    free(th); free(jobs);
}

void orc_h16_to_f32(const h16* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = (float)src[i];
}

void orc_f32_to_h16(const float* src, h16* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = (h16)src[i];
}

/* cuDNN BOOLEAN tensors hold one bit per element, least significant bit first,
 * indexed by the flat NHWC element index (tests/op/cbr_amp_test_utils.hpp:115-145). */
void orc_mask_pack(const int8_t* bytes, uint8_t* bits, int64_t n) {
    memset(bits, 0, (size_t)((n + 7) / 8));
    for (int64_t i = 0; i < n; ++i)
        if (bytes[i]) bits[i >> 3] |= (uint8_t)(1u << (i & 7));
}

void orc_mask_unpack(const uint8_t* bits, int8_t* bytes, int64_t n) {
    for (int64_t i = 0; i < n; ++i) bytes[i] = (int8_t)((bits[i >> 3] >> (i & 7)) & 1u);
}

/* ------------------------------------------------------------------------- */
/* convolution, FP32 (groups = 1)                                             */
/* ------------------------------------------------------------------------- */

static inline int out_extent(int in, int pad, int k, int stride) {
    return (in + 2 * pad - k) / stride + 1;
}

/* Y[n,oh,ow,k] = sum_{r,s,c} X[n,oh*st+r-p,ow*st+s-p,c] * Wt[k,r,s,c], float
 * accumulation in (r,s,c) order as conv_op.cpp:664-729. */
typedef struct {
    const float *a, *b; float* out;
    int N, H, W, C, K, R, S, pad, stride, OH, OW;
} conv_ctx;

static void conv_fwd_rows(int64_t begin, int64_t end, void* p) {
    const conv_ctx* q = (const conv_ctx*)p;
    const float *X = q->a, *Wt = q->b; float* Y = q->out;
    const int H = q->H, W = q->W, C = q->C, K = q->K, R = q->R, S = q->S;
    const int pad = q->pad, stride = q->stride, OH = q->OH, OW = q->OW;
    for (int64_t row = begin; row < end; ++row) {   /* row = n*OH + oh */
        const int n = (int)(row / OH), oh = (int)(row % OH);
            for (int ow = 0; ow < OW; ++ow) {
                float* y = Y + (((int64_t)n * OH + oh) * OW + ow) * K;
                for (int k = 0; k < K; ++k) {
                    float acc = 0.0f;
                    for (int r = 0; r < R; ++r) {
                        const int ih = oh * stride + r - pad;
                        if (ih < 0 || ih >= H) continue;
                        for (int s = 0; s < S; ++s) {
                            const int iw = ow * stride + s - pad;
                            if (iw < 0 || iw >= W) continue;
                            const float* x = X + (((int64_t)n * H + ih) * W + iw) * C;
                            const float* w = Wt + (((int64_t)k * R + r) * S + s) * C;
                            for (int c = 0; c < C; ++c) acc += x[c] * w[c];
                        }
                    }
                    y[k] = acc;
                }
            }
    }
}

void orc_conv_fwd_f32(const float* X, const float* Wt, float* Y,
                      int N, int H, int W, int C, int K, int R, int S,
                      int pad, int stride) {
    conv_ctx q = {X, Wt, Y, N, H, W, C, K, R, S, pad, stride,
                  out_extent(H, pad, R, stride), out_extent(W, pad, S, stride)};
    orc_parallel_for((int64_t)N * q.OH, conv_fwd_rows, &q);
}

/* Data gradient.  The reference scatters dX += dY*W in (n,oh,ow,k,r,s,c) order
 * (conv_op.cpp:780-812); for one dX element that is ascending (oh,ow,k).  This
 * gather form visits the same terms in the same order, so the float sum is the
 * same, and rows of dX are independent (safe to run in parallel). */
static void conv_dgrad_rows(int64_t begin, int64_t end, void* p) {
    const conv_ctx* q = (const conv_ctx*)p;
    const float *dY = q->a, *Wt = q->b; float* dX = q->out;
    const int H = q->H, W = q->W, C = q->C, K = q->K, R = q->R, S = q->S;
    const int pad = q->pad, stride = q->stride, OH = q->OH, OW = q->OW;
    for (int64_t row = begin; row < end; ++row) {   /* row = n*H + ih */
        const int n = (int)(row / H), ih = (int)(row % H);
            for (int iw = 0; iw < W; ++iw) {
                float* dx = dX + (((int64_t)n * H + ih) * W + iw) * C;
                for (int c = 0; c < C; ++c) dx[c] = 0.0f;
                for (int oh = 0; oh < OH; ++oh) {
                    const int r = ih + pad - oh * stride;
                    if (r < 0 || r >= R) continue;
                    for (int ow = 0; ow < OW; ++ow) {
                        const int s = iw + pad - ow * stride;
                        if (s < 0 || s >= S) continue;
                        const float* dy = dY + (((int64_t)n * OH + oh) * OW + ow) * K;
                        for (int k = 0; k < K; ++k) {
                            const float g = dy[k];
                            const float* w = Wt + (((int64_t)k * R + r) * S + s) * C;
                            for (int c = 0; c < C; ++c) dx[c] += g * w[c];
                        }
                    }
                }
            }
    }
}

void orc_conv_dgrad_f32(const float* dY, const float* Wt, float* dX,
                        int N, int H, int W, int C, int K, int R, int S,
                        int pad, int stride) {
    conv_ctx q = {dY, Wt, dX, N, H, W, C, K, R, S, pad, stride,
                  out_extent(H, pad, R, stride), out_extent(W, pad, S, stride)};
    orc_parallel_for((int64_t)N * H, conv_dgrad_rows, &q);
}

/* Weight gradient.  Reference order (conv_op.cpp:817-848): for one dW element
 * the terms arrive in ascending (n,oh,ow).  Each (k,r,s) row of dW is
 * accumulated here by one thread in that order. */
static void conv_wgrad_rows(int64_t begin, int64_t end, void* p) {
    const conv_ctx* q = (const conv_ctx*)p;
    const float *dY = q->a, *X = q->b; float* dW = q->out;
    const int N = q->N, H = q->H, W = q->W, C = q->C, K = q->K, R = q->R, S = q->S;
    const int pad = q->pad, stride = q->stride, OH = q->OH, OW = q->OW;
    for (int64_t row = begin; row < end; ++row) {   /* row = (k*R + r)*S + s */
        const int k = (int)(row / (R * S)), r = (int)((row / S) % R), s = (int)(row % S);
            {
                float* dw = dW + (((int64_t)k * R + r) * S + s) * C;
                for (int c = 0; c < C; ++c) dw[c] = 0.0f;
                for (int n = 0; n < N; ++n)
                    for (int oh = 0; oh < OH; ++oh) {
                        const int ih = oh * stride + r - pad;
                        if (ih < 0 || ih >= H) continue;
                        for (int ow = 0; ow < OW; ++ow) {
                            const int iw = ow * stride + s - pad;
                            if (iw < 0 || iw >= W) continue;
                            const float g = dY[(((int64_t)n * OH + oh) * OW + ow) * K + k];
                            const float* x = X + (((int64_t)n * H + ih) * W + iw) * C;
                            for (int c = 0; c < C; ++c) dw[c] += g * x[c];
                        }
                    }
            }
    }
}

void orc_conv_wgrad_f32(const float* dY, const float* X, float* dW,
                        int N, int H, int W, int C, int K, int R, int S,
                        int pad, int stride) {
    conv_ctx q = {dY, X, dW, N, H, W, C, K, R, S, pad, stride,
                  out_extent(H, pad, R, stride), out_extent(W, pad, S, stride)};
    orc_parallel_for((int64_t)K * R * S, conv_wgrad_rows, &q);
}

/* ------------------------------------------------------------------------- */
/* batch norm, FP32 (bn_op.cpp:55-168)                                        */
/* ------------------------------------------------------------------------- */

/* Training forward: double sums, biased variance for inv_std, unbiased for the
 * running variance, running stats updated in place. */
void orc_bn_fwd_f32(const float* x, const float* gamma, const float* beta,
                    float* running_mean, float* running_var,
                    float* y, float* saved_mean, float* saved_inv_std,
                    int64_t M, int C, float eps, float momentum) {
    for (int c = 0; c < C; ++c) {
        double sum = 0.0;
        for (int64_t i = 0; i < M; ++i) sum += x[i * C + c];
        const float mean = (float)(sum / (double)M);
        double sq = 0.0;
        for (int64_t i = 0; i < M; ++i) {
            const float d = x[i * C + c] - mean;
            sq += d * d;
        }
        const float var = (float)(sq / (double)M);
        const float inv_std = 1.0f / sqrtf(var + eps);
        saved_mean[c] = mean;
        saved_inv_std[c] = inv_std;
        if (running_mean) running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * mean;
        if (running_var) {
            const float unb = (M > 1) ? (float)(sq / (double)(M - 1)) : var;
            running_var[c] = (1.0f - momentum) * running_var[c] + momentum * unb;
        }
        if (y)
            for (int64_t i = 0; i < M; ++i)
                y[i * C + c] = gamma[c] * (x[i * C + c] - mean) * inv_std + beta[c];
    }
}

/* Training backward (bn_op.cpp:119-168): double channel sums, then
 * dx = g*is*(dy - sum_dy/M - (sum_dy_xmu/M)*is*is*(x-mu)). */
void orc_bn_bwd_f32(const float* dy, const float* x, const float* gamma,
                    const float* saved_mean, const float* saved_inv_std,
                    float* dx, float* dgamma, float* dbeta, int64_t M, int C) {
    for (int c = 0; c < C; ++c) {
        const float mean = saved_mean[c], is = saved_inv_std[c];
        double s_dy = 0.0, s_dyxmu = 0.0;
        for (int64_t i = 0; i < M; ++i) {
            const float g = dy[i * C + c];
            s_dy += g;
            s_dyxmu += g * (x[i * C + c] - mean);
        }
        dbeta[c] = (float)s_dy;
        dgamma[c] = (float)(s_dyxmu * is);
        if (dx) {
            const float inv_m = 1.0f / (float)M;
            for (int64_t i = 0; i < M; ++i) {
                const float xmu = x[i * C + c] - mean;
                dx[i * C + c] = gamma[c] * is *
                                (dy[i * C + c] - inv_m * (float)s_dy -
                                 inv_m * (float)s_dyxmu * is * is * xmu);
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* ReLU with byte mask (relu_op.cpp:348-419)                                  */
/* ------------------------------------------------------------------------- */

void orc_relu_fwd_f32(const float* x, float* y, int8_t* mask, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i];
        y[i] = v > 0.0f ? v : 0.0f;
        mask[i] = v > 0.0f ? 1 : 0;
    }
}

void orc_relu_bwd_f32(const float* dy, const int8_t* mask, float* dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dx[i] = mask[i] ? dy[i] : 0.0f;
}

/* ------------------------------------------------------------------------- */
/* softmax + cross entropy                                                    */
/* ------------------------------------------------------------------------- */

/* CPU operator (softmax_ce_op.cpp:114-156): probs are written twice (exp, then
 * normalised), eps sits in 1/(sum+1e-8) and log(p+1e-8), the loss is ADDED to
 * *loss and then the whole *loss is multiplied by `scaling`. */
void orc_softmax_ce_fwd_cpu(const float* logits, const int32_t* labels,
                            float* loss, float* inv_scaling, float* probs,
                            int batch, int classes, float scaling, float ls) {
    const float inv_b = 1.0f / (float)batch;
    *inv_scaling = inv_b;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    for (int b = 0; b < batch; ++b) {
        const float* z = logits + (int64_t)b * classes;
        float* p = probs + (int64_t)b * classes;
        float zmax = -INFINITY;
        for (int c = 0; c < classes; ++c) if (z[c] > zmax) zmax = z[c];
        float sum = 0.0f;
        for (int c = 0; c < classes; ++c) { p[c] = expf(z[c] - zmax); sum += p[c]; }
        const float inv_sum = 1.0f / (sum + 1e-8f);
        float sum_log = 0.0f;
        for (int c = 0; c < classes; ++c) { p[c] *= inv_sum; sum_log += logf(p[c] + 1e-8f); }
        const float ly = logf(p[labels[b]] + 1e-8f);
        *loss += (-keep * ly - spread * sum_log) * inv_b;
    }
    *loss *= scaling;
}

/* Backward, shared by CPU and GPU (softmax_ce_op.cpp:237-256,
 * softmax_ce_op.cu:438-468): g = (p - ls/K - [c==y](1-ls)) * scale. */
void orc_softmax_ce_bwd(const float* probs, const int32_t* labels, float* dlogits,
                        int batch, int classes, float scale, float ls) {
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < classes; ++c) {
            float g = probs[(int64_t)b * classes + c] - spread;
            if (c == labels[b]) g -= keep;
            dlogits[(int64_t)b * classes + c] = g * scale;
        }
}

/* GPU AMP operator semantics (softmax_ce_op.cu:63-177, 372-429, 438-468):
 * fp16 logits with a row stride, fp32 probs, per-row loss partial already
 * multiplied by 1/batch, loss = plain sum of partials (NOT multiplied by
 * `scaling`), inv_scaling = 1/batch, d_logits = half(g * scaling * inv_scaling).
 * Row sums are taken in double here; the kernels' float tree order is free. */
typedef struct {
    const h16* logits; int64_t logits_stride; const int32_t* labels;
    float *probs, *loss_partial; h16* dlogits; int64_t dlogits_stride;
    int batch, classes; float scaling, ls;
} sce_ctx;

static void sce_rows(int64_t begin, int64_t end, void* p) {
    const sce_ctx* q = (const sce_ctx*)p;
    const h16* logits = q->logits; const int64_t logits_stride = q->logits_stride;
    const int32_t* labels = q->labels;
    float *probs = q->probs, *loss_partial = q->loss_partial;
    h16* dlogits = q->dlogits; const int64_t dlogits_stride = q->dlogits_stride;
    const int classes = q->classes; const float scaling = q->scaling, ls = q->ls;
    const float inv_b = 1.0f / (float)q->batch;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    for (int64_t b = begin; b < end; ++b) {
        const h16* z = logits + (int64_t)b * logits_stride;
        float zmax = -INFINITY;
        for (int c = 0; c < classes; ++c) { const float v = (float)z[c]; if (v > zmax) zmax = v; }
        double sum = 0.0;
        for (int c = 0; c < classes; ++c) sum += (double)expf((float)z[c] - zmax);
        const float inv_sum = 1.0f / ((float)sum + 1e-8f);
        double sum_log = 0.0;
        float py = 0.0f;
        const float scale = scaling * inv_b;
        for (int c = 0; c < classes; ++c) {
            const float p = expf((float)z[c] - zmax) * inv_sum;
            if (probs) probs[(int64_t)b * classes + c] = p;
            sum_log += (double)logf(p + 1e-8f);
            if (c == labels[b]) py = p;
            if (dlogits) {
                float g = p - spread;
                if (c == labels[b]) g -= keep;
                dlogits[(int64_t)b * dlogits_stride + c] = (h16)(g * scale);
            }
        }
        if (loss_partial)
            loss_partial[b] = (-keep * logf(py + 1e-8f) - spread * (float)sum_log) * inv_b;
    }
}

void orc_softmax_ce_amp(const h16* logits, int64_t logits_stride, const int32_t* labels,
                        float* probs, float* loss_partial, float* loss, float* inv_scaling,
                        h16* dlogits, int64_t dlogits_stride,
                        int batch, int classes, float scaling, float ls) {
    sce_ctx q = {logits, logits_stride, labels, probs, loss_partial, dlogits, dlogits_stride,
                 batch, classes, scaling, ls};
    if (inv_scaling) *inv_scaling = 1.0f / (float)batch;
    orc_parallel_for(batch, sce_rows, &q);
    if (loss && loss_partial) {
        double tot = 0.0;
        for (int b = 0; b < batch; ++b) tot += (double)loss_partial[b];
        *loss = (float)tot;
    }
}

/* ------------------------------------------------------------------------- */
/* FC and SGD (config-1 MLP on the reference CPU backend)                     */
/* ------------------------------------------------------------------------- */

void orc_fc_fwd_f32(const float* x, const float* w, const float* b, float* y,
                    int batch, int in_f, int out_f) {
    for (int n = 0; n < batch; ++n)
        for (int o = 0; o < out_f; ++o) {
            float acc = 0.0f;
            for (int i = 0; i < in_f; ++i) acc += x[(int64_t)n * in_f + i] * w[(int64_t)o * in_f + i];
            if (b) acc += b[o];
            y[(int64_t)n * out_f + o] = acc;
        }
}

void orc_fc_bwd_f32(const float* dy, const float* w, const float* x,
                    float* dx, float* dw, float* db, int batch, int in_f, int out_f) {
    if (db)
        for (int o = 0; o < out_f; ++o) {
            float acc = 0.0f;
            for (int n = 0; n < batch; ++n) acc += dy[(int64_t)n * out_f + o];
            db[o] = acc;
        }
    if (dw) {
        for (int o = 0; o < out_f; ++o)
            for (int i = 0; i < in_f; ++i) {
                float acc = 0.0f;
                for (int n = 0; n < batch; ++n)
                    acc += dy[(int64_t)n * out_f + o] * x[(int64_t)n * in_f + i];
                dw[(int64_t)o * in_f + i] = acc;
            }
    }
    if (dx) {
        for (int n = 0; n < batch; ++n)
            for (int i = 0; i < in_f; ++i) {
                float acc = 0.0f;
                for (int o = 0; o < out_f; ++o)
                    acc += dy[(int64_t)n * out_f + o] * w[(int64_t)o * in_f + i];
                dx[(int64_t)n * in_f + i] = acc;
            }
    }
}

/* w <- w*(1 - lr*wd) - lr*g/scaling   (optimizer_op.cpp:297-304) */
void orc_sgd_f32(float* w, const float* g, int64_t n, float lr, float wd, float scaling) {
    const float inv = scaling != 0.0f ? 1.0f / scaling : 1.0f;
    for (int64_t i = 0; i < n; ++i) w[i] = w[i] * (1.0f - lr * wd) - lr * g[i] * inv;
}

/* m <- beta*m + g/scaling ; w <- w*(1 - lr*wd) - lr*m   (optimizer_op.cpp:306-316,
 * optimizer_op.cu:40-60) */
void orc_momentum_f32(float* w, const float* g, float* m, int64_t n,
                      float lr, float wd, float beta, float scaling) {
    const float inv = scaling != 0.0f ? 1.0f / scaling : 1.0f;
    for (int64_t i = 0; i < n; ++i) {
        m[i] = m[i] * beta + g[i] * inv;
        w[i] = w[i] * (1.0f - lr * wd) - lr * m[i];
    }
}

/* m_new = m*beta + g/scaling ; w <- w*(1 - lr*wd) - lr*(m_new*beta + g/scaling)
 * (update_nesterov_kernel, optimizer_op.cu:68-93) */
void orc_nesterov_f32(float* w, const float* g, float* m, int64_t n,
                      float lr, float wd, float beta, float scaling) {
    const float inv = scaling != 0.0f ? 1.0f / scaling : 1.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float gi = g[i] * inv;
        const float mn = m[i] * beta + gi;
        m[i] = mn;
        w[i] = w[i] * (1.0f - lr * wd) - lr * (mn * beta + gi);
    }
}

/* NaN: flag, value kept; otherwise clamp to [-clip, clip] (check_nan_and_clip_kernel, check_op.cu:54-79).
 * Returns the flag. */
int orc_check_nan_and_clip_f32(float* g, int64_t n, float clip) {
    int flag = 0;
    for (int64_t i = 0; i < n; ++i) {
        const float v = g[i];
        if (v != v) { flag = 1; continue; }
        const float c = v < -clip ? -clip : (v > clip ? clip : v);
        if (c != v) g[i] = c;
    }
    return flag;
}

/* loss-scale back-off (grad_scaling_kernel, grad_scaling_op.cu:15-22) */
float orc_grad_scaling(int has_nan, float scaling) {
    if (has_nan != 0) {
        const float s = scaling * 0.5f;
        return s < 1.0f ? 1.0f : s;
    }
    return scaling;
}

/* ------------------------------------------------------------------------- */
/* fused AMP block (CBR): what the reference asks cuDNN for                   */
/* ------------------------------------------------------------------------- */

/* Forward (cbr_op.cpp:430-718): conv with float accumulation -> conv_out half;
 * per-channel sum / sum of squares in float ("genstats", taken from the float
 * accumulator); bn_finalize -> saved_mean, saved_inv_std, eq_scale, eq_bias;
 * y = relu(t), mask = t > 0 with t = half(half(x*eq_scale) + eq_bias) when
 * round_steps != 0 (the virtual tensors are declared HALF, cbr_op.cpp:568-577)
 * or t = x*eq_scale + eq_bias kept in float when round_steps == 0.
 * stats_from_half != 0 takes the statistics from the half-rounded conv output
 * (a separate pass over the stored tensor) instead of the float accumulator. */
void orc_cbr_fwd_amp(const h16* X, const h16* Wt, const float* gamma, const float* beta,
                     float* running_mean, float* running_var,
                     h16* conv_out, float* ch_sum, float* ch_sqsum,
                     float* saved_mean, float* saved_inv_std,
                     float* eq_scale, float* eq_bias,
                     h16* relu_out, uint8_t* mask_bits,
                     int N, int H, int W, int C, int K, int R, int S, int pad, int stride,
                     float eps, float momentum, int round_steps, int stats_from_half) {
    const int OH = out_extent(H, pad, R, stride), OW = out_extent(W, pad, S, stride);
    const int64_t M = (int64_t)N * OH * OW;
    const int64_t ne = M * K;
    float* acc = (float*)malloc(sizeof(float) * (size_t)ne);
    float* xf = (float*)malloc(sizeof(float) * (size_t)N * H * W * C);
    float* wf = (float*)malloc(sizeof(float) * (size_t)K * R * S * C);
    orc_h16_to_f32(X, xf, (int64_t)N * H * W * C);
    orc_h16_to_f32(Wt, wf, (int64_t)K * R * S * C);
    orc_conv_fwd_f32(xf, wf, acc, N, H, W, C, K, R, S, pad, stride);
    free(xf); free(wf);
    for (int64_t i = 0; i < ne; ++i) conv_out[i] = (h16)acc[i];
    for (int k = 0; k < K; ++k) {
        double s = 0.0, q = 0.0;
        for (int64_t i = 0; i < M; ++i) {
            /* stats_from_half: statistics of the stored half tensor instead of the float accumulator */
            const double v = stats_from_half ? (double)(float)conv_out[i * K + k] : (double)acc[i * K + k];
            s += v; q += v * v;
        }
        ch_sum[k] = (float)s; ch_sqsum[k] = (float)q;
        const float mean = (float)(s / (double)M);
        float var = (float)(q / (double)M - (s / (double)M) * (s / (double)M));
        if (var < 0.0f) var = 0.0f;
        const float is = 1.0f / sqrtf(var + eps);
        saved_mean[k] = mean; saved_inv_std[k] = is;
        eq_scale[k] = gamma[k] * is;
        eq_bias[k] = beta[k] - mean * eq_scale[k];
        if (running_mean) running_mean[k] = (1.0f - momentum) * running_mean[k] + momentum * mean;
        if (running_var) {
            const float unb = M > 1 ? var * (float)((double)M / (double)(M - 1)) : var;
            running_var[k] = (1.0f - momentum) * running_var[k] + momentum * unb;
        }
    }
    free(acc);
    memset(mask_bits, 0, ((size_t)ne + 7) / 8);
    for (int64_t i = 0; i < ne; ++i) {
        const int k = (int)(i % K);
        const float x = (float)conv_out[i];
        float t;
        if (round_steps) {
            const h16 a = (h16)(x * eq_scale[k]);
            t = (float)(h16)((float)a + eq_bias[k]);
        } else {
            t = x * eq_scale[k] + eq_bias[k];
        }
        const int on = t > 0.0f;
        if (relu_out) relu_out[i] = on ? (h16)t : (h16)0.0f;
        if (on) mask_bits[i >> 3] |= (uint8_t)(1u << (i & 7));
    }
}

/* BN+ReLU backward of the block (cbr_op.cpp:1259-1353):
 * dy_m = half(dY * mask); dbeta = sum dy_m; dgamma = sum dy_m*(x-mu)*is;
 * dconv = half(g*is*(dy_m - dbeta/M - xhat*dgamma/M)).  Channel sums in double. */
typedef struct {
    const h16* dY; const uint8_t* mask_bits; const h16* conv_out;
    const float *gamma, *saved_mean, *saved_inv_std;
    h16* dconv; float *dgamma, *dbeta; int64_t M; int C;
} bnb_ctx;

static void bnrelu_bwd_channels(int64_t begin, int64_t end, void* p) {
    const bnb_ctx* q = (const bnb_ctx*)p;
    const h16 *dY = q->dY, *conv_out = q->conv_out; const uint8_t* mask_bits = q->mask_bits;
    const float *gamma = q->gamma, *saved_mean = q->saved_mean, *saved_inv_std = q->saved_inv_std;
    h16* dconv = q->dconv; float *dgamma = q->dgamma, *dbeta = q->dbeta;
    const int64_t M = q->M; const int C = q->C;
    for (int64_t c = begin; c < end; ++c) {
        const float mu = saved_mean[c], is = saved_inv_std[c];
        double s1 = 0.0, s2 = 0.0;
        for (int64_t i = 0; i < M; ++i) {
            const int64_t e = i * C + c;
            const int on = (mask_bits[e >> 3] >> (e & 7)) & 1;
            const float g = on ? (float)dY[e] : 0.0f;
            s1 += g;
            s2 += (double)(g * (((float)conv_out[e] - mu) * is));
        }
        dbeta[c] = (float)s1;
        dgamma[c] = (float)s2;
        if (dconv) {
            const float inv_m = 1.0f / (float)M;
            const float mb = (float)s1 * inv_m, mg = (float)s2 * inv_m;
            for (int64_t i = 0; i < M; ++i) {
                const int64_t e = i * C + c;
                const int on = (mask_bits[e >> 3] >> (e & 7)) & 1;
                const float g = on ? (float)dY[e] : 0.0f;
                const float xhat = ((float)conv_out[e] - mu) * is;
                dconv[e] = (h16)(gamma[c] * is * (g - mb - xhat * mg));
            }
        }
    }
}

void orc_bnrelu_bwd_amp(const h16* dY, const uint8_t* mask_bits, const h16* conv_out,
                        const float* gamma, const float* saved_mean, const float* saved_inv_std,
                        h16* dconv, float* dgamma, float* dbeta, int64_t M, int C) {
    bnb_ctx q = {dY, mask_bits, conv_out, gamma, saved_mean, saved_inv_std,
                 dconv, dgamma, dbeta, M, C};
    orc_parallel_for(C, bnrelu_bwd_channels, &q);
}

/* Whole block backward: BN+ReLU backward, then wgrad and dgrad from the
 * half-rounded dconv with float accumulation, outputs rounded to half
 * (cbr_op.cpp:763-917, 1359-1522).  dX may be NULL (first-layer variant,
 * cbr_op.cpp:1528-1651). */
void orc_cbr_bwd_amp(const h16* dY, const h16* Wt, const float* gamma,
                     const float* saved_mean, const float* saved_inv_std,
                     const uint8_t* mask_bits, const h16* X, const h16* conv_out,
                     h16* dX, h16* dW, float* dgamma, float* dbeta, h16* dconv,
                     int N, int H, int W, int C, int K, int R, int S, int pad, int stride) {
    const int OH = out_extent(H, pad, R, stride), OW = out_extent(W, pad, S, stride);
    const int64_t M = (int64_t)N * OH * OW;
    orc_bnrelu_bwd_amp(dY, mask_bits, conv_out, gamma, saved_mean, saved_inv_std,
                       dconv, dgamma, dbeta, M, K);
    const int64_t nx = (int64_t)N * H * W * C, nw = (int64_t)K * R * S * C;
    float* gf = (float*)malloc(sizeof(float) * (size_t)(M * K));
    float* xf = (float*)malloc(sizeof(float) * (size_t)nx);
    float* wf = (float*)malloc(sizeof(float) * (size_t)nw);
    float* of = (float*)malloc(sizeof(float) * (size_t)(nx > nw ? nx : nw));
    orc_h16_to_f32(dconv, gf, M * K);
    orc_h16_to_f32(X, xf, nx);
    orc_h16_to_f32(Wt, wf, nw);
    orc_conv_wgrad_f32(gf, xf, of, N, H, W, C, K, R, S, pad, stride);
    orc_f32_to_h16(of, dW, nw);
    if (dX) {
        orc_conv_dgrad_f32(gf, wf, of, N, H, W, C, K, R, S, pad, stride);
        orc_f32_to_h16(of, dX, nx);
    }
    free(gf); free(xf); free(wf); free(of);
}

/* ------------------------------------------------------------------------- */
/* max pooling, NHWC half (maxpool_op.cu:23-217): forward keeps the argmax    */
/* position, backward routes the gradient to it (first maximum wins).         */
/* ------------------------------------------------------------------------- */

void orc_maxpool2x2_fwd_h16(const h16* x, h16* y, uint8_t* argmax,
                            int N, int H, int W, int C) {
    const int OH = H / 2, OW = W / 2;
    for (int n = 0; n < N; ++n)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow)
                for (int c = 0; c < C; ++c) {
                    float best = -INFINITY; int bi = 0;
                    for (int j = 0; j < 4; ++j) {
                        const int ih = oh * 2 + (j >> 1), iw = ow * 2 + (j & 1);
                        const float v = (float)x[(((int64_t)n * H + ih) * W + iw) * C + c];
                        if (v > best) { best = v; bi = j; }
                    }
                    const int64_t o = (((int64_t)n * OH + oh) * OW + ow) * C + c;
                    y[o] = (h16)best;
                    if (argmax) argmax[o] = (uint8_t)bi;
                }
}

void orc_maxpool2x2_bwd_h16(const h16* dy, const uint8_t* argmax, h16* dx,
                            int N, int H, int W, int C) {
    const int OH = H / 2, OW = W / 2;
    memset(dx, 0, sizeof(h16) * (size_t)N * H * W * C);
    for (int n = 0; n < N; ++n)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow)
                for (int c = 0; c < C; ++c) {
                    const int64_t o = (((int64_t)n * OH + oh) * OW + ow) * C + c;
                    const int j = argmax[o];
                    const int ih = oh * 2 + (j >> 1), iw = ow * 2 + (j & 1);
                    dx[(((int64_t)n * H + ih) * W + iw) * C + c] = dy[o];
                }
}
