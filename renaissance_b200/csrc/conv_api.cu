// C entry points for the convolution gradients and the whole-block backward.
#include "common.cuh"
#include "conv.cuh"

#include <atomic>

namespace trb {

int device_status_read_and_clear(int* out);
int wait_timeout_selftest(unsigned long long limit_ns, int* out4, cudaStream_t st);
int softmax_status_read_and_clear(int* out);
int bn_status_read_and_clear(int* out);
size_t bnrelu_pool_bwd_workspace(int n, int h, int w, int c);
int bnrelu_pool_bwd_launch(const void* dy_pooled, const void* argmax, const void* mask_bits, const void* x,
                           const float* gamma, const float* saved_mean, const float* saved_inv_std, void* dconv,
                           float* dgamma, float* dbeta, int n, int h, int w, int c, void* workspace,
                           size_t workspace_bytes, cudaStream_t s);
int bnrelu_bwd_launch(const void* dy, const void* mask_bits, const void* x, const float* gamma,
                      const float* saved_mean, const float* saved_inv_std, void* dconv, float* dgamma,
                      float* dbeta, int64_t m, int c, void* workspace, size_t workspace_bytes, cudaStream_t s,
                      int dtype);

namespace {
std::atomic<int> g_backend{0};   // 0 = automatic, 1 = direct kernels only

bool use_igemm(const trb200_conv_desc& d, int which) { return g_backend.load() == 0 && igemm_supports(d, which); }
bool use_strided(const trb200_conv_desc& d, int which) { return g_backend.load() == 0 && strided_supports(d, which); }
// the in-kernel 3x3 first-layer variant (half) comes first; every other 4-channel first layer is lowered
bool use_stem(const trb200_conv_desc& d, int which) {
    return g_backend.load() == 0 && !igemm_supports(d, which) && stem_supports(d, which);
}
}  // namespace

int validate_conv_desc(const trb200_conv_desc* d, const char* who) {
    TRB_REQUIRE(d, TRB200_ERR_INVALID_ARGUMENT, "%s: null descriptor", who);
    TRB_REQUIRE(d->n > 0 && d->h > 0 && d->w > 0 && d->c > 0 && d->k > 0 && d->r > 0 && d->s > 0,
                TRB200_ERR_INVALID_ARGUMENT, "%s: sizes must be positive", who);
    TRB_REQUIRE(d->stride_h > 0 && d->stride_w > 0 && d->pad_h >= 0 && d->pad_w >= 0, TRB200_ERR_INVALID_ARGUMENT,
                "%s: bad stride or padding", who);
    TRB_REQUIRE(d->h + 2 * d->pad_h >= d->r && d->w + 2 * d->pad_w >= d->s, TRB200_ERR_INVALID_ARGUMENT,
                "%s: filter larger than the padded input", who);
    TRB_REQUIRE((int64_t)d->n * d->h * d->w * d->c < (int64_t)1 << 40, TRB200_ERR_UNSUPPORTED, "%s: tensor too large",
                who);
    TRB_REQUIRE(valid_dtype(d->dtype), TRB200_ERR_INVALID_ARGUMENT, "%s: unknown dtype %d", who, d->dtype);
    return TRB200_OK;
}

}  // namespace trb

using trb::use_igemm;
using trb::use_strided;
using trb::use_stem;

extern "C" int trb200_set_conv_backend(int backend) {
    TRB_REQUIRE(backend == 0 || backend == 1, TRB200_ERR_INVALID_ARGUMENT, "set_conv_backend: 0 or 1 expected");
    trb::g_backend.store(backend);
    return TRB200_OK;
}

extern "C" int trb200_conv_uses_tensor_cores(const trb200_conv_desc* d, int which) {
    if (!d || which < 0 || which > 2) return 0;
    return (use_igemm(*d, which) || use_strided(*d, which) || use_stem(*d, which)) ? 1 : 0;
}

extern "C" int trb200_device_status(void) {
    int v = 0, v2 = 0;
    int rc = trb::device_status_read_and_clear(&v);
    if (rc) return rc;
    rc = trb::softmax_status_read_and_clear(&v2);
    if (rc) return rc;
    if (v == 0) v = v2;
    rc = trb::bn_status_read_and_clear(&v2);
    if (rc) return rc;
    if (v == 0) v = v2;
    if (v != 0)
        return trb::fail(TRB200_ERR_DEVICE_TIMEOUT, "a device-side wait gave up (role code %d)", v);
    return TRB200_OK;
}

extern "C" int trb200_selftest_wait_timeout(uint64_t limit_ns, int32_t* out4, void* stream) {
    return trb::wait_timeout_selftest((unsigned long long)limit_ns, out4, trb::as_stream(stream));
}

extern "C" size_t trb200_conv_wgrad_workspace_bytes(const trb200_conv_desc* d) {
    if (trb::validate_conv_desc(d, "conv_wgrad_workspace_bytes")) return 0;
    if (use_igemm(*d, 0)) return trb::igemm_wgrad_workspace(*d);
    if (use_strided(*d, 0)) return trb::strided_workspace(*d, 0);
    if (use_stem(*d, 0)) return trb::stem_workspace(*d, 0);
    return trb::wgrad_direct_workspace(*d);
}

extern "C" size_t trb200_conv_dgrad_workspace_bytes(const trb200_conv_desc* d) {
    if (trb::validate_conv_desc(d, "conv_dgrad_workspace_bytes")) return 0;
    if (use_igemm(*d, 1)) return trb::igemm_dgrad_workspace(*d);
    return use_strided(*d, 1) ? trb::strided_workspace(*d, 1) : 0;
}

extern "C" int trb200_conv_wgrad(const trb200_conv_desc* d, const void* dy, const void* x, void* dw, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    int rc = trb::validate_conv_desc(d, "conv_wgrad");
    if (rc) return rc;
    TRB_REQUIRE(dy && x && dw, TRB200_ERR_INVALID_ARGUMENT, "conv_wgrad: null pointer");
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(x) && trb::aligned16(dw), TRB200_ERR_INVALID_ARGUMENT,
                "conv_wgrad: tensors must be 16-byte aligned");
    if (use_igemm(*d, 0)) return trb::igemm_wgrad(*d, dy, x, dw, workspace, workspace_bytes, trb::as_stream(stream));
    if (use_strided(*d, 0)) return trb::strided_wgrad(*d, dy, x, dw, workspace, workspace_bytes, trb::as_stream(stream));
    if (use_stem(*d, 0)) return trb::stem_wgrad(*d, dy, x, dw, workspace, workspace_bytes, trb::as_stream(stream));
    return trb::wgrad_direct(*d, dy, x, dw, workspace, workspace_bytes, trb::as_stream(stream));
}

extern "C" int trb200_conv_dgrad(const trb200_conv_desc* d, const void* dy, const void* w, void* dx, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    int rc = trb::validate_conv_desc(d, "conv_dgrad");
    if (rc) return rc;
    TRB_REQUIRE(dy && w && dx, TRB200_ERR_INVALID_ARGUMENT, "conv_dgrad: null pointer");
    TRB_REQUIRE(dx != dy && dx != w, TRB200_ERR_INVALID_ARGUMENT, "conv_dgrad: dx must not alias dy or w");
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(w) && trb::aligned16(dx), TRB200_ERR_INVALID_ARGUMENT,
                "conv_dgrad: tensors must be 16-byte aligned");
    if (use_igemm(*d, 1)) return trb::igemm_dgrad(*d, dy, w, dx, workspace, workspace_bytes, trb::as_stream(stream));
    if (use_strided(*d, 1)) return trb::strided_dgrad(*d, dy, w, dx, workspace, workspace_bytes, trb::as_stream(stream));
    return trb::dgrad_direct(*d, dy, w, dx, trb::as_stream(stream));
}

extern "C" size_t trb200_conv_fprop_workspace_bytes(const trb200_conv_desc* d) {
    if (trb::validate_conv_desc(d, "conv_fprop_workspace_bytes")) return 0;
    if (trb::igemm_supports(*d, 2)) return trb::igemm_fprop_workspace(*d);
    if (trb::strided_supports(*d, 2)) return trb::strided_workspace(*d, 2);
    return trb::stem_supports(*d, 2) ? trb::stem_workspace(*d, 2) : 0;
}

extern "C" int trb200_conv_fprop(const trb200_conv_desc* d, const void* x, const void* w, void* y, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    int rc = trb::validate_conv_desc(d, "conv_fprop");
    if (rc) return rc;
    TRB_REQUIRE(x && w && y, TRB200_ERR_INVALID_ARGUMENT, "conv_fprop: null pointer");
    TRB_REQUIRE(y != x && y != w, TRB200_ERR_INVALID_ARGUMENT, "conv_fprop: y must not alias x or w");
    TRB_REQUIRE(trb::aligned16(x) && trb::aligned16(w) && trb::aligned16(y), TRB200_ERR_INVALID_ARGUMENT,
                "conv_fprop: tensors must be 16-byte aligned");
    if (!trb::igemm_supports(*d, 2) && trb::strided_supports(*d, 2))
        return trb::strided_fprop(*d, x, w, y, workspace, workspace_bytes, trb::as_stream(stream));
    if (!trb::igemm_supports(*d, 2) && trb::stem_supports(*d, 2))
        return trb::stem_fprop(*d, x, w, y, workspace, workspace_bytes, trb::as_stream(stream));
    TRB_REQUIRE(trb::igemm_supports(*d, 2), TRB200_ERR_UNSUPPORTED,
                "conv_fprop: only 3x3 pad 1 (c = 4 at stride 1, or a multiple of 64) and 1x1 pad 0 (c a multiple of 64) "
                "at stride 1 or 2, with k = 64, 128 or a multiple of 256");
    return trb::igemm_fprop(*d, x, w, y, workspace, workspace_bytes, trb::as_stream(stream));
}

extern "C" size_t trb200_conv_fprop_bn_stats_workspace_bytes(const trb200_conv_desc* d) {
    if (trb::validate_conv_desc(d, "conv_fprop_bn_stats_workspace_bytes")) return 0;
    if (trb::igemm_s2_supports(*d, 2)) return trb::igemm_fprop_stats_bytes(*d);
    if (!trb::igemm_supports(*d, 2)) return 0;
    return (size_t)trb::align_up((int64_t)trb::igemm_fprop_workspace(*d), 256) + trb::igemm_fprop_stats_bytes(*d);
}

extern "C" int trb200_conv_fprop_bn_stats(const trb200_conv_desc* d, const void* x, const void* w, void* y,
                                          const float* gamma, const float* beta, float eps, float momentum,
                                          float* ch_sum, float* ch_sqsum, float* saved_mean, float* saved_inv_std,
                                          float* eq_scale, float* eq_bias, float* running_mean, float* running_var,
                                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = trb::validate_conv_desc(d, "conv_fprop_bn_stats");
    if (rc) return rc;
    TRB_REQUIRE(x && w && y && gamma && beta && saved_mean && saved_inv_std && eq_scale && eq_bias,
                TRB200_ERR_INVALID_ARGUMENT, "conv_fprop_bn_stats: null pointer");
    TRB_REQUIRE(y != x && y != w, TRB200_ERR_INVALID_ARGUMENT, "conv_fprop_bn_stats: y must not alias x or w");
    TRB_REQUIRE(trb::aligned16(x) && trb::aligned16(w) && trb::aligned16(y), TRB200_ERR_INVALID_ARGUMENT,
                "conv_fprop_bn_stats: tensors must be 16-byte aligned");
    const bool s2 = trb::igemm_s2_supports(*d, 2);
    TRB_REQUIRE(s2 || trb::igemm_supports(*d, 2), TRB200_ERR_UNSUPPORTED,
                "conv_fprop_bn_stats: only 3x3 pad 1 (c = 4 at stride 1, or a multiple of 64 at stride 1 or 2) and 1x1 pad 0 "
                "(c a multiple of 64, stride 1 or 2), with k = 64, 128 or a multiple of 256");
    const size_t need = trb200_conv_fprop_bn_stats_workspace_bytes(d);
    TRB_REQUIRE(workspace && workspace_bytes >= need, TRB200_ERR_WORKSPACE,
                "conv_fprop_bn_stats: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv_fprop_bn_stats: workspace must be 256-byte aligned");
    // the statistics scratch sits at the END of the workspace so that a caller can hand over an
    // activation-sized buffer followed by a small tail
    unsigned char* base = static_cast<unsigned char*>(workspace);
    const size_t stats_bytes = trb::igemm_fprop_stats_bytes(*d);
    float* partial = reinterpret_cast<float*>(base + (workspace_bytes - stats_bytes) / 256 * 256);
    int strips = 0;
    if (s2) rc = trb::igemm_s2_fprop(*d, x, w, y, trb::as_stream(stream), partial, &strips);
    else rc = trb::igemm_fprop(*d, x, w, y, workspace, workspace_bytes - stats_bytes, trb::as_stream(stream), partial, &strips);
    if (rc) return rc;
    const int oh = trb::conv_out(d->h, d->pad_h, d->r, d->stride_h), ow = trb::conv_out(d->w, d->pad_w, d->s, d->stride_w);
    return trb::bn_finalize_from_partials(partial, strips, d->k, (int64_t)d->n * oh * ow, gamma, beta, eps, momentum,
                                          ch_sum, ch_sqsum, saved_mean, saved_inv_std, eq_scale, eq_bias, running_mean,
                                          running_var, trb::as_stream(stream));
}

// ---------------------------------------------------------------------------
// Whole block.  Workspace layout: [bnrelu partials][wgrad scratch][dgrad scratch],
// each 256-byte aligned, so that the three stages can run on three streams.
// ---------------------------------------------------------------------------
namespace {
struct BlockWs {
    size_t bn_off, bn_bytes, wg_off, wg_bytes, dg_off, dg_bytes, total;
};

BlockWs block_ws(const trb200_conv_desc& d, bool first_layer) {
    const int oh = trb::conv_out(d.h, d.pad_h, d.r, d.stride_h), ow = trb::conv_out(d.w, d.pad_w, d.s, d.stride_w);
    BlockWs b;
    b.bn_off = 0;
    b.bn_bytes = trb200_bnrelu_bwd_workspace_bytes((int64_t)d.n * oh * ow, d.k);
    if (oh % 2 == 0 && ow % 2 == 0) {       // room for the pooled variant of stage 1 as well
        const size_t pooled = trb::bnrelu_pool_bwd_workspace(d.n, oh, ow, d.k);
        if (pooled > b.bn_bytes) b.bn_bytes = pooled;
    }
    b.wg_off = (size_t)trb::align_up((int64_t)b.bn_bytes, 256);
    b.wg_bytes = trb200_conv_wgrad_workspace_bytes(&d);
    b.dg_off = b.wg_off + (size_t)trb::align_up((int64_t)b.wg_bytes, 256);
    b.dg_bytes = first_layer ? 0 : trb200_conv_dgrad_workspace_bytes(&d);
    b.total = b.dg_off + (size_t)trb::align_up((int64_t)b.dg_bytes, 256);
    return b;
}
}  // namespace

extern "C" size_t trb200_cbr_bwd_workspace_bytes(const trb200_conv_desc* d, int first_layer) {
    if (trb::validate_conv_desc(d, "cbr_bwd_workspace_bytes")) return 0;
    return block_ws(*d, first_layer != 0).total;
}

extern "C" int trb200_cbr_bwd(const trb200_cbr_bwd_args* a) {
    TRB_REQUIRE(a, TRB200_ERR_INVALID_ARGUMENT, "cbr_bwd: null argument block");
    const trb200_conv_desc& d = a->conv;
    int rc = trb::validate_conv_desc(&d, "cbr_bwd");
    if (rc) return rc;
    TRB_REQUIRE(a->dy && a->w && a->gamma && a->saved_mean && a->saved_inv_std && a->mask_bits && a->x && a->dw &&
                    a->dgamma && a->dbeta && a->conv_out && a->bn_scratch,
                TRB200_ERR_INVALID_ARGUMENT, "cbr_bwd: null pointer");
    TRB_REQUIRE(d.k % 8 == 0, TRB200_ERR_UNSUPPORTED, "cbr_bwd: k must be a multiple of 8 (k=%d)", d.k);
    const bool first = a->dx == nullptr;
    const BlockWs ws = block_ws(d, first);
    TRB_REQUIRE(ws.total == 0 || (a->workspace && a->workspace_bytes >= ws.total), TRB200_ERR_WORKSPACE,
                "cbr_bwd: workspace of %zu bytes needed, %zu given", ws.total, a->workspace_bytes);
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "cbr_bwd: workspace must be 256-byte aligned");
    cudaStream_t s_bn = trb::as_stream(a->stream_bn), s_wg = trb::as_stream(a->stream_wgrad),
                 s_dg = trb::as_stream(a->stream_dgrad);
    const bool multi = (s_wg != s_bn) || (s_dg != s_bn);
    TRB_REQUIRE(!multi || (a->ev_bn && a->ev_wgrad && (first || a->ev_dgrad)), TRB200_ERR_INVALID_ARGUMENT,
                "cbr_bwd: events are required when the streams differ");
    unsigned char* wsp = static_cast<unsigned char*>(a->workspace);
    const int oh = trb::conv_out(d.h, d.pad_h, d.r, d.stride_h), ow = trb::conv_out(d.w, d.pad_w, d.s, d.stride_w);

    if (a->ev_time[0]) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_time[0]), s_bn));
    // 1) BN + ReLU backward: dconv -> bn_scratch, dgamma, dbeta
    TRB_REQUIRE(!a->pool_argmax || d.dtype == TRB200_DTYPE_F16, TRB200_ERR_UNSUPPORTED,
                "cbr_bwd: the pooled variant is built for half tensors only");
    if (a->pool_argmax)
        rc = trb::bnrelu_pool_bwd_launch(a->dy, a->pool_argmax, a->mask_bits, a->conv_out, a->gamma, a->saved_mean,
                                         a->saved_inv_std, a->bn_scratch, a->dgamma, a->dbeta, d.n, oh, ow, d.k,
                                         wsp + ws.bn_off, ws.bn_bytes, s_bn);
    else
        rc = trb::bnrelu_bwd_launch(a->dy, a->mask_bits, a->conv_out, a->gamma, a->saved_mean, a->saved_inv_std,
                                    a->bn_scratch, a->dgamma, a->dbeta, (int64_t)d.n * oh * ow, d.k, wsp + ws.bn_off,
                                    ws.bn_bytes, s_bn, d.dtype);
    if (rc) return rc;
    if (a->ev_bn) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_bn), s_bn));
    if (a->ev_time[1]) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_time[1]), s_bn));

    // 2) wgrad(dconv, x) -> dw
    if (s_wg != s_bn) TRB_CUDA_TRY(cudaStreamWaitEvent(s_wg, trb::as_event(a->ev_bn), 0));
    rc = trb200_conv_wgrad(&d, a->bn_scratch, a->x, a->dw, wsp + ws.wg_off, ws.wg_bytes, s_wg);
    if (rc) return rc;
    if (a->ev_wgrad) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_wgrad), s_wg));
    if (a->ev_time[2]) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_time[2]), s_wg));

    // 3) dgrad(dconv, w) -> dx, after wgrad has read x (dx is x's buffer)
    if (!first) {
        if (s_dg != s_wg) TRB_CUDA_TRY(cudaStreamWaitEvent(s_dg, trb::as_event(a->ev_wgrad), 0));
        rc = trb200_conv_dgrad(&d, a->bn_scratch, a->w, a->dx, wsp + ws.dg_off, ws.dg_bytes, s_dg);
        if (rc) return rc;
        if (a->ev_dgrad) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_dgrad), s_dg));
        if (a->ev_time[3]) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_time[3]), s_dg));
    }

    // 4) join back onto the BN stream
    if (s_wg != s_bn) TRB_CUDA_TRY(cudaStreamWaitEvent(s_bn, trb::as_event(a->ev_wgrad), 0));
    if (!first && s_dg != s_bn) TRB_CUDA_TRY(cudaStreamWaitEvent(s_bn, trb::as_event(a->ev_dgrad), 0));
    if (a->ev_bn) TRB_CUDA_TRY(cudaEventRecord(trb::as_event(a->ev_bn), s_bn));
    return TRB200_OK;
}
