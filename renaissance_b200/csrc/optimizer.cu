// Gradient post-processing after the all-reduce, as one sweep over the flat
// parameter range: non-finite check (loss-scale guard), SGD with momentum on the
// float master weights, and the half working copy.
//
// Reference counterparts: check_nan_kernel (src/backend/ops/range/check_op.cu:15-79),
// momentum update (src/backend/ops/range/optimizer_op.cu:40-60; CPU form
// optimizer_op.cpp:306-313: m = beta*m + g/scaling, w = w*(1-lr*wd) - lr*m; the
// kernels return early when the NaN flag is set, optimizer_op.cu:28) and
// RANGE_CAST_FP32_TO_FP16 of the weights (cast_op.cu:18-37).
#include "common.cuh"

namespace trb {
namespace {

__global__ void __launch_bounds__(256)
check_nonfinite_kernel(const float* __restrict__ g, int64_t n, int* __restrict__ flag) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    bool bad = false;
    const int64_t n4 = n >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = g4[i];
        bad |= !(isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && isfinite(v.w));
    }
    for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        bad |= !isfinite(g[i]);
    if (bad) *flag = 1;
}

__global__ void __launch_bounds__(256)
sgd_momentum_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
                    __half* __restrict__ w16, int64_t n, float lr, float wd, float beta,
                    const float* __restrict__ scaling, const int* __restrict__ skip_flag) {
    if (skip_flag && *skip_flag) return;
    const float sc = scaling ? scaling[0] : 1.0f;
    const float inv = sc != 0.f ? 1.0f / sc : 1.0f;
    const float decay = 1.0f - lr * wd;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n4 = n >> 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 wv = reinterpret_cast<float4*>(w)[i];
        const float4 gv = reinterpret_cast<const float4*>(g)[i];
        float4 mv = reinterpret_cast<float4*>(m)[i];
        mv.x = mv.x * beta + gv.x * inv; mv.y = mv.y * beta + gv.y * inv;
        mv.z = mv.z * beta + gv.z * inv; mv.w = mv.w * beta + gv.w * inv;
        wv.x = wv.x * decay - lr * mv.x; wv.y = wv.y * decay - lr * mv.y;
        wv.z = wv.z * decay - lr * mv.z; wv.w = wv.w * decay - lr * mv.w;
        reinterpret_cast<float4*>(m)[i] = mv;
        reinterpret_cast<float4*>(w)[i] = wv;
        if (w16) {
            const __half2 a = __floats2half2_rn(wv.x, wv.y), b = __floats2half2_rn(wv.z, wv.w);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&a);
            o.y = *reinterpret_cast<const uint32_t*>(&b);
            reinterpret_cast<uint2*>(w16)[i] = o;
        }
    }
    for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float mv = m[i] * beta + g[i] * inv;
        const float wv = w[i] * decay - lr * mv;
        m[i] = mv;
        w[i] = wv;
        if (w16) w16[i] = __float2half_rn(wv);
    }
}

int grid_for(int64_t items) {
    int64_t b = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

}  // namespace
}  // namespace trb

extern "C" int trb200_check_nonfinite(const float* grads, int64_t n, int32_t* flag, void* stream) {
    TRB_REQUIRE(flag && (grads || n == 0) && n >= 0, TRB200_ERR_INVALID_ARGUMENT, "check_nonfinite: bad argument");
    if (n == 0) return TRB200_OK;
    TRB_REQUIRE(trb::aligned16(grads), TRB200_ERR_INVALID_ARGUMENT, "check_nonfinite: grads must be 16-byte aligned");
    trb::check_nonfinite_kernel<<<trb::grid_for((n + 3) / 4), 256, 0, trb::as_stream(stream)>>>(grads, n, flag);
    TRB_LAUNCH_CHECK("check_nonfinite");
    return TRB200_OK;
}

extern "C" int trb200_sgd_momentum(float* weights, const float* grads, float* momentum, void* weights_half,
                                   int64_t n, float lr, float weight_decay, float beta, const float* scaling,
                                   const int32_t* skip_flag, void* stream) {
    TRB_REQUIRE((weights && grads && momentum) || n == 0, TRB200_ERR_INVALID_ARGUMENT, "sgd_momentum: null pointer");
    TRB_REQUIRE(n >= 0, TRB200_ERR_INVALID_ARGUMENT, "sgd_momentum: negative size");
    if (n == 0) return TRB200_OK;
    TRB_REQUIRE(trb::aligned16(weights) && trb::aligned16(grads) && trb::aligned16(momentum) &&
                    (!weights_half || (reinterpret_cast<uintptr_t>(weights_half) & 7u) == 0),
                TRB200_ERR_INVALID_ARGUMENT, "sgd_momentum: buffers must be 16-byte aligned (half copy: 8)");
    trb::sgd_momentum_kernel<<<trb::grid_for((n + 3) / 4), 256, 0, trb::as_stream(stream)>>>(
        weights, grads, momentum, static_cast<__half*>(weights_half), n, lr, weight_decay, beta, scaling, skip_flag);
    TRB_LAUNCH_CHECK("sgd_momentum");
    return TRB200_OK;
}
