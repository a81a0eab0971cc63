// Gradient post-processing after the all-reduce, as one sweep over the flat
// parameter range: non-finite check (loss-scale guard) with its clipping variant, the
// loss-scale back-off, SGD / momentum / Nesterov on the float master weights, and the
// half working copy.
//
// Reference counterparts: check_nan_kernel (src/backend/ops/range/check_op.cu:15-79),
// momentum update (src/backend/ops/range/optimizer_op.cu:40-60; CPU form
// optimizer_op.cpp:306-313: m = beta*m + g/scaling, w = w*(1-lr*wd) - lr*m; the
// kernels return early when the NaN flag is set, optimizer_op.cu:28) and
// RANGE_CAST_FP32_TO_FP16 of the weights (cast_op.cu:18-37); check_nan_and_clip_kernel
// (check_op.cu:54-79); grad_scaling_kernel (grad_scaling_op.cu:15-22); update_sgd_kernel and
// update_nesterov_kernel (optimizer_op.cu:22-38, 68-93).
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

// KIND 0: plain SGD (m unused); 1: momentum m = beta*m + g, step m; 2: Nesterov m = beta*m + g, step beta*m + g
template <int KIND>
__device__ __forceinline__ void update_one(float& w, float g, float& m, float inv, float decay, float lr, float beta) {
    const float gi = g * inv;
    if (KIND == 0) {
        w = w * decay - lr * gi;
    } else {
        const float mn = m * beta + gi;
        m = mn;
        w = w * decay - lr * (KIND == 2 ? mn * beta + gi : mn);
    }
}

template <int KIND>
__global__ void __launch_bounds__(256)
sgd_update_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
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
        float4 mv = KIND ? reinterpret_cast<float4*>(m)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        update_one<KIND>(wv.x, gv.x, mv.x, inv, decay, lr, beta);
        update_one<KIND>(wv.y, gv.y, mv.y, inv, decay, lr, beta);
        update_one<KIND>(wv.z, gv.z, mv.z, inv, decay, lr, beta);
        update_one<KIND>(wv.w, gv.w, mv.w, inv, decay, lr, beta);
        if (KIND) reinterpret_cast<float4*>(m)[i] = mv;
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
        float wv = w[i], mv = KIND ? m[i] : 0.f;
        update_one<KIND>(wv, g[i], mv, inv, decay, lr, beta);
        if (KIND) m[i] = mv;
        w[i] = wv;
        if (w16) w16[i] = __float2half_rn(wv);
    }
}

// NaN: raise the flag and leave the value; anything else (infinities included) is clamped to [-clip, clip]
__global__ void __launch_bounds__(256)
check_nan_and_clip_kernel(float* __restrict__ g, int64_t n, float clip, int* __restrict__ flag) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = g[i];
        if (isnan(v)) {
            bad = true;
        } else {
            const float c = fminf(fmaxf(v, -clip), clip);
            if (c != v) g[i] = c;
        }
    }
    if (bad) *flag = 1;
}

// the loss scale halves after a step that saw a NaN, never below 1
__global__ void grad_scaling_kernel(int* __restrict__ has_nan, float* __restrict__ scaling, int clear_flag) {
    if (*has_nan != 0) {
        const float s = *scaling * 0.5f;
        *scaling = s < 1.0f ? 1.0f : s;
        if (clear_flag) *has_nan = 0;
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

static int sgd_update(int kind, float* weights, const float* grads, float* momentum, void* weights_half, int64_t n,
                      float lr, float weight_decay, float beta, const float* scaling, const int32_t* skip_flag,
                      void* stream, const char* who) {
    TRB_REQUIRE((weights && grads && (momentum || kind == 0)) || n == 0, TRB200_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    TRB_REQUIRE(n >= 0, TRB200_ERR_INVALID_ARGUMENT, "%s: negative size", who);
    if (n == 0) return TRB200_OK;
    TRB_REQUIRE(trb::aligned16(weights) && trb::aligned16(grads) && (kind == 0 || trb::aligned16(momentum)) &&
                    (!weights_half || (reinterpret_cast<uintptr_t>(weights_half) & 7u) == 0),
                TRB200_ERR_INVALID_ARGUMENT, "%s: buffers must be 16-byte aligned (half copy: 8)", who);
    const int grid = trb::grid_for((n + 3) / 4);
    cudaStream_t st = trb::as_stream(stream);
    __half* w16 = static_cast<__half*>(weights_half);
    if (kind == 0)
        trb::sgd_update_kernel<0><<<grid, 256, 0, st>>>(weights, grads, momentum, w16, n, lr, weight_decay, beta, scaling, skip_flag);
    else if (kind == 1)
        trb::sgd_update_kernel<1><<<grid, 256, 0, st>>>(weights, grads, momentum, w16, n, lr, weight_decay, beta, scaling, skip_flag);
    else
        trb::sgd_update_kernel<2><<<grid, 256, 0, st>>>(weights, grads, momentum, w16, n, lr, weight_decay, beta, scaling, skip_flag);
    TRB_LAUNCH_CHECK(who);
    return TRB200_OK;
}

extern "C" int trb200_sgd_momentum(float* weights, const float* grads, float* momentum, void* weights_half,
                                   int64_t n, float lr, float weight_decay, float beta, const float* scaling,
                                   const int32_t* skip_flag, void* stream) {
    return sgd_update(1, weights, grads, momentum, weights_half, n, lr, weight_decay, beta, scaling, skip_flag, stream,
                      "sgd_momentum");
}

extern "C" int trb200_sgd_nesterov(float* weights, const float* grads, float* momentum, void* weights_half,
                                   int64_t n, float lr, float weight_decay, float beta, const float* scaling,
                                   const int32_t* skip_flag, void* stream) {
    return sgd_update(2, weights, grads, momentum, weights_half, n, lr, weight_decay, beta, scaling, skip_flag, stream,
                      "sgd_nesterov");
}

extern "C" int trb200_sgd_plain(float* weights, const float* grads, void* weights_half, int64_t n, float lr,
                                float weight_decay, const float* scaling, const int32_t* skip_flag, void* stream) {
    return sgd_update(0, weights, grads, nullptr, weights_half, n, lr, weight_decay, 0.f, scaling, skip_flag, stream,
                      "sgd_plain");
}

extern "C" int trb200_check_nan_and_clip(float* grads, int64_t n, float clip, int32_t* flag, void* stream) {
    TRB_REQUIRE(flag && (grads || n == 0) && n >= 0, TRB200_ERR_INVALID_ARGUMENT, "check_nan_and_clip: bad argument");
    TRB_REQUIRE(clip >= 0.f, TRB200_ERR_INVALID_ARGUMENT, "check_nan_and_clip: negative clip value");
    if (n == 0) return TRB200_OK;
    trb::check_nan_and_clip_kernel<<<trb::grid_for(n), 256, 0, trb::as_stream(stream)>>>(grads, n, clip, flag);
    TRB_LAUNCH_CHECK("check_nan_and_clip");
    return TRB200_OK;
}

extern "C" int trb200_grad_scaling(int32_t* has_nan, float* scaling, int32_t clear_flag, void* stream) {
    TRB_REQUIRE(has_nan && scaling, TRB200_ERR_INVALID_ARGUMENT, "grad_scaling: null pointer");
    trb::grad_scaling_kernel<<<1, 1, 0, trb::as_stream(stream)>>>(has_nan, scaling, clear_flag);
    TRB_LAUNCH_CHECK("grad_scaling");
    return TRB200_OK;
}
