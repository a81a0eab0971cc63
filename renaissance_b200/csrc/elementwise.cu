// Small streaming kernels either side of the gradient all-reduce.
#include "common.cuh"

namespace trb {
namespace {

// data[i] *= f  (tr_scale_fp32_kernel, src/backend/ops/range/infra_kernels.cu:82-96)
__global__ void __launch_bounds__(256) scale_f32_kernel(float* __restrict__ data, int64_t n, float f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n4 = n >> 2;
    float4* d4 = reinterpret_cast<float4*>(data);
    for (int64_t v = i; v < n4; v += stride) {
        float4 t = d4[v];
        t.x *= f; t.y *= f; t.z *= f; t.w *= f;
        d4[v] = t;
    }
    for (int64_t t = (n4 << 2) + i; t < n; t += stride) data[t] *= f;
}

// dst[i] = float(src[i]) * f  (cast_fp16_to_fp32_kernel, src/backend/ops/range/cast_op.cu:18-37)
__global__ void __launch_bounds__(256)
cast_f16_f32_kernel(const __half* __restrict__ src, float* __restrict__ dst, int64_t n, float f, int vec_ok) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t n8 = n >> 3;
        for (int64_t v = i; v < n8; v += stride) {
            const uint4 raw = reinterpret_cast<const uint4*>(src)[v];
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
            float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
            float2 c = __half22float2(h[2]), d = __half22float2(h[3]);
            reinterpret_cast<float4*>(dst)[2 * v] = make_float4(a.x * f, a.y * f, b.x * f, b.y * f);
            reinterpret_cast<float4*>(dst)[2 * v + 1] = make_float4(c.x * f, c.y * f, d.x * f, d.y * f);
        }
        done = n8 << 3;
    }
    for (int64_t t = done + i; t < n; t += stride) dst[t] = __half2float(src[t]) * f;
}

int grid_for(int64_t work_items) {
    int64_t blocks = (work_items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace
}  // namespace trb

extern "C" int trb200_scale_f32(float* data, int64_t n, float factor, void* stream) {
    TRB_REQUIRE(data || n == 0, TRB200_ERR_INVALID_ARGUMENT, "scale_f32: null pointer");
    TRB_REQUIRE(n >= 0, TRB200_ERR_INVALID_ARGUMENT, "scale_f32: negative size");
    if (n == 0) return TRB200_OK;
    TRB_REQUIRE(trb::aligned16(data), TRB200_ERR_INVALID_ARGUMENT, "scale_f32: data must be 16-byte aligned");
    trb::scale_f32_kernel<<<trb::grid_for((n + 3) / 4), 256, 0, trb::as_stream(stream)>>>(data, n, factor);
    TRB_LAUNCH_CHECK("scale_f32");
    return TRB200_OK;
}

extern "C" int trb200_cast_f16_to_f32(const void* src, float* dst, int64_t n, float factor, void* stream) {
    TRB_REQUIRE((src && dst) || n == 0, TRB200_ERR_INVALID_ARGUMENT, "cast_f16_to_f32: null pointer");
    TRB_REQUIRE(n >= 0, TRB200_ERR_INVALID_ARGUMENT, "cast_f16_to_f32: negative size");
    if (n == 0) return TRB200_OK;
    const int vec_ok = trb::aligned16(src) && trb::aligned16(dst);
    trb::cast_f16_f32_kernel<<<trb::grid_for((n + 7) / 8), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const __half*>(src), dst, n, factor, vec_ok);
    TRB_LAUNCH_CHECK("cast_f16_to_f32");
    return TRB200_OK;
}
