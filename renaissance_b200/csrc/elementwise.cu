// Small streaming kernels either side of the gradient all-reduce, and the element-wise pieces of a residual
// block (sum of two branches, ReLU with the block's bit-packed mask, its backward).
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

// Residual join.  One thread = 8 elements (16 bytes) and, where there is a mask, one mask byte.
//   MODE 0: out = round16(a + b)                                 (AXPY with alpha = 1, axpy_op.cu:30-58, on 16-bit data)
//   MODE 1: t = round16(a + b); out = max(t, 0); mask bit = t > 0 (that AXPY followed by relu_fwd_amp_mask_kernel,
//           relu_op.cu:101-114, the mask bit-packed like the block's)
template <bool BF16, int MODE>
// `out` may be `a` or `b` (in-place join), so none of the three tensor pointers is declared restrict
__device__ __forceinline__ void add_body(const uint4* a, const uint4* b, uint4* out, uint8_t* __restrict__ mask,
                                         int64_t vecs) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        float fa[8], fb[8];
        unpack8_t<BF16>(a[v], fa);
        unpack8_t<BF16>(b[v], fb);
        uint32_t w[4], bits = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[j] = pack2_t<BF16>(fa[2 * j] + fb[2 * j], fa[2 * j + 1] + fb[2 * j + 1]);
            if (MODE == 1) {
                const float2 t = unpack2_t<BF16>(w[j]);            // the rounded sum decides, as in the reference
                const bool p0 = t.x > 0.f, p1 = t.y > 0.f;
                bits |= (p0 ? 1u : 0u) << (2 * j) | (p1 ? 1u : 0u) << (2 * j + 1);
                w[j] = (p0 ? w[j] & 0xffffu : 0u) | (p1 ? w[j] & 0xffff0000u : 0u);
            }
        }
        out[v] = make_uint4(w[0], w[1], w[2], w[3]);
        if (MODE == 1) mask[v] = (uint8_t)bits;
    }
}

__global__ void __launch_bounds__(256)
add16_kernel(const uint4* a, const uint4* b, uint4* out, int64_t vecs, int bf16) {
    if (bf16) add_body<true, 0>(a, b, out, nullptr, vecs);
    else add_body<false, 0>(a, b, out, nullptr, vecs);
}

__global__ void __launch_bounds__(256)
add_relu_mask_kernel(const uint4* a, const uint4* b, uint4* out, uint8_t* __restrict__ mask, int64_t vecs, int bf16) {
    if (bf16) add_body<true, 1>(a, b, out, mask, vecs);
    else add_body<false, 1>(a, b, out, mask, vecs);
}

// dx = mask bit ? dy : 0 (relu_bwd_amp_kernel, relu_op.cu:116-126, with the bit-packed mask); a pure select on
// 16-bit words, so the same for half and bfloat16
__global__ void __launch_bounds__(256)
relu_mask_bwd_kernel(const uint4* dy, const uint8_t* __restrict__ mask, uint4* dx,   // dx may be dy
                     int64_t vecs) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        const uint4 g = dy[v];
        const uint32_t m = mask[v];
        const uint32_t w[4] = {g.x, g.y, g.z, g.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = ((m >> (2 * j)) & 1u ? w[j] & 0xffffu : 0u) | ((m >> (2 * j + 1)) & 1u ? w[j] & 0xffff0000u : 0u);
        dx[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
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

namespace {
int check_join(const void* a, const void* b, const void* out, int64_t n, int32_t dtype, const char* who) {
    TRB_REQUIRE(n >= 0 && n % 8 == 0, TRB200_ERR_INVALID_ARGUMENT, "%s: the element count must be a multiple of 8", who);
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "%s: unknown dtype %d", who, dtype);
    TRB_REQUIRE((a && b && out) || n == 0, TRB200_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    TRB_REQUIRE(trb::aligned16(a) && trb::aligned16(b) && trb::aligned16(out), TRB200_ERR_INVALID_ARGUMENT,
                "%s: tensors must be 16-byte aligned", who);
    return TRB200_OK;
}
}  // namespace

extern "C" int trb200_add16(const void* a, const void* b, void* out, int64_t n, int32_t dtype, void* stream) {
    int rc = check_join(a, b, out, n, dtype, "add16");
    if (rc || n == 0) return rc;
    trb::add16_kernel<<<trb::grid_for(n / 8), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint4*>(out), n / 8,
        dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("add16");
    return TRB200_OK;
}

extern "C" int trb200_add_relu_mask(const void* a, const void* b, void* out, void* mask_bits, int64_t n, int32_t dtype,
                                    void* stream) {
    int rc = check_join(a, b, out, n, dtype, "add_relu_mask");
    if (rc || n == 0) return rc;
    TRB_REQUIRE(mask_bits, TRB200_ERR_INVALID_ARGUMENT, "add_relu_mask: null mask");
    trb::add_relu_mask_kernel<<<trb::grid_for(n / 8), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint4*>(out),
        static_cast<uint8_t*>(mask_bits), n / 8, dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("add_relu_mask");
    return TRB200_OK;
}

extern "C" int trb200_relu_mask_bwd(const void* dy, const void* mask_bits, void* dx, int64_t n, void* stream) {
    int rc = check_join(dy, dy, dx, n, TRB200_DTYPE_F16, "relu_mask_bwd");
    if (rc || n == 0) return rc;
    TRB_REQUIRE(mask_bits, TRB200_ERR_INVALID_ARGUMENT, "relu_mask_bwd: null mask");
    trb::relu_mask_bwd_kernel<<<trb::grid_for(n / 8), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(dy), static_cast<const uint8_t*>(mask_bits), static_cast<uint4*>(dx), n / 8);
    TRB_LAUNCH_CHECK("relu_mask_bwd");
    return TRB200_OK;
}
