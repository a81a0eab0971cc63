// Max pooling with any window, stride and padding, and global average pooling, on NHWC 16-bit tensors: the two
// pooling operators of a ResNet (3x3 stride-2 pad-1 after the stem, the average over 7x7 before the classifier).
// One thread = 8 adjacent channels (one 16-byte vector) of one pixel.
//
// Reference counterparts:
//   maxpool_amp_fwd_mask_kernel, src/backend/ops/dtensor/maxpool_op.cu:83-133 (mask byte = kh*k + kw of the first
//     maximum, strict comparison in float, -1 for a window with no pixel inside the image);
//   maxpool_bwd_deterministic_kernel, maxpool_op.cu:155-217 (every input pixel gathers, in (oh, ow) order and in
//     float, the dy of the windows whose mask points at it);
//   global average pool: y = sum * (1 / (H*W)), gap_op.cpp:137-155; dx = dy * (1 / (H*W)), gap_op.cu:92-112.
#include "common.cuh"

namespace trb {
namespace {

template <bool BF16>
__device__ __forceinline__ void maxpool_fwd_body(const uint4* __restrict__ x, uint4* __restrict__ y,
                                                 uint2* __restrict__ argmax, int n, int h, int w, int vec, int oh_n,
                                                 int ow_n, int k, int stride, int pad) {
    const int64_t total = (int64_t)n * oh_n * ow_n * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        int64_t pix = i / vec;
        const int ow = (int)(pix % ow_n);
        pix /= ow_n;
        const int oh = (int)(pix % oh_n);
        const int64_t img = pix / oh_n;
        float best[8];
        int pos[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; pos[j] = -1; }
        for (int kh = 0; kh < k; ++kh) {
            const int ih = oh * stride - pad + kh;
            if (ih < 0 || ih >= h) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int iw = ow * stride - pad + kw;
                if (iw < 0 || iw >= w) continue;
                float f[8];
                unpack8_t<BF16>(x[((img * h + ih) * w + iw) * vec + v], f);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (f[j] > best[j]) { best[j] = f[j]; pos[j] = kh * k + kw; }
            }
        }
        uint32_t o[4], a[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = pack2_t<BF16>(best[2 * j], best[2 * j + 1]);   // exact: inputs of this type
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j >> 2] |= (uint32_t)(pos[j] & 0xff) << (8 * (j & 3));
        y[i] = make_uint4(o[0], o[1], o[2], o[3]);
        argmax[i] = make_uint2(a[0], a[1]);
    }
}

__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, uint2* __restrict__ argmax, int n, int h, int w,
                   int vec, int oh_n, int ow_n, int k, int stride, int pad, int bf16) {
    if (bf16) maxpool_fwd_body<true>(x, y, argmax, n, h, w, vec, oh_n, ow_n, k, stride, pad);
    else maxpool_fwd_body<false>(x, y, argmax, n, h, w, vec, oh_n, ow_n, k, stride, pad);
}

template <bool BF16>
__device__ __forceinline__ void maxpool_bwd_body(const uint4* __restrict__ dy, const uint2* __restrict__ argmax,
                                                 uint4* __restrict__ dx, int n, int h, int w, int vec, int oh_n,
                                                 int ow_n, int k, int stride, int pad) {
    const int64_t total = (int64_t)n * h * w * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        int64_t pix = i / vec;
        const int iw = (int)(pix % w);
        pix /= w;
        const int ih = (int)(pix % h);
        const int64_t img = pix / h;
        // output windows that can contain this pixel
        int oh0 = (ih + pad - k + 1 + stride - 1) / stride, oh1 = (ih + pad) / stride + 1;
        int ow0 = (iw + pad - k + 1 + stride - 1) / stride, ow1 = (iw + pad) / stride + 1;
        if (ih + pad - k + 1 < 0) oh0 = 0;              // the division above rounds toward zero, not down
        if (iw + pad - k + 1 < 0) ow0 = 0;
        if (oh1 > oh_n) oh1 = oh_n;
        if (ow1 > ow_n) ow1 = ow_n;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int oh = oh0; oh < oh1; ++oh) {
            const int kh = ih - (oh * stride - pad);
            for (int ow = ow0; ow < ow1; ++ow) {
                const int kw = iw - (ow * stride - pad);
                const int64_t o = ((img * oh_n + oh) * ow_n + ow) * vec + v;
                const uint2 a = argmax[o];
                const uint32_t want = (uint32_t)(kh * k + kw);
                float g[8];
                unpack8_t<BF16>(dy[o], g);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t p = ((j < 4 ? a.x : a.y) >> (8 * (j & 3))) & 0xffu;
                    if (p == want) acc[j] += g[j];
                }
            }
        }
        uint32_t o4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o4[j] = pack2_t<BF16>(acc[2 * j], acc[2 * j + 1]);
        dx[i] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const uint4* __restrict__ dy, const uint2* __restrict__ argmax, uint4* __restrict__ dx, int n, int h,
                   int w, int vec, int oh_n, int ow_n, int k, int stride, int pad, int bf16) {
    if (bf16) maxpool_bwd_body<true>(dy, argmax, dx, n, h, w, vec, oh_n, ow_n, k, stride, pad);
    else maxpool_bwd_body<false>(dy, argmax, dx, n, h, w, vec, oh_n, ow_n, k, stride, pad);
}

// y[n][c] = (sum over h, w in that order, float) * scale
__global__ void __launch_bounds__(256)
avgpool_global_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int n, int hw, int vec, float scale,
                          int bf16) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * vec) return;
    const int v = i % vec;
    const int64_t img = i / vec;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < hw; ++p) {
        float f[8];
        const uint4 raw = x[(img * hw + p) * vec + v];
        if (bf16) unpack8_t<true>(raw, f);
        else unpack8_t<false>(raw, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = bf16 ? pack2_t<true>(acc[2 * j] * scale, acc[2 * j + 1] * scale)
                    : pack2_t<false>(acc[2 * j] * scale, acc[2 * j + 1] * scale);
    y[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// dx[n][h][w][c] = dy[n][c] * scale
__global__ void __launch_bounds__(256)
avgpool_global_bwd_kernel(const uint4* __restrict__ dy, uint4* __restrict__ dx, int n, int hw, int vec, float scale,
                          int bf16) {
    const int64_t total = (int64_t)n * hw * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        const int64_t img = i / ((int64_t)hw * vec);
        float g[8];
        const uint4 raw = dy[img * vec + v];
        if (bf16) unpack8_t<true>(raw, g);
        else unpack8_t<false>(raw, g);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = bf16 ? pack2_t<true>(g[2 * j] * scale, g[2 * j + 1] * scale)
                        : pack2_t<false>(g[2 * j] * scale, g[2 * j + 1] * scale);
        dx[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

int pool_blocks(int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

int check_pool(int n, int h, int w, int c, int k, int stride, int pad, int dtype, const char* who) {
    TRB_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "%s: need positive sizes and c a multiple of 8 (n=%d h=%d w=%d c=%d)", who, n, h, w, c);
    TRB_REQUIRE(k >= 1 && k <= 15 && stride >= 1 && pad >= 0 && pad < k && h + 2 * pad >= k && w + 2 * pad >= k,
                TRB200_ERR_INVALID_ARGUMENT, "%s: bad window (k=%d stride=%d pad=%d)", who, k, stride, pad);
    TRB_REQUIRE(valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "%s: unknown dtype %d", who, dtype);
    return TRB200_OK;
}

}  // namespace
}  // namespace trb

extern "C" int trb200_maxpool_fwd(const void* x, void* y, void* argmax, int32_t n, int32_t h, int32_t w, int32_t c,
                                  int32_t k, int32_t stride, int32_t pad, int32_t dtype, void* stream) {
    int rc = trb::check_pool(n, h, w, c, k, stride, pad, dtype, "maxpool_fwd");
    if (rc) return rc;
    TRB_REQUIRE(x && y && argmax, TRB200_ERR_INVALID_ARGUMENT, "maxpool_fwd: null pointer");
    TRB_REQUIRE(trb::aligned16(x) && trb::aligned16(y) && (reinterpret_cast<uintptr_t>(argmax) & 7u) == 0,
                TRB200_ERR_INVALID_ARGUMENT, "maxpool_fwd: tensors must be 16-byte aligned (argmax: 8)");
    const int oh = trb::conv_out(h, pad, k, stride), ow = trb::conv_out(w, pad, k, stride);
    trb::maxpool_fwd_kernel<<<trb::pool_blocks((int64_t)n * oh * ow * (c / 8)), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(y), static_cast<uint2*>(argmax), n, h, w, c / 8, oh, ow, k,
        stride, pad, dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("maxpool_fwd_kernel");
    return TRB200_OK;
}

extern "C" int trb200_maxpool_bwd(const void* dy, const void* argmax, void* dx, int32_t n, int32_t h, int32_t w,
                                  int32_t c, int32_t k, int32_t stride, int32_t pad, int32_t dtype, void* stream) {
    int rc = trb::check_pool(n, h, w, c, k, stride, pad, dtype, "maxpool_bwd");
    if (rc) return rc;
    TRB_REQUIRE(dy && argmax && dx, TRB200_ERR_INVALID_ARGUMENT, "maxpool_bwd: null pointer");
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(dx) && (reinterpret_cast<uintptr_t>(argmax) & 7u) == 0,
                TRB200_ERR_INVALID_ARGUMENT, "maxpool_bwd: tensors must be 16-byte aligned (argmax: 8)");
    const int oh = trb::conv_out(h, pad, k, stride), ow = trb::conv_out(w, pad, k, stride);
    trb::maxpool_bwd_kernel<<<trb::pool_blocks((int64_t)n * h * w * (c / 8)), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(dy), static_cast<const uint2*>(argmax), static_cast<uint4*>(dx), n, h, w, c / 8, oh,
        ow, k, stride, pad, dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("maxpool_bwd_kernel");
    return TRB200_OK;
}

extern "C" int trb200_avgpool_global_fwd(const void* x, void* y, int32_t n, int32_t h, int32_t w, int32_t c,
                                         int32_t dtype, void* stream) {
    int rc = trb::check_pool(n, h, w, c, 1, 1, 0, dtype, "avgpool_global_fwd");
    if (rc) return rc;
    TRB_REQUIRE(x && y && trb::aligned16(x) && trb::aligned16(y), TRB200_ERR_INVALID_ARGUMENT,
                "avgpool_global_fwd: null or unaligned pointer");
    const int items = n * (c / 8);
    trb::avgpool_global_fwd_kernel<<<(items + 255) / 256, 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(y), n, h * w, c / 8, 1.0f / (float)(h * w),
        dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("avgpool_global_fwd_kernel");
    return TRB200_OK;
}

extern "C" int trb200_avgpool_global_bwd(const void* dy, void* dx, int32_t n, int32_t h, int32_t w, int32_t c,
                                         int32_t dtype, void* stream) {
    int rc = trb::check_pool(n, h, w, c, 1, 1, 0, dtype, "avgpool_global_bwd");
    if (rc) return rc;
    TRB_REQUIRE(dy && dx && trb::aligned16(dy) && trb::aligned16(dx), TRB200_ERR_INVALID_ARGUMENT,
                "avgpool_global_bwd: null or unaligned pointer");
    trb::avgpool_global_bwd_kernel<<<trb::pool_blocks((int64_t)n * h * w * (c / 8)), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(dy), static_cast<uint4*>(dx), n, h * w, c / 8, 1.0f / (float)(h * w),
        dtype == TRB200_DTYPE_BF16);
    TRB_LAUNCH_CHECK("avgpool_global_bwd_kernel");
    return TRB200_OK;
}
