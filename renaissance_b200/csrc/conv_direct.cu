// Direct (CUDA-core) convolution gradients for every geometry the tensor-core
// kernels do not take: any filter size, stride and padding, any channel count.
// Same arithmetic as the tensor-core path: 16-bit operands (half or bfloat16), float
// accumulation, 16-bit results; the weight gradient is split over rows of the output image and
// the splits are added in split order, so results are bitwise reproducible.
//
// Reference counterparts: cuDNN-FE conv_dgrad / conv_wgrad graphs,
// src/backend/ops/dtensor/cbr_op.cpp:763-917.
#include "common.cuh"
#include "conv.cuh"

namespace trb {
namespace {

template <bool BF16>
__device__ __forceinline__ void
dgrad_direct_body(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ w,
                  uint16_t* __restrict__ dx, const trb200_conv_desc& d, int oh_n, int ow_n) {
    const int64_t total = (int64_t)d.n * d.h * d.w * d.c;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % d.c);
        int64_t pix = idx / d.c;
        const int iw = (int)(pix % d.w);
        pix /= d.w;
        const int ih = (int)(pix % d.h);
        const int n = (int)(pix / d.h);
        float acc = 0.f;
        for (int r = 0; r < d.r; ++r) {
            const int t = ih + d.pad_h - r;
            if (t < 0 || t % d.stride_h) continue;
            const int oh = t / d.stride_h;
            if (oh >= oh_n) continue;
            for (int s = 0; s < d.s; ++s) {
                const int u = iw + d.pad_w - s;
                if (u < 0 || u % d.stride_w) continue;
                const int ow = u / d.stride_w;
                if (ow >= ow_n) continue;
                const uint16_t* g = dy + (((int64_t)n * oh_n + oh) * ow_n + ow) * d.k;
                const uint16_t* wp = w + ((int64_t)r * d.s + s) * d.c + c;
                const int64_t wk = (int64_t)d.r * d.s * d.c;
                for (int k = 0; k < d.k; ++k)
                    acc = fmaf(load16_t<BF16>(g + k), load16_t<BF16>(wp + k * wk), acc);
            }
        }
        dx[idx] = round16_t<BF16>(acc);
    }
}

__global__ void __launch_bounds__(256)
dgrad_direct_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ w, uint16_t* __restrict__ dx,
                    trb200_conv_desc d, int oh_n, int ow_n) {
    dgrad_direct_body<false>(dy, w, dx, d, oh_n, ow_n);
}

__global__ void __launch_bounds__(256)
dgrad_direct_kernel_bf16(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ w, uint16_t* __restrict__ dx,
                         trb200_conv_desc d, int oh_n, int ow_n) {
    dgrad_direct_body<true>(dy, w, dx, d, oh_n, ow_n);
}

// One thread per dW element and split; split = a range of output rows (n, oh).
template <bool BF16>
__device__ __forceinline__ void
wgrad_direct_body(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x,
                  float* __restrict__ partial, const trb200_conv_desc& d, int oh_n, int ow_n,
                  int rows_per_split) {
    const int n_out = d.k * d.r * d.s * d.c;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    const int c = o % d.c;
    const int s = (o / d.c) % d.s;
    const int r = (o / (d.c * d.s)) % d.r;
    const int k = o / (d.c * d.s * d.r);
    const int total_rows = d.n * oh_n;
    const int q0 = blockIdx.y * rows_per_split;
    const int q1 = min(q0 + rows_per_split, total_rows);
    float acc = 0.f;
    for (int q = q0; q < q1; ++q) {
        const int n = q / oh_n, oh = q % oh_n;
        const int ih = oh * d.stride_h + r - d.pad_h;
        if (ih < 0 || ih >= d.h) continue;
        const uint16_t* g = dy + ((int64_t)q * ow_n) * d.k + k;
        const uint16_t* xr = x + (((int64_t)n * d.h + ih) * d.w) * d.c + c;
        for (int ow = 0; ow < ow_n; ++ow) {
            const int iw = ow * d.stride_w + s - d.pad_w;
            if (iw < 0 || iw >= d.w) continue;
            acc = fmaf(load16_t<BF16>(g + (int64_t)ow * d.k), load16_t<BF16>(xr + (int64_t)iw * d.c), acc);
        }
    }
    partial[(int64_t)blockIdx.y * n_out + o] = acc;
}

__global__ void __launch_bounds__(256)
wgrad_direct_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x, float* __restrict__ partial,
                    trb200_conv_desc d, int oh_n, int ow_n, int rows_per_split) {
    wgrad_direct_body<false>(dy, x, partial, d, oh_n, ow_n, rows_per_split);
}

__global__ void __launch_bounds__(256)
wgrad_direct_kernel_bf16(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x, float* __restrict__ partial,
                         trb200_conv_desc d, int oh_n, int ow_n, int rows_per_split) {
    wgrad_direct_body<true>(dy, x, partial, d, oh_n, ow_n, rows_per_split);
}

__global__ void __launch_bounds__(256)
wgrad_direct_reduce(const float* __restrict__ partial, uint16_t* __restrict__ dw, int n_out, int splits, int bf16) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    float acc = 0.f;
    for (int sp = 0; sp < splits; ++sp) acc += partial[(int64_t)sp * n_out + o];
    dw[o] = bf16 ? round16_t<true>(acc) : round16_t<false>(acc);
}

int direct_splits(const trb200_conv_desc& d) {
    const int oh = conv_out(d.h, d.pad_h, d.r, d.stride_h);
    const int rows = d.n * oh;
    const int n_out = d.k * d.r * d.s * d.c;
    const int blocks_x = (n_out + 255) / 256;
    int want = (sm_count() * 8 + blocks_x - 1) / blocks_x;
    if (want > rows) want = rows;
    if (want > 2048) want = 2048;
    if (want < 1) want = 1;
    return want;
}

}  // namespace

size_t wgrad_direct_workspace(const trb200_conv_desc& d) {
    return (size_t)direct_splits(d) * d.k * d.r * d.s * d.c * sizeof(float);
}

int wgrad_direct(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws,
                 size_t ws_bytes, cudaStream_t st) {
    const int oh = conv_out(d.h, d.pad_h, d.r, d.stride_h), ow = conv_out(d.w, d.pad_w, d.s, d.stride_w);
    const int n_out = d.k * d.r * d.s * d.c;
    const int splits = direct_splits(d);
    const size_t need = wgrad_direct_workspace(d);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE,
                "conv_wgrad: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    const int rows = d.n * oh;
    const int rows_per_split = (rows + splits - 1) / splits;
    dim3 grid((n_out + 255) / 256, splits);
    const bool bf16 = d.dtype == TRB200_DTYPE_BF16;
    (bf16 ? wgrad_direct_kernel_bf16 : wgrad_direct_kernel)<<<grid, 256, 0, st>>>(
        static_cast<const uint16_t*>(dy), static_cast<const uint16_t*>(x), static_cast<float*>(ws), d, oh, ow,
        rows_per_split);
    TRB_LAUNCH_CHECK("wgrad_direct_kernel");
    wgrad_direct_reduce<<<(n_out + 255) / 256, 256, 0, st>>>(static_cast<const float*>(ws),
                                                            static_cast<uint16_t*>(dw), n_out, splits, bf16 ? 1 : 0);
    TRB_LAUNCH_CHECK("wgrad_direct_reduce");
    return TRB200_OK;
}

int dgrad_direct(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, cudaStream_t st) {
    const int oh = conv_out(d.h, d.pad_h, d.r, d.stride_h), ow = conv_out(d.w, d.pad_w, d.s, d.stride_w);
    const int64_t total = (int64_t)d.n * d.h * d.w * d.c;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    (d.dtype == TRB200_DTYPE_BF16 ? dgrad_direct_kernel_bf16 : dgrad_direct_kernel)<<<(int)blocks, 256, 0, st>>>(
        static_cast<const uint16_t*>(dy), static_cast<const uint16_t*>(w), static_cast<uint16_t*>(dx), d, oh, ow);
    TRB_LAUNCH_CHECK("dgrad_direct_kernel");
    return TRB200_OK;
}

}  // namespace trb
