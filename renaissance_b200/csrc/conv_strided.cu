// Stride-2 convolutions (3x3 pad 1 and 1x1 pad 0, the two kinds ResNet-50 has besides its 7x7 stem) on the
// tensor-core kernels.
//
// Channel counts the implicit-GEMM kernels tile (multiples of 64 with 64, 128 or a multiple of 256 on the output
// side) run without any resampling (conv_igemm_sm100.cu, igemm_s2_*): forward and weight gradient read x through a
// tensor map that steps two pixels, the 3x3 data gradient is four stride-1 convolutions of dy, one per parity class
// of the dx pixel, with 1 + 2 + 2 + 4 taps.  What is left takes the stride-1 kernels plus one resampling pass:
//
//   3x3 s2 p1   y  = even pixels of the stride-1 convolution of x                 (forward)
//               dx = stride-1 data gradient of dy with zeros put between its pixels
//               dW = stride-1 weight gradient of that zero-stuffed dy against x
//   1x1 s2 p0   y  = 1x1 convolution of the even pixels of x
//               dW = 1x1 weight gradient of dy against the even pixels of x
//               dx = 1x1 data gradient of dy, written to the even pixels of a zeroed dx   (always this route)
//
// The 3x3 resampling route spends four times the flops of the native one.  Results equal the strided convolution's
// exactly up to summation order: the extra terms are exact zeros.
//
// A network's first convolution (4 input channels = RGB + 1 pad, any filter size, stride and padding; ResNet-50's
// 7x7 stride-2 stem) is lowered instead: every output pixel's receptive field is written out as one row of
// r*s*4 values padded to a multiple of 64, after which the forward convolution and the weight gradient are 1x1
// convolutions over that buffer on the same kernels.  The buffer is written and read once (n*oh*ow*2*Kpad bytes,
// 1.6 GB for the stem at batch 256), a millisecond of HBM time against the tens of milliseconds of the direct
// kernels.
//
// Reference counterparts: the same cuDNN-FE conv_dgrad / conv_wgrad / conv_fprop graphs with stride 2,
// src/backend/ops/dtensor/cbr_op.cpp:622-917.
#include "common.cuh"
#include "conv.cuh"

namespace trb {
namespace {

// out[n][oh][ow][:] = in[n][2*oh][2*ow][:], 16-byte vectors (vec = channels / 8)
__global__ void __launch_bounds__(256)
subsample2_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int n, int h, int w, int oh_n, int ow_n,
                  int vec) {
    const int64_t total = (int64_t)n * oh_n * ow_n * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        int64_t pix = i / vec;
        const int ow = (int)(pix % ow_n);
        pix /= ow_n;
        const int oh = (int)(pix % oh_n);
        const int64_t img = pix / oh_n;
        out[i] = in[((img * h + 2 * oh) * w + 2 * ow) * vec + v];
    }
}

// out[n][ih][iw][:] = (ih, iw both even) ? in[n][ih/2][iw/2][:] : 0
__global__ void __launch_bounds__(256)
upsample_zero2_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int n, int h, int w, int oh_n, int ow_n,
                      int vec) {
    const int64_t total = (int64_t)n * h * w * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec);
        int64_t pix = i / vec;
        const int iw = (int)(pix % w);
        pix /= w;
        const int ih = (int)(pix % h);
        const int64_t img = pix / h;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (!(ih & 1) && !(iw & 1)) val = in[((img * oh_n + (ih >> 1)) * ow_n + (iw >> 1)) * vec + v];
        out[i] = val;
    }
}

int resample_blocks(int64_t total) {
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

int subsample2(const void* in, void* out, int n, int h, int w, int ch, cudaStream_t st) {
    const int oh = (h - 1) / 2 + 1, ow = (w - 1) / 2 + 1;
    subsample2_kernel<<<resample_blocks((int64_t)n * oh * ow * (ch / 8)), 256, 0, st>>>(
        static_cast<const uint4*>(in), static_cast<uint4*>(out), n, h, w, oh, ow, ch / 8);
    TRB_LAUNCH_CHECK("subsample2_kernel");
    return TRB200_OK;
}

int upsample_zero2(const void* in, void* out, int n, int h, int w, int ch, cudaStream_t st) {
    const int oh = (h - 1) / 2 + 1, ow = (w - 1) / 2 + 1;
    upsample_zero2_kernel<<<resample_blocks((int64_t)n * h * w * (ch / 8)), 256, 0, st>>>(
        static_cast<const uint4*>(in), static_cast<uint4*>(out), n, h, w, oh, ow, ch / 8);
    TRB_LAUNCH_CHECK("upsample_zero2_kernel");
    return TRB200_OK;
}

bool is_3x3_s2_p1(const trb200_conv_desc& d) {
    return d.r == 3 && d.s == 3 && d.pad_h == 1 && d.pad_w == 1 && d.stride_h == 2 && d.stride_w == 2;
}
bool is_1x1_s2_p0(const trb200_conv_desc& d) {
    return d.r == 1 && d.s == 1 && d.pad_h == 0 && d.pad_w == 0 && d.stride_h == 2 && d.stride_w == 2;
}

int out_h(const trb200_conv_desc& d) { return (d.h - 1) / 2 + 1; }
int out_w(const trb200_conv_desc& d) { return (d.w - 1) / 2 + 1; }

// The stride-1 problem the tensor-core kernels are given: the 3x3 one at the input's resolution, the 1x1 one
// at the output's.
trb200_conv_desc dense_desc(const trb200_conv_desc& d) {
    trb200_conv_desc e = d;
    e.stride_h = e.stride_w = 1;
    if (is_1x1_s2_p0(d)) { e.h = out_h(d); e.w = out_w(d); }
    return e;
}

// bytes of the resampled tensor that sits at the front of the workspace
size_t temp_bytes(const trb200_conv_desc& d, int which) {
    int64_t elems;
    if (is_3x3_s2_p1(d)) elems = (int64_t)d.n * d.h * d.w * d.k;                          // y or dy at full resolution
    else elems = (int64_t)d.n * out_h(d) * out_w(d) * d.c;                                // x or dx at half resolution
    (void)which;
    return (size_t)align_up(elems * 2, 256);
}

size_t inner_bytes(const trb200_conv_desc& d, int which) {
    const trb200_conv_desc e = dense_desc(d);
    if (which == 0) return igemm_wgrad_workspace(e);
    if (which == 1) return igemm_dgrad_workspace(e);
    return igemm_fprop_workspace(e);
}

// ---- first-layer lowering (c = 4)
bool is_stem(const trb200_conv_desc& d) { return d.c == 4 && d.r * d.s * 4 <= 1024; }
int stem_kpad(const trb200_conv_desc& d) { return (int)align_up((int64_t)d.r * d.s * 4, 64); }
int stem_oh(const trb200_conv_desc& d) { return conv_out(d.h, d.pad_h, d.r, d.stride_h); }
int stem_ow(const trb200_conv_desc& d) { return conv_out(d.w, d.pad_w, d.s, d.stride_w); }

// the 1x1 problem over the lowered buffer: [n, oh, ow, Kpad] -> k filters
trb200_conv_desc stem_desc(const trb200_conv_desc& d) {
    trb200_conv_desc e = d;
    e.h = stem_oh(d); e.w = stem_ow(d);
    e.c = stem_kpad(d);
    e.r = e.s = 1;
    e.pad_h = e.pad_w = 0;
    e.stride_h = e.stride_w = 1;
    return e;
}

// rows[pixel][slot] (8 bytes = 4 channels): slot = r * S + s holds x[n, oh*stride + r - pad, ow*stride + s - pad, :],
// zeros outside the image and in the padding slots
__global__ void __launch_bounds__(256)
lower_c4_kernel(const uint2* __restrict__ x, uint2* __restrict__ rows, trb200_conv_desc d, int oh_n, int ow_n,
                int slots) {
    const int64_t total = (int64_t)d.n * oh_n * ow_n * slots;
    const int taps = d.r * d.s;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int slot = (int)(i % slots);
        int64_t pix = i / slots;
        const int ow = (int)(pix % ow_n);
        pix /= ow_n;
        const int oh = (int)(pix % oh_n);
        const int64_t img = pix / oh_n;
        uint2 v = make_uint2(0, 0);
        if (slot < taps) {
            const int ih = oh * d.stride_h + slot / d.s - d.pad_h, iw = ow * d.stride_w + slot % d.s - d.pad_w;
            if (ih >= 0 && ih < d.h && iw >= 0 && iw < d.w) v = x[(img * d.h + ih) * d.w + iw];
        }
        rows[i] = v;
    }
}

// wp[k][j] = j < cols ? w[k][j] : 0, and back (16-bit elements of either type)
__global__ void pad_rows_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wp, int kk, int cols, int kpad) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kk * kpad) return;
    const int k = i / kpad, j = i % kpad;
    wp[i] = j < cols ? w[k * cols + j] : (uint16_t)0;
}
__global__ void unpad_rows_kernel(const uint16_t* __restrict__ dwp, uint16_t* __restrict__ dw, int kk, int cols,
                                  int kpad) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kk * cols) return;
    dw[i] = dwp[(i / cols) * kpad + i % cols];
}

size_t stem_rows_bytes(const trb200_conv_desc& d) {
    return (size_t)align_up((int64_t)d.n * stem_oh(d) * stem_ow(d) * stem_kpad(d) * 2, 256);
}
size_t stem_filter_bytes(const trb200_conv_desc& d) { return (size_t)align_up((int64_t)d.k * stem_kpad(d) * 2, 256); }

int stem_lower(const trb200_conv_desc& d, const void* x, void* rows, cudaStream_t st) {
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 7u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv: a 4-channel input must be 8-byte aligned");
    const int slots = stem_kpad(d) / 4;
    lower_c4_kernel<<<resample_blocks((int64_t)d.n * stem_oh(d) * stem_ow(d) * slots), 256, 0, st>>>(
        static_cast<const uint2*>(x), static_cast<uint2*>(rows), d, stem_oh(d), stem_ow(d), slots);
    TRB_LAUNCH_CHECK("lower_c4_kernel");
    return TRB200_OK;
}

}  // namespace

// First layer through the lowering: forward (which = 2) and weight gradient (0); it has no data gradient.
bool stem_supports(const trb200_conv_desc& d, int which) {
    if (!is_stem(d) || which == 1) return false;
    return igemm_supports(stem_desc(d), which);
}

size_t stem_workspace(const trb200_conv_desc& d, int which) {
    const trb200_conv_desc e = stem_desc(d);
    const size_t inner = which == 0 ? igemm_wgrad_workspace(e) : igemm_fprop_workspace(e);
    return stem_rows_bytes(d) + stem_filter_bytes(d) + (size_t)align_up((int64_t)inner, 256);
}

#define TRB_STEM_PROLOGUE(who)                                                                                 \
    const size_t need = stem_workspace(d, which);                                                              \
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, who ": workspace of %zu bytes needed, %zu given", \
                need, ws_bytes);                                                                               \
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,                     \
                who ": workspace must be 256-byte aligned");                                                   \
    unsigned char* rows = static_cast<unsigned char*>(ws);                                                     \
    unsigned char* filt = rows + stem_rows_bytes(d);                                                           \
    unsigned char* inner = filt + stem_filter_bytes(d);                                                        \
    const size_t inner_size = ws_bytes - stem_rows_bytes(d) - stem_filter_bytes(d);                            \
    const trb200_conv_desc e = stem_desc(d);                                                                   \
    const int cols = d.r * d.s * 4, kpad = stem_kpad(d)

int stem_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
               cudaStream_t st) {
    const int which = 0;
    TRB_STEM_PROLOGUE("conv_wgrad");
    int rc = stem_lower(d, x, rows, st);
    if (rc) return rc;
    rc = igemm_wgrad(e, dy, rows, filt, inner, inner_size, st);
    if (rc) return rc;
    unpad_rows_kernel<<<(d.k * cols + 255) / 256, 256, 0, st>>>(reinterpret_cast<const uint16_t*>(filt),
                                                                static_cast<uint16_t*>(dw), d.k, cols, kpad);
    TRB_LAUNCH_CHECK("unpad_rows_kernel");
    return TRB200_OK;
}

int stem_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
               cudaStream_t st) {
    const int which = 2;
    TRB_STEM_PROLOGUE("conv_fprop");
    int rc = stem_lower(d, x, rows, st);
    if (rc) return rc;
    pad_rows_kernel<<<(d.k * kpad + 255) / 256, 256, 0, st>>>(static_cast<const uint16_t*>(w),
                                                              reinterpret_cast<uint16_t*>(filt), d.k, cols, kpad);
    TRB_LAUNCH_CHECK("pad_rows_kernel");
    return igemm_fprop(e, rows, filt, y, inner, inner_size, st);
}

bool strided_supports(const trb200_conv_desc& d, int which) {
    if (!is_3x3_s2_p1(d) && !is_1x1_s2_p0(d)) return false;
    if (d.c % 64 != 0 || d.k % 64 != 0) return false;
    return igemm_supports(dense_desc(d), which);
}

size_t strided_workspace(const trb200_conv_desc& d, int which) {
    if (igemm_s2_supports(d, which)) return igemm_s2_workspace(d, which);
    return temp_bytes(d, which) + (size_t)align_up((int64_t)inner_bytes(d, which), 256);
}

#define TRB_STRIDED_PROLOGUE(who)                                                                              \
    const size_t need = strided_workspace(d, which);                                                           \
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, who ": workspace of %zu bytes needed, %zu given", \
                need, ws_bytes);                                                                               \
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,                     \
                who ": workspace must be 256-byte aligned");                                                   \
    unsigned char* temp = static_cast<unsigned char*>(ws);                                                     \
    unsigned char* inner = temp + temp_bytes(d, which);                                                        \
    const size_t inner_size = ws_bytes - temp_bytes(d, which);                                                 \
    const trb200_conv_desc e = dense_desc(d)

int strided_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
    const int which = 0;
    if (igemm_s2_supports(d, which)) return igemm_s2_wgrad(d, dy, x, dw, ws, ws_bytes, st);
    TRB_STRIDED_PROLOGUE("conv_wgrad");
    int rc;
    if (is_3x3_s2_p1(d)) {
        rc = upsample_zero2(dy, temp, d.n, d.h, d.w, d.k, st);
        if (rc) return rc;
        return igemm_wgrad(e, temp, x, dw, inner, inner_size, st);
    }
    rc = subsample2(x, temp, d.n, d.h, d.w, d.c, st);
    if (rc) return rc;
    return igemm_wgrad(e, dy, temp, dw, inner, inner_size, st);
}

int strided_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
    const int which = 1;
    if (igemm_s2_supports(d, which)) return igemm_s2_dgrad(d, dy, w, dx, ws, ws_bytes, st);
    TRB_STRIDED_PROLOGUE("conv_dgrad");
    int rc;
    if (is_3x3_s2_p1(d)) {
        rc = upsample_zero2(dy, temp, d.n, d.h, d.w, d.k, st);
        if (rc) return rc;
        return igemm_dgrad(e, temp, w, dx, inner, inner_size, st);
    }
    rc = igemm_dgrad(e, dy, w, temp, inner, inner_size, st);
    if (rc) return rc;
    return upsample_zero2(temp, dx, d.n, d.h, d.w, d.c, st);
}

int strided_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
    const int which = 2;
    if (igemm_s2_supports(d, which)) return igemm_s2_fprop(d, x, w, y, st);
    TRB_STRIDED_PROLOGUE("conv_fprop");
    int rc;
    if (is_3x3_s2_p1(d)) {
        rc = igemm_fprop(e, x, w, temp, inner, inner_size, st);
        if (rc) return rc;
        return subsample2(temp, y, d.n, d.h, d.w, d.k, st);
    }
    rc = subsample2(x, temp, d.n, d.h, d.w, d.c, st);
    if (rc) return rc;
    return igemm_fprop(e, temp, w, y, inner, inner_size, st);
}

}  // namespace trb
