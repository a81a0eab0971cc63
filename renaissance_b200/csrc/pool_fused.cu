// Blocks that are followed by a 2x2 max pool: the pool fused into the block's
// HBM-bound kernels, so that the full-resolution ReLU output (forward) and the
// full-resolution gradient of it (backward) never travel through HBM.
//
//   forward : conv_out -> mask bits (full resolution), pool_out, argmax
//             = bn_apply_relu_mask followed by maxpool2x2_fwd
//   backward: pooled dy + argmax + mask + conv_out -> dconv, dgamma, dbeta
//             = maxpool2x2_bwd followed by bnrelu_bwd
// Reference counterparts: the BN-apply/ReLU/mask graph of the block
// (src/backend/ops/dtensor/cbr_op.cpp:534-616), the max-pool kernels
// (src/backend/ops/dtensor/maxpool_op.cu:23-217) and the BN backward graph
// (cbr_op.cpp:1259-1353); the results are those of the unfused sequence bit for bit
// (forward) and to the summation order of the channel sums (backward).
//
// One work item = one pooled pixel x 8 channels = a 2x2 window of 16-byte vectors.
// Bytes per full-resolution element: forward 2 + 1/8 + (2 + 1)/4 = 2.875 instead of
// 6.875; backward 2 x (2 + 1/8 + 3/4) + 2 = 7.75 instead of 14.75.
#include "common.cuh"

#include <cuda_fp16.h>

namespace trb {
namespace {

constexpr int kThreads = 256;

struct PoolPlan {
    int tpr, bx, by, gy, gx;
    int64_t rows_per_strip;     // pooled pixels per strip
};

PoolPlan make_pool_plan(int64_t pooled_rows, int c) {
    PoolPlan p;
    p.tpr = c / 8;
    p.bx = p.tpr < kThreads ? p.tpr : kThreads;
    p.by = kThreads / p.bx;
    if (p.by < 1) p.by = 1;
    p.gy = (p.tpr + p.bx - 1) / p.bx;
    // strips of at least 4 loop trips, at most 4 waves of 2 resident blocks per SM, whole waves
    int64_t want = (pooled_rows + (int64_t)p.by * 4 - 1) / ((int64_t)p.by * 4);
    int64_t resident = (int64_t)sm_count() * 2 / p.gy;
    if (resident < 1) resident = 1;
    int64_t g = want < resident * 4 ? want : resident * 4;
    if (g > resident) g = g / resident * resident;
    p.gx = (int)(g < 1 ? 1 : g);
    int64_t rps = (pooled_rows + p.gx - 1) / p.gx;
    rps = (rps + p.by - 1) / p.by * p.by;
    p.rows_per_strip = rps;
    p.gx = (int)((pooled_rows + rps - 1) / rps);
    return p;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// full-resolution vector index of window position q (q = kh*2 + kw) of pooled pixel pr.
// Measured, not obvious: cheaper forms of this index (32-bit divisions; one division, using that pooled row t
// starts at full-resolution row 2 * t) made all three pool kernels 7-18 % SLOWER at every size, although they
// execute fewer instructions; the kernels are bound by memory latency, not by issue, and this form stays.
__device__ __forceinline__ int64_t window_base(int64_t pr, int oh_n, int ow_n, int w, int tpr, int vec) {
    const int ow = (int)(pr % ow_n);
    const int64_t t = pr / ow_n;
    const int oh = (int)(t % oh_n);
    const int64_t img = t / oh_n;
    return ((img * (2 * oh_n) + 2 * oh) * (int64_t)w + 2 * ow) * tpr + vec;
}

// t = half(half(x * s) + b) for 8 channels, two per packed conversion (the roundings are those of the scalar form)
__device__ __forceinline__ void bn_apply8(const uint4& v, const float (&sc)[8], const float (&bi)[8], __half2 (&t)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        const float2 a = __half22float2(__floats2half2_rn(f.x * sc[2 * i], f.y * sc[2 * i + 1]));
        t[i] = __floats2half2_rn(a.x + bi[2 * i], a.y + bi[2 * i + 1]);
    }
}

// One mask byte from four packed comparison results (0xffff per true lane): a byte of each lane is gathered, each
// byte keeps its own bit, and a multiply adds the four bytes up in the top byte.
__device__ __forceinline__ uint32_t mask_byte(const uint32_t (&on)[4]) {
    const uint32_t lo = __byte_perm(on[0], on[1], 0x6420) & 0x08040201u;
    const uint32_t hi = __byte_perm(on[2], on[3], 0x6420) & 0x08040201u;
    return ((lo * 0x01010101u) >> 24) | (((hi * 0x01010101u) >> 24) << 4);
}

// One pooled pixel x 8 channels: ReLU output (to relu_out if asked), mask byte of each of the four window positions,
// window maximum and the position of its first occurrence.  Comparisons and selections run on packed halfs.
__device__ __forceinline__ void pool_window(const uint4 (&v)[4], const int64_t (&idx)[4], const float (&sc)[8],
                                            const float (&bi)[8], uint4* __restrict__ relu_out,
                                            uint8_t* __restrict__ mask, uint4& best_out, uint2& am_out) {
    const __half2 zero2 = __float2half2_rn(0.f);
    uint32_t best[4], am[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { best[i] = 0xfc00fc00u; am[i] = 0u; }        // -inf, position 0
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        __half2 t[4];
        bn_apply8(v[q], sc, bi, t);
        uint32_t y[4], on[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            on[i] = __hgt2_mask(t[i], zero2);                                  // 0xffff per lane with t > 0
            y[i] = *reinterpret_cast<const uint32_t*>(&t[i]) & on[i];          // ReLU: +0 where off
            const uint32_t gt = __hgt2_mask(*reinterpret_cast<const __half2*>(&y[i]),
                                            *reinterpret_cast<const __half2*>(&best[i]));   // strictly greater: first wins
            best[i] = (y[i] & gt) | (best[i] & ~gt);
            am[i] = ((uint32_t)(q | (q << 16)) & gt) | (am[i] & ~gt);
        }
        mask[idx[q]] = (uint8_t)mask_byte(on);
        if (relu_out) relu_out[idx[q]] = make_uint4(y[0], y[1], y[2], y[3]);
    }
    best_out = make_uint4(best[0], best[1], best[2], best[3]);
    am_out.x = __byte_perm(am[0], am[1], 0x6420);        // one byte per channel
    am_out.y = __byte_perm(am[2], am[3], 0x6420);
}

__global__ void __launch_bounds__(kThreads)
bn_apply_relu_mask_pool_kernel(const uint4* __restrict__ x, const float* __restrict__ eq_scale,
                               const float* __restrict__ eq_bias, uint4* __restrict__ relu_out,
                               uint8_t* __restrict__ mask, uint4* __restrict__ pool_out,
                               uint2* __restrict__ argmax, int64_t pooled_rows, int oh_n, int ow_n, int w,
                               int tpr, int bx, int by, int64_t rows_per_strip) {
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    if (vec >= tpr || ty >= by) return;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < pooled_rows) ? r0 + rows_per_strip : pooled_rows;
    float sc[8], bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sc[j] = eq_scale[vec * 8 + j]; bi[j] = eq_bias[vec * 8 + j]; }
    const int64_t row_step = (int64_t)w * tpr;       // one image row down
    // two windows (eight 16-byte loads) in flight per thread
    for (int64_t pr = r0 + ty; pr < r1; pr += 2 * (int64_t)by) {
        const int64_t pr2 = pr + by;
        const bool two = pr2 < r1;
        const int64_t b0 = window_base(pr, oh_n, ow_n, w, tpr, vec);
        const int64_t b1 = two ? window_base(pr2, oh_n, ow_n, w, tpr, vec) : b0;
        const int64_t idx0[4] = {b0, b0 + tpr, b0 + row_step, b0 + row_step + tpr};
        const int64_t idx1[4] = {b1, b1 + tpr, b1 + row_step, b1 + row_step + tpr};
        uint4 v0[4], v1[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v0[q] = x[idx0[q]];
#pragma unroll
        for (int q = 0; q < 4; ++q) v1[q] = x[idx1[q]];
        uint4 bv;
        uint2 a;
        pool_window(v0, idx0, sc, bi, relu_out, mask, bv, a);
        pool_out[pr * tpr + vec] = bv;
        argmax[pr * tpr + vec] = a;
        if (two) {
            pool_window(v1, idx1, sc, bi, relu_out, mask, bv, a);
            pool_out[pr2 * tpr + vec] = bv;
            argmax[pr2 * tpr + vec] = a;
        }
    }
}

__global__ void __launch_bounds__(kThreads)
bnrelu_pool_bwd_reduce(const uint4* __restrict__ dy, const uint2* __restrict__ argmax,
                       const uint8_t* __restrict__ mask, const uint4* __restrict__ x,
                       const float* __restrict__ mean, const float* __restrict__ inv_std,
                       float* __restrict__ partial, int64_t pooled_rows, int c, int oh_n, int ow_n, int w,
                       int tpr, int bx, int by, int64_t rows_per_strip) {
    __shared__ float s_red[kThreads * 16];
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    const bool ok = vec < tpr && ty < by;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < pooled_rows) ? r0 + rows_per_strip : pooled_rows;
    float sb[8], sg[8], mu[8], is[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sb[j] = 0.f; sg[j] = 0.f; mu[j] = 0.f; is[j] = 0.f; }
    if (ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { mu[j] = mean[vec * 8 + j]; is[j] = inv_std[vec * 8 + j]; }
        const int64_t row_step = (int64_t)w * tpr;
        for (int64_t pr = r0 + ty; pr < r1; pr += by) {
            const int64_t b0 = window_base(pr, oh_n, ow_n, w, tpr, vec);
            const int64_t idx[4] = {b0, b0 + tpr, b0 + row_step, b0 + row_step + tpr};
            const int64_t po = pr * tpr + vec;
            const uint4 g4 = dy[po];
            const uint2 a2 = argmax[po];
            uint4 xv[4];
            uint32_t mb[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) { xv[q] = x[idx[q]]; mb[q] = mask[idx[q]]; }
            float g[8];
            unpack8(g4, g);
            const uint8_t* ab = reinterpret_cast<const uint8_t*>(&a2);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float xf[8];
                unpack8(xv[q], xf);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float gm = (ab[j] == q && ((mb[q] >> j) & 1u)) ? g[j] : 0.f;
                    sb[j] += gm;
                    sg[j] += gm * ((xf[j] - mu[j]) * is[j]);
                }
            }
        }
    }
    float* mine = s_red + (size_t)threadIdx.x * 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = sb[j]; mine[8 + j] = sg[j]; }
    __syncthreads();
    for (int t = threadIdx.x; t < bx * 16; t += kThreads) {
        const int otx = t / 16, j = t % 16;
        const int ovec = blockIdx.y * bx + otx;
        if (ovec >= tpr) continue;
        float acc = 0.f;
        for (int y = 0; y < by; ++y) acc += s_red[(size_t)(y * bx + otx) * 16 + j];
        partial[((size_t)blockIdx.x * 2 + (j >> 3)) * c + ovec * 8 + (j & 7)] = acc;
    }
}

__global__ void __launch_bounds__(256)
bnrelu_pool_bwd_finalize(const float* __restrict__ partial, float* __restrict__ dgamma,
                         float* __restrict__ dbeta, int c, int strips) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= 2 * c) return;
    const int stat = i / c, ch = i % c;
    // same order of additions as a plain loop over this lane's strips; eight loads are in flight at a time
    // (one dependent load per strip made this kernel as long as its strip count)
    double acc = 0.0;
    for (int s0 = lane; s0 < strips; s0 += 32 * 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int s = s0 + 32 * u;
            v[u] = s < strips ? partial[((size_t)s * 2 + stat) * c + ch] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (s0 + 32 * u < strips) acc += (double)v[u];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) (stat == 0 ? dbeta : dgamma)[ch] = (float)acc;
}

__global__ void __launch_bounds__(kThreads)
bnrelu_pool_bwd_apply(const uint4* __restrict__ dy, const uint2* __restrict__ argmax,
                      const uint8_t* __restrict__ mask, const uint4* __restrict__ x,
                      const float* __restrict__ gamma, const float* __restrict__ mean,
                      const float* __restrict__ inv_std, const float* __restrict__ dgamma,
                      const float* __restrict__ dbeta, uint4* __restrict__ out, int64_t pooled_rows,
                      int64_t m_full, int oh_n, int ow_n, int w, int tpr, int bx, int by,
                      int64_t rows_per_strip) {
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    if (vec >= tpr || ty >= by) return;
    const int strip = gridDim.x - 1 - blockIdx.x;     // the rows the reduce kernel read last are still in L2
    const int64_t r0 = (int64_t)strip * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < pooled_rows) ? r0 + rows_per_strip : pooled_rows;
    float ca[8], cmb[8], cmu[8], ck[8];
    const float inv_m = 1.0f / (float)m_full;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int ch = vec * 8 + j;
        const float is = inv_std[ch];
        ca[j] = gamma[ch] * is;
        cmb[j] = dbeta[ch] * inv_m;
        cmu[j] = mean[ch];
        ck[j] = is * (dgamma[ch] * inv_m);
    }
    const int64_t row_step = (int64_t)w * tpr;
    for (int64_t pr = r0 + ty; pr < r1; pr += by) {
        const int64_t b0 = window_base(pr, oh_n, ow_n, w, tpr, vec);
        const int64_t idx[4] = {b0, b0 + tpr, b0 + row_step, b0 + row_step + tpr};
        const int64_t po = pr * tpr + vec;
        const uint4 g4 = dy[po];
        const uint2 a2 = argmax[po];
        uint4 xv[4];
        uint32_t mb[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { xv[q] = x[idx[q]]; mb[q] = mask[idx[q]]; }
        float g[8];
        unpack8(g4, g);
        const uint8_t* ab = reinterpret_cast<const uint8_t*>(&a2);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float xf[8];
            unpack8(xv[q], xf);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int j0 = 2 * j, j1 = 2 * j + 1;
                const float g0 = (ab[j0] == q && ((mb[q] >> j0) & 1u)) ? g[j0] : 0.f;
                const float g1 = (ab[j1] == q && ((mb[q] >> j1) & 1u)) ? g[j1] : 0.f;
                const float o0 = ca[j0] * (g0 - cmb[j0] - (xf[j0] - cmu[j0]) * ck[j0]);
                const float o1 = ca[j1] * (g1 - cmb[j1] - (xf[j1] - cmu[j1]) * ck[j1]);
                oh[j] = __floats2half2_rn(o0, o1);
            }
            out[idx[q]] = o;
        }
    }
}

int check_pool_shape(int n, int h, int w, int c, const char* who) {
    TRB_REQUIRE(n > 0 && h > 0 && w > 0 && h % 2 == 0 && w % 2 == 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "%s: need even h, w and c a positive multiple of 8 (n=%d h=%d w=%d c=%d)", who, n, h, w, c);
    return TRB200_OK;
}

}  // namespace

size_t bnrelu_pool_bwd_workspace(int n, int h, int w, int c) {
    const PoolPlan p = make_pool_plan((int64_t)n * (h / 2) * (w / 2), c);
    return (size_t)p.gx * 2 * (size_t)c * sizeof(float);
}

int bnrelu_pool_bwd_launch(const void* dy_pooled, const void* argmax, const void* mask_bits, const void* x,
                           const float* gamma, const float* saved_mean, const float* saved_inv_std, void* dconv,
                           float* dgamma, float* dbeta, int n, int h, int w, int c, void* workspace,
                           size_t workspace_bytes, cudaStream_t s) {
    int rc = check_pool_shape(n, h, w, c, "bnrelu_pool_bwd");
    if (rc) return rc;
    TRB_REQUIRE(dy_pooled && argmax && mask_bits && x && gamma && saved_mean && saved_inv_std && dconv && dgamma && dbeta,
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_pool_bwd: null pointer");
    TRB_REQUIRE(aligned16(dy_pooled) && aligned16(x) && aligned16(dconv) && (reinterpret_cast<uintptr_t>(argmax) & 7u) == 0,
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_pool_bwd: tensors must be 16-byte aligned (argmax: 8)");
    TRB_REQUIRE(dconv != x && dconv != dy_pooled, TRB200_ERR_INVALID_ARGUMENT, "bnrelu_pool_bwd: dconv must not alias an input");
    const size_t need = bnrelu_pool_bwd_workspace(n, h, w, c);
    TRB_REQUIRE(workspace && workspace_bytes >= need, TRB200_ERR_WORKSPACE,
                "bnrelu_pool_bwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    const int64_t pooled = (int64_t)n * (h / 2) * (w / 2);
    const PoolPlan p = make_pool_plan(pooled, c);
    float* partial = static_cast<float*>(workspace);
    dim3 grid(p.gx, p.gy);
    bnrelu_pool_bwd_reduce<<<grid, kThreads, 0, s>>>(
        static_cast<const uint4*>(dy_pooled), static_cast<const uint2*>(argmax), static_cast<const uint8_t*>(mask_bits),
        static_cast<const uint4*>(x), saved_mean, saved_inv_std, partial, pooled, c, h / 2, w / 2, w, p.tpr, p.bx, p.by,
        p.rows_per_strip);
    TRB_LAUNCH_CHECK("bnrelu_pool_bwd_reduce");
    bnrelu_pool_bwd_finalize<<<(2 * c + 7) / 8, 256, 0, s>>>(partial, dgamma, dbeta, c, p.gx);
    TRB_LAUNCH_CHECK("bnrelu_pool_bwd_finalize");
    bnrelu_pool_bwd_apply<<<grid, kThreads, 0, s>>>(
        static_cast<const uint4*>(dy_pooled), static_cast<const uint2*>(argmax), static_cast<const uint8_t*>(mask_bits),
        static_cast<const uint4*>(x), gamma, saved_mean, saved_inv_std, dgamma, dbeta, static_cast<uint4*>(dconv), pooled,
        (int64_t)n * h * w, h / 2, w / 2, w, p.tpr, p.bx, p.by, p.rows_per_strip);
    TRB_LAUNCH_CHECK("bnrelu_pool_bwd_apply");
    return TRB200_OK;
}

}  // namespace trb

extern "C" int trb200_bn_apply_relu_mask_pool(const void* conv_out, const float* eq_scale, const float* eq_bias,
                                              void* relu_out, void* mask_bits, void* pool_out, void* argmax,
                                              int32_t n, int32_t h, int32_t w, int32_t c, void* stream) {
    int rc = trb::check_pool_shape(n, h, w, c, "bn_apply_relu_mask_pool");
    if (rc) return rc;
    TRB_REQUIRE(conv_out && eq_scale && eq_bias && mask_bits && pool_out && argmax, TRB200_ERR_INVALID_ARGUMENT,
                "bn_apply_relu_mask_pool: null pointer");
    TRB_REQUIRE(trb::aligned16(conv_out) && trb::aligned16(pool_out) && (!relu_out || trb::aligned16(relu_out)) &&
                    (reinterpret_cast<uintptr_t>(argmax) & 7u) == 0,
                TRB200_ERR_INVALID_ARGUMENT, "bn_apply_relu_mask_pool: tensors must be 16-byte aligned (argmax: 8)");
    const int64_t pooled = (int64_t)n * (h / 2) * (w / 2);
    const trb::PoolPlan p = trb::make_pool_plan(pooled, c);
    trb::bn_apply_relu_mask_pool_kernel<<<dim3(p.gx, p.gy), trb::kThreads, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(conv_out), eq_scale, eq_bias, static_cast<uint4*>(relu_out),
        static_cast<uint8_t*>(mask_bits), static_cast<uint4*>(pool_out), static_cast<uint2*>(argmax), pooled, h / 2,
        w / 2, w, p.tpr, p.bx, p.by, p.rows_per_strip);
    TRB_LAUNCH_CHECK("bn_apply_relu_mask_pool_kernel");
    return TRB200_OK;
}

extern "C" size_t trb200_bnrelu_pool_bwd_workspace_bytes(int32_t n, int32_t h, int32_t w, int32_t c) {
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || h % 2 || w % 2 || c % 8) return 0;
    return trb::bnrelu_pool_bwd_workspace(n, h, w, c);
}

extern "C" int trb200_bnrelu_pool_bwd(const void* dy_pooled, const void* argmax, const void* mask_bits, const void* x,
                                      const float* gamma, const float* saved_mean, const float* saved_inv_std,
                                      void* dconv, float* dgamma, float* dbeta, int32_t n, int32_t h, int32_t w,
                                      int32_t c, void* workspace, size_t workspace_bytes, void* stream) {
    return trb::bnrelu_pool_bwd_launch(dy_pooled, argmax, mask_bits, x, gamma, saved_mean, saved_inv_std, dconv, dgamma,
                                       dbeta, n, h, w, c, workspace, workspace_bytes, trb::as_stream(stream));
}
