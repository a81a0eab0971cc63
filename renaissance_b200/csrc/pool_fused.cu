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
#include "sm100_ptx.cuh"

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

// ---------------------------------------------------------------------------------------------------------------
// Backward on a ring of bulk copies.  The kernels above keep one window per thread in flight (ten dependent loads,
// then ~300 instructions), so their time follows the SM clock and they lose a third of their bandwidth inside a
// power-capped training step.  Here one thread of a producer warp streams whole row segments into shared memory
// with bulk copies (four stages, ~40 KB each: what is in flight no longer depends on the consumers), and the
// consumer warps work from shared memory.  One item = one pooled image row (or an aligned part of it): two
// full-resolution rows of x and of the mask, one row of pooled dy and of the argmax.
//
// The selection runs on packed halfs: the gradient of a pooled pixel reaches ONE window position per channel (the
// argmax), and only if the ReLU mask bit there is set.
constexpr int kRingStages = 4;
constexpr int kRingMaxConsumers = 512;

struct RingPlan {
    int ok;
    int nchunk, cols_p;                // parts of a pooled row, pooled pixels per part
    int ppp, consumers;                // pooled pixels per pass of the consumers, consumer threads
    uint32_t x_bytes, dy_bytes, am_bytes, m_bytes, stage_bytes;
    int64_t items;
    int grid;
};

RingPlan make_ring_plan(int n, int h, int w, int c) {
    RingPlan p{};
    const int tpr = c / 8, ow = w / 2, oh = h / 2;
    if (tpr > kRingMaxConsumers || (tpr & (tpr - 1)) != 0) return p;     // a thread keeps its channels: tpr | consumers
    if (((int64_t)w * c) % 128 != 0) return p;                             // mask rows start on 16-byte boundaries
    for (int nchunk = 1; nchunk <= ow; ++nchunk) {
        if (ow % nchunk) continue;
        const int cols_p = ow / nchunk;
        if (((int64_t)cols_p * c) % 64 != 0) continue;                     // every segment a multiple of 16 bytes
        const int64_t x_bytes = (int64_t)2 * cols_p * c * 2, dy_bytes = (int64_t)cols_p * c * 2,
                      am_bytes = (int64_t)cols_p * c, m_bytes = (int64_t)2 * cols_p * c / 8;
        const int64_t stage = align_up(2 * x_bytes + dy_bytes + am_bytes + 2 * m_bytes, 128);
        if (stage > 48 * 1024) continue;
        p.nchunk = nchunk;
        p.cols_p = cols_p;
        p.x_bytes = (uint32_t)x_bytes;
        p.dy_bytes = (uint32_t)dy_bytes;
        p.am_bytes = (uint32_t)am_bytes;
        p.m_bytes = (uint32_t)m_bytes;
        p.stage_bytes = (uint32_t)stage;
        break;
    }
    if (p.nchunk == 0) return p;
    // consumer threads: whole warps, pixels per pass chosen for the fewest idle lanes in the last pass
    int best = 0;
    double best_waste = 1e30;
    for (int ppp = kRingMaxConsumers / tpr; ppp >= 1; --ppp) {
        if ((ppp * tpr) % 32) continue;
        const double waste = (double)((p.cols_p + ppp - 1) / ppp * ppp) / p.cols_p;
        if (waste < best_waste - 1e-9 && ppp * tpr >= 128) { best_waste = waste; best = ppp; }
    }
    if (best == 0) return p;
    p.ppp = best;
    p.consumers = best * tpr;
    p.items = (int64_t)n * oh * p.nchunk;
    p.grid = (int)(p.items < sm_count() ? p.items : sm_count());
    p.ok = 1;
    return p;
}

struct WindowSelect {
    uint32_t eq[4][4];      // [position][channel pair]: 0xffff in the half whose argmax is this position
    uint32_t gsel[4];       // dy of the pooled pixel (packed halfs), zero where the mask bit at the argmax is clear
};

// m4: the mask bytes of window positions 0..3 in bytes 0..3
__device__ __forceinline__ void window_select(const uint4& g4, const uint2& a2, uint32_t m4, WindowSelect& s) {
    // argmax byte of a channel -> the half 1 + a / 1024 (a normal number, so the packed compare is exact)
    const uint32_t am[4] = {__byte_perm(a2.x, 0x3c3c3c3cu, 0x4140), __byte_perm(a2.x, 0x3c3c3c3cu, 0x4342),
                            __byte_perm(a2.y, 0x3c3c3c3cu, 0x4140), __byte_perm(a2.y, 0x3c3c3c3cu, 0x4342)};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t qq = 0x3c003c00u | (uint32_t)q | ((uint32_t)q << 16);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            s.eq[q][i] = __heq2_mask(*reinterpret_cast<const __half2*>(&am[i]), *reinterpret_cast<const __half2*>(&qq));
    }
    // mask bit of channel j at its argmax position a: bit 8 a + j of m4, moved to bit 31 by a shift of
    // 31 - j - 8 a (one byte per channel, no borrow between the bytes) and spread over the half by a sign-replicating
    // byte permute
    const uint32_t sh[2] = {0x1c1d1e1fu - (a2.x << 3), 0x18191a1bu - (a2.y << 3)};
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t s2 = sh[i >> 1] >> (16 * (i & 1));
        const uint32_t lo = __funnelshift_l(0u, m4, s2), hi = __funnelshift_l(0u, m4, s2 >> 8);
        s.gsel[i] = gw[i] & ptx::prmt_b32(lo, hi, 0xffbbu);
    }
}

template <bool APPLY>
__global__ void __launch_bounds__(kRingMaxConsumers + 32)
bnrelu_pool_bwd_ring(const unsigned char* __restrict__ dy, const unsigned char* __restrict__ argmax,
                     const unsigned char* __restrict__ mask, const unsigned char* __restrict__ x,
                     const float* __restrict__ gamma, const float* __restrict__ mean,
                     const float* __restrict__ inv_std, const float* __restrict__ dgamma,
                     const float* __restrict__ dbeta, float* __restrict__ partial, uint4* __restrict__ out,
                     int64_t m_full, int c, int oh_n, int ow_n, int w, int tpr, RingPlan pl, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kRingStages], s_empty[kRingStages];
    __shared__ int s_abort;
    const int tid = threadIdx.x;
    const int consumers = pl.consumers;
    const uint32_t buf0 = ptx::smem_u32(smem_raw);
    const uint32_t full0 = ptx::smem_u32(&s_full[0]), empty0 = ptx::smem_u32(&s_empty[0]);
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < kRingStages; ++i) {
            ptx::mbar_init(full0 + 8u * i, 1);
            ptx::mbar_init(empty0 + 8u * i, (uint32_t)(consumers >> 5));
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();

    const int64_t row_c = (int64_t)w * c;                       // elements of one full-resolution image row
    // the apply pass walks the items backwards: what the reduce pass read last is still in L2
    auto item_of = [&](int64_t k) -> int64_t {
        const int64_t it = (int64_t)blockIdx.x + k * gridDim.x;
        return APPLY ? pl.items - 1 - it : it;
    };
    const int64_t my_items = (pl.items - blockIdx.x + gridDim.x - 1) / gridDim.x;

    if (tid >= consumers) {
        // ---------------- producer: one thread
        if (tid == consumers) {
            for (int64_t k = 0; k < my_items; ++k) {
                const int st = (int)(k % kRingStages);
                if (k >= kRingStages &&
                    !ptx::mbar_wait_relaxed(empty0 + 8u * st, (uint32_t)((k / kRingStages - 1) & 1), &s_abort, status, 21))
                    break;
                const int64_t it = item_of(k);
                const int64_t prow = it / pl.nchunk;
                const int ch = (int)(it % pl.nchunk);
                const int64_t img = prow / oh_n;
                const int oh = (int)(prow % oh_n);
                const int64_t e0 = ((img * 2 * oh_n + 2 * oh) * (int64_t)w + (int64_t)ch * 2 * pl.cols_p) * c;   // x element
                const int64_t p0 = (prow * ow_n + (int64_t)ch * pl.cols_p) * c;                                   // pooled element
                const uint32_t dst = buf0 + (uint32_t)st * pl.stage_bytes;
                const uint32_t bar = full0 + 8u * st;
                ptx::mbar_expect_tx(bar, 2 * pl.x_bytes + pl.dy_bytes + pl.am_bytes + 2 * pl.m_bytes);
                ptx::bulk_load_1d(dst, x + e0 * 2, pl.x_bytes, bar);
                ptx::bulk_load_1d(dst + pl.x_bytes, x + (e0 + row_c) * 2, pl.x_bytes, bar);
                ptx::bulk_load_1d(dst + 2 * pl.x_bytes, dy + p0 * 2, pl.dy_bytes, bar);
                ptx::bulk_load_1d(dst + 2 * pl.x_bytes + pl.dy_bytes, argmax + p0, pl.am_bytes, bar);
                ptx::bulk_load_1d(dst + 2 * pl.x_bytes + pl.dy_bytes + pl.am_bytes, mask + e0 / 8, pl.m_bytes, bar);
                ptx::bulk_load_1d(dst + 2 * pl.x_bytes + pl.dy_bytes + pl.am_bytes + pl.m_bytes, mask + (e0 + row_c) / 8,
                                  pl.m_bytes, bar);
            }
        }
    } else {
        // ---------------- consumers: a thread keeps its 8 channels, the passes walk the pooled pixels of the item
        const int vec = tid % tpr, lane_p = tid / tpr;
        float k0[8], k1[8], k2[8], k3[8];
        // reduce: k0 = mean, k1 = inv_std, k2 / k3 = the two sums;  apply: dconv = (x - k0) * k1 + (k2 * g + k3)
        const float inv_m = 1.0f / (float)m_full;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int chn = vec * 8 + j;
            k0[j] = mean[chn];
            if (APPLY) {
                const float is = inv_std[chn];
                k2[j] = gamma[chn] * is;
                k1[j] = -k2[j] * (is * (dgamma[chn] * inv_m));
                k3[j] = -k2[j] * (dbeta[chn] * inv_m);
            } else {
                k1[j] = inv_std[chn];
                k2[j] = 0.f;
                k3[j] = 0.f;
            }
        }
        for (int64_t k = 0; k < my_items; ++k) {
            const int st = (int)(k % kRingStages);
            if (!ptx::mbar_wait(full0 + 8u * st, (uint32_t)((k / kRingStages) & 1), &s_abort, status, 22)) break;
            const unsigned char* sx = smem_raw + (size_t)st * pl.stage_bytes;
            const unsigned char* sdy = sx + 2 * pl.x_bytes;
            const unsigned char* sam = sdy + pl.dy_bytes;
            const unsigned char* sm0 = sam + pl.am_bytes;
            int64_t o0 = 0;
            if (APPLY) {
                const int64_t it = item_of(k);
                const int64_t prow = it / pl.nchunk;
                const int chk = (int)(it % pl.nchunk);
                const int64_t img = prow / oh_n;
                const int oh = (int)(prow % oh_n);
                o0 = ((img * 2 * oh_n + 2 * oh) * (int64_t)w + (int64_t)chk * 2 * pl.cols_p) * tpr;     // 16-byte vectors
            }
            for (int p = lane_p; p < pl.cols_p; p += pl.ppp) {
                const int v0 = (2 * p) * tpr + vec;                 // vector index inside a row segment
                const uint4 g4 = *reinterpret_cast<const uint4*>(sdy + (size_t)(p * tpr + vec) * 16);
                const uint2 a2 = *reinterpret_cast<const uint2*>(sam + (size_t)(p * tpr + vec) * 8);
                uint4 xv[4];
                xv[0] = *reinterpret_cast<const uint4*>(sx + (size_t)v0 * 16);
                xv[1] = *reinterpret_cast<const uint4*>(sx + (size_t)(v0 + tpr) * 16);
                xv[2] = *reinterpret_cast<const uint4*>(sx + pl.x_bytes + (size_t)v0 * 16);
                xv[3] = *reinterpret_cast<const uint4*>(sx + pl.x_bytes + (size_t)(v0 + tpr) * 16);
                const uint32_t m4 = (uint32_t)sm0[v0] | ((uint32_t)sm0[v0 + tpr] << 8) |
                                    ((uint32_t)sm0[pl.m_bytes + v0] << 16) | ((uint32_t)sm0[pl.m_bytes + v0 + tpr] << 24);
                WindowSelect ws;
                window_select(g4, a2, m4, ws);
                const uint32_t xw[4][4] = {{xv[0].x, xv[0].y, xv[0].z, xv[0].w}, {xv[1].x, xv[1].y, xv[1].z, xv[1].w},
                                           {xv[2].x, xv[2].y, xv[2].z, xv[2].w}, {xv[3].x, xv[3].y, xv[3].z, xv[3].w}};
                if (!APPLY) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t xa = (xw[0][i] & ws.eq[0][i]) | (xw[1][i] & ws.eq[1][i]) | (xw[2][i] & ws.eq[2][i]) |
                                            (xw[3][i] & ws.eq[3][i]);          // x at the channel's argmax position
                        const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&ws.gsel[i]));
                        const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xa));
                        k2[2 * i] += gf.x;
                        k2[2 * i + 1] += gf.y;
                        k3[2 * i] += gf.x * ((xf.x - k0[2 * i]) * k1[2 * i]);
                        k3[2 * i + 1] += gf.y * ((xf.y - k0[2 * i + 1]) * k1[2 * i + 1]);
                    }
                } else {
                    const int64_t ov[4] = {o0 + v0, o0 + v0 + tpr, o0 + v0 + (int64_t)w * tpr, o0 + v0 + (int64_t)w * tpr + tpr};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        __half2* ohh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t gq = ws.gsel[i] & ws.eq[q][i];
                            const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gq));
                            const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[q][i]));
                            const float o0f = fmaf(xf.x - k0[2 * i], k1[2 * i], fmaf(k2[2 * i], gf.x, k3[2 * i]));
                            const float o1f = fmaf(xf.y - k0[2 * i + 1], k1[2 * i + 1], fmaf(k2[2 * i + 1], gf.y, k3[2 * i + 1]));
                            ohh[i] = __floats2half2_rn(o0f, o1f);
                        }
                        out[ov[q]] = o;
                    }
                }
            }
            __syncwarp();
            if ((tid & 31) == 0) ptx::mbar_arrive(empty0 + 8u * st);
        }
        if (!APPLY) {
            // block sums in a fixed order: the ring is idle now (every copy issued has been waited for), its first
            // bytes hold the per-thread sums
            ptx::named_barrier(1, consumers);
            float* s_red = reinterpret_cast<float*>(smem_raw);
            float* mine = s_red + (size_t)tid * 16;
#pragma unroll
            for (int j = 0; j < 8; ++j) { mine[j] = k2[j]; mine[8 + j] = k3[j]; }
            ptx::named_barrier(1, consumers);
            for (int t = tid; t < tpr * 16; t += consumers) {
                const int ovec = t / 16, j = t % 16;
                float acc = 0.f;
                for (int y = 0; y < pl.ppp; ++y) acc += s_red[(size_t)(y * tpr + ovec) * 16 + j];
                partial[((size_t)blockIdx.x * 2 + (j >> 3)) * c + ovec * 8 + (j & 7)] = acc;
            }
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
    const RingPlan rp = make_ring_plan(n, h, w, c);
    const int strips = rp.ok && rp.grid > p.gx ? rp.grid : p.gx;
    return (size_t)strips * 2 * (size_t)c * sizeof(float);
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
    float* partial = static_cast<float*>(workspace);
    const RingPlan rp = make_ring_plan(n, h, w, c);
    if (rp.ok) {
        static bool attr_done[64] = {false};
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            const int lim = kRingStages * 48 * 1024;
            TRB_CUDA_TRY(cudaFuncSetAttribute(bnrelu_pool_bwd_ring<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(bnrelu_pool_bwd_ring<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            attr_done[dev] = true;
        }
        int* status = nullptr;
        {
            const int rc2 = ring_status_ptr(&status);
            if (rc2) return rc2;
        }
        size_t smem = (size_t)kRingStages * rp.stage_bytes;
        if (smem < (size_t)rp.consumers * 64) smem = (size_t)rp.consumers * 64;     // the block's sums at the end
        const int threads = rp.consumers + 32;
        auto b = [](const void* q) { return static_cast<const unsigned char*>(q); };
        bnrelu_pool_bwd_ring<false><<<rp.grid, threads, smem, s>>>(
            b(dy_pooled), b(argmax), b(mask_bits), b(x), gamma, saved_mean, saved_inv_std, dgamma, dbeta, partial, nullptr,
            (int64_t)n * h * w, c, h / 2, w / 2, w, c / 8, rp, status);
        TRB_LAUNCH_CHECK("bnrelu_pool_bwd_ring<reduce>");
        bnrelu_pool_bwd_finalize<<<(2 * c + 7) / 8, 256, 0, s>>>(partial, dgamma, dbeta, c, rp.grid);
        TRB_LAUNCH_CHECK("bnrelu_pool_bwd_finalize");
        bnrelu_pool_bwd_ring<true><<<rp.grid, threads, smem, s>>>(
            b(dy_pooled), b(argmax), b(mask_bits), b(x), gamma, saved_mean, saved_inv_std, dgamma, dbeta, partial,
            static_cast<uint4*>(dconv), (int64_t)n * h * w, c, h / 2, w / 2, w, c / 8, rp, status);
        TRB_LAUNCH_CHECK("bnrelu_pool_bwd_ring<apply>");
        return TRB200_OK;
    }
    const PoolPlan p = make_pool_plan(pooled, c);
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
