// Forward side of the Conv+BN+ReLU block that is HBM-bound: batch statistics of
// the conv output, bn_finalize, and BN-apply + ReLU + bit mask; plus 2x2 max
// pooling.  These produce the inputs of the backward hot path.
//
// Reference counterparts (cuDNN-FE graphs in src/backend/ops/dtensor/cbr_op.cpp):
//   genstats (sum, sum of squares per channel)            cbr_op.cpp:622-718
//   bn_finalize -> eq_scale, eq_bias, saved stats, running stats   cbr_op.cpp:430-528
//   y = relu(t), mask = t > 0, t = half(half(x*eq_scale) + eq_bias) cbr_op.cpp:534-616
//   max pooling with argmax byte (kh*k + kw, first maximum wins)    maxpool_op.cu:23-217
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <cuda_fp16.h>
#include "conv.cuh"

namespace trb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kBlocksPerSm = 2;     // resident blocks per SM at the kernels' register use

struct RowPlan {
    int tpr, bx, by, gy, gx;
    int64_t rows_per_strip;
};

RowPlan make_row_plan(int64_t m, int c) {
    RowPlan p;
    p.tpr = c / 8;
    p.bx = p.tpr < kThreads ? p.tpr : kThreads;
    p.by = kThreads / p.bx;
    if (p.by < 1) p.by = 1;
    p.gy = (p.tpr + p.bx - 1) / p.bx;
    // strips of at least 8 loop trips, at most 4 waves of resident blocks, whole waves when
    // there is more than one (equal strips: a partial last wave would idle most SMs)
    int64_t want = (m + (int64_t)p.by * kUnroll * 8 - 1) / ((int64_t)p.by * kUnroll * 8);
    int64_t resident = (int64_t)sm_count() * kBlocksPerSm / p.gy;
    if (resident < 1) resident = 1;
    int64_t g = want < resident * 4 ? want : resident * 4;
    if (g > resident) g = g / resident * resident;
    p.gx = (int)(g < 1 ? 1 : g);
    int64_t rps = (m + p.gx - 1) / p.gx;
    rps = (rps + p.by - 1) / p.by * p.by;
    p.rows_per_strip = rps;
    p.gx = (int)((m + rps - 1) / rps);
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

// per-strip partial sums of x and x*x, 8 channels per thread
__global__ void __launch_bounds__(kThreads)
bn_stats_partial(const uint4* __restrict__ x, float* __restrict__ partial, int64_t m, int c, int tpr, int bx,
                 int by, int64_t rows_per_strip, int bf16) {
    __shared__ float s_red[kThreads * 16];
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    const bool ok = vec < tpr && ty < by;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < m) ? r0 + rows_per_strip : m;
    float s1[8], s2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { s1[j] = 0.f; s2[j] = 0.f; }
    if (ok) {
        for (int64_t row = r0 + ty; row < r1; row += (int64_t)by * kUnroll) {
            uint4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int64_t r = row + (int64_t)u * by;
                v[u] = r < r1 ? x[r * tpr + vec] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                float f[8];
                if (bf16) unpack8_t<true>(v[u], f);
                else unpack8(v[u], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) { s1[j] += f[j]; s2[j] = fmaf(f[j], f[j], s2[j]); }
            }
        }
    }
    float* mine = s_red + (size_t)threadIdx.x * 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = s1[j]; mine[8 + j] = s2[j]; }
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

// One warp per channel: lanes add every 32nd strip in double, a fixed butterfly adds
// the lanes (the order of additions never changes), lane 0 finalizes the statistics.
__global__ void __launch_bounds__(256)
bn_stats_finalize(const float* __restrict__ partial, int strips, int c, int64_t m,
                  const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                  float momentum, float* __restrict__ ch_sum, float* __restrict__ ch_sqsum,
                  float* __restrict__ saved_mean, float* __restrict__ saved_inv_std,
                  float* __restrict__ eq_scale, float* __restrict__ eq_bias,
                  float* __restrict__ running_mean, float* __restrict__ running_var) {
    const int ch = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (ch >= c) return;
    double s = 0.0, q = 0.0;
    for (int i = lane; i < strips; i += 32) {
        s += (double)partial[((size_t)i * 2) * c + ch];
        q += (double)partial[((size_t)i * 2 + 1) * c + ch];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    if (lane != 0) return;
    if (ch_sum) ch_sum[ch] = (float)s;
    if (ch_sqsum) ch_sqsum[ch] = (float)q;
    const double mean_d = s / (double)m;
    const float mean = (float)mean_d;
    float var = (float)(q / (double)m - mean_d * mean_d);
    if (var < 0.f) var = 0.f;
    const float is = 1.0f / sqrtf(var + eps);
    saved_mean[ch] = mean;
    saved_inv_std[ch] = is;
    const float es = gamma[ch] * is;
    eq_scale[ch] = es;
    eq_bias[ch] = beta[ch] - mean * es;
    if (running_mean) running_mean[ch] = (1.0f - momentum) * running_mean[ch] + momentum * mean;
    if (running_var) {
        const float unb = m > 1 ? var * (float)((double)m / (double)(m - 1)) : var;
        running_var[ch] = (1.0f - momentum) * running_var[ch] + momentum * unb;
    }
}

// t = half(half(x*s) + b); y = max(t, 0); mask bit = t > 0
__global__ void __launch_bounds__(kThreads)
bn_apply_relu_mask(const uint4* __restrict__ x, const float* __restrict__ eq_scale,
                   const float* __restrict__ eq_bias, uint4* __restrict__ y, uint8_t* __restrict__ mask,
                   int64_t m, int tpr, int bx, int by, int64_t rows_per_strip) {
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    if (vec >= tpr || ty >= by) return;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < m) ? r0 + rows_per_strip : m;
    float sc[8], bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sc[j] = eq_scale[vec * 8 + j]; bi[j] = eq_bias[vec * 8 + j]; }
    for (int64_t row = r0 + ty; row < r1; row += (int64_t)by * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t r = row + (int64_t)u * by;
            if (r < r1) v[u] = x[r * tpr + vec];
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t r = row + (int64_t)u * by;
            if (r >= r1) continue;
            // two channels per packed conversion and comparison; the roundings are those of the scalar form
            const __half2* h = reinterpret_cast<const __half2*>(&v[u]);
            const __half2 zero2 = __float2half2_rn(0.f);
            uint32_t o[4], on[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                const float2 a = __half22float2(__floats2half2_rn(f.x * sc[2 * i], f.y * sc[2 * i + 1]));
                const __half2 t = __floats2half2_rn(a.x + bi[2 * i], a.y + bi[2 * i + 1]);
                on[i] = __hgt2_mask(t, zero2);                                 // 0xffff per lane with t > 0
                o[i] = *reinterpret_cast<const uint32_t*>(&t) & on[i];         // ReLU: +0 where off
            }
            // one byte of each lane's result gathered, each byte keeps its own bit, a multiply adds them up
            const uint32_t lo = __byte_perm(on[0], on[1], 0x6420) & 0x08040201u;
            const uint32_t hi = __byte_perm(on[2], on[3], 0x6420) & 0x08040201u;
            y[r * tpr + vec] = make_uint4(o[0], o[1], o[2], o[3]);
            mask[r * tpr + vec] = (uint8_t)(((lo * 0x01010101u) >> 24) | (((hi * 0x01010101u) >> 24) << 4));
        }
    }
}

// The same on a ring of bulk copies, for tensors of four or more items per SM: one thread of a producer warp streams
// runs of 1024 vectors into shared memory (eight stages of 16 KB: what is in flight does not depend on the consumers'
// progress or on the SM clock), 512 consumer threads, each keeping its 8 channels, write y and the mask bytes from
// registers.  Vectors past the last whole item are handled by block 0 with plain loads.
constexpr int kApplyRingStages = 8;
constexpr int kApplyRingConsumers = 512;
constexpr int kApplyRingPasses = 2;

__device__ __forceinline__ void apply_relu_mask_vector(const uint4& v, const float (&sc)[8], const float (&bi)[8],
                                                       uint4& yv, uint8_t& mbyte) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    const __half2 zero2 = __float2half2_rn(0.f);
    uint32_t o[4], on[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        const float2 a = __half22float2(__floats2half2_rn(f.x * sc[2 * i], f.y * sc[2 * i + 1]));
        const __half2 t = __floats2half2_rn(a.x + bi[2 * i], a.y + bi[2 * i + 1]);
        on[i] = __hgt2_mask(t, zero2);
        o[i] = *reinterpret_cast<const uint32_t*>(&t) & on[i];
    }
    const uint32_t lo = __byte_perm(on[0], on[1], 0x6420) & 0x08040201u;
    const uint32_t hi = __byte_perm(on[2], on[3], 0x6420) & 0x08040201u;
    yv = make_uint4(o[0], o[1], o[2], o[3]);
    mbyte = (uint8_t)(((lo * 0x01010101u) >> 24) | (((hi * 0x01010101u) >> 24) << 4));
}

__global__ void __launch_bounds__(kApplyRingConsumers + 32)
bn_apply_relu_mask_ring(const unsigned char* __restrict__ x, const float* __restrict__ eq_scale,
                        const float* __restrict__ eq_bias, uint4* __restrict__ y, uint8_t* __restrict__ mask,
                        int64_t vectors, int tpr, int64_t items, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kApplyRingStages], s_empty[kApplyRingStages];
    __shared__ int s_abort;
    constexpr int kItemVectors = kApplyRingConsumers * kApplyRingPasses;
    constexpr uint32_t kStageBytes = kItemVectors * 16u;
    const int tid = threadIdx.x;
    const uint32_t buf0 = ptx::smem_u32(smem_raw);
    const uint32_t full0 = ptx::smem_u32(&s_full[0]), empty0 = ptx::smem_u32(&s_empty[0]);
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < kApplyRingStages; ++i) {
            ptx::mbar_init(full0 + 8u * i, 1);
            ptx::mbar_init(empty0 + 8u * i, kApplyRingConsumers / 32);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const int64_t my_items = (items - blockIdx.x + gridDim.x - 1) / gridDim.x;
    if (tid >= kApplyRingConsumers) {
        if (tid == kApplyRingConsumers) {
            for (int64_t k = 0; k < my_items; ++k) {
                const int st = (int)(k % kApplyRingStages);
                if (k >= kApplyRingStages &&
                    !ptx::mbar_wait_relaxed(empty0 + 8u * st, (uint32_t)((k / kApplyRingStages - 1) & 1), &s_abort, status, 27))
                    break;
                const int64_t v0 = ((int64_t)blockIdx.x + k * gridDim.x) * kItemVectors;
                ptx::mbar_expect_tx(full0 + 8u * st, kStageBytes);
                ptx::bulk_load_1d(buf0 + (uint32_t)st * kStageBytes, x + v0 * 16, kStageBytes, full0 + 8u * st);
            }
        }
        return;
    }
    const int vec = tid % tpr;
    float sc[8], bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sc[j] = eq_scale[vec * 8 + j]; bi[j] = eq_bias[vec * 8 + j]; }
    for (int64_t k = 0; k < my_items; ++k) {
        const int st = (int)(k % kApplyRingStages);
        if (!ptx::mbar_wait(full0 + 8u * st, (uint32_t)((k / kApplyRingStages) & 1), &s_abort, status, 28)) break;
        const unsigned char* sx = smem_raw + (size_t)st * kStageBytes;
        const int64_t v0 = ((int64_t)blockIdx.x + k * gridDim.x) * kItemVectors;
#pragma unroll
        for (int ps = 0; ps < kApplyRingPasses; ++ps) {
            const int v = ps * kApplyRingConsumers + tid;
            uint4 yv;
            uint8_t mb;
            apply_relu_mask_vector(*reinterpret_cast<const uint4*>(sx + (size_t)v * 16), sc, bi, yv, mb);
            y[v0 + v] = yv;
            mask[v0 + v] = mb;
        }
        __syncwarp();
        if ((tid & 31) == 0) ptx::mbar_arrive(empty0 + 8u * st);
    }
    if (blockIdx.x == 0) {
        for (int64_t v = items * kItemVectors + tid; v < vectors; v += kApplyRingConsumers) {
            uint4 yv;
            uint8_t mb;
            apply_relu_mask_vector(*reinterpret_cast<const uint4*>(x + v * 16), sc, bi, yv, mb);
            y[v] = yv;
            mask[v] = mb;
        }
    }
}

// 2x2 / stride 2 max pooling, 8 channels per thread
__global__ void __launch_bounds__(256)
maxpool2x2_fwd(const uint4* __restrict__ x, uint4* __restrict__ y, uint2* __restrict__ argmax, int n, int h,
               int w, int tpr) {
    const int oh_n = h / 2, ow_n = w / 2;
    const int64_t total = (int64_t)n * oh_n * ow_n * tpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int vec = (int)(i % tpr);
        int64_t p = i / tpr;
        const int ow = (int)(p % ow_n);
        p /= ow_n;
        const int oh = (int)(p % oh_n);
        const int img = (int)(p / oh_n);
        float best[8];
        uint8_t am[8];
        uint4 bv = make_uint4(0, 0, 0, 0);
        __half* bh = reinterpret_cast<__half*>(&bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; am[j] = 0; }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int ih = oh * 2 + (q >> 1), iw = ow * 2 + (q & 1);
            const uint4 v = x[(((int64_t)img * h + ih) * w + iw) * tpr + vec];
            const __half* vh = reinterpret_cast<const __half*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = __half2float(vh[j]);
                if (f > best[j]) { best[j] = f; am[j] = (uint8_t)q; bh[j] = vh[j]; }
            }
        }
        y[i] = bv;
        uint2 a;
        a.x = am[0] | (am[1] << 8) | (am[2] << 16) | (am[3] << 24);
        a.y = am[4] | (am[5] << 8) | (am[6] << 16) | (am[7] << 24);
        argmax[i] = a;
    }
}

__global__ void __launch_bounds__(256)
maxpool2x2_bwd(const uint4* __restrict__ dy, const uint2* __restrict__ argmax, uint4* __restrict__ dx, int n,
               int h, int w, int tpr) {
    const int oh_n = h / 2, ow_n = w / 2;
    const int64_t total = (int64_t)n * oh_n * ow_n * tpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int vec = (int)(i % tpr);
        int64_t p = i / tpr;
        const int ow = (int)(p % ow_n);
        p /= ow_n;
        const int oh = (int)(p % oh_n);
        const int img = (int)(p / oh_n);
        const uint4 g = dy[i];
        const uint2 a = argmax[i];
        const uint16_t* gh = reinterpret_cast<const uint16_t*>(&g);
        const uint8_t* ab = reinterpret_cast<const uint8_t*>(&a);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 o;
            uint16_t* oh16 = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) oh16[j] = ab[j] == q ? gh[j] : (uint16_t)0;
            const int ih = oh * 2 + (q >> 1), iw = ow * 2 + (q & 1);
            dx[(((int64_t)img * h + ih) * w + iw) * tpr + vec] = o;
        }
    }
}

int grid_for(int64_t items) {
    int64_t b = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

}  // namespace

int bn_finalize_from_partials(const float* partial, int strips, int c, int64_t m, const float* gamma,
                              const float* beta, float eps, float momentum, float* ch_sum, float* ch_sqsum,
                              float* saved_mean, float* saved_inv_std, float* eq_scale, float* eq_bias,
                              float* running_mean, float* running_var, cudaStream_t st) {
    bn_stats_finalize<<<(c + 7) / 8, 256, 0, st>>>(partial, strips, c, m, gamma, beta, eps, momentum, ch_sum, ch_sqsum,
                                                   saved_mean, saved_inv_std, eq_scale, eq_bias, running_mean,
                                                   running_var);
    TRB_LAUNCH_CHECK("bn_stats_finalize");
    return TRB200_OK;
}

}  // namespace trb

extern "C" size_t trb200_bn_stats_workspace_bytes(int64_t m, int32_t c) {
    if (m <= 0 || c <= 0 || c % 8 != 0) return 0;
    const trb::RowPlan p = trb::make_row_plan(m, c);
    return (size_t)p.gx * 2 * (size_t)c * sizeof(float);
}

static int bn_stats_finalize_any(const void* conv_out, const float* gamma, const float* beta, float eps,
                                 float momentum, float* ch_sum, float* ch_sqsum, float* saved_mean,
                                 float* saved_inv_std, float* eq_scale, float* eq_bias,
                                 float* running_mean, float* running_var, int64_t m, int32_t c,
                                 void* workspace, size_t workspace_bytes, void* stream, int bf16) {
    TRB_REQUIRE(conv_out && gamma && beta && saved_mean && saved_inv_std && eq_scale && eq_bias,
                TRB200_ERR_INVALID_ARGUMENT, "bn_stats_finalize: null pointer");
    TRB_REQUIRE(m > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "bn_stats_finalize: need m > 0 and c a positive multiple of 8 (m=%lld c=%d)", (long long)m, c);
    TRB_REQUIRE(trb::aligned16(conv_out), TRB200_ERR_INVALID_ARGUMENT, "bn_stats_finalize: conv_out must be 16-byte aligned");
    const size_t need = trb200_bn_stats_workspace_bytes(m, c);
    TRB_REQUIRE(workspace && workspace_bytes >= need, TRB200_ERR_WORKSPACE,
                "bn_stats_finalize: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    const trb::RowPlan p = trb::make_row_plan(m, c);
    cudaStream_t s = trb::as_stream(stream);
    float* partial = static_cast<float*>(workspace);
    trb::bn_stats_partial<<<dim3(p.gx, p.gy), trb::kThreads, 0, s>>>(static_cast<const uint4*>(conv_out), partial, m, c,
                                                                     p.tpr, p.bx, p.by, p.rows_per_strip, bf16);
    TRB_LAUNCH_CHECK("bn_stats_partial");
    trb::bn_stats_finalize<<<(c + 7) / 8, 256, 0, s>>>(partial, p.gx, c, m, gamma, beta, eps, momentum, ch_sum,
                                                          ch_sqsum, saved_mean, saved_inv_std, eq_scale, eq_bias,
                                                          running_mean, running_var);
    TRB_LAUNCH_CHECK("bn_stats_finalize");
    return TRB200_OK;
}

extern "C" int trb200_bn_stats_finalize(const void* conv_out, const float* gamma, const float* beta, float eps,
                                        float momentum, float* ch_sum, float* ch_sqsum, float* saved_mean,
                                        float* saved_inv_std, float* eq_scale, float* eq_bias,
                                        float* running_mean, float* running_var, int64_t m, int32_t c,
                                        void* workspace, size_t workspace_bytes, void* stream) {
    return bn_stats_finalize_any(conv_out, gamma, beta, eps, momentum, ch_sum, ch_sqsum, saved_mean, saved_inv_std,
                                 eq_scale, eq_bias, running_mean, running_var, m, c, workspace, workspace_bytes, stream,
                                 0);
}

extern "C" int trb200_bn_stats_finalize_dtype(const void* conv_out, const float* gamma, const float* beta, float eps,
                                              float momentum, float* ch_sum, float* ch_sqsum, float* saved_mean,
                                              float* saved_inv_std, float* eq_scale, float* eq_bias,
                                              float* running_mean, float* running_var, int64_t m, int32_t c,
                                              int32_t dtype, void* workspace, size_t workspace_bytes, void* stream) {
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "bn_stats_finalize: unknown dtype %d", dtype);
    return bn_stats_finalize_any(conv_out, gamma, beta, eps, momentum, ch_sum, ch_sqsum, saved_mean, saved_inv_std,
                                 eq_scale, eq_bias, running_mean, running_var, m, c, workspace, workspace_bytes, stream,
                                 dtype == TRB200_DTYPE_BF16);
}

namespace trb {
namespace {
// The apply stage for either storage type, with or without the ReLU: t = round16(round16(x*s) + b);
// RELU: y = max(t, 0) and mask bit = t > 0; otherwise y = t and no mask (a BN in front of a residual join).
template <bool BF16, bool RELU>
__device__ __forceinline__ void bn_apply_body(const uint4* __restrict__ x, const float* __restrict__ eq_scale,
                                              const float* __restrict__ eq_bias, uint4* __restrict__ y,
                                              uint8_t* __restrict__ mask, int64_t m, int tpr) {
    const int64_t total = m * tpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int vec = (int)(i % tpr);
        float f[8];
        unpack8_t<BF16>(x[i], f);
        uint32_t o[4], bits = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = unpack2_t<BF16>(pack2_t<BF16>(f[2 * j] * eq_scale[vec * 8 + 2 * j],
                                                           f[2 * j + 1] * eq_scale[vec * 8 + 2 * j + 1]));
            o[j] = pack2_t<BF16>(a.x + eq_bias[vec * 8 + 2 * j], a.y + eq_bias[vec * 8 + 2 * j + 1]);
            if (RELU) {
                const float2 t = unpack2_t<BF16>(o[j]);
                const bool p0 = t.x > 0.f, p1 = t.y > 0.f;
                bits |= (p0 ? 1u : 0u) << (2 * j) | (p1 ? 1u : 0u) << (2 * j + 1);
                o[j] = (p0 ? o[j] & 0xffffu : 0u) | (p1 ? o[j] & 0xffff0000u : 0u);
            }
        }
        y[i] = make_uint4(o[0], o[1], o[2], o[3]);
        if (RELU) mask[i] = (uint8_t)bits;
    }
}

__global__ void __launch_bounds__(256)
bn_apply_any_kernel(const uint4* __restrict__ x, const float* __restrict__ eq_scale, const float* __restrict__ eq_bias,
                    uint4* __restrict__ y, uint8_t* __restrict__ mask, int64_t m, int tpr, int bf16, int relu) {
    if (bf16) {
        if (relu) bn_apply_body<true, true>(x, eq_scale, eq_bias, y, mask, m, tpr);
        else bn_apply_body<true, false>(x, eq_scale, eq_bias, y, mask, m, tpr);
    } else {
        if (relu) bn_apply_body<false, true>(x, eq_scale, eq_bias, y, mask, m, tpr);
        else bn_apply_body<false, false>(x, eq_scale, eq_bias, y, mask, m, tpr);
    }
}
}  // namespace
}  // namespace trb

extern "C" int trb200_bn_apply_dtype(const void* conv_out, const float* eq_scale, const float* eq_bias, void* out,
                                     void* mask_bits, int64_t m, int32_t c, int32_t relu, int32_t dtype,
                                     void* stream) {
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "bn_apply: unknown dtype %d", dtype);
    TRB_REQUIRE(conv_out && eq_scale && eq_bias && out && (!relu || mask_bits), TRB200_ERR_INVALID_ARGUMENT,
                "bn_apply: null pointer");
    TRB_REQUIRE(m > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "bn_apply: need m > 0 and c a positive multiple of 8 (m=%lld c=%d)", (long long)m, c);
    TRB_REQUIRE(trb::aligned16(conv_out) && trb::aligned16(out), TRB200_ERR_INVALID_ARGUMENT,
                "bn_apply: tensors must be 16-byte aligned");
    // the tuned kernel covers the half + ReLU case of the VGG path
    if (dtype == TRB200_DTYPE_F16 && relu)
        return trb200_bn_apply_relu_mask(conv_out, eq_scale, eq_bias, out, mask_bits, m, c, stream);
    const int64_t items = m * (c / 8);
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)trb::sm_count() * 16;
    if (blocks > cap) blocks = cap;
    trb::bn_apply_any_kernel<<<(int)blocks, 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(conv_out), eq_scale, eq_bias, static_cast<uint4*>(out),
        static_cast<uint8_t*>(mask_bits), m, c / 8, dtype == TRB200_DTYPE_BF16, relu != 0);
    TRB_LAUNCH_CHECK("bn_apply_any_kernel");
    return TRB200_OK;
}

extern "C" int trb200_bn_apply_relu_mask(const void* conv_out, const float* eq_scale, const float* eq_bias,
                                         void* relu_out, void* mask_bits, int64_t m, int32_t c, void* stream) {
    TRB_REQUIRE(conv_out && eq_scale && eq_bias && relu_out && mask_bits, TRB200_ERR_INVALID_ARGUMENT,
                "bn_apply_relu_mask: null pointer");
    TRB_REQUIRE(m > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "bn_apply_relu_mask: need m > 0 and c a positive multiple of 8 (m=%lld c=%d)", (long long)m, c);
    TRB_REQUIRE(trb::aligned16(conv_out) && trb::aligned16(relu_out), TRB200_ERR_INVALID_ARGUMENT,
                "bn_apply_relu_mask: tensors must be 16-byte aligned");
    {
        const int tpr = c / 8;
        const int64_t vectors = m * tpr;
        const int64_t items = vectors / (trb::kApplyRingConsumers * trb::kApplyRingPasses);
        if (tpr <= trb::kApplyRingConsumers && (tpr & (tpr - 1)) == 0 && items >= 4 * (int64_t)trb::sm_count()) {
            static bool attr_done[64] = {false};
            int dev = 0;
            TRB_CUDA_TRY(cudaGetDevice(&dev));
            const size_t smem = (size_t)trb::kApplyRingStages * trb::kApplyRingConsumers * trb::kApplyRingPasses * 16;
            if (dev >= 0 && dev < 64 && !attr_done[dev]) {
                TRB_CUDA_TRY(cudaFuncSetAttribute(trb::bn_apply_relu_mask_ring, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)smem));
                attr_done[dev] = true;
            }
            int* status = nullptr;
            const int rc = trb::ring_status_ptr(&status);
            if (rc) return rc;
            trb::bn_apply_relu_mask_ring<<<trb::sm_count(), trb::kApplyRingConsumers + 32, smem, trb::as_stream(stream)>>>(
                static_cast<const unsigned char*>(conv_out), eq_scale, eq_bias, static_cast<uint4*>(relu_out),
                static_cast<uint8_t*>(mask_bits), vectors, tpr, items, status);
            TRB_LAUNCH_CHECK("bn_apply_relu_mask_ring");
            return TRB200_OK;
        }
    }
    const trb::RowPlan p = trb::make_row_plan(m, c);
    trb::bn_apply_relu_mask<<<dim3(p.gx, p.gy), trb::kThreads, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(conv_out), eq_scale, eq_bias, static_cast<uint4*>(relu_out),
        static_cast<uint8_t*>(mask_bits), m, p.tpr, p.bx, p.by, p.rows_per_strip);
    TRB_LAUNCH_CHECK("bn_apply_relu_mask");
    return TRB200_OK;
}

extern "C" int trb200_maxpool2x2_fwd(const void* x, void* y, void* argmax, int32_t n, int32_t h, int32_t w,
                                     int32_t c, void* stream) {
    TRB_REQUIRE(x && y && argmax, TRB200_ERR_INVALID_ARGUMENT, "maxpool2x2_fwd: null pointer");
    TRB_REQUIRE(n > 0 && h > 0 && w > 0 && h % 2 == 0 && w % 2 == 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "maxpool2x2_fwd: need even h, w and c a multiple of 8");
    TRB_REQUIRE(trb::aligned16(x) && trb::aligned16(y) && trb::aligned16(argmax), TRB200_ERR_INVALID_ARGUMENT,
                "maxpool2x2_fwd: tensors must be 16-byte aligned");
    const int64_t total = (int64_t)n * (h / 2) * (w / 2) * (c / 8);
    trb::maxpool2x2_fwd<<<trb::grid_for(total), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(y), static_cast<uint2*>(argmax), n, h, w, c / 8);
    TRB_LAUNCH_CHECK("maxpool2x2_fwd");
    return TRB200_OK;
}

extern "C" int trb200_maxpool2x2_bwd(const void* dy, const void* argmax, void* dx, int32_t n, int32_t h, int32_t w,
                                     int32_t c, void* stream) {
    TRB_REQUIRE(dy && dx && argmax, TRB200_ERR_INVALID_ARGUMENT, "maxpool2x2_bwd: null pointer");
    TRB_REQUIRE(n > 0 && h > 0 && w > 0 && h % 2 == 0 && w % 2 == 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "maxpool2x2_bwd: need even h, w and c a multiple of 8");
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(dx) && trb::aligned16(argmax), TRB200_ERR_INVALID_ARGUMENT,
                "maxpool2x2_bwd: tensors must be 16-byte aligned");
    TRB_REQUIRE(dx != dy, TRB200_ERR_INVALID_ARGUMENT, "maxpool2x2_bwd: dx must not alias dy");
    const int64_t total = (int64_t)n * (h / 2) * (w / 2) * (c / 8);
    trb::maxpool2x2_bwd<<<trb::grid_for(total), 256, 0, trb::as_stream(stream)>>>(
        static_cast<const uint4*>(dy), static_cast<const uint2*>(argmax), static_cast<uint4*>(dx), n, h, w, c / 8);
    TRB_LAUNCH_CHECK("maxpool2x2_bwd");
    return TRB200_OK;
}
