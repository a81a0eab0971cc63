// Softmax + cross entropy with label smoothing (AMP: half logits, float math).
//
// Reference kernels: softmax_ce_fwd_kernel<true>, softmax_ce_reduce_kernel and
// softmax_ce_bwd_kernel<true>, src/backend/ops/dtensor/softmax_ce_op.cu:63-177,
// 372-429, 438-468.  Arithmetic kept from there:
//   e_c   = exp(z_c - max_c z)            p_c = e_c * (1 / (sum_c e_c + 1e-8))
//   loss_partial[b] = (-(1-ls) * log(p_y + 1e-8) - ls/C * sum_c log(p_c + 1e-8)) / batch
//   loss  = sum_b loss_partial[b]  (fixed order, one block)     inv_scaling = 1/batch
//   g_c   = (p_c - ls/C - [c==y](1-ls)) * scaling * inv_scaling   -> half
//
// The reference sweeps a row three times in global memory and keeps probs in
// fp32 between its forward and backward kernels.  Here one kernel reads each
// logit once (row held in registers for C <= 2048, in shared memory above that)
// and writes d_logits directly; probs are written only when asked for.
// HBM bytes per element: 2 read + 2 written (+4 when probs are kept).
#include "common.cuh"

namespace trb {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct RowOut {
    float* probs;          // may be null
    int64_t probs_stride;
    __half* dlogits;       // may be null
    int64_t dlogits_stride;
    float* loss_partial;   // may be null
};

// One warp per row, the row lives in registers: lane l holds vectors l, l+32, ...
// of 8 halfs each.  Needs 16-byte aligned rows.
template <int VPL>
__global__ void __launch_bounds__(256)
softmax_ce_rows_warp(const __half* __restrict__ logits, int64_t logits_stride,
                     const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                     const float* __restrict__ label_smoothing, RowOut out, int batch, int classes) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= batch) return;
    const __half* z = logits + (int64_t)row * logits_stride;
    const int nvec = (classes + 7) >> 3;

    float v[VPL][8];
    float zmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        uint4 raw = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);   // -inf halfs
        if (vec < nvec) raw = *reinterpret_cast<const uint4*>(z + vec * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 t = __half22float2(h[j]);
            v[i][2 * j] = t.x;
            v[i][2 * j + 1] = t.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (vec * 8 + j >= classes) v[i][j] = -INFINITY;   // padding inside the last vector
            zmax = fmaxf(zmax, v[i][j]);
        }
    }
    zmax = warp_max(zmax);
    const float shift = -zmax * kLog2e;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[i][j] = fast_exp2(fmaf(v[i][j], kLog2e, shift));
            sum += v[i][j];
        }
    sum = warp_sum(sum);
    const float inv_sum = 1.0f / (sum + 1e-8f);

    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const int y = labels[row];
    const float inv_b = 1.0f / (float)batch;
    const float gscale = (scaling ? scaling[0] : 1.0f) * inv_b;
    float sum_log = 0.f, py = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        if (vec >= nvec) continue;
        float p[8];
        uint4 graw;
        __half2* gh = reinterpret_cast<__half2*>(&graw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int cidx = vec * 8 + j;
            p[j] = v[i][j] * inv_sum;
            if (cidx == y) py = p[j];
            if (ls != 0.f && cidx < classes) sum_log += fast_log2(p[j] + 1e-8f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float g0 = p[2 * j] - spread, g1 = p[2 * j + 1] - spread;
            if (vec * 8 + 2 * j == y) g0 -= keep;
            if (vec * 8 + 2 * j + 1 == y) g1 -= keep;
            gh[j] = __floats2half2_rn(g0 * gscale, g1 * gscale);
        }
        const bool full = vec * 8 + 8 <= classes;
        if (out.dlogits) {
            __half* d = out.dlogits + (int64_t)row * out.dlogits_stride + vec * 8;
            if (full && (out.dlogits_stride & 7) == 0) {
                *reinterpret_cast<uint4*>(d) = graw;
            } else {
                const __half* gs = reinterpret_cast<const __half*>(&graw);
                for (int j = 0; j < 8 && vec * 8 + j < classes; ++j) d[j] = gs[j];
            }
        }
        if (out.probs) {
            float* pr = out.probs + (int64_t)row * out.probs_stride + vec * 8;
            if (full && (out.probs_stride & 3) == 0) {
                reinterpret_cast<float4*>(pr)[0] = make_float4(p[0], p[1], p[2], p[3]);
                reinterpret_cast<float4*>(pr)[1] = make_float4(p[4], p[5], p[6], p[7]);
            } else {
                for (int j = 0; j < 8 && vec * 8 + j < classes; ++j) pr[j] = p[j];
            }
        }
    }
    if (out.loss_partial) {
        py = warp_sum(py);   // exactly one lane holds a non-zero value
        sum_log = warp_sum(sum_log) * kLn2;
        if (lane == 0)
            out.loss_partial[row] = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
    }
}

// One block per row, the row is staged once in shared memory as floats' source
// halfs (classes * 2 bytes); used when the row does not fit a warp's registers
// or is not 16-byte aligned.  cache == 0 re-reads global memory instead (rows
// beyond the shared-memory size).
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_ce_rows_block(const __half* __restrict__ logits, int64_t logits_stride,
                      const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                      const float* __restrict__ label_smoothing, RowOut out, int batch, int classes,
                      int cache, int vec_ok) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* srow = reinterpret_cast<__half*>(smem_raw);
    __shared__ float s_red[THREADS / 32];
    __shared__ float s_bcast;
    const int row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __half* z = logits + (int64_t)row * logits_stride;

    auto block_reduce = [&](float val, bool is_max) -> float {
        val = is_max ? warp_max(val) : warp_sum(val);
        __syncthreads();
        if (lane == 0) s_red[warp] = val;
        __syncthreads();
        if (warp == 0) {
            float t = lane < THREADS / 32 ? s_red[lane] : (is_max ? -INFINITY : 0.f);
            t = is_max ? warp_max(t) : warp_sum(t);
            if (lane == 0) s_bcast = t;
        }
        __syncthreads();
        return s_bcast;
    };

    // sweep 1: global -> shared, running max
    float zmax = -INFINITY;
    if (vec_ok) {
        const int nfull = classes >> 3;
        for (int vec = tid; vec < nfull; vec += THREADS) {
            const uint4 raw = *reinterpret_cast<const uint4*>(z + vec * 8);
            if (cache) *reinterpret_cast<uint4*>(srow + vec * 8) = raw;
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __half22float2(h[j]);
                zmax = fmaxf(zmax, fmaxf(t.x, t.y));
            }
        }
        for (int cidx = nfull * 8 + tid; cidx < classes; cidx += THREADS) {
            const __half hv = z[cidx];
            if (cache) srow[cidx] = hv;
            zmax = fmaxf(zmax, __half2float(hv));
        }
    } else {
        for (int cidx = tid; cidx < classes; cidx += THREADS) {
            const __half hv = z[cidx];
            if (cache) srow[cidx] = hv;
            zmax = fmaxf(zmax, __half2float(hv));
        }
    }
    zmax = block_reduce(zmax, true);
    const __half* src = cache ? srow : z;
    const float shift = -zmax * kLog2e;

    // sweep 2: sum of exponentials
    float sum = 0.f;
    for (int cidx = tid; cidx < classes; cidx += THREADS)
        sum += fast_exp2(fmaf(__half2float(src[cidx]), kLog2e, shift));
    sum = block_reduce(sum, false);
    const float inv_sum = 1.0f / (sum + 1e-8f);

    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const int y = labels[row];
    const float inv_b = 1.0f / (float)batch;
    const float gscale = (scaling ? scaling[0] : 1.0f) * inv_b;

    // sweep 3: outputs (pairs of classes so that half2 stores are possible)
    float sum_log = 0.f;
    const bool pair_ok = out.dlogits && ((out.dlogits_stride & 1) == 0) &&
                         ((reinterpret_cast<uintptr_t>(out.dlogits) & 3) == 0);
    const int npairs = (classes + 1) >> 1;
    for (int pr = tid; pr < npairs; pr += THREADS) {
        const int c0 = pr * 2, c1 = c0 + 1;
        const float p0 = fast_exp2(fmaf(__half2float(src[c0]), kLog2e, shift)) * inv_sum;
        const float p1 = c1 < classes ? fast_exp2(fmaf(__half2float(src[c1]), kLog2e, shift)) * inv_sum : 0.f;
        if (ls != 0.f) {
            sum_log += fast_log2(p0 + 1e-8f);
            if (c1 < classes) sum_log += fast_log2(p1 + 1e-8f);
        }
        if (out.probs) {
            float* prow = out.probs + (int64_t)row * out.probs_stride;
            prow[c0] = p0;
            if (c1 < classes) prow[c1] = p1;
        }
        if (out.dlogits) {
            float g0 = p0 - spread, g1 = p1 - spread;
            if (c0 == y) g0 -= keep;
            if (c1 == y) g1 -= keep;
            __half* d = out.dlogits + (int64_t)row * out.dlogits_stride;
            if (pair_ok && c1 < classes) {
                *reinterpret_cast<__half2*>(d + c0) = __floats2half2_rn(g0 * gscale, g1 * gscale);
            } else {
                d[c0] = __float2half_rn(g0 * gscale);
                if (c1 < classes) d[c1] = __float2half_rn(g1 * gscale);
            }
        }
    }
    if (out.loss_partial) {
        sum_log = block_reduce(sum_log, false) * kLn2;
        if (tid == 0) {
            const float py = fast_exp2(fmaf(__half2float(src[y]), kLog2e, shift)) * inv_sum;
            out.loss_partial[row] = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
        }
    }
}

// Fixed-order sum of the per-row partials (one block, strided adds then a
// shared-memory tree), as softmax_ce_reduce_kernel does; also writes 1/batch.
__global__ void __launch_bounds__(256)
softmax_ce_loss_reduce(const float* __restrict__ partial, float* __restrict__ loss,
                       float* __restrict__ inv_scaling, int batch) {
    __shared__ float s[256];
    float acc = 0.f;
    if (partial)
        for (int i = threadIdx.x; i < batch; i += 256) acc += partial[i];
    s[threadIdx.x] = acc;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w) s[threadIdx.x] += s[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (loss && partial) *loss = s[0];
        if (inv_scaling) *inv_scaling = 1.0f / (float)batch;
    }
}

// Backward node on stored probs: grid.y = rows, grid.x covers the row in chunks.
__global__ void __launch_bounds__(256)
softmax_ce_bwd_rows(const float* __restrict__ probs, int64_t probs_stride,
                    const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                    const float* __restrict__ inv_scaling, const float* __restrict__ label_smoothing,
                    __half* __restrict__ dlogits, int64_t dlogits_stride, int classes, int vec_ok) {
    const int row = blockIdx.y;
    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float gscale = scaling[0] * inv_scaling[0];
    const int y = labels[row];
    const float* p = probs + (int64_t)row * probs_stride;
    __half* d = dlogits + (int64_t)row * dlogits_stride;
    if (vec_ok) {
        const int vec = blockIdx.x * blockDim.x + threadIdx.x;
        const int c0 = vec * 8;
        if (c0 >= classes) return;
        if (c0 + 8 <= classes) {
            const float4 a = reinterpret_cast<const float4*>(p + c0)[0];
            const float4 b = reinterpret_cast<const float4*>(p + c0)[1];
            float g[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                g[j] -= spread;
                if (c0 + j == y) g[j] -= keep;
                g[j] *= gscale;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(g[2 * j], g[2 * j + 1]);
            *reinterpret_cast<uint4*>(d + c0) = o;
        } else {
            for (int cidx = c0; cidx < classes; ++cidx) {
                float g = p[cidx] - spread;
                if (cidx == y) g -= keep;
                d[cidx] = __float2half_rn(g * gscale);
            }
        }
    } else {
        const int cidx = blockIdx.x * blockDim.x + threadIdx.x;
        if (cidx >= classes) return;
        float g = p[cidx] - spread;
        if (cidx == y) g -= keep;
        d[cidx] = __float2half_rn(g * gscale);
    }
}

int launch_rows(const void* logits, int64_t logits_stride, const int32_t* labels,
                const float* scaling, const float* label_smoothing, RowOut out, float* loss,
                float* inv_scaling, int batch, int classes, cudaStream_t s) {
    const __half* z = static_cast<const __half*>(logits);
    const bool rows_aligned = aligned16(logits) && (logits_stride % 8 == 0);
    if (rows_aligned && classes <= 2048) {
        const int warps = 8;
        dim3 grid((batch + warps - 1) / warps), block(warps * 32);
        if (classes <= 256)
            softmax_ce_rows_warp<1><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else if (classes <= 512)
            softmax_ce_rows_warp<2><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else if (classes <= 1024)
            softmax_ce_rows_warp<4><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else
            softmax_ce_rows_warp<8><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        TRB_LAUNCH_CHECK("softmax_ce_rows_warp");
    } else {
        constexpr int kT = 512;
        const size_t row_bytes = (size_t)align_up((int64_t)classes * 2, 16);
        const int cache = row_bytes <= 200 * 1024 ? 1 : 0;
        const size_t smem = cache ? row_bytes : 0;
        static bool attr_done[64] = {false};
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<kT>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_done[dev] = true;
        }
        softmax_ce_rows_block<kT><<<batch, kT, smem, s>>>(z, logits_stride, labels, scaling, label_smoothing,
                                                          out, batch, classes, cache, rows_aligned ? 1 : 0);
        TRB_LAUNCH_CHECK("softmax_ce_rows_block");
    }
    if (loss || inv_scaling) {
        softmax_ce_loss_reduce<<<1, 256, 0, s>>>(out.loss_partial, loss, inv_scaling, batch);
        TRB_LAUNCH_CHECK("softmax_ce_loss_reduce");
    }
    return TRB200_OK;
}

}  // namespace
}  // namespace trb

extern "C" int trb200_softmax_ce_fwd(const void* logits, int64_t logits_stride, const int32_t* labels,
                                     const float* label_smoothing, float* probs, int64_t probs_stride,
                                     float* loss_partial, float* loss, float* inv_scaling,
                                     int32_t batch, int32_t classes, void* stream) {
    TRB_REQUIRE(logits && labels && loss_partial, TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fwd: null pointer");
    TRB_REQUIRE(batch > 0 && classes > 0 && logits_stride >= classes && (!probs || probs_stride >= classes),
                TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fwd: bad sizes (batch=%d classes=%d)", batch, classes);
    trb::RowOut out{probs, probs_stride, nullptr, 0, loss_partial};
    return trb::launch_rows(logits, logits_stride, labels, nullptr, label_smoothing, out, loss, inv_scaling,
                            batch, classes, trb::as_stream(stream));
}

extern "C" int trb200_softmax_ce_fused(const void* logits, int64_t logits_stride, const int32_t* labels,
                                       const float* scaling, const float* label_smoothing, float* probs,
                                       int64_t probs_stride, void* dlogits, int64_t dlogits_stride,
                                       float* loss_partial, float* loss, float* inv_scaling,
                                       int32_t batch, int32_t classes, void* stream) {
    TRB_REQUIRE(logits && labels && dlogits && scaling, TRB200_ERR_INVALID_ARGUMENT,
                "softmax_ce_fused: null pointer");
    TRB_REQUIRE(batch > 0 && classes > 0 && logits_stride >= classes && dlogits_stride >= classes &&
                    (!probs || probs_stride >= classes),
                TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fused: bad sizes (batch=%d classes=%d)", batch, classes);
    TRB_REQUIRE(!loss || loss_partial, TRB200_ERR_INVALID_ARGUMENT,
                "softmax_ce_fused: loss needs loss_partial");
    TRB_REQUIRE(dlogits != logits, TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fused: dlogits must not alias logits");
    trb::RowOut out{probs, probs_stride, static_cast<__half*>(dlogits), dlogits_stride, loss_partial};
    return trb::launch_rows(logits, logits_stride, labels, scaling, label_smoothing, out, loss, inv_scaling,
                            batch, classes, trb::as_stream(stream));
}

extern "C" int trb200_softmax_ce_bwd(const float* probs, int64_t probs_stride, const int32_t* labels,
                                     const float* scaling, const float* inv_scaling,
                                     const float* label_smoothing, void* dlogits, int64_t dlogits_stride,
                                     int32_t batch, int32_t classes, void* stream) {
    TRB_REQUIRE(probs && labels && scaling && inv_scaling && dlogits, TRB200_ERR_INVALID_ARGUMENT,
                "softmax_ce_bwd: null pointer");
    TRB_REQUIRE(batch > 0 && classes > 0 && probs_stride >= classes && dlogits_stride >= classes,
                TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_bwd: bad sizes (batch=%d classes=%d)", batch, classes);
    TRB_REQUIRE(batch <= 65535 * 1024, TRB200_ERR_UNSUPPORTED, "softmax_ce_bwd: batch too large");
    const int vec_ok = trb::aligned16(probs) && trb::aligned16(dlogits) && probs_stride % 4 == 0 &&
                       dlogits_stride % 8 == 0;
    const int per_row = vec_ok ? (classes + 7) / 8 : classes;
    // grid.y is limited to 65535 rows: larger batches go in slices
    for (int r0 = 0; r0 < batch; r0 += 65535) {
        const int rows = batch - r0 < 65535 ? batch - r0 : 65535;
        dim3 grid((per_row + 255) / 256, rows);
        trb::softmax_ce_bwd_rows<<<grid, 256, 0, trb::as_stream(stream)>>>(
            probs + (int64_t)r0 * probs_stride, probs_stride, labels + r0, scaling, inv_scaling, label_smoothing,
            static_cast<__half*>(dlogits) + (int64_t)r0 * dlogits_stride, dlogits_stride, classes, vec_ok);
        TRB_LAUNCH_CHECK("softmax_ce_bwd_rows");
    }
    return TRB200_OK;
}
