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
#include "sm100_ptx.cuh"

#include <atomic>
#include <mutex>

namespace trb {

__device__ int g_softmax_status = 0;   // set when a bounded wait of the staged kernel gives up

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

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ void half8_to_float(const uint4& raw, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = __half22float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
    }
}

// max of the 8 halfs of a 16-byte vector, taken with packed half2 instructions
__device__ __forceinline__ float half8_max(const uint4& raw) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
    const __half2 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(__low2float(m), __high2float(m));
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
__global__ void __launch_bounds__(256, VPL >= 8 ? 1 : 3)
softmax_ce_rows_warp(const __half* __restrict__ logits, int64_t logits_stride,
                     const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                     const float* __restrict__ label_smoothing, RowOut out, int batch, int classes) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nvec = (classes + 7) >> 3;
    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float inv_b = 1.0f / (float)batch;
    const float gscale = (scaling ? scaling[0] : 1.0f) * inv_b;
    const bool dvec = out.dlogits && (out.dlogits_stride & 7) == 0 && aligned16_dev(out.dlogits);
    const bool pvec = out.probs && (out.probs_stride & 3) == 0 && aligned16_dev(out.probs);

    const uint4 kNegInf = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);   // -inf halfs
    const int row_first = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // the next row's vectors are requested before the current row is processed
    uint4 nxt[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        nxt[i] = kNegInf;
        if (row_first < batch && vec < nvec)
            nxt[i] = *reinterpret_cast<const uint4*>(logits + (int64_t)row_first * logits_stride + vec * 8);
    }
    for (int row = row_first; row < batch; row += warps) {
        float v[VPL][8];
        float zmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPL; ++i) half8_to_float(nxt[i], v[i]);
        {
            const int row_n = row + warps;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int vec = i * 32 + lane;
                nxt[i] = kNegInf;
                if (row_n < batch && vec < nvec)
                    nxt[i] = *reinterpret_cast<const uint4*>(logits + (int64_t)row_n * logits_stride + vec * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int vec = i * 32 + lane;
            if (vec * 8 + 8 > classes) {                      // padding inside the row's last vector
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (vec * 8 + j >= classes) v[i][j] = -INFINITY;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) zmax = fmaxf(zmax, v[i][j]);
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
        const int y_raw = labels[row];
        const int y = (unsigned)y_raw < (unsigned)classes ? y_raw : -1;   // out of range: matches no class
        float sum_log = 0.f, py = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int vec = i * 32 + lane;
            if (vec >= nvec) continue;
            const int c0 = vec * 8;
            float p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) p[j] = v[i][j] * inv_sum;
            if (ls != 0.f) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (c0 + j < classes) sum_log += fast_log2(p[j] + 1e-8f);
            }
            const bool full = c0 + 8 <= classes;
            if (out.probs) {
                float* pr = out.probs + (int64_t)row * out.probs_stride + c0;
                if (full && pvec) {
                    reinterpret_cast<float4*>(pr)[0] = make_float4(p[0], p[1], p[2], p[3]);
                    reinterpret_cast<float4*>(pr)[1] = make_float4(p[4], p[5], p[6], p[7]);
                } else {
                    for (int j = 0; j < 8 && c0 + j < classes; ++j) pr[j] = p[j];
                }
            }
            const int jy = y - c0;                               // the label sits in at most one vector of the row
            if ((unsigned)jy < 8u) {
#pragma unroll
                for (int j = 0; j < 8; ++j) py += (j == jy) ? p[j] : 0.f;
            }
            if (out.dlogits) {
#pragma unroll
                for (int j = 0; j < 8; ++j) p[j] -= spread;
                if ((unsigned)jy < 8u) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) p[j] -= (j == jy) ? keep : 0.f;
                }
                uint4 graw;
                __half2* gh = reinterpret_cast<__half2*>(&graw);
#pragma unroll
                for (int j = 0; j < 4; ++j) gh[j] = __floats2half2_rn(p[2 * j] * gscale, p[2 * j + 1] * gscale);
                __half* d = out.dlogits + (int64_t)row * out.dlogits_stride + c0;
                if (full && dvec) {
                    *reinterpret_cast<uint4*>(d) = graw;
                } else {
                    const __half* gs = reinterpret_cast<const __half*>(&graw);
                    for (int j = 0; j < 8 && c0 + j < classes; ++j) d[j] = gs[j];
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
}

// The same for the common training call: gradient and loss only (no probabilities kept), rows
// of whole 16-byte vectors.  Per class: one conversion, one FMA and one exponential for the
// sum, one FMA and half a pack for the gradient; the maximum is taken on packed halfs; the
// label's class is patched by one lane after the row's vectors are stored, from a float
// recomputation that also gives the loss.  Label smoothing adds a logarithm per class for the
// loss and nothing to the gradient's cost.
// Completion counters for the loss: every block of a row kernel leaves the sum of its rows'
// losses (added in a fixed order) in a slot of a small library-owned array, and the last block to
// finish adds the slots in block order and writes the loss; the result does not depend on which
// block that is, and the separate one-block reduction launch is saved.  A launch takes the next
// counter (and slot array) of the pool, so fewer calls than the pool holds may be in flight at a time.
constexpr int kLossTickets = 64;
constexpr int kLossTailBlocks = 2048;          // largest grid that finishes its loss this way
__device__ unsigned int g_loss_tickets[kLossTickets];
__device__ float g_loss_block_sums[kLossTickets][kLossTailBlocks];

struct LossTail {
    float* loss;              // may be null
    float* inv_scaling;       // may be null
    unsigned int* ticket;     // null: the caller launches softmax_ce_loss_reduce instead
    float* block_sums;        // this launch's slots, one per block
};

// called by every thread of every block once its rows are done; `mine` = the losses this thread wrote
__device__ __forceinline__ void loss_tail(const LossTail& t, float mine, int batch) {
    if (!t.ticket) return;
    __shared__ int s_last;
    __shared__ float s_part[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float v = warp_sum(mine);
    if (lane == 0) s_part[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = 0.f;
        for (int w = 0; w < nw; ++w) b += s_part[w];
        t.block_sums[blockIdx.x] = b;
        __threadfence();                   // the slot is visible device-wide before the ticket is
        s_last = atomicAdd(t.ticket, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float a = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) a += __ldcg(t.block_sums + i);
    v = warp_sum(a);
    __syncthreads();
    if (lane == 0) s_part[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int w = 0; w < nw; ++w) total += s_part[w];
        if (t.loss) *t.loss = total;
        if (t.inv_scaling) *t.inv_scaling = 1.0f / (float)batch;
        *t.ticket = 0u;                    // ready for the next launch that draws this counter
    }
}

template <int VPL, bool BF16>
__device__ __forceinline__ void
softmax_ce_rows_warp_lean_body(const uint16_t* __restrict__ logits, int64_t logits_stride,
                               const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                               const float* __restrict__ label_smoothing, uint16_t* __restrict__ dlogits,
                               int64_t dlogits_stride, float* __restrict__ loss_partial, int batch, int classes,
                               LossTail tail) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nvec = classes >> 3;
    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float inv_b = 1.0f / (float)batch;
    const float gscale = scaling[0] * inv_b;
    constexpr uint32_t kNegInf2 = BF16 ? 0xff80ff80u : 0xfc00fc00u;                         // two -inf values
    const uint4 kNegInf = make_uint4(kNegInf2, kNegInf2, kNegInf2, kNegInf2);
    const int row_first = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // the next row's vectors are requested before the current row is processed
    uint4 nxt[VPL];
    float my_loss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int vec = i * 32 + lane;
        nxt[i] = kNegInf;
        if (row_first < batch && vec < nvec)
            nxt[i] = *reinterpret_cast<const uint4*>(logits + (int64_t)row_first * logits_stride + vec * 8);
    }
    for (int row = row_first; row < batch; row += warps) {
        uint4 cur[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) cur[i] = nxt[i];
        // a label outside [0, classes) matches no class: nothing is read or written through it, its
        // probability counts as 0 in the loss and no entry of the gradient gets the -(1 - ls) term
        const int y_raw = labels[row];
        const bool y_ok = (unsigned)y_raw < (unsigned)classes;
        const int y = y_ok ? y_raw : 0;
        const float zy = load16_t<BF16>(logits + (int64_t)row * logits_stride + y);
        {
            const int row_n = row + warps;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int vec = i * 32 + lane;
                nxt[i] = kNegInf;
                if (row_n < batch && vec < nvec)
                    nxt[i] = *reinterpret_cast<const uint4*>(logits + (int64_t)row_n * logits_stride + vec * 8);
            }
        }
        float zmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            if constexpr (BF16) {
                float f[8];
                unpack8_t<true>(cur[i], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) zmax = fmaxf(zmax, f[j]);
            } else {
                zmax = fmaxf(zmax, half8_max(cur[i]));
            }
        }
        zmax = warp_max(zmax);
        const float shift = -zmax * kLog2e;
        float e[VPL][8];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            unpack8_t<BF16>(cur[i], e[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                e[i][j] = fast_exp2(fmaf(e[i][j], kLog2e, shift));
                sum += e[i][j];
            }
        }
        sum = warp_sum(sum);
        const float inv_sum = 1.0f / (sum + 1e-8f);
        const float ga = inv_sum * gscale, gb = -spread * gscale;
        uint16_t* drow = dlogits + (int64_t)row * dlogits_stride;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int vec = i * 32 + lane;
            if (vec < nvec) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    o[j] = pack2_t<BF16>(fmaf(e[i][2 * j], ga, gb), fmaf(e[i][2 * j + 1], ga, gb));
                *reinterpret_cast<uint4*>(drow + vec * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        float sum_log = 0.f;
        if (ls != 0.f && loss_partial) {
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (i * 32 + lane < nvec) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) sum_log += fast_log2(fmaf(e[i][j], inv_sum, 1e-8f));
                }
            sum_log = warp_sum(sum_log) * kLn2;
        }
        // the label's class, by the lane that stored its vector
        if (((y >> 3) & 31) == lane) {
            const float py = y_ok ? fast_exp2(fmaf(zy, kLog2e, shift)) * inv_sum : 0.f;
            if (y_ok) drow[y] = round16_t<BF16>((py - spread - keep) * gscale);
            const float row_loss = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
            if (loss_partial) loss_partial[row] = row_loss;
            my_loss += row_loss;
        }
    }
    loss_tail(tail, my_loss, batch);
}

// The kernels proper: the half instantiation under the plain name, the bfloat16 one beside it.
template <int VPL>
__global__ void __launch_bounds__(256, VPL >= 8 ? 2 : 3)
softmax_ce_rows_warp_lean(const __half* __restrict__ logits, int64_t logits_stride,
                          const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                          const float* __restrict__ label_smoothing, __half* __restrict__ dlogits,
                          int64_t dlogits_stride, float* __restrict__ loss_partial, int batch, int classes,
                          LossTail tail) {
    softmax_ce_rows_warp_lean_body<VPL, false>(reinterpret_cast<const uint16_t*>(logits), logits_stride, labels, scaling,
                                               label_smoothing, reinterpret_cast<uint16_t*>(dlogits), dlogits_stride,
                                               loss_partial, batch, classes, tail);
}

template <int VPL>
__global__ void __launch_bounds__(256, VPL >= 8 ? 2 : 3)
softmax_ce_rows_warp_lean_bf16(const __half* __restrict__ logits, int64_t logits_stride,
                               const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                               const float* __restrict__ label_smoothing, __half* __restrict__ dlogits,
                               int64_t dlogits_stride, float* __restrict__ loss_partial, int batch, int classes,
                               LossTail tail) {
    softmax_ce_rows_warp_lean_body<VPL, true>(reinterpret_cast<const uint16_t*>(logits), logits_stride, labels, scaling,
                                              label_smoothing, reinterpret_cast<uint16_t*>(dlogits), dlogits_stride,
                                              loss_partial, batch, classes, tail);
}

// One block per row, the row is staged once in shared memory as halfs (classes * 2
// bytes); used when the row does not fit a warp's registers or is not 16-byte
// aligned.  cache == 0 re-reads global memory instead (rows beyond the
// shared-memory size).  All three sweeps work on 16-byte vectors of 8 classes when
// the rows are 16-byte aligned (vec_ok): the kernel is otherwise bound by its own
// instruction count, not by memory.
// E_HALF (only when probs are not kept and the row is staged): sweep 2 overwrites the
// staged logits with exp(z - max) rounded to half, so that sweep 3 is one FMA per class
// instead of a second exponential; d_logits are half anyway and the loss is taken from a
// float recomputation of the label's class.
template <int THREADS, bool E_HALF>
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

    const int nfull = vec_ok ? (classes >> 3) : 0;       // whole 8-class vectors
    const int tail0 = nfull * 8;                         // first class handled one by one

    // sweep 1: global -> shared, running max; four independent loads in flight per thread
    float zmax = -INFINITY;
    for (int vec0 = tid; vec0 < nfull; vec0 += 4 * THREADS) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int vec = vec0 + u * THREADS;
            raw[u] = vec < nfull ? *reinterpret_cast<const uint4*>(z + vec * 8)
                                 : make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int vec = vec0 + u * THREADS;
            if (cache && vec < nfull) *reinterpret_cast<uint4*>(srow + vec * 8) = raw[u];
            zmax = fmaxf(zmax, half8_max(raw[u]));
        }
    }
    for (int cidx = tail0 + tid; cidx < classes; cidx += THREADS) {
        const __half hv = z[cidx];
        if (cache) srow[cidx] = hv;
        zmax = fmaxf(zmax, __half2float(hv));
    }
    zmax = block_reduce(zmax, true);
    const __half* src = cache ? srow : z;
    const float shift = -zmax * kLog2e;

    // sweep 2: sum of exponentials
    float sum = 0.f;
    const int y_raw = labels[row];                        // out of range: matches no class, see softmax_ce_rows_warp_lean
    const bool y_ok = (unsigned)y_raw < (unsigned)classes;
    const int y = y_ok ? y_raw : -1;
    const float zy = y_ok ? __half2float(z[y]) : 0.f;     // from global: the staged row is about to be overwritten
    for (int vec = tid; vec < nfull; vec += THREADS) {
        float f[8];
        half8_to_float(*reinterpret_cast<const uint4*>(src + vec * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            f[j] = fast_exp2(fmaf(f[j], kLog2e, shift));
            sum += f[j];
        }
        if (E_HALF) {
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
            *reinterpret_cast<uint4*>(srow + vec * 8) = o;
        }
    }
    for (int cidx = tail0 + tid; cidx < classes; cidx += THREADS) {
        const float e = fast_exp2(fmaf(__half2float(src[cidx]), kLog2e, shift));
        sum += e;
        if (E_HALF) srow[cidx] = __float2half_rn(e);
    }
    sum = block_reduce(sum, false);
    const float inv_sum = 1.0f / (sum + 1e-8f);

    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float inv_b = 1.0f / (float)batch;
    const float gscale = (scaling ? scaling[0] : 1.0f) * inv_b;
    const bool want_log = ls != 0.f;

    // sweep 3: outputs
    float sum_log = 0.f;
    __half* drow = out.dlogits ? out.dlogits + (int64_t)row * out.dlogits_stride : nullptr;
    float* prow = out.probs ? out.probs + (int64_t)row * out.probs_stride : nullptr;
    const bool dvec = drow && (out.dlogits_stride & 7) == 0 && aligned16_dev(out.dlogits);
    const bool pvec = prow && (out.probs_stride & 3) == 0 && aligned16_dev(out.probs);
    for (int vec = tid; vec < nfull; vec += THREADS) {
        float f[8];
        half8_to_float(*reinterpret_cast<const uint4*>(src + vec * 8), f);
        const int c0 = vec * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            f[j] = (E_HALF ? f[j] : fast_exp2(fmaf(f[j], kLog2e, shift))) * inv_sum;
            if (want_log) sum_log += fast_log2(f[j] + 1e-8f);
        }
        if (prow) {
            if (pvec) {
                reinterpret_cast<float4*>(prow + c0)[0] = make_float4(f[0], f[1], f[2], f[3]);
                reinterpret_cast<float4*>(prow + c0)[1] = make_float4(f[4], f[5], f[6], f[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) prow[c0 + j] = f[j];
            }
        }
        if (drow) {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] -= spread;
            const int jy = y - c0;
            if ((unsigned)jy < 8u) {                             // at most one vector of the row holds the label
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] -= (j == jy) ? keep : 0.f;
            }
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j] * gscale, f[2 * j + 1] * gscale);
            if (dvec) {
                *reinterpret_cast<uint4*>(drow + c0) = o;
            } else {
                const __half* os = reinterpret_cast<const __half*>(&o);
#pragma unroll
                for (int j = 0; j < 8; ++j) drow[c0 + j] = os[j];
            }
        }
    }
    for (int cidx = tail0 + tid; cidx < classes; cidx += THREADS) {
        const float pv = (E_HALF ? __half2float(src[cidx]) : fast_exp2(fmaf(__half2float(src[cidx]), kLog2e, shift))) * inv_sum;
        if (want_log) sum_log += fast_log2(pv + 1e-8f);
        if (prow) prow[cidx] = pv;
        if (drow) {
            float g = pv - spread;
            if (cidx == y) g -= keep;
            drow[cidx] = __float2half_rn(g * gscale);
        }
    }
    if (out.loss_partial) {
        sum_log = block_reduce(sum_log, false) * kLn2;
        if (tid == 0) {
            const float py = y_ok ? fast_exp2(fmaf(zy, kLog2e, shift)) * inv_sum : 0.f;
            out.loss_partial[row] = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
        }
    }
}

// Persistent variant for long, 16-byte aligned rows with classes % 8 == 0: a block walks
// rows blockIdx.x, blockIdx.x + gridDim.x, ...; each row is brought into shared memory by
// ONE bulk (TMA) copy that completes on an mbarrier, into one of two buffers, so that the
// copy of the next row is in flight while the three sweeps of the current row run.
// Arithmetic and E_HALF as in softmax_ce_rows_block.
template <int THREADS, bool E_HALF>
__global__ void __launch_bounds__(THREADS)
softmax_ce_rows_staged(const __half* __restrict__ logits, int64_t logits_stride,
                       const int32_t* __restrict__ labels, const float* __restrict__ scaling,
                       const float* __restrict__ label_smoothing, RowOut out, int batch, int classes,
                       uint32_t buf_stride, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ float s_red[THREADS / 32];
    __shared__ float s_bcast;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t row_bytes = (uint32_t)classes * 2u;
    const uint32_t buf0 = ptx::smem_u32(smem_raw);
    const uint32_t bar0 = ptx::smem_u32(&s_bar[0]);
    if (tid == 0) {
        s_abort = 0;
        ptx::mbar_init(bar0, 1);
        ptx::mbar_init(bar0 + 8, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();

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

    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float inv_b = 1.0f / (float)batch;
    const float gscale = (scaling ? scaling[0] : 1.0f) * inv_b;
    const bool want_log = ls != 0.f;
    const int nvec = classes >> 3;
    const bool dvec = out.dlogits && (out.dlogits_stride & 7) == 0 && aligned16_dev(out.dlogits);
    const bool pvec = out.probs && (out.probs_stride & 3) == 0 && aligned16_dev(out.probs);

    int row = blockIdx.x;
    if (tid == 0 && row < batch) {
        ptx::mbar_expect_tx(bar0, row_bytes);
        ptx::bulk_load_1d(buf0, logits + (int64_t)row * logits_stride, row_bytes, bar0);
    }
    for (int it = 0; row < batch; row += gridDim.x, ++it) {
        const int b = it & 1;
        const int next = row + gridDim.x;
        if (tid == 0 && next < batch) {       // the other buffer was released by the barrier that ended the last row
            ptx::mbar_expect_tx(bar0 + 8u * (b ^ 1), row_bytes);
            ptx::bulk_load_1d(buf0 + (uint32_t)(b ^ 1) * buf_stride, logits + (int64_t)next * logits_stride, row_bytes,
                              bar0 + 8u * (b ^ 1));
        }
        const bool ok = ptx::mbar_wait(bar0 + 8u * b, ((uint32_t)it >> 1) & 1u, &s_abort, status, 4);
        if (__syncthreads_or(ok ? 0 : 1)) break;
        __half* srow = reinterpret_cast<__half*>(smem_raw + (size_t)b * buf_stride);
        const int y_raw = labels[row];                    // out of range: matches no class
        const bool y_ok = (unsigned)y_raw < (unsigned)classes;
        const int y = y_ok ? y_raw : -1;
        const float zy = y_ok ? __half2float(logits[(int64_t)row * logits_stride + y]) : 0.f;

        float zmax = -INFINITY;
        for (int vec = tid; vec < nvec; vec += THREADS)
            zmax = fmaxf(zmax, half8_max(*reinterpret_cast<const uint4*>(srow + vec * 8)));
        zmax = block_reduce(zmax, true);
        const float shift = -zmax * kLog2e;

        float sum = 0.f;
        for (int vec = tid; vec < nvec; vec += THREADS) {
            float f[8];
            half8_to_float(*reinterpret_cast<const uint4*>(srow + vec * 8), f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                f[j] = fast_exp2(fmaf(f[j], kLog2e, shift));
                sum += f[j];
            }
            if (E_HALF) {
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                *reinterpret_cast<uint4*>(srow + vec * 8) = o;
            }
        }
        sum = block_reduce(sum, false);
        const float inv_sum = 1.0f / (sum + 1e-8f);

        float sum_log = 0.f;
        __half* drow = out.dlogits ? out.dlogits + (int64_t)row * out.dlogits_stride : nullptr;
        float* prow = out.probs ? out.probs + (int64_t)row * out.probs_stride : nullptr;
        if (E_HALF && !want_log && dvec) {
            // gradient only: g = e * (inv_sum * gscale) - spread * gscale, one FMA per class
            const float ga = inv_sum * gscale, gb = -spread * gscale, gk = keep * gscale;
            for (int vec = tid; vec < nvec; vec += THREADS) {
                float f[8];
                half8_to_float(*reinterpret_cast<const uint4*>(srow + vec * 8), f);
                const int c0 = vec * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], ga, gb);
                const int jy = y - c0;
                if ((unsigned)jy < 8u) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] -= (j == jy) ? gk : 0.f;
                }
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                *reinterpret_cast<uint4*>(drow + c0) = o;
            }
        } else
        for (int vec = tid; vec < nvec; vec += THREADS) {
            float f[8];
            half8_to_float(*reinterpret_cast<const uint4*>(srow + vec * 8), f);
            const int c0 = vec * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                f[j] = (E_HALF ? f[j] : fast_exp2(fmaf(f[j], kLog2e, shift))) * inv_sum;
                if (want_log) sum_log += fast_log2(f[j] + 1e-8f);
            }
            if (prow) {
                if (pvec) {
                    reinterpret_cast<float4*>(prow + c0)[0] = make_float4(f[0], f[1], f[2], f[3]);
                    reinterpret_cast<float4*>(prow + c0)[1] = make_float4(f[4], f[5], f[6], f[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) prow[c0 + j] = f[j];
                }
            }
            if (drow) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] -= spread;
                const int jy = y - c0;
                if ((unsigned)jy < 8u) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] -= (j == jy) ? keep : 0.f;
                }
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j] * gscale, f[2 * j + 1] * gscale);
                if (dvec) {
                    *reinterpret_cast<uint4*>(drow + c0) = o;
                } else {
                    const __half* os = reinterpret_cast<const __half*>(&o);
#pragma unroll
                    for (int j = 0; j < 8; ++j) drow[c0 + j] = os[j];
                }
            }
        }
        if (out.loss_partial) {
            sum_log = block_reduce(sum_log, false) * kLn2;
            if (tid == 0) {
                const float py = y_ok ? fast_exp2(fmaf(zy, kLog2e, shift)) * inv_sum : 0.f;
                out.loss_partial[row] = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
            }
        }
        // this buffer is refilled by a bulk copy two rows from now: order the generic-proxy
        // accesses above before it
        ptx::fence_proxy_async_smem();
        __syncthreads();
    }
    if (*(volatile int*)&s_abort) {     // a wait gave up: let a copy that may still be in flight land before the block ends
        const unsigned long long t0 = ptx::global_ns();
        while (ptx::global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
}

// One block per row with the row in the block's registers: gradient and loss only (no
// probabilities kept), rows of whole 16-byte vectors, THREADS x VPT vectors at most.  A persistent
// block walks rows blockIdx.x, + gridDim.x, ...; thread 0 keeps the next row on its way into the
// other half of a two-row shared-memory buffer with a bulk copy, the block picks its vectors up
// from there once and never writes them back.  Maximum and sum meet in ONE block-wide step: every
// thread takes exponentials against its own maximum, (max, sum) pairs are merged by rescaling
// (warp shuffles, then one exchange through shared memory that every warp reads back), and the
// thread's factor exp(own max - row max) / sum goes into the single FMA that makes the gradient.
constexpr int kRegsMaxBuf = 4;

template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? 3 : (THREADS == 512 ? 2 : 1))
softmax_ce_rows_regs(const __half* __restrict__ logits, int64_t logits_stride, const int32_t* __restrict__ labels,
                     const float* __restrict__ scaling, const float* __restrict__ label_smoothing,
                     __half* __restrict__ dlogits, int64_t dlogits_stride, float* __restrict__ loss_partial, int batch,
                     int classes, uint32_t buf_stride, int nbuf, int* status, LossTail tail) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[kRegsMaxBuf];
    __shared__ float s_m[32], s_s[32], s_l[32];
    __shared__ int s_abort;
    constexpr int kWarps = THREADS / 32;
    constexpr float kFloor = -1.0e30f;             // stands in for -inf so that differences of maxima stay finite
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t row_bytes = (uint32_t)classes * 2u;
    const uint32_t buf0 = ptx::smem_u32(smem_raw);
    const uint32_t bar0 = ptx::smem_u32(&s_bar[0]);
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < nbuf; ++i) ptx::mbar_init(bar0 + 8u * i, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();

    const float ls = label_smoothing ? label_smoothing[0] : 0.f;
    const float keep = 1.0f - ls, spread = ls / (float)classes;
    const float inv_b = 1.0f / (float)batch;
    const float gscale = scaling[0] * inv_b;
    const float gb = -spread * gscale;
    const int nvec = classes >> 3;
    const uint4 kNegInf = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);

    // merges (m, s) of the other lane / warp into this one: s counts exponentials taken against m
    auto merge = [](float& m, float& s, float m2, float s2) {
        const float mn = fmaxf(m, m2);
        s = s * fast_exp2((m - mn) * kLog2e) + s2 * fast_exp2((m2 - mn) * kLog2e);
        m = mn;
    };

    float my_loss = 0.f;
    // rows blockIdx.x + k * gridDim.x; row k lives in buffer k % nbuf, and the rows up to nbuf - 1 ahead are on their way
    int row = blockIdx.x;
    if (tid == 0) {
        for (int k = 0; k < nbuf - 1; ++k) {
            const int64_t r = (int64_t)row + (int64_t)k * gridDim.x;
            if (r < batch) {
                ptx::mbar_expect_tx(bar0 + 8u * k, row_bytes);
                ptx::bulk_load_1d(buf0 + (uint32_t)k * buf_stride, logits + r * logits_stride, row_bytes, bar0 + 8u * k);
            }
        }
    }
    int b = 0;
    uint32_t phase = 0;
    for (; row < batch; row += gridDim.x) {
        {
            // the buffer of the row before this one was released by the barrier that ended it: refill it
            const int64_t r = (int64_t)row + (int64_t)(nbuf - 1) * gridDim.x;
            const int bn = b == 0 ? nbuf - 1 : b - 1;
            if (tid == 0 && r < batch) {
                ptx::mbar_expect_tx(bar0 + 8u * bn, row_bytes);
                ptx::bulk_load_1d(buf0 + (uint32_t)bn * buf_stride, logits + r * logits_stride, row_bytes,
                                  bar0 + 8u * bn);
            }
        }
        const bool ok = ptx::mbar_wait(bar0 + 8u * b, phase, &s_abort, status, 4);
        if (__syncthreads_or(ok ? 0 : 1)) break;
        const __half* srow = reinterpret_cast<const __half*>(smem_raw + (size_t)b * buf_stride);
        const int y_raw = labels[row];                    // out of range: matches no class
        const bool y_ok = (unsigned)y_raw < (unsigned)classes;
        const int y = y_ok ? y_raw : 0;
        const float zy = __half2float(srow[y]);

        uint4 raw[VPT];
        float m_t = kFloor;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = i * THREADS + tid;
            raw[i] = vec < nvec ? *reinterpret_cast<const uint4*>(srow + vec * 8) : kNegInf;
            m_t = fmaxf(m_t, half8_max(raw[i]));
        }
        const float sh_t = -m_t * kLog2e;
        float e[VPT][8];
        float s_t = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            half8_to_float(raw[i], e[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                e[i][j] = fast_exp2(fmaf(e[i][j], kLog2e, sh_t));
                s_t += e[i][j];
            }
        }
        float m = m_t, ssum = s_t;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
            merge(m, ssum, m2, s2);
        }
        if (lane == 0) { s_m[warp] = m; s_s[warp] = ssum; }
        __syncthreads();
        m = lane < kWarps ? s_m[lane] : kFloor;
        ssum = lane < kWarps ? s_s[lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
            merge(m, ssum, m2, s2);
        }
        // m = row maximum, ssum = sum of exponentials against it (the same in every thread)
        const float inv_sum = 1.0f / (ssum + 1e-8f);
        const float pf = fast_exp2((m_t - m) * kLog2e) * inv_sum;      // e * pf = probability
        const float ga = pf * gscale;
        __half* drow = dlogits + (int64_t)row * dlogits_stride;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vec = i * THREADS + tid;
            if (vec < nvec) {
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    oh[j] = __floats2half2_rn(fmaf(e[i][2 * j], ga, gb), fmaf(e[i][2 * j + 1], ga, gb));
                *reinterpret_cast<uint4*>(drow + vec * 8) = o;
            }
        }
        float sum_log = 0.f;
        if (ls != 0.f && loss_partial) {          // the same branch in every thread of the block
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
                if (i * THREADS + tid < nvec) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) t += fast_log2(fmaf(e[i][j], pf, 1e-8f));
                }
            t = warp_sum(t);
            if (lane == 0) s_l[warp] = t;
            __syncthreads();
            t = lane < kWarps ? s_l[lane] : 0.f;
            sum_log = warp_sum(t) * kLn2;
        }
        // the label's class, by the thread that stored its vector
        if (((y >> 3) % THREADS) == tid) {
            const float py = y_ok ? fast_exp2((zy - m) * kLog2e) * inv_sum : 0.f;
            if (y_ok) drow[y] = __float2half_rn((py - spread - keep) * gscale);
            const float row_loss = (-keep * logf(py + 1e-8f) - spread * sum_log) * inv_b;
            if (loss_partial) loss_partial[row] = row_loss;
            my_loss += row_loss;
        }
        // this buffer is refilled by a bulk copy at the top of the next row: order the generic-proxy
        // reads above before it (the barrier also frees s_m / s_s / s_l for the next row)
        ptx::fence_proxy_async_smem();
        __syncthreads();
        if (++b == nbuf) { b = 0; phase ^= 1u; }
    }
    if (*(volatile int*)&s_abort) {     // a wait gave up: let a copy that may still be in flight land before the block ends
        const unsigned long long t0 = ptx::global_ns();
        while (ptx::global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    loss_tail(tail, my_loss, batch);
}

// Fixed-order sum of the per-row partials (one block: every thread adds a fixed
// strided subset four values at a time, then a shared-memory tree), as
// softmax_ce_reduce_kernel does; also writes 1/batch.
__global__ void __launch_bounds__(1024)
softmax_ce_loss_reduce(const float* __restrict__ partial, float* __restrict__ loss,
                       float* __restrict__ inv_scaling, int batch) {
    __shared__ float s[1024];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (partial) {
        int i = threadIdx.x;
        for (; i + 3 * 1024 < batch; i += 4 * 1024) {       // four independent loads in flight
            a0 += partial[i];
            a1 += partial[i + 1024];
            a2 += partial[i + 2048];
            a3 += partial[i + 3072];
        }
        for (; i < batch; i += 1024) a0 += partial[i];
    }
    s[threadIdx.x] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    for (int w = 512; w > 0; w >>= 1) {
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
                float* inv_scaling, int batch, int classes, cudaStream_t s, int dtype = TRB200_DTYPE_F16) {
    const __half* z = static_cast<const __half*>(logits);
    const bool rows_aligned = aligned16(logits) && (logits_stride % 8 == 0);
    const bool bf16 = dtype == TRB200_DTYPE_BF16;
    // bfloat16 logits: the warp-per-row fused kernel only (what a 1000-class head needs)
    TRB_REQUIRE(!bf16 || (rows_aligned && classes <= 2048 && classes % 8 == 0 && !out.probs && out.dlogits && scaling &&
                          out.dlogits_stride % 8 == 0 && aligned16(out.dlogits)),
                TRB200_ERR_UNSUPPORTED,
                "softmax_ce: bfloat16 logits need the fused call without probs, 16-byte aligned rows and at most 2048 "
                "classes in whole vectors of 8 (classes=%d)", classes);
    // kernels that finish the loss themselves draw a completion counter; `fused_tail` says one did
    LossTail tail{loss, inv_scaling, nullptr, nullptr};
    bool fused_tail = false;
#ifndef TRB200_NO_LOSS_TAIL
    // only the two kernels that finish the loss themselves need a counter
    const bool lean_path = rows_aligned && classes <= 2048 && classes % 8 == 0 && !out.probs && out.dlogits && scaling &&
                           out.dlogits_stride % 8 == 0 && aligned16(out.dlogits);
    const bool regs_path = !lean_path && !(rows_aligned && classes <= 2048) && rows_aligned && classes % 8 == 0 &&
                           classes <= 32768 && !out.probs && out.dlogits && scaling && out.dlogits_stride % 8 == 0 &&
                           aligned16(out.dlogits);
    if ((loss || inv_scaling) && (lean_path || regs_path)) {
        // The counter (and its per-block sums) belongs to the (device, stream) of the call: work on one stream runs in
        // order, so two launches never share a counter while both are in flight.  64 (device, stream) pairs get one; a
        // call from a further stream does the loss with the separate reduction launch instead.
        static std::mutex slot_mutex;
        static struct { int dev; cudaStream_t stream; } owners[kLossTickets];
        static int owners_used = 0;
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
        int slot = -1;
        {
            std::lock_guard<std::mutex> lock(slot_mutex);
            for (int i = 0; i < owners_used; ++i)
                if (owners[i].dev == dev && owners[i].stream == s) { slot = i; break; }
            if (slot < 0 && owners_used < kLossTickets) {
                slot = owners_used++;
                owners[slot].dev = dev;
                owners[slot].stream = s;
            }
        }
        if (slot >= 0) {
            unsigned int* pool = nullptr;
            float* sums = nullptr;
            TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&pool), g_loss_tickets));
            TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&sums), g_loss_block_sums));
            tail.ticket = pool + slot;
            tail.block_sums = sums + (size_t)slot * kLossTailBlocks;
        }
    }
#endif
    if (rows_aligned && classes <= 2048 && classes % 8 == 0 && !out.probs && out.dlogits && scaling &&
        out.dlogits_stride % 8 == 0 && aligned16(out.dlogits)) {
        const int warps = 8;
        int blocks = (batch + warps - 1) / warps;
        // exactly the blocks that are resident at once (3 per SM, 2 for the widest rows): warps loop over rows, and a
        // grid of several partial waves would leave the last one half empty
        const int resident = sm_count() * (classes > 1024 ? 2 : 3);
        if (blocks > resident) blocks = resident;
        if (blocks > kLossTailBlocks) blocks = kLossTailBlocks;
        dim3 grid(blocks), block(warps * 32);
#define TRB_LEAN_LAUNCH(V)                                                                                        \
    (bf16 ? softmax_ce_rows_warp_lean_bf16<V> : softmax_ce_rows_warp_lean<V>)<<<grid, block, 0, s>>>(              \
        z, logits_stride, labels, scaling, label_smoothing, out.dlogits, out.dlogits_stride, out.loss_partial, batch, \
        classes, tail)
        if (classes <= 256) TRB_LEAN_LAUNCH(1);
        else if (classes <= 512) TRB_LEAN_LAUNCH(2);
        else if (classes <= 1024) TRB_LEAN_LAUNCH(4);
        else TRB_LEAN_LAUNCH(8);
#undef TRB_LEAN_LAUNCH
        TRB_LAUNCH_CHECK("softmax_ce_rows_warp_lean");
        fused_tail = tail.ticket != nullptr;
    } else if (rows_aligned && classes <= 2048) {
        const int warps = 8;
        int blocks = (batch + warps - 1) / warps;
        if (blocks > sm_count() * 8) blocks = sm_count() * 8;      // warps loop over rows
        dim3 grid(blocks), block(warps * 32);
        if (classes <= 256)
            softmax_ce_rows_warp<1><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else if (classes <= 512)
            softmax_ce_rows_warp<2><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else if (classes <= 1024)
            softmax_ce_rows_warp<4><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        else
            softmax_ce_rows_warp<8><<<grid, block, 0, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, batch, classes);
        TRB_LAUNCH_CHECK("softmax_ce_rows_warp");
    } else if (rows_aligned && classes % 8 == 0 && classes <= 32768 && !out.probs && out.dlogits && scaling &&
               out.dlogits_stride % 8 == 0 && aligned16(out.dlogits)) {
        // row in the block's registers: 256 threads x 2-5 vectors, 512 x 3-4 or 1024 x 3-4
        const uint32_t buf_stride = (uint32_t)align_up((int64_t)classes * 2, 128);
        const int nvec = classes / 8;
        const int threads = nvec <= 1280 ? 256 : (nvec <= 2048 ? 512 : 1024);
        const int vpt = (nvec + threads - 1) / threads;
        int* status = nullptr;
        TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_softmax_status));
        // as many blocks per SM as the registers allow, then as deep a ring as shared memory allows
        int per_sm = threads == 256 ? 3 : (threads == 512 ? 2 : 1);
        while (per_sm > 1 && (size_t)per_sm * 2 * buf_stride > 200 * 1024) --per_sm;
        int nbuf = (int)((200 * 1024) / ((size_t)per_sm * buf_stride));
        if (nbuf > kRegsMaxBuf) nbuf = kRegsMaxBuf;
        if (nbuf < 2) nbuf = 2;
        const size_t smem = (size_t)buf_stride * nbuf;
        int grid = sm_count() * per_sm;
        if (grid > batch) grid = batch;
        if (grid > kLossTailBlocks) grid = kLossTailBlocks;
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
#define TRB_RG_LAUNCH(T, V)                                                                                          \
    do {                                                                                                             \
        static bool done[64] = {false};                                                                              \
        if (dev >= 0 && dev < 64 && !done[dev]) {                                                                    \
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_regs<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                              200 * 1024));                                                          \
            done[dev] = true;                                                                                        \
        }                                                                                                            \
        softmax_ce_rows_regs<T, V><<<grid, T, smem, s>>>(z, logits_stride, labels, scaling, label_smoothing,         \
                                                         out.dlogits, out.dlogits_stride, out.loss_partial, batch,   \
                                                         classes, buf_stride, nbuf, status, tail);                   \
    } while (0)
        if (threads == 256) {
            if (vpt <= 2) TRB_RG_LAUNCH(256, 2);
            else if (vpt == 3) TRB_RG_LAUNCH(256, 3);
            else if (vpt == 4) TRB_RG_LAUNCH(256, 4);
            else TRB_RG_LAUNCH(256, 5);
        } else if (threads == 512) {
            if (vpt <= 3) TRB_RG_LAUNCH(512, 3);
            else TRB_RG_LAUNCH(512, 4);
        } else {
            if (vpt <= 3) TRB_RG_LAUNCH(1024, 3);
            else TRB_RG_LAUNCH(1024, 4);
        }
#undef TRB_RG_LAUNCH
        TRB_LAUNCH_CHECK("softmax_ce_rows_regs");
        fused_tail = tail.ticket != nullptr;
    } else if (rows_aligned && classes % 8 == 0 && (size_t)align_up((int64_t)classes * 2, 128) <= 48 * 1024) {
        const uint32_t buf_stride = (uint32_t)align_up((int64_t)classes * 2, 128);
        const size_t smem = (size_t)buf_stride * 2;
        static bool staged_attr_done[64] = {false};
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !staged_attr_done[dev]) {
            const int lim = 200 * 1024;
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<512, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<1024, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<512, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_staged<1024, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            staged_attr_done[dev] = true;
        }
        int* status = nullptr;
        TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_softmax_status));
        const int threads = classes <= 12288 ? 256 : (classes <= 24576 ? 512 : 1024);
        int per_sm = (int)((200 * 1024) / smem);
        if (per_sm > 2048 / threads) per_sm = 2048 / threads;
        if (per_sm < 1) per_sm = 1;
        int grid = sm_count() * per_sm;
        if (grid > batch) grid = batch;
        const bool e_half = !out.probs && out.dlogits;
#define TRB_ST_LAUNCH(T, E)                                                                                      \
    softmax_ce_rows_staged<T, E><<<grid, T, smem, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, \
                                                       batch, classes, buf_stride, status)
        if (threads == 256) { if (e_half) TRB_ST_LAUNCH(256, true); else TRB_ST_LAUNCH(256, false); }
        else if (threads == 512) { if (e_half) TRB_ST_LAUNCH(512, true); else TRB_ST_LAUNCH(512, false); }
        else { if (e_half) TRB_ST_LAUNCH(1024, true); else TRB_ST_LAUNCH(1024, false); }
#undef TRB_ST_LAUNCH
        TRB_LAUNCH_CHECK("softmax_ce_rows_staged");
    } else {
        const size_t row_bytes = (size_t)align_up((int64_t)classes * 2, 16);
        const int cache = row_bytes <= 200 * 1024 ? 1 : 0;
        const size_t smem = cache ? row_bytes : 0;
        static bool attr_done[64] = {false};
        int dev = 0;
        TRB_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_done[dev]) {
            const int lim = 200 * 1024;
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<512, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<1024, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<512, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            TRB_CUDA_TRY(cudaFuncSetAttribute(softmax_ce_rows_block<1024, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
            attr_done[dev] = true;
        }
        const int vec_ok = rows_aligned ? 1 : 0;
        const bool e_half = cache && !out.probs && out.dlogits;
#define TRB_SM_LAUNCH(T, E)                                                                                  \
    softmax_ce_rows_block<T, E><<<batch, T, smem, s>>>(z, logits_stride, labels, scaling, label_smoothing, out, \
                                                       batch, classes, cache, vec_ok)
        // four to eight 8-class vectors per thread and sweep; rows beyond 64 K classes take 1024 threads
        if (classes <= 8192) {
            if (e_half) TRB_SM_LAUNCH(256, true); else TRB_SM_LAUNCH(256, false);
        } else if (classes <= 65536) {
            if (e_half) TRB_SM_LAUNCH(512, true); else TRB_SM_LAUNCH(512, false);
        } else {
            if (e_half) TRB_SM_LAUNCH(1024, true); else TRB_SM_LAUNCH(1024, false);
        }
#undef TRB_SM_LAUNCH
        TRB_LAUNCH_CHECK("softmax_ce_rows_block");
    }
    if ((loss || inv_scaling) && !fused_tail) {
        softmax_ce_loss_reduce<<<1, 1024, 0, s>>>(out.loss_partial, loss, inv_scaling, batch);
        TRB_LAUNCH_CHECK("softmax_ce_loss_reduce");
    }
    return TRB200_OK;
}

}  // namespace

int softmax_status_read_and_clear(int* out) {
    int v = 0;
    TRB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_softmax_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        TRB_CUDA_TRY(cudaMemcpyToSymbol(g_softmax_status, &zero, sizeof(int)));
    }
    *out = v;
    return TRB200_OK;
}

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

extern "C" int trb200_softmax_ce_fused_dtype(const void* logits, int64_t logits_stride, const int32_t* labels,
                                             const float* scaling, const float* label_smoothing, void* dlogits,
                                             int64_t dlogits_stride, float* loss_partial, float* loss,
                                             float* inv_scaling, int32_t batch, int32_t classes, int32_t dtype,
                                             void* stream) {
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fused: unknown dtype %d", dtype);
    TRB_REQUIRE(logits && labels && dlogits && scaling, TRB200_ERR_INVALID_ARGUMENT,
                "softmax_ce_fused: null pointer");
    TRB_REQUIRE(batch > 0 && classes > 0 && logits_stride >= classes && dlogits_stride >= classes,
                TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fused: bad sizes (batch=%d classes=%d)", batch, classes);
    TRB_REQUIRE(!loss || loss_partial, TRB200_ERR_INVALID_ARGUMENT,
                "softmax_ce_fused: loss needs loss_partial");
    TRB_REQUIRE(dlogits != logits, TRB200_ERR_INVALID_ARGUMENT, "softmax_ce_fused: dlogits must not alias logits");
    trb::RowOut out{nullptr, 0, static_cast<__half*>(dlogits), dlogits_stride, loss_partial};
    return trb::launch_rows(logits, logits_stride, labels, scaling, label_smoothing, out, loss, inv_scaling,
                            batch, classes, trb::as_stream(stream), dtype);
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
