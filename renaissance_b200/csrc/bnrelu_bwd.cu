// BN + ReLU backward of the fused Conv+BN+ReLU block (HBM-bound, two sweeps).
//
// Replaces the cuDNN-FE graph MUL(dY, BOOLEAN mask) -> batchnorm_backward of the
// reference (src/backend/ops/dtensor/cbr_op.cpp:1259-1353).
//
// Data layout: dy, x, dconv are [m rows][c channels] half, c % 8 == 0, so one
// row is c/8 16-byte vectors and the mask byte that covers a vector has the same
// index as the vector (1 bit per element, least significant bit first).
//
// Sweep 1 (bnrelu_bwd_reduce): every thread owns 8 adjacent channels and walks a
//   strip of rows with 128-bit loads, keeping 2x8 float sums in registers; the
//   block adds its threads' sums in a fixed order through shared memory and
//   writes one partial per block.  bnrelu_bwd_finalize adds the partials of all
//   blocks in block order in double.  No float atomics anywhere, so dgamma and
//   dbeta are bitwise reproducible.
// Sweep 2 (bnrelu_bwd_apply): dconv = a*(dy_m - dbeta/m - (x-mean)*k) per channel,
//   written as 128-bit stores.  It walks the row strips in the opposite order of sweep 1 so
//   that the rows sweep 1 read last, still resident in L2, are consumed first.
//
// Algorithmic HBM bytes: 2 x (2 + 2 + 1/8) read + 2 written = 10.25 B / element.
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <mutex>

namespace trb {

__device__ int g_bn_status = 0;   // set when a bounded wait of the ring kernels gives up

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kBlocksPerSm = 2;     // resident blocks per SM at the kernels' register use

struct BnPlan {
    int tpr;     // 16-byte vectors per row
    int bx;      // threads along the row (vectors handled per block row)
    int by;      // rows handled per block step
    int gy;      // column chunks
    int gx;      // row strips
    int64_t rows_per_strip;
};

BnPlan make_plan(int64_t m, int c) {
    BnPlan p;
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
    // strips are multiples of the block's row step so that every strip starts on a
    // 16-byte boundary of the mask as well
    rps = (rps + p.by - 1) / p.by * p.by;
    p.rows_per_strip = rps;
    p.gx = (int)((m + rps - 1) / rps);
    return p;
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <bool BF16>
__device__ __forceinline__ void
bnrelu_bwd_reduce_body(const uint4* __restrict__ dy, const uint8_t* __restrict__ mask,
                       const uint4* __restrict__ x, const float* __restrict__ mean,
                       const float* __restrict__ inv_std, float* __restrict__ partial,
                       int64_t m, int c, int tpr, int bx, int by, int64_t rows_per_strip) {
    __shared__ float s_red[kThreads * 16];
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;           // vector (8-channel group) in the row
    const bool col_ok = vec < tpr && ty < by;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < m) ? r0 + rows_per_strip : m;

    float sb[8], sg[8], mu[8], is[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sb[j] = 0.f; sg[j] = 0.f; mu[j] = 0.f; is[j] = 0.f; }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { mu[j] = mean[vec * 8 + j]; is[j] = inv_std[vec * 8 + j]; }
        for (int64_t row = r0 + ty; row < r1; row += (int64_t)by * kUnroll) {
            uint4 vdy[kUnroll], vx[kUnroll];
            uint32_t mb[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int64_t r = row + (int64_t)u * by;
                if (r < r1) {
                    const int64_t v = r * tpr + vec;
                    vdy[u] = ld_stream(dy + v);
                    vx[u] = ld_stream(x + v);
                    mb[u] = mask ? mask[v] : 0xffu;
                } else {
                    vdy[u] = make_uint4(0, 0, 0, 0);
                    vx[u] = make_uint4(0, 0, 0, 0);
                    mb[u] = 0;
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                float g[8], xv[8];
                unpack8_t<BF16>(vdy[u], g);
                unpack8_t<BF16>(vx[u], xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float gm = (mb[u] >> j) & 1u ? g[j] : 0.f;
                    sb[j] += gm;
                    sg[j] += gm * ((xv[j] - mu[j]) * is[j]);
                }
            }
        }
    }
    // block reduction over ty in ascending order
    float* mine = s_red + (size_t)threadIdx.x * 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = sb[j]; mine[8 + j] = sg[j]; }
    __syncthreads();
    // thread t < bx*16 owns value (tx = t / 16, j = t % 16)
    for (int t = threadIdx.x; t < bx * 16; t += kThreads) {
        const int otx = t / 16, j = t % 16;
        const int ovec = blockIdx.y * bx + otx;
        if (ovec >= tpr) continue;
        float acc = 0.f;
        for (int y = 0; y < by; ++y) acc += s_red[(size_t)(y * bx + otx) * 16 + j];
        const int ch = ovec * 8 + (j & 7);
        // partial[strip][stat][c], stat 0 = dbeta, 1 = dgamma
        partial[((size_t)blockIdx.x * 2 + (j >> 3)) * c + ch] = acc;
    }
}

// One warp per (statistic, channel): lanes add every 32nd strip in double, then a
// fixed butterfly adds the lanes, so the order of additions never changes.
#define TRB_BN_REDUCE_ARGS                                                                                   \
    const uint4 *__restrict__ dy, const uint8_t *__restrict__ mask, const uint4 *__restrict__ x,                 \
        const float *__restrict__ mean, const float *__restrict__ inv_std, float *__restrict__ partial, int64_t m, \
        int c, int tpr, int bx, int by, int64_t rows_per_strip

__global__ void __launch_bounds__(kThreads) bnrelu_bwd_reduce(TRB_BN_REDUCE_ARGS) {
    bnrelu_bwd_reduce_body<false>(dy, mask, x, mean, inv_std, partial, m, c, tpr, bx, by, rows_per_strip);
}

__global__ void __launch_bounds__(kThreads) bnrelu_bwd_reduce_bf16(TRB_BN_REDUCE_ARGS) {
    bnrelu_bwd_reduce_body<true>(dy, mask, x, mean, inv_std, partial, m, c, tpr, bx, by, rows_per_strip);
}

__global__ void __launch_bounds__(256)
bnrelu_bwd_finalize(const float* __restrict__ partial, float* __restrict__ dgamma,
                    float* __restrict__ dbeta, int c, int strips) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // i in [0, 2c)
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

template <bool BF16>
__device__ __forceinline__ void
bnrelu_bwd_apply_body(const uint4* __restrict__ dy, const uint8_t* __restrict__ mask,
                      const uint4* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ mean, const float* __restrict__ inv_std,
                      const float* __restrict__ dgamma, const float* __restrict__ dbeta,
                      uint4* __restrict__ out, int64_t m, int tpr, int bx, int by,
                      int64_t rows_per_strip) {
    const int tx = threadIdx.x % bx, ty = threadIdx.x / bx;
    const int vec = blockIdx.y * bx + tx;
    if (vec >= tpr || ty >= by) return;
    // reverse strip order: see the header of this file
    const int strip = gridDim.x - 1 - blockIdx.x;
    const int64_t r0 = (int64_t)strip * rows_per_strip;
    const int64_t r1 = (r0 + rows_per_strip < m) ? r0 + rows_per_strip : m;

    // out = a * (g - mb - (x - mu) * k), a = gamma*inv_std, mb = dbeta/m, k = inv_std * dgamma/m
    float ca[8], cmb[8], cmu[8], ck[8];
    const float inv_m = 1.0f / (float)m;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int ch = vec * 8 + j;
        const float is = inv_std[ch];
        ca[j] = gamma[ch] * is;
        cmb[j] = dbeta[ch] * inv_m;
        cmu[j] = mean[ch];
        ck[j] = is * (dgamma[ch] * inv_m);
    }
    for (int64_t row = r0 + ty; row < r1; row += (int64_t)by * kUnroll) {
        uint4 vdy[kUnroll], vx[kUnroll];
        uint32_t mb[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t r = row + (int64_t)u * by;
            if (r < r1) {
                const int64_t v = r * tpr + vec;
                vdy[u] = ld_stream(dy + v);
                vx[u] = ld_stream(x + v);
                mb[u] = mask ? mask[v] : 0xffu;
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t r = row + (int64_t)u * by;
            if (r >= r1) continue;
            float g[8], xv[8];
            unpack8_t<BF16>(vdy[u], g);
            unpack8_t<BF16>(vx[u], xv);
            uint4 o;
            uint32_t* oh = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g0 = (mb[u] >> (2 * j)) & 1u ? g[2 * j] : 0.f;
                const float g1 = (mb[u] >> (2 * j + 1)) & 1u ? g[2 * j + 1] : 0.f;
                const float o0 = ca[2 * j] * (g0 - cmb[2 * j] - (xv[2 * j] - cmu[2 * j]) * ck[2 * j]);
                const float o1 = ca[2 * j + 1] * (g1 - cmb[2 * j + 1] - (xv[2 * j + 1] - cmu[2 * j + 1]) * ck[2 * j + 1]);
                oh[j] = pack2_t<BF16>(o0, o1);
            }
            out[r * tpr + vec] = o;
        }
    }
}

#define TRB_BN_APPLY_ARGS                                                                                     \
    const uint4 *__restrict__ dy, const uint8_t *__restrict__ mask, const uint4 *__restrict__ x,                  \
        const float *__restrict__ gamma, const float *__restrict__ mean, const float *__restrict__ inv_std,       \
        const float *__restrict__ dgamma, const float *__restrict__ dbeta, uint4 *__restrict__ out, int64_t m,    \
        int tpr, int bx, int by, int64_t rows_per_strip

__global__ void __launch_bounds__(kThreads) bnrelu_bwd_apply(TRB_BN_APPLY_ARGS) {
    bnrelu_bwd_apply_body<false>(dy, mask, x, gamma, mean, inv_std, dgamma, dbeta, out, m, tpr, bx, by,
                                 rows_per_strip);
}

__global__ void __launch_bounds__(kThreads) bnrelu_bwd_apply_bf16(TRB_BN_APPLY_ARGS) {
    bnrelu_bwd_apply_body<true>(dy, mask, x, gamma, mean, inv_std, dgamma, dbeta, out, m, tpr, bx, by,
                                rows_per_strip);
}

// ---------------------------------------------------------------------------------------------------------------
// The same two sweeps on a ring of bulk copies.  In the kernels above a thread keeps four rows in flight and then
// works through them, so what is in flight follows the SM clock and the occupancy; inside a power-capped training
// step they lose 10-25 % of the bandwidth they reach alone.  Here one thread of a producer warp streams the three
// operands of a run of rows into shared memory with bulk copies (stages of ~33 KB), and 512 consumer threads, each
// keeping its 8 channels, work from shared memory.  The ReLU mask is applied on packed halfs (two channels per
// operation).  Rows beyond the last whole item are read with plain loads by block 0.
constexpr int kRingStages = 5;
constexpr int kRingConsumers = 512;
constexpr int kRingPasses = 2;       // rows of an item = passes x (consumers / vectors per row)

struct BnRingPlan {
    int ok;
    int ppp, item_rows, grid;
    uint32_t v_bytes, m_bytes, stage_bytes;     // one operand of an item, its mask bytes, a stage
    int64_t items;                              // whole items
};

BnRingPlan make_bn_ring_plan(int64_t m, int c) {
    BnRingPlan p{};
    const int tpr = c / 8;
    if (tpr > kRingConsumers || (tpr & (tpr - 1)) != 0) return p;
    p.ppp = kRingConsumers / tpr;
    p.item_rows = p.ppp * kRingPasses;
    p.items = m / p.item_rows;
    if (p.items < 4 * (int64_t)sm_count()) return p;          // short tensors stay on the strip kernels
    p.v_bytes = (uint32_t)kRingConsumers * kRingPasses * 16u;
    p.m_bytes = (uint32_t)kRingConsumers * kRingPasses;
    p.stage_bytes = 2 * p.v_bytes + p.m_bytes;
    p.grid = sm_count();
    p.ok = 1;
    return p;
}

// lane masks (0xffff per half) of the four channel pairs from one mask byte: the low and the high nibble are
// spread to the top bits of four bytes by one multiply each, a sign-replicating byte permute widens them
__device__ __forceinline__ void lane_masks(uint32_t mb, uint32_t (&lm)[4]) {
    const uint32_t lo = (mb & 15u) * 0x10204080u, hi = (mb >> 4) * 0x10204080u;
    lm[0] = ptx::prmt_b32(lo, 0u, 0x9988u);
    lm[1] = ptx::prmt_b32(lo, 0u, 0xbbaau);
    lm[2] = ptx::prmt_b32(hi, 0u, 0x9988u);
    lm[3] = ptx::prmt_b32(hi, 0u, 0xbbaau);
}

template <bool APPLY, bool BF16, bool MASK>
__global__ void __launch_bounds__(kRingConsumers + 32)
bnrelu_bwd_ring(const unsigned char* __restrict__ dy, const unsigned char* __restrict__ mask,
                const unsigned char* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ mean,
                const float* __restrict__ inv_std, const float* __restrict__ dgamma, const float* __restrict__ dbeta,
                float* __restrict__ partial, uint4* __restrict__ out, int64_t m, int c, int tpr, BnRingPlan pl,
                int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kRingStages], s_empty[kRingStages];
    __shared__ int s_abort;
    const int tid = threadIdx.x;
    const uint32_t buf0 = ptx::smem_u32(smem_raw);
    const uint32_t full0 = ptx::smem_u32(&s_full[0]), empty0 = ptx::smem_u32(&s_empty[0]);
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < kRingStages; ++i) {
            ptx::mbar_init(full0 + 8u * i, 1);
            ptx::mbar_init(empty0 + 8u * i, kRingConsumers / 32);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();

    // the apply pass walks the items backwards: what the reduce pass read last is still in L2
    auto item_of = [&](int64_t k) -> int64_t {
        const int64_t it = (int64_t)blockIdx.x + k * gridDim.x;
        return APPLY ? pl.items - 1 - it : it;
    };
    const int64_t my_items = (pl.items - blockIdx.x + gridDim.x - 1) / gridDim.x;

    if (tid >= kRingConsumers) {
        if (tid == kRingConsumers) {
            for (int64_t k = 0; k < my_items; ++k) {
                const int st = (int)(k % kRingStages);
                if (k >= kRingStages &&
                    !ptx::mbar_wait_relaxed(empty0 + 8u * st, (uint32_t)((k / kRingStages - 1) & 1), &s_abort, status, 23))
                    break;
                const int64_t v0 = item_of(k) * (int64_t)(kRingConsumers * kRingPasses);     // first 16-byte vector
                const uint32_t dst = buf0 + (uint32_t)st * pl.stage_bytes;
                const uint32_t bar = full0 + 8u * st;
                ptx::mbar_expect_tx(bar, 2 * pl.v_bytes + (MASK ? pl.m_bytes : 0u));
                ptx::bulk_load_1d(dst, dy + v0 * 16, pl.v_bytes, bar);
                ptx::bulk_load_1d(dst + pl.v_bytes, x + v0 * 16, pl.v_bytes, bar);
                if (MASK) ptx::bulk_load_1d(dst + 2 * pl.v_bytes, mask + v0, pl.m_bytes, bar);
            }
        }
        return;
    }

    // ---------------- consumers
    const int vec = tid % tpr;
    float k0[8], k1[8], k2[8], k3[8];
    // reduce: k0 = mean, k2 = sum dy_m, k3 = sum dy_m (x - mean);  apply: dconv = (x - k0) * k1 + (k2 * g + k3)
    const float inv_m = 1.0f / (float)m;
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
            k1[j] = 0.f;
            k2[j] = 0.f;
            k3[j] = 0.f;
        }
    }
    auto work = [&](const uint4& g4, const uint4& x4, uint32_t mb, int64_t ovec) {
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, xw[4] = {x4.x, x4.y, x4.z, x4.w};
        uint32_t lm[4];
        if (MASK) lane_masks(mb, lm);
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 gf = unpack2_t<BF16>(MASK ? (gw[i] & lm[i]) : gw[i]);
            const float2 xf = unpack2_t<BF16>(xw[i]);
            if (!APPLY) {
                k2[2 * i] += gf.x;
                k2[2 * i + 1] += gf.y;
                k3[2 * i] = fmaf(gf.x, xf.x - k0[2 * i], k3[2 * i]);
                k3[2 * i + 1] = fmaf(gf.y, xf.y - k0[2 * i + 1], k3[2 * i + 1]);
            } else {
                ow[i] = pack2_t<BF16>(fmaf(xf.x - k0[2 * i], k1[2 * i], fmaf(k2[2 * i], gf.x, k3[2 * i])),
                                      fmaf(xf.y - k0[2 * i + 1], k1[2 * i + 1], fmaf(k2[2 * i + 1], gf.y, k3[2 * i + 1])));
            }
        }
        if (APPLY) out[ovec] = o;
    };
    auto tail = [&]() {
        // rows past the last whole item: block 0, plain loads
        if (blockIdx.x != 0) return;
        const int64_t v_end = m * tpr;
        for (int64_t v = pl.items * (int64_t)(kRingConsumers * kRingPasses) + tid; v < v_end; v += kRingConsumers) {
            const uint4 g4 = *reinterpret_cast<const uint4*>(dy + v * 16);
            const uint4 x4 = *reinterpret_cast<const uint4*>(x + v * 16);
            work(g4, x4, MASK ? (uint32_t)mask[v] : 0xffu, v);
        }
    };
    if (APPLY) tail();
    for (int64_t k = 0; k < my_items; ++k) {
        const int st = (int)(k % kRingStages);
        if (!ptx::mbar_wait(full0 + 8u * st, (uint32_t)((k / kRingStages) & 1), &s_abort, status, 24)) break;
        const unsigned char* sdy = smem_raw + (size_t)st * pl.stage_bytes;
        const unsigned char* sx = sdy + pl.v_bytes;
        const unsigned char* sm = sx + pl.v_bytes;
        const int64_t v0 = APPLY ? item_of(k) * (int64_t)(kRingConsumers * kRingPasses) : 0;
#pragma unroll
        for (int ps = 0; ps < kRingPasses; ++ps) {
            const int v = ps * kRingConsumers + tid;            // consecutive threads, consecutive vectors
            work(*reinterpret_cast<const uint4*>(sdy + (size_t)v * 16), *reinterpret_cast<const uint4*>(sx + (size_t)v * 16),
                 MASK ? (uint32_t)sm[v] : 0xffu, v0 + v);
        }
        __syncwarp();
        if ((tid & 31) == 0) ptx::mbar_arrive(empty0 + 8u * st);
    }
    if (!APPLY) {
        tail();
        // block sums in a fixed order; the ring is idle now (every copy issued has been waited for)
        ptx::named_barrier(1, kRingConsumers);
        float* s_red = reinterpret_cast<float*>(smem_raw);
        float* mine = s_red + (size_t)tid * 16;
#pragma unroll
        for (int j = 0; j < 8; ++j) { mine[j] = k2[j]; mine[8 + j] = k3[j]; }
        ptx::named_barrier(1, kRingConsumers);
        for (int t = tid; t < tpr * 16; t += kRingConsumers) {
            const int ovec = t / 16, j = t % 16;
            float acc = 0.f;
            for (int y = 0; y < pl.ppp; ++y) acc += s_red[(size_t)(y * tpr + ovec) * 16 + j];
            const int chn = ovec * 8 + (j & 7);
            if (j >> 3) acc *= inv_std[chn];                    // sum dy_m (x - mean) -> sum dy_m x_hat
            partial[((size_t)blockIdx.x * 2 + (j >> 3)) * c + chn] = acc;
        }
    }
}

}  // namespace

namespace {

template <bool BF16, bool MASK>
int bnrelu_bwd_ring_launch_t(const BnRingPlan& rp, const void* dy, const void* mask_bits, const void* x, const float* gamma,
                             const float* saved_mean, const float* saved_inv_std, void* dconv, float* dgamma,
                             float* dbeta, float* partial, int64_t m, int c, cudaStream_t s) {
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    const size_t smem = (size_t)kRingStages * rp.stage_bytes;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(bnrelu_bwd_ring<false, BF16, MASK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
        TRB_CUDA_TRY(cudaFuncSetAttribute(bnrelu_bwd_ring<true, BF16, MASK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_bn_status));
    auto b = [](const void* q) { return static_cast<const unsigned char*>(q); };
    const int threads = kRingConsumers + 32;
    bnrelu_bwd_ring<false, BF16, MASK><<<rp.grid, threads, smem, s>>>(b(dy), b(mask_bits), b(x), gamma, saved_mean,
                                                                      saved_inv_std, dgamma, dbeta, partial, nullptr, m, c,
                                                                      c / 8, rp, status);
    TRB_LAUNCH_CHECK("bnrelu_bwd_ring<reduce>");
    bnrelu_bwd_finalize<<<(2 * c + 7) / 8, 256, 0, s>>>(partial, dgamma, dbeta, c, rp.grid);
    TRB_LAUNCH_CHECK("bnrelu_bwd_finalize");
    if (dconv) {
        bnrelu_bwd_ring<true, BF16, MASK><<<rp.grid, threads, smem, s>>>(b(dy), b(mask_bits), b(x), gamma, saved_mean,
                                                                         saved_inv_std, dgamma, dbeta, partial,
                                                                         static_cast<uint4*>(dconv), m, c, c / 8, rp, status);
        TRB_LAUNCH_CHECK("bnrelu_bwd_ring<apply>");
    }
    return TRB200_OK;
}

int bnrelu_bwd_ring_launch(const BnRingPlan& rp, const void* dy, const void* mask_bits, const void* x, const float* gamma,
                           const float* saved_mean, const float* saved_inv_std, void* dconv, float* dgamma, float* dbeta,
                           float* partial, int64_t m, int c, cudaStream_t s, bool bf16) {
#define TRB_RING_CASE(B, M)                                                                                              \
    return bnrelu_bwd_ring_launch_t<B, M>(rp, dy, mask_bits, x, gamma, saved_mean, saved_inv_std, dconv, dgamma, dbeta, \
                                          partial, m, c, s)
    if (bf16) {
        if (mask_bits) TRB_RING_CASE(true, true);
        TRB_RING_CASE(true, false);
    }
    if (mask_bits) TRB_RING_CASE(false, true);
    TRB_RING_CASE(false, false);
#undef TRB_RING_CASE
}

}  // namespace

// device address of the status word the bulk-copy ring kernels (this file, pool_fused.cu, block_fwd.cu) report to
int ring_status_ptr(int** out) {
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(out), g_bn_status));
    return TRB200_OK;
}

int bn_status_read_and_clear(int* out) {
    int v = 0;
    TRB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_bn_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        TRB_CUDA_TRY(cudaMemcpyToSymbol(g_bn_status, &zero, sizeof(int)));
    }
    *out = v;
    return TRB200_OK;
}

int bnrelu_bwd_launch(const void* dy, const void* mask_bits, const void* x, const float* gamma,
                      const float* saved_mean, const float* saved_inv_std, void* dconv,
                      float* dgamma, float* dbeta, int64_t m, int c, void* workspace,
                      size_t workspace_bytes, cudaStream_t s, int dtype) {
    TRB_REQUIRE(valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "bnrelu_bwd: unknown dtype %d", dtype);
    const bool bf16 = dtype == TRB200_DTYPE_BF16;
    // mask_bits may be NULL: no ReLU behind this BN (every element kept), the plain batch-norm backward
    TRB_REQUIRE(dy && x && gamma && saved_mean && saved_inv_std && dgamma && dbeta,
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_bwd: null pointer");
    TRB_REQUIRE(m > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "bnrelu_bwd: need m > 0 and c a positive multiple of 8 (m=%lld c=%d)", (long long)m, c);
    TRB_REQUIRE(aligned16(dy) && aligned16(x) && (!dconv || aligned16(dconv)),
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_bwd: dy, x and dconv must be 16-byte aligned");
    TRB_REQUIRE(dconv != dy && dconv != x, TRB200_ERR_INVALID_ARGUMENT,
                "bnrelu_bwd: dconv must not alias dy or x");
    const size_t need = trb200_bnrelu_bwd_workspace_bytes(m, c);
    TRB_REQUIRE(workspace && workspace_bytes >= need, TRB200_ERR_WORKSPACE,
                "bnrelu_bwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    float* partial = static_cast<float*>(workspace);
    const BnRingPlan rp = make_bn_ring_plan(m, c);
    if (rp.ok && (!mask_bits || aligned16(mask_bits))) {
        const int rc = bnrelu_bwd_ring_launch(rp, dy, mask_bits, x, gamma, saved_mean, saved_inv_std, dconv, dgamma, dbeta,
                                              partial, m, c, s, bf16);
        if (rc != TRB200_ERR_UNSUPPORTED) return rc;
    }
    const BnPlan p = make_plan(m, c);
    dim3 grid(p.gx, p.gy);
    (bf16 ? bnrelu_bwd_reduce_bf16 : bnrelu_bwd_reduce)<<<grid, kThreads, 0, s>>>(
        static_cast<const uint4*>(dy), static_cast<const uint8_t*>(mask_bits),
        static_cast<const uint4*>(x), saved_mean, saved_inv_std, partial, m, c, p.tpr, p.bx, p.by,
        p.rows_per_strip);
    TRB_LAUNCH_CHECK("bnrelu_bwd_reduce");
    bnrelu_bwd_finalize<<<(2 * c + 7) / 8, 256, 0, s>>>(partial, dgamma, dbeta, c, p.gx);
    TRB_LAUNCH_CHECK("bnrelu_bwd_finalize");
    if (dconv) {
        (bf16 ? bnrelu_bwd_apply_bf16 : bnrelu_bwd_apply)<<<grid, kThreads, 0, s>>>(
            static_cast<const uint4*>(dy), static_cast<const uint8_t*>(mask_bits),
            static_cast<const uint4*>(x), gamma, saved_mean, saved_inv_std, dgamma, dbeta,
            static_cast<uint4*>(dconv), m, p.tpr, p.bx, p.by, p.rows_per_strip);
        TRB_LAUNCH_CHECK("bnrelu_bwd_apply");
    }
    return TRB200_OK;
}

int bn_ring_strips(int64_t m, int c) {
    const BnRingPlan rp = make_bn_ring_plan(m, c);
    return rp.ok ? rp.grid : 0;
}

}  // namespace trb

extern "C" size_t trb200_bnrelu_bwd_workspace_bytes(int64_t m, int32_t c) {
    if (m <= 0 || c <= 0 || c % 8 != 0) return 0;
    const trb::BnPlan p = trb::make_plan(m, c);
    const int ring = trb::bn_ring_strips(m, c);
    return (size_t)(ring > p.gx ? ring : p.gx) * 2 * (size_t)c * sizeof(float);
}

extern "C" int trb200_bnrelu_bwd(const void* dy, const void* mask_bits, const void* x,
                                 const float* gamma, const float* saved_mean,
                                 const float* saved_inv_std, void* dconv, float* dgamma,
                                 float* dbeta, int64_t m, int32_t c, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    return trb::bnrelu_bwd_launch(dy, mask_bits, x, gamma, saved_mean, saved_inv_std, dconv, dgamma,
                                  dbeta, m, c, workspace, workspace_bytes, trb::as_stream(stream), TRB200_DTYPE_F16);
}

extern "C" int trb200_bnrelu_bwd_dtype(const void* dy, const void* mask_bits, const void* x,
                                       const float* gamma, const float* saved_mean,
                                       const float* saved_inv_std, void* dconv, float* dgamma,
                                       float* dbeta, int64_t m, int32_t c, int32_t dtype, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    return trb::bnrelu_bwd_launch(dy, mask_bits, x, gamma, saved_mean, saved_inv_std, dconv, dgamma,
                                  dbeta, m, c, workspace, workspace_bytes, trb::as_stream(stream), dtype);
}

// ---------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they need
// the operator: a replay-only runtime whose memory plan is frozen after start-up, a
// plugin that runs inside another framework's stream capture, or a process that has
// handed all of the GPU's memory to its own arena.  For them the per-strip partial
// sums live in a fixed array that is part of the library image instead of a
// caller-provided workspace.  Every GPU that loads the library holds these 4 MiB
// until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticPartialFloats = 1u << 20;                  // 4 MiB
constexpr int kStaticMaxChannels = 4096;
static __device__ __align__(256) float g_bnrelu_static_partials[kStaticPartialFloats];

// Same strip layout as make_plan(), with fewer strips when c is large so that
// strips * 2 * c floats fit the fixed array.
static trb::BnPlan make_static_plan(int64_t m, int c) {
    trb::BnPlan p = trb::make_plan(m, c);
    const int64_t cap = (int64_t)(kStaticPartialFloats / (2 * (size_t)c));
    if (p.gx > cap) {
        p.gx = (int)cap;
        int64_t rps = (m + p.gx - 1) / p.gx;
        rps = (rps + p.by - 1) / p.by * p.by;
        p.rows_per_strip = rps;
        p.gx = (int)((m + rps - 1) / rps);
    }
    return p;
}

// Device address of the fixed array on the CURRENT device, looked up once per device.
// In host code the array's name only stands for the symbol; the address a kernel can
// use comes from cudaGetSymbolAddress.
static int static_partials_ptr(float** out) {
    static std::mutex mu;
    static float* cached[64] = {nullptr};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    TRB_REQUIRE(dev >= 0 && dev < 64, TRB200_ERR_UNSUPPORTED, "bnrelu_bwd_static: device ordinal %d not covered", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        float* ptr = nullptr;
        TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_bnrelu_static_partials));
        TRB_REQUIRE(ptr != nullptr, TRB200_ERR_CUDA, "bnrelu_bwd_static: no device address for the fixed scratch");
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return TRB200_OK;
}

extern "C" int trb200_bnrelu_bwd_static(const void* dy, const void* mask_bits, const void* x,
                                        const float* gamma, const float* saved_mean,
                                        const float* saved_inv_std, void* dconv, float* dgamma,
                                        float* dbeta, int64_t m, int32_t c, void* stream) {
    TRB_REQUIRE(dy && mask_bits && x && gamma && saved_mean && saved_inv_std && dgamma && dbeta,
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_bwd_static: null pointer");
    TRB_REQUIRE(m > 0 && c > 0 && c % 8 == 0, TRB200_ERR_UNSUPPORTED,
                "bnrelu_bwd_static: need m > 0 and c a positive multiple of 8 (m=%lld c=%d)", (long long)m, c);
    TRB_REQUIRE(c <= kStaticMaxChannels, TRB200_ERR_UNSUPPORTED,
                "bnrelu_bwd_static: c=%d is beyond the %d channels the fixed 4 MiB scratch covers; "
                "use trb200_bnrelu_bwd with a workspace", c, kStaticMaxChannels);
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(x) && (!dconv || trb::aligned16(dconv)),
                TRB200_ERR_INVALID_ARGUMENT, "bnrelu_bwd_static: dy, x and dconv must be 16-byte aligned");
    TRB_REQUIRE(dconv != dy && dconv != x, TRB200_ERR_INVALID_ARGUMENT,
                "bnrelu_bwd_static: dconv must not alias dy or x");
    float* partial = nullptr;
    const int rc = static_partials_ptr(&partial);
    if (rc) return rc;
    const trb::BnPlan p = make_static_plan(m, c);
    cudaStream_t s = trb::as_stream(stream);
    dim3 grid(p.gx, p.gy);
    // every strip overwrites all of its partials before the finalize kernel reads them,
    // so nothing left in the array by an earlier call is ever read
    trb::bnrelu_bwd_reduce<<<grid, trb::kThreads, 0, s>>>(
        static_cast<const uint4*>(dy), static_cast<const uint8_t*>(mask_bits), static_cast<const uint4*>(x),
        saved_mean, saved_inv_std, partial, m, c, p.tpr, p.bx, p.by, p.rows_per_strip);
    TRB_LAUNCH_CHECK("bnrelu_bwd_reduce (static scratch)");
    trb::bnrelu_bwd_finalize<<<(2 * c + 7) / 8, 256, 0, s>>>(partial, dgamma, dbeta, c, p.gx);
    TRB_LAUNCH_CHECK("bnrelu_bwd_finalize (static scratch)");
    if (dconv) {
        trb::bnrelu_bwd_apply<<<grid, trb::kThreads, 0, s>>>(
            static_cast<const uint4*>(dy), static_cast<const uint8_t*>(mask_bits), static_cast<const uint4*>(x),
            gamma, saved_mean, saved_inv_std, dgamma, dbeta, static_cast<uint4*>(dconv), m, p.tpr, p.bx, p.by,
            p.rows_per_strip);
        TRB_LAUNCH_CHECK("bnrelu_bwd_apply (static scratch)");
    }
    return TRB200_OK;
}
