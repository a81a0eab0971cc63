// 3x3 / stride 1 / pad 1 weight gradient with the (tap, input-channel block) units on the
// MMA's N dimension.
//
//   dW[k][tap][c] = sum_pixels dconv[p][k] * X[p + tap offset][c]
//   D[k][u * 64 + c'] with unit u = tap * (C / 64) + c / 64: in KRSC order row k of dW is
//   exactly the 9 * C columns u * 64 + c', so the accumulator tile is a piece of dW as stored.
//   M = 128 filters k (A operand = dconv, 64 pixels x 64-filter blocks, MN-major),
//   N = up to 4 units = 256 columns (B operand = tap-shifted boxes of X, MN-major),
//   K loop = pixels, 64 per stage.
//
// The thread that issues the MMAs pays about 55 clocks per tcgen05.mma, commit or barrier probe, so its ~460
// clocks per K step of four MMAs hide behind the tensor pipe only at N = 256 (4 x 128 clocks): with the filters on N
// (wgrad_igemm_kernel) a 64-filter layer needs one instruction per two units and 16 pixels, here one per four units.
//
// Work item = (split of the pixel range, block of 128 filters, group of units); every item
// leaves a float partial tile and wgrad_unitn_reduce adds the splits in split order (bitwise
// reproducible) and writes half KRSC.  A group is 4 units, or 3 for 64 input channels: they have 9 units, and groups
// of 4, 4, 1 make the last third of the work items a third as long as the others
// (the kernel runs as long as its longest item); groups of 3, 3, 3 at N = 192 keep the pipe as busy and the items
// equal (0.46 -> 0.39 ms at 256 x 112 x 112, 64 -> 128).  With 64 filters the second half of the A operand is
// never loaded and lanes 64-127 of the accumulator are never read.
//
// This file is included by conv_igemm_sm100.cu inside its anonymous namespace.
#pragma once

struct WgradUnitnParams {
    int cblocks;        // C / 64
    int units;          // 9 * cblocks
    int upg;            // units per group: 4, or 3 when that divides the units (9 units: groups of 3, 3, 3 instead of
                        // 4, 4, 1, so that every work item is the same length)
    int n_tiles;        // ceil(units / upg)
    int k_blocks;       // ceil(K / 128)
    int k_halves;       // 64-filter blocks in a filter block: 1 (K = 64) or 2
    int splits;
    int pix_tiles;
    int tw, th;
    int bw, bh, bn;     // 64-pixel box
    int kk, cc;         // K, C
    int bf16;           // operands and dW are bfloat16 instead of half
};

constexpr int kUnABytes = 2 * kStageTileBytes;     // 64 pixels x 128 filters
constexpr int kUnBBytes = 4 * kStageTileBytes;     // 64 pixels x 4 units
constexpr int kUnStageBytes = kUnABytes + kUnBBytes;
constexpr int kUnStages = 4;
constexpr int kUnSmemTotal = kUnStages * kUnStageBytes + 2048;
static_assert(kUnSmemTotal <= kSmemBudget, "shared memory budget");

__global__ void __launch_bounds__(kThreads, 1)
wgrad_unitn_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                   float* __restrict__ partial, const WgradUnitnParams p, int* status) {
    constexpr int kStages = kUnStages;
    constexpr uint32_t kTmemCols = 256;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_base = base;
    const uint32_t b_base = base + kStages * kUnABytes;
    const uint32_t bar_base = b_base + kStages * kUnBBytes;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    const uint32_t done_bar = bar_base + 8u * (2 * kStages);
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        // a stage is full once the dconv boxes and both pairs of unit boxes have landed
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, 3); mbar_init(empty0 + 8u * s, 1); }
        mbar_init(done_bar, 1);
        fence_barrier_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_dy);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&s_tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    volatile int* abort_flag = &s_abort;

    // work item -> (split, filter block, unit group)
    const int item = blockIdx.x;
    const int nt = item % p.n_tiles;
    const int kb = (item / p.n_tiles) % p.k_blocks;
    const int split = item / (p.n_tiles * p.k_blocks);
    const int pt0 = (int)((long)p.pix_tiles * split / p.splits);
    const int pt1 = (int)((long)p.pix_tiles * (split + 1) / p.splits);
    const int u0 = nt * p.upg;
    const int nu = p.units - u0 < p.upg ? p.units - u0 : p.upg;  // units of this group
    // pixel tiles are walked with running box origins (w fastest, then h, then n)
    const int w_first = (pt0 % p.tw) * p.bw, h_first = ((pt0 / p.tw) % p.th) * p.bh;
    const int n_first = (pt0 / (p.tw * p.th)) * p.bn;
    const int w_end = p.tw * p.bw, h_end = p.th * p.bh;

    if (warp == 0) {
        // producer A: the stage's 64-filter boxes of dconv
        const int k_off = kb * 128;
        const uint32_t tx_bytes = (uint32_t)p.k_halves * kStageTileBytes;
        uint32_t stage = 0, phase = 0;
        int w0 = w_first, h0 = h_first, n0 = n_first;
        for (int pt = pt0; pt < pt1; ++pt) {
            if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
            const uint32_t fb = full0 + 8u * stage;
            const uint32_t a_dst = a_base + stage * kUnABytes;
            if (lane == 0) {
                mbar_expect_tx(fb, tx_bytes);
                tma_load_4d(a_dst, &tm_dy, fb, k_off, w0, h0, n0);
                if (p.k_halves == 2) tma_load_4d(a_dst + kStageTileBytes, &tm_dy, fb, k_off + 64, w0, h0, n0);
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            w0 += p.bw;
            if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
        }
    } else if (warp == 2 || warp == 3) {
        // producers B: warp 2 fetches the group's units 0 and 1, warp 3 units 2 and 3 (tap-shifted boxes of x)
        const int j0 = (warp - 2) * 2;
        const int mine = nu - j0 >= 2 ? 2 : (nu - j0 >= 1 ? 1 : 0);
        int dw[2] = {0, 0}, dh[2] = {0, 0}, c0[2] = {0, 0};
        for (int j = 0; j < mine; ++j) {
            const int u = u0 + j0 + j;
            const int tap = u / p.cblocks;
            c0[j] = (u % p.cblocks) * 64;
            dw[j] = tap % 3 - 1;
            dh[j] = tap / 3 - 1;
        }
        uint32_t stage = 0, phase = 0;
        int w0 = w_first, h0 = h_first, n0 = n_first;
        RT_DECL;
        for (int pt = pt0; pt < pt1; ++pt) {
            RT_ADD(1);
            if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
            RT_ADD(0);
            const uint32_t fb = full0 + 8u * stage;
            const uint32_t b_dst = b_base + stage * kUnBBytes + j0 * kStageTileBytes;
            if (lane == 0) {
                if (mine == 0) mbar_arrive(fb);
                else mbar_expect_tx(fb, (uint32_t)mine * kStageTileBytes);
                if (mine >= 1) tma_load_4d(b_dst, &tm_x, fb, c0[0], w0 + dw[0], h0 + dh[0], n0);
                if (mine >= 2) tma_load_4d(b_dst + kStageTileBytes, &tm_x, fb, c0[1], w0 + dw[1], h0 + dh[1], n0);
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            w0 += p.bw;
            if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
        }
        RT_ADD(1);
        if (lane == 0 && warp == 2) RT_STORE(0);
    } else if (warp == 1) {
        // MMA issuer: M = 128 filters, N = 64 columns per unit of the group
        const uint32_t idesc = idesc_f16(128, nu * 64, true, true) | (p.bf16 ? idesc_ab_bf16() : 0u);
        // MN-major: 64-element blocks of M/N are one 8 KB tile apart, 8 pixels are 1024 bytes apart
        constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
        const uint32_t a_lo0 = smem_desc_lo(a_base, kStageTileBytes), b_lo0 = smem_desc_lo(b_base, kStageTileBytes);
        uint32_t stage = 0, phase = 0;
        uint32_t accumulate = 0;
        bool ok = true;
        RT_DECL;
        for (int pt = pt0; pt < pt1; ++pt) {
            RT_ADD(2);
            ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
            RT_ADD(1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + stage * (kUnABytes >> 4);
            const uint32_t b_lo = b_lo0 + stage * (kUnBBytes >> 4);
            // 4 x (K = 16 pixels = 2048 bytes: +128 in the address field)
            if (lane == 0) {
                umma_f16_lohi(tmem_base, a_lo, desc_hi, b_lo, desc_hi, idesc, accumulate);
                umma_f16_lohi(tmem_base, a_lo + 128, desc_hi, b_lo + 128, desc_hi, idesc, 1u);
                umma_f16_lohi(tmem_base, a_lo + 256, desc_hi, b_lo + 256, desc_hi, idesc, 1u);
                umma_f16_lohi(tmem_base, a_lo + 384, desc_hi, b_lo + 384, desc_hi, idesc, 1u);
                umma_commit(empty0 + 8u * stage);
            }
            __syncwarp();
            accumulate = 1u;
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok && lane == 0) umma_commit(done_bar);
        __syncwarp();
        RT_ADD(2);
        if (lane == 0) RT_STORE(1);
    } else if (warp >= 4) {
        // epilogue: lane = filter; rows that are no filter (K = 64: lanes 64-127) are skipped by whole warps
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool live = q * 32 < p.k_halves * 64;          // warp-uniform
        float* dst = partial + ((size_t)item * 128 + row) * 256;
        if (pt1 > pt0) {
            if (mbar_wait_relaxed(done_bar, 0, abort_flag, status, kStatusEpilogueTimeout) && live) {
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < nu * 64; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(dst + c0)[j] =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                }
            }
        } else if (live) {
            for (int c0 = 0; c0 < nu * 64; c0 += 4) *reinterpret_cast<float4*>(dst + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    abort_drain(abort_flag);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// dW[k][col] = half or bfloat16(sum over splits, in split order, of partial[split][kb][nt][k % 128][col % (64 upg)]);
// one thread = 4 consecutive columns of one filter row.
__global__ void __launch_bounds__(256)
wgrad_unitn_reduce(const float* __restrict__ partial, uint16_t* __restrict__ dw, WgradUnitnParams p) {
    const int cols = 9 * p.cc;                    // columns of a filter row
    const int quads = cols / 4;
    const long total = (long)p.kk * quads;
    const size_t item_elems = (size_t)128 * 256;
    const size_t split_stride = (size_t)p.k_blocks * p.n_tiles * item_elems;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int k = (int)(i / quads), col = (int)(i % quads) * 4;
        const int gcols = p.upg * 64;                 // columns of one unit group
        const size_t off = ((size_t)(k / 128) * p.n_tiles + col / gcols) * item_elems + (size_t)(k % 128) * 256 + col % gcols;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < p.splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s * split_stride + off);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint2 o;
        o.x = p.bf16 ? pack2_t<true>(acc.x, acc.y) : pack2_t<false>(acc.x, acc.y);
        o.y = p.bf16 ? pack2_t<true>(acc.z, acc.w) : pack2_t<false>(acc.z, acc.w);
        *reinterpret_cast<uint2*>(dw + (size_t)k * cols + col) = o;
    }
}

WgradUnitnParams wgrad_unitn_plan(const trb200_conv_desc& d, const TileShape& t) {
    WgradUnitnParams p;
    p.cblocks = d.c / 64;
    p.units = 9 * p.cblocks;
    p.upg = p.units == 9 ? 3 : 4;      // 18 units (128 channels) stay at 4, 4, 4, 4, 2: N = 192 MMAs are paced by their issue
    p.n_tiles = (p.units + p.upg - 1) / p.upg;
    p.k_blocks = (d.k + 127) / 128;
    p.k_halves = d.k >= 128 ? 2 : 1;
    p.pix_tiles = t.tw * t.th * t.tn;
    const int items = p.n_tiles * p.k_blocks;
    int splits = sm_count() / items;
    if (splits < 1) splits = 1;
    if (splits > p.pix_tiles) splits = p.pix_tiles;
    p.splits = splits;
    p.tw = t.tw; p.th = t.th;
    p.bw = t.bw; p.bh = t.bh; p.bn = t.bn;
    p.kk = d.k; p.cc = d.c;
    p.bf16 = d.dtype == TRB200_DTYPE_BF16 ? 1 : 0;
    return p;
}

// filters: 64 or a multiple of 128; channels: a multiple of 64
inline bool wgrad_unitn_supports(const trb200_conv_desc& d) {
    return d.c % 64 == 0 && (d.k == 64 || d.k % 128 == 0);
}

size_t wgrad_unitn_partial_bytes(const trb200_conv_desc& d) {
    const TileShape t = pick_tile(d.n, d.h, d.w, 64);
    const WgradUnitnParams p = wgrad_unitn_plan(d, t);
    return (size_t)p.splits * p.k_blocks * p.n_tiles * 128 * 256 * sizeof(float);
}

int wgrad_unitn_run(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, float* partial,
                    cudaStream_t st) {
    const TileShape t = pick_tile(d.n, d.h, d.w, 64);
    const WgradUnitnParams p = wgrad_unitn_plan(d, t);
    CUtensorMap tx, tdy;
    int rc = make_act_tmap(&tdy, dy, d.n, d.h, d.w, d.k, t, "wgrad dy");
    if (rc) return rc;
    rc = make_act_tmap(&tx, x, d.n, d.h, d.w, d.c, t, "wgrad x");
    if (rc) return rc;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(wgrad_unitn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kUnSmemTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = p.n_tiles * p.k_blocks * p.splits;
    wgrad_unitn_kernel<<<grid, kThreads, kUnSmemTotal, st>>>(tx, tdy, partial, p, status);
    TRB_LAUNCH_CHECK("wgrad_unitn_kernel");
    const long total = (long)d.k * (9 * d.c / 4);
    long blocks = (total + 255) / 256;
    if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
    wgrad_unitn_reduce<<<(int)blocks, 256, 0, st>>>(partial, static_cast<uint16_t*>(dw), p);
    TRB_LAUNCH_CHECK("wgrad_unitn_reduce");
    return TRB200_OK;
}
