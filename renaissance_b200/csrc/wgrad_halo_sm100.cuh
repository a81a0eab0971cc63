// 3x3 / stride 1 / pad 1 weight gradient for 64 input channels and 64 filters, with the 3x3 neighbourhood of a
// pixel patch fetched ONCE and every filter tap read from that one shared-memory copy.
//
//   dW[k][tap][c] = sum_pixels dy[p][k] * x[p + tap offset][c]
//
// With 64 filters on M a tcgen05.mma uses half of the tensor pipe, so the GEMM is laid out the other way round:
//   D[(tap, c)][k]:  M = 128 = two taps x 64 input channels (A operand = x),  N = 64 filters (B operand = dy),
//   K = pixels, 16 per instruction (two rows of an 8 x 16 pixel patch).
// Both operands are MN-major (a pixel is one 128-byte row of 64 channels, the reduction runs over rows).
//
// A operand.  The patch plus a one-pixel halo is one TMA box of 10 x 18 pixels (out-of-image pixels zero-filled = the
// padding), 180 rows of 128 bytes in shared memory, row = yy*10 + xx.  For tap t = (r, s) the operand starts
// (r*10 + s) rows into the box; its 8-pixel groups (the K direction) are one box row = 1280 bytes apart (stride byte
// offset), and the second 64-row block of M (the leading byte offset) is simply the NEXT tap: taps t and t + 1 start
// 1 row (same r) or 8 rows (s = 2 -> next r, s = 0) apart.  The swizzle follows the absolute shared-memory address,
// for the TMA write and for the tensor core alike, so none of these starts needs a 1024-byte boundary.  Five tap
// pairs (0,1) (2,3) (4,5) (6,7) (8,-) cover the nine taps; the second half of the last pair reads valid shared
// memory and is never written out.
//
// B operand: the patch of dy, a dense 8 x 16 x 64 box (128 rows), 16 pixels = 2048 bytes per K step.
//
// Each of the five pairs has its own accumulator (5 x 64 columns of tensor memory), so consecutive MMAs are
// independent and three warps issue them (pairs dealt in turn; measured 6 % faster than one or two: the MN-major
// 128 x 64 x 16 instruction occupies the pipe for ~54 clocks); a stage is released by all of them.  A persistent
// CTA walks its share of the patches with everything accumulating in tensor memory and writes one float partial
// per CTA at the end; wgrad_halo_reduce adds the partials in a fixed order (bitwise reproducible).  Pixels outside the
// image contribute nothing: their dy is zero-filled by the copy.
//
// This file is included by conv_igemm_sm100.cu inside its anonymous namespace.
#pragma once

constexpr int kWhPairs = 5;
#ifndef TRB200_WH_ISSUERS
#define TRB200_WH_ISSUERS 3
#endif
constexpr int kWhIssuers = TRB200_WH_ISSUERS;                         // warps 1 .. kWhIssuers issue MMAs
constexpr int kWhDyBytes = 128 * 128;                                // 8 x 16 pixels x 64 filters
constexpr int kWhStageBytes = kHaloStageBytes + kWhDyBytes;          // 23552 + 16384
constexpr int kWhStages = 5;
constexpr int kWhSmemTotal = kWhStages * kWhStageBytes + 2048;
constexpr int kWhPartialFloats = kWhPairs * 128 * 64;                // per CTA
static_assert(kWhSmemTotal <= kSmemBudget, "shared memory budget");

struct WgradHaloParams {
    int pw, ph;         // patches along w and h per image
    int patches;        // n * ph * pw
    int bf16;
};

__global__ void __launch_bounds__(kThreads, 1)
wgrad_halo_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                  float* __restrict__ partial, const WgradHaloParams p, int* status) {
    constexpr int kStages = kWhStages;
    constexpr uint32_t kTmemCols = 512;                              // 5 x 64 used
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t bar_base = base + kStages * kWhStageBytes;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    const uint32_t done_bar = bar_base + 8u * (2 * kStages);
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, kWhIssuers); }
        mbar_init(done_bar, kWhIssuers);
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

    const int my_patches = p.patches > (int)blockIdx.x ? (p.patches - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int per_image = p.pw * p.ph;

    if (warp == 0) {
        // producer: the halo box of x and the patch of dy
        uint32_t stage = 0, phase = 0;
        for (int j = 0; j < my_patches; ++j) {
            const int q = (int)blockIdx.x + j * (int)gridDim.x;
            const int img = q / per_image, rem = q - img * per_image;
            const int py = rem / p.pw, px = rem - py * p.pw;
            if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
            if (lane == 0) {
                const uint32_t fb = full0 + 8u * stage;
                const uint32_t dst = base + stage * kWhStageBytes;
                mbar_expect_tx(fb, kHaloBoxBytes + kWhDyBytes);
                tma_load_4d(dst, &tm_x, fb, 0, px * kHaloW - 1, py * kHaloH - 1, img);
                tma_load_4d(dst + kHaloStageBytes, &tm_dy, fb, 0, px * kHaloW, py * kHaloH, img);
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
    } else if (warp >= 1 && warp <= kWhIssuers) {
        // MMA issuers: the tap pairs are dealt to the issuing warps in turn; all of them read every stage
        const int issuer = warp - 1;
        const uint32_t idesc = idesc_f16(128, 64, true, true) | (p.bf16 ? idesc_ab_bf16() : 0u);
        constexpr uint32_t a_hi = smem_desc_hi_sw128(kHaloBoxW * 128);      // 8-pixel groups one box row apart
        constexpr uint32_t b_hi = smem_desc_hi_sw128(1024);
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        RT_DECL;
        for (int j = 0; j < my_patches && ok; ++j) {
            RT_ADD(2);
            // a polite wait: the warp with fewer pairs is ahead of the other one, and a tight mbarrier poll slows the
            // other warp's MMA issue down
            ok = mbar_wait_relaxed(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
            RT_ADD(1);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t x_addr = base + stage * kWhStageBytes;
                const uint32_t b_lo0 = smem_desc_lo(x_addr + kHaloStageBytes, 1024);
                const uint32_t accumulate = j ? 1u : 0u;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
                    for (int pair = 0; pair < kWhPairs; ++pair) {
                        if (pair % kWhIssuers != issuer) continue;
                        const int t0 = 2 * pair, t1 = 2 * pair + 1;
                        const int off0 = (t0 / 3) * kHaloBoxW + t0 % 3, off1 = (t1 / 3) * kHaloBoxW + t1 % 3;
                        // start (address field, 16-byte units) and leading byte offset = distance to the next tap
                        const uint32_t a_lo = (((x_addr >> 4) + (uint32_t)((off0 + kk * 2 * kHaloBoxW) * 8)) & 0x3FFFu) |
                                              ((uint32_t)(((off1 - off0) * 128) >> 4) << 16);
                        umma_f16_lohi(tmem_base + (uint32_t)(pair * 64), a_lo, a_hi, b_lo0 + (uint32_t)(kk * 128), b_hi,
                                      idesc, kk ? 1u : accumulate);
                    }
                }
                umma_commit(empty0 + 8u * stage);
            }
            __syncwarp();
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok && lane == 0) umma_commit(done_bar);
        __syncwarp();
        RT_ADD(2);
        if (lane == 0) RT_STORE(issuer);
    } else if (warp >= 4) {
        // epilogue, once: accumulator row m = (tap in pair) * 64 + c, 64 columns k per pair -> partial[block][pair][m][k]
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        float* dst = partial + ((size_t)blockIdx.x * kWhPairs * 128 + row) * 64;
        if (my_patches > 0) {
            if (mbar_wait_relaxed(done_bar, 0, abort_flag, status, kStatusEpilogueTimeout)) {
                tc_fence_after();
#pragma unroll 1
                for (int pair = 0; pair < kWhPairs; ++pair)
#pragma unroll 1
                    for (int c0 = 0; c0 < 64; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(pair * 64 + c0), v);
                        tmem_ld_wait();
                        float4* o = reinterpret_cast<float4*>(dst + (size_t)pair * 128 * 64 + c0);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            o[e] = make_float4(__uint_as_float(v[4 * e]), __uint_as_float(v[4 * e + 1]),
                                               __uint_as_float(v[4 * e + 2]), __uint_as_float(v[4 * e + 3]));
                    }
            }
        } else {
            for (int pair = 0; pair < kWhPairs; ++pair)
                for (int c0 = 0; c0 < 64; c0 += 4)
                    *reinterpret_cast<float4*>(dst + (size_t)pair * 128 * 64 + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
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

// dW[k][tap][c] = half or bfloat16(sum over the CTAs' partials partial[b][tap / 2][(tap % 2) * 64 + c][k]).
// One block = one (tap, c): thread (slice, k4) adds the partials b = slice, slice + 16, ... of four consecutive k
// (independent loads, one memory round trip), then the 16 slices are added in slice order: a fixed order, so the
// result is bitwise reproducible.
__global__ void __launch_bounds__(256)
wgrad_halo_reduce(const float* __restrict__ partial, uint16_t* __restrict__ dw, int blocks, int bf16) {
    __shared__ float4 part[16][16];
    const int tap = blockIdx.x >> 6, c = blockIdx.x & 63;
    const int k4 = threadIdx.x & 15, slice = threadIdx.x >> 4;
    const float* src = partial + ((size_t)(tap >> 1) * 128 + (size_t)((tap & 1) * 64 + c)) * 64 + k4 * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int b = slice; b < blocks; b += 16) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src + (size_t)b * kWhPartialFloats));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    part[slice][k4] = acc;
    __syncthreads();
    if (threadIdx.x < 16) {
        float4 t = part[0][k4];
#pragma unroll
        for (int sl = 1; sl < 16; ++sl) {
            const float4 v = part[sl][k4];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        const float r[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            dw[((size_t)(k4 * 4 + e) * 9 + tap) * 64 + c] = bf16 ? round16_t<true>(r[e]) : round16_t<false>(r[e]);
    }
}

inline bool wgrad_halo_supports(const trb200_conv_desc& d) { return d.r == 3 && d.c == 64 && d.k == 64; }

inline int wgrad_halo_grid(const trb200_conv_desc& d) {
    const long patches = (long)d.n * ((d.w + kHaloW - 1) / kHaloW) * ((d.h + kHaloH - 1) / kHaloH);
    return (int)(patches < sm_count() ? patches : sm_count());
}

size_t wgrad_halo_partial_bytes(const trb200_conv_desc& d) {
    (void)d;
    return (size_t)sm_count() * kWhPartialFloats * sizeof(float);
}

int wgrad_halo_run(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, float* partial, cudaStream_t st) {
    WgradHaloParams p;
    p.pw = (d.w + kHaloW - 1) / kHaloW;
    p.ph = (d.h + kHaloH - 1) / kHaloH;
    p.patches = d.n * p.pw * p.ph;
    p.bf16 = d.dtype == TRB200_DTYPE_BF16 ? 1 : 0;
    CUtensorMap tx, tdy;
    int rc = make_act_tmap(&tx, x, d.n, d.h, d.w, d.c, TileShape{kHaloBoxW, kHaloBoxH, 1, 0, 0, 0}, "wgrad x (halo box)");
    if (rc) return rc;
    rc = make_act_tmap(&tdy, dy, d.n, d.h, d.w, d.k, TileShape{kHaloW, kHaloH, 1, 0, 0, 0}, "wgrad dy (patch)");
    if (rc) return rc;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(wgrad_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWhSmemTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = wgrad_halo_grid(d);
    wgrad_halo_kernel<<<grid, kThreads, kWhSmemTotal, st>>>(tx, tdy, partial, p, status);
    TRB_LAUNCH_CHECK("wgrad_halo_kernel");
    wgrad_halo_reduce<<<9 * 64, 256, 0, st>>>(partial, static_cast<uint16_t*>(dw), grid, p.bf16);
    TRB_LAUNCH_CHECK("wgrad_halo_reduce");
    return TRB200_OK;
}
