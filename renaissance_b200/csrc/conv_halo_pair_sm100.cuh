// 3x3 / stride 1 / pad 1 convolution (forward and data gradient) for layers with 64 or 128 output channels and
// 64 or 128 input channels, on MMAs that span a CTA pair (tcgen05.mma.cta_group::2), with the whole 3x3
// neighbourhood of a tile fetched from global memory ONCE.
//
//   out[n,y,x,co] = sum_{tap=(r,s)} sum_{ci} in[n, y+r-1, x+s-1, ci] * Wv[tap][co][ci]
//
// Tile: a patch of 8 x 16 output pixels of one image per CTA (M = 128 rows, row = y*8 + x), two patches per pair
// (M = 256 for the instruction), N = NT output channels (each CTA holds NT/2 filter rows), K = 64 input channels
// per slice.
//
// Halo box.  One TMA box of 10 x 18 pixels x 64 channels (the patch plus one pixel all round; pixels outside the
// image are zero-filled, which is the padding) lands in shared memory as 180 rows of 128 bytes, row = yy*10 + xx,
// 128-byte swizzled.  The A operand of tap (r, s) is that same buffer read through a K-major descriptor whose start
// address is moved by (r*10 + s) rows and whose 8-row groups are 1280 bytes (one box row of 10 pixels) apart: the
// eight rows of group y are pixels (y + r, s .. s + 7) of the box, exactly the patch row moved by the tap.  The
// tensor core applies the swizzle to the absolute shared-memory address, as the TMA write did, so a start address
// that is not on a 1024-byte boundary needs no base offset.  One load per (patch, 64-channel slice) instead of
// nine: 1.4 x the activation bytes cross L2 -> shared memory instead of 9 x.
//
// Filters are resident.  All 9 x (Cin / 64) filter tiles of this CTA's NT/2 output channels (36 .. 144 KB) are
// loaded once when the kernel starts and stay in shared memory; the main loop moves activations only.
//
// Issue.  One thread issues a 256 x NT x 16 MMA about every 50-56 clocks, while the tensor pipe needs 43 (NT = 64)
// or 64 (NT = 128) clocks for it, so with NT = 64 two warps issue, on alternate tiles with two accumulators each
// (the MMAs of one accumulator form a dependent chain; MMAs of different accumulators overlap).  The 36 MMAs of a
// slice are unrolled with constant descriptor offsets: a lone thread pays for every scalar instruction.
//
// Roles (256 threads per CTA; both CTAs of a pair run all roles except the MMA issue, which is the leader's):
//   warp 0  halo producer: one box per (tile, slice) into a ring; completion is counted on the LEADER's barrier
//   warp 1  MMA issuer 0 (leader) and tensor-memory allocation (both CTAs)
//   warp 2  MMA issuer 1 (leader, NT = 64)
//   warp 3  filter loader (once)
//   warps 4-7 epilogue: own 128 accumulator rows -> half -> swizzled staging -> TMA store of the 8 x 16 patch;
//           forward: batch statistics of the rounded output from the staged tile
// Barriers: full[stage] and filters-ready live in the leader (they count the bytes of both CTAs); empty[stage]
// and accumulator-full[a] exist in both CTAs and get their arrival from the leader's tcgen05.commit; accumulator-
// empty[a] lives in the leader and gets one (remote) arrival from each CTA's epilogue.  Every wait is bounded.
//
// This file is included by conv_igemm_sm100.cu inside its anonymous namespace.
#pragma once

struct HaloParams {
    int pw, ph;             // patches along w and h per image
    int patches;            // n * ph * pw
    int pair_tiles;         // ceil(patches / 2)
    int b_tap_is_dim1;      // filter view is (ci, tap, co) instead of (ci, co, tap)
    int cout;
    int ext_w, ext_h, ext_n;
    int has_padding;        // some patch hangs over an image edge, or the patch count is odd
    float* stats_partial;   // [strip = block][2][cout]
};

constexpr int kHaloW = 8, kHaloH = 16;                              // patch
constexpr int kHaloBoxW = kHaloW + 2, kHaloBoxH = kHaloH + 2;       // box with halo
constexpr int kHaloBoxBytes = kHaloBoxW * kHaloBoxH * 128;          // 23040
constexpr int kHaloStageBytes = (kHaloBoxBytes + 1023) / 1024 * 1024;
constexpr int kHaloEpiBufBytes = 128 * 128;                         // 128 pixels x 64 channels

template <int NT, int S>
struct HaloCfg {
    static constexpr int kIssuers = NT == 64 ? 2 : 1;
    static constexpr int kAccs = 2 * kIssuers;
    static constexpr int kBTileBytes = (NT / 2) * 128;              // one (tap, slice) tile of this CTA's filter half
    static constexpr int kBBytes = S * 9 * kBTileBytes;
    static constexpr int kEpiBufs = 2;
    static constexpr int kFixed = kBBytes + kEpiBufs * kHaloEpiBufBytes + 2048;
    static constexpr int kFit = (kSmemBudget - kFixed) / kHaloStageBytes;
    // a stage keeps its issuer: the ring is a multiple of (issuers x slices per tile)
    static constexpr int kUnit = kIssuers * S;
    static constexpr int kStagesRaw = kFit / kUnit * kUnit;
    static constexpr int kStages = kStagesRaw > 8 ? 8 / kUnit * kUnit : kStagesRaw;
    static constexpr int kTotal = kFixed + kStages * kHaloStageBytes;
    static constexpr uint32_t kTmemCols = kAccs * NT;               // 256 or 256
    static_assert(kStages >= kUnit && kStages >= 2, "the activation ring does not fit");
};

template <int NT, int S, bool STATS, bool BF16>
__device__ __forceinline__ void
conv3x3_halo_pair_body(const CUtensorMap& tm_in, const CUtensorMap& tm_w, const CUtensorMap& tm_out, const HaloParams& p,
                       int* status) {
    using L = HaloCfg<NT, S>;
    constexpr int kStages = L::kStages;
    constexpr int kIssuers = L::kIssuers, kAccs = L::kAccs;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t b_base = base;
    const uint32_t a_base = b_base + L::kBBytes;
    const uint32_t epi_base = a_base + kStages * kHaloStageBytes;
    const uint32_t bar_base = epi_base + L::kEpiBufs * kHaloEpiBufBytes;
    // barriers: full[kStages], empty[kStages], tfull[kAccs], tempty[kAccs], bfull
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + kAccs + a); };
    const uint32_t bfull = bar_base + 8u * (2 * kStages + 2 * kAccs);
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_epi_fail;
    __shared__ uint32_t s_valid[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_epi_fail = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
        for (int a = 0; a < kAccs; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2); }
        mbar_init(bfull, 1);
        fence_barrier_init();
        prefetch_tmap(&tm_in);
        prefetch_tmap(&tm_w);
        prefetch_tmap(&tm_out);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&s_tmem_base), L::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    volatile int* abort_flag = &s_abort;

    // tiles of this pair: pt = cluster, cluster + clusters, ...; local index j
    const int cluster = (int)cluster_id_x(), clusters = (int)num_clusters_x();
    const int my_tiles = p.pair_tiles > cluster ? (p.pair_tiles - cluster + clusters - 1) / clusters : 0;
    const int per_image = p.pw * p.ph;

    if (warp == 0) {
        // halo producer (both CTAs): box origin = patch origin - (1, 1)
        const uint32_t lead_full0 = map_to_cta(full0, 0);
        bool ok = true;
        uint32_t stage = 0, phase = 0;
        for (int j = 0; j < my_tiles && ok; ++j) {
            const int q = 2 * (cluster + j * clusters) + (int)rank;
            const int img = q / per_image, rem = q - img * per_image;
            const int py = rem / p.pw, px = rem - py * p.pw;
            for (int sl = 0; sl < S; ++sl) {
                ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                if (!ok) break;
                if (lane == 0) {
                    if (rank == 0) mbar_expect_tx(full0 + 8u * stage, 2u * kHaloBoxBytes);
                    tma_load_4d_pair(a_base + stage * kHaloStageBytes, &tm_in, lead_full0 + 8u * stage, sl * 64,
                                     px * kHaloW - 1, py * kHaloH - 1, img);
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 3) {
        // filter loader (both CTAs): this CTA's NT/2 output channels of every (slice, tap) tile, once
        if (lane == 0 && my_tiles > 0) {
            const uint32_t lead_bfull = map_to_cta(bfull, 0);
            if (rank == 0) mbar_expect_tx(bfull, 2u * (uint32_t)L::kBBytes);
            const int co0 = (int)rank * (NT / 2);
            for (int sl = 0; sl < S; ++sl)
                for (int tap = 0; tap < 9; ++tap) {
                    const uint32_t dst = b_base + (uint32_t)((sl * 9 + tap) * L::kBTileBytes);
                    if (p.b_tap_is_dim1) tma_load_3d_pair(dst, &tm_w, lead_bfull, sl * 64, tap, co0);
                    else tma_load_3d_pair(dst, &tm_w, lead_bfull, sl * 64, co0, tap);
                }
        }
        __syncwarp();
    } else if ((warp == 1 || (warp == 2 && kIssuers == 2)) && rank == 0) {
        // MMA issuers (leader): issuer i takes the local tiles j = i, i + kIssuers, ...; tile j accumulates in
        // accumulator j % kAccs and reads the stages (j*S + sl) % kStages
        const int issuer = warp - 1;
        constexpr uint32_t idesc = idesc_f16(256, NT, false, false) | (BF16 ? idesc_ab_bf16() : 0u);
        constexpr uint32_t a_hi = smem_desc_hi_sw128(kHaloBoxW * 128);       // 8-row groups one box row apart
        constexpr uint32_t b_hi = smem_desc_hi_sw128(1024);
        bool ok = my_tiles > issuer ? mbar_wait(bfull, 0, abort_flag, status, kStatusMmaTimeout) : true;
        tc_fence_after();
        const uint32_t b_lo0 = smem_desc_lo(b_base, 16);
        RT_DECL;
        for (int j = issuer; j < my_tiles && ok; j += kIssuers) {
            const int acc = j % kAccs;
            RT_ADD(3);
            ok = mbar_wait(tempty_bar(acc), (((uint32_t)(j / kAccs)) & 1u) ^ 1u, abort_flag, status, kStatusMmaTimeout);
            RT_ADD(0);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * NT);
#pragma unroll
            for (int sl = 0; sl < S; ++sl) {
                const int it = j * S + sl;
                const uint32_t stage = (uint32_t)(it % kStages), phase = (uint32_t)((it / kStages) & 1);
                RT_ADD(3);
                ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
                RT_ADD(1);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_lo0 = smem_desc_lo(a_base + stage * kHaloStageBytes, 16);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const uint32_t a_lo = a_lo0 + (uint32_t)(((tap / 3) * kHaloBoxW + tap % 3) * 8);
                        const uint32_t b_lo = b_lo0 + (uint32_t)(((sl * 9 + tap) * L::kBTileBytes) >> 4);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_pair_f16_lohi(d_tmem, a_lo + 2 * k, a_hi, b_lo + 2 * k, b_hi, idesc,
                                               (sl | tap | k) ? 1u : 0u);
                    }
                    umma_pair_commit(empty0 + 8u * stage, 3);
                }
                __syncwarp();
                RT_ADD(2);
            }
            if (ok && lane == 0) umma_pair_commit(tfull_bar(acc), 3);
            __syncwarp();
        }
        RT_ADD(3);
        if (lane == 0) RT_STORE(issuer == 0 ? 1 : 0);
    } else if (warp >= 4) {
        // epilogue (both CTAs): thread = accumulator row = pixel (y = row / 8, x = row % 8) of this CTA's patch
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        const bool leader = threadIdx.x == 128;
        const uint32_t lead_tempty0 = map_to_cta(tempty_bar(0), 0);
        const int st_cc = (threadIdx.x - 128) & 7, st_rg = (threadIdx.x - 128) >> 3;
        float run_s[NT / 64][8], run_q[NT / 64][8];
#pragma unroll
        for (int i = 0; i < NT / 64; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) { run_s[i][e] = 0.f; run_q[i][e] = 0.f; }
        int chunk_count = 0;
        RT_DECL;
        for (int j = 0; j < my_tiles; ++j) {
            const int acc = j % kAccs;
            const int q = 2 * (cluster + j * clusters) + (int)rank;
            const int img = q / per_image, rem = q - img * per_image;
            const int py = rem / p.pw, px = rem - py * p.pw;
            const int w0 = px * kHaloW, h0 = py * kHaloH;
            const bool patch_real = q < p.patches;
            if (STATS && p.has_padding) {
                const bool real = patch_real && (w0 + (row & 7) < p.ext_w) && (h0 + (row >> 3) < p.ext_h);
                const uint32_t m = __ballot_sync(0xffffffffu, real);
                if (lane == 0) s_valid[q4] = m;
            }
#ifdef TRB200_RT_FINE
            RT_ADD(3);
#else
            RT_ADD(2);
#endif
            if (!mbar_wait_relaxed(tfull_bar(acc), ((uint32_t)(j / kAccs)) & 1u, abort_flag, status, kStatusEpilogueTimeout))
                s_epi_fail = 1;
            named_barrier(2, kEpiThreads);
#ifdef TRB200_RT_FINE
            RT_ADD(3);
#else
            RT_ADD(0);
#endif
            if (*(volatile int*)&s_epi_fail) break;
            tc_fence_after();
            uint32_t vm = 0xffu;
            if (STATS && p.has_padding) vm = (s_valid[st_rg >> 2] >> ((st_rg & 3) * 8)) & 0xffu;
#pragma unroll
            for (int chunk = 0; chunk < NT / 64; ++chunk, ++chunk_count) {
                const uint32_t buf = epi_base + (uint32_t)(chunk_count & 1) * kHaloEpiBufBytes;
#ifdef TRB200_RT_FINE
                RT_ADD(3);
#else
                RT_ADD(2);
#endif
                if (leader) tma_store_wait_read<1>();     // the store that last read this buffer is done
                named_barrier(1, kEpiThreads);
#ifdef TRB200_RT_FINE
                RT_ADD(3);
#else
                RT_ADD(1);
#endif
                const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(acc * NT + chunk * 64);
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(taddr, v0);
                tmem_ld_32x32(taddr + 32, v1);
                tmem_ld_wait();
                const uint32_t row_addr = buf + (uint32_t)row * 128u;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t* src = c < 4 ? &v0[c * 8] : &v1[(c - 4) * 8];
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        pk[e] = pack2_t<BF16>(__uint_as_float(src[2 * e]), __uint_as_float(src[2 * e + 1]));
                    const uint32_t dst = row_addr + (uint32_t)((c ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]),
                                 "r"(pk[2]), "r"(pk[3])
                                 : "memory");
                }
                RT_ADD(3);
                fence_proxy_async_smem();
                named_barrier(1, kEpiThreads);
#ifdef TRB200_RT_FINE
                RT_ADD(0);
#endif
                if (leader && patch_real) {
                    tma_store_4d(&tm_out, buf, chunk * 64, w0, h0, img);
                    tma_store_commit();
                }
#ifdef TRB200_RT_FINE
                RT_ADD(1);
#endif
                if (STATS) {
                    const uint32_t rows0 = buf + (uint32_t)(st_rg * 8) * 128u;
                    uint32_t hw[8][4];
#pragma unroll
                    for (int i = 0; i < 8; ++i)          // row st_rg * 8 + i: its swizzle phase is i
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(hw[i][0]), "=r"(hw[i][1]), "=r"(hw[i][2]), "=r"(hw[i][3])
                                     : "r"(rows0 + (uint32_t)i * 128u + (uint32_t)((st_cc ^ i) << 4)));
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const bool real = (vm >> i) & 1u;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float2 f = unpack2_t<BF16>(hw[i][e]);
                            if (!real) f = make_float2(0.f, 0.f);
                            run_s[chunk][2 * e] += f.x;
                            run_s[chunk][2 * e + 1] += f.y;
                            run_q[chunk][2 * e] = fmaf(f.x, f.x, run_q[chunk][2 * e]);
                            run_q[chunk][2 * e + 1] = fmaf(f.y, f.y, run_q[chunk][2 * e + 1]);
                        }
                    }
                }
            }
            // this CTA's 128 rows of the accumulator are read: one arrival on the leader's barrier
            tc_fence_before();
            named_barrier(1, kEpiThreads);
            if (threadIdx.x == 128 + 32) mbar_arrive_remote(lead_tempty0 + 8u * (uint32_t)acc);   // not the thread with stores in flight
#ifdef TRB200_RT_FINE
            RT_ADD(2);
#endif
        }
        if (leader) tma_store_wait_all();
        RT_ADD(2);
        if (leader) RT_STORE(2);
        if (STATS && !*(volatile int*)&s_epi_fail) {
            // the 16 row groups meet through the (now idle) staging buffers: red[rg][sum | sumsq][NT]
            named_barrier(1, kEpiThreads);
            float* red = reinterpret_cast<float*>(smem_dyn + (epi_base - smem_u32(smem_dyn)));
#pragma unroll
            for (int i = 0; i < NT / 64; ++i) {
                float4* ds = reinterpret_cast<float4*>(red + (st_rg * 2) * NT + i * 64 + st_cc * 8);
                float4* dq = reinterpret_cast<float4*>(red + (st_rg * 2 + 1) * NT + i * 64 + st_cc * 8);
                ds[0] = make_float4(run_s[i][0], run_s[i][1], run_s[i][2], run_s[i][3]);
                ds[1] = make_float4(run_s[i][4], run_s[i][5], run_s[i][6], run_s[i][7]);
                dq[0] = make_float4(run_q[i][0], run_q[i][1], run_q[i][2], run_q[i][3]);
                dq[1] = make_float4(run_q[i][4], run_q[i][5], run_q[i][6], run_q[i][7]);
            }
            named_barrier(1, kEpiThreads);
            const int strip = blockIdx.x;
            for (int ch = threadIdx.x - 128; ch < NT; ch += kEpiThreads) {
                float s1 = 0.f, s2 = 0.f;
#pragma unroll
                for (int g = 0; g < 16; ++g) {
                    s1 += red[(g * 2) * NT + ch];
                    s2 += red[(g * 2 + 1) * NT + ch];
                }
                p.stats_partial[((size_t)strip * 2) * p.cout + ch] = s1;
                p.stats_partial[((size_t)strip * 2 + 1) * p.cout + ch] = s2;
            }
        }
    }

    abort_drain(abort_flag);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // neither CTA leaves while the other may still signal its barriers or read its operands
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, L::kTmemCols);
    }
}

template <int NT, int S, bool STATS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
conv3x3_halo_pair_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_out, const HaloParams p, int* status) {
    conv3x3_halo_pair_body<NT, S, STATS, false>(tm_in, tm_w, tm_out, p, status);
}

template <int NT, int S, bool STATS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
conv3x3_halo_pair_kernel_bf16(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                              const __grid_constant__ CUtensorMap tm_out, const HaloParams p, int* status) {
    conv3x3_halo_pair_body<NT, S, STATS, true>(tm_in, tm_w, tm_out, p, status);
}

// CTAs of the persistent grid: two per pair, at most one CTA per SM (an even count)
inline int halo_pair_grid(int pair_tiles) {
    const int pairs_max = sm_count() / 2;
    return 2 * (pair_tiles < pairs_max ? pair_tiles : pairs_max);
}

template <int NT, int S, bool STATS>
int launch_halo_pair(const CUtensorMap& tin, const CUtensorMap& tw, const CUtensorMap& tout, const HaloParams& p,
                     cudaStream_t st, bool bf16) {
    using L = HaloCfg<NT, S>;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_halo_pair_kernel<NT, S, STATS>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_halo_pair_kernel_bf16<NT, S, STATS>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = halo_pair_grid(p.pair_tiles);
    if (bf16) conv3x3_halo_pair_kernel_bf16<NT, S, STATS><<<grid, kThreads, L::kTotal, st>>>(tin, tw, tout, p, status);
    else conv3x3_halo_pair_kernel<NT, S, STATS><<<grid, kThreads, L::kTotal, st>>>(tin, tw, tout, p, status);
    TRB_LAUNCH_CHECK("conv3x3_halo_pair_kernel");
    return TRB200_OK;
}

// layers this kernel takes: 3x3, 64 or 128 channels on either side
inline bool halo_pair_preferred(int cin, int cout, int taps) {
    return taps == 9 && (cout == 64 || cout == 128) && (cin == 64 || cin == 128);
}

// Same contract as conv3x3_run (taps = 9).
int conv3x3_halo_pair_run(const void* in, const void* wv, int tap_is_dim1, void* out, int n, int h, int w, int cin,
                          int cout, cudaStream_t st, float* stats_partial, int* stats_strips, bool bf16) {
    HaloParams p;
    p.pw = (w + kHaloW - 1) / kHaloW;
    p.ph = (h + kHaloH - 1) / kHaloH;
    p.patches = n * p.pw * p.ph;
    p.pair_tiles = (p.patches + 1) / 2;
    p.b_tap_is_dim1 = tap_is_dim1;
    p.cout = cout;
    p.ext_w = w; p.ext_h = h; p.ext_n = n;
    p.has_padding = (p.pw * kHaloW != w) || (p.ph * kHaloH != h) || (p.patches & 1);
    p.stats_partial = stats_partial;
    CUtensorMap tin, tw, tout;
    int rc = make_act_tmap(&tin, in, n, h, w, cin, TileShape{kHaloBoxW, kHaloBoxH, 1, 0, 0, 0}, "conv input (halo box)");
    if (rc) return rc;
    rc = make_act_tmap(&tout, out, n, h, w, cout, TileShape{kHaloW, kHaloH, 1, 0, 0, 0}, "conv output (patch)");
    if (rc) return rc;
    const int half_rows = cout / 2;
    if (tap_is_dim1) {
        const uint64_t dims[3] = {(uint64_t)cin, 9, (uint64_t)cout};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)9 * cin * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)half_rows};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,tap,co)");
    } else {
        const uint64_t dims[3] = {(uint64_t)cin, (uint64_t)cout, 9};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)cout * cin * 2};
        const uint32_t box[3] = {64, (uint32_t)half_rows, 1};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,co,tap)");
    }
    if (rc) return rc;
    if (stats_partial && stats_strips) *stats_strips = halo_pair_grid(p.pair_tiles);
    const bool stats = stats_partial != nullptr;
#define TRB_HALO_CASE(NT_, S_)                                                                      \
    if (cout == NT_ && cin == 64 * S_)                                                              \
        return stats ? launch_halo_pair<NT_, S_, true>(tin, tw, tout, p, st, bf16)                  \
                     : launch_halo_pair<NT_, S_, false>(tin, tw, tout, p, st, bf16);
    TRB_HALO_CASE(64, 1)
    TRB_HALO_CASE(64, 2)
    TRB_HALO_CASE(128, 1)
    TRB_HALO_CASE(128, 2)
#undef TRB_HALO_CASE
    return fail(TRB200_ERR_UNSUPPORTED, "conv3x3 halo-pair: cin=%d cout=%d not covered", cin, cout);
}
