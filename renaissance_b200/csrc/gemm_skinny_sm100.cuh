// GEMMs of the classifier: one dimension is the batch (256), the other two are thousands wide, so every operand
// is touched once or twice and the kernels are bound by HBM (205 MB of weights in VGG16's first FC layer).
//
//   D[m][n] = sum_k A[m][k] * B[n][k]        tile: MA x 128 rows, 256 columns, 64 of k per stage
//
// Each operand is a row-major half matrix in global memory and is either K-MAJOR (the contraction runs along its
// rows' contiguous direction: box {64 k, rows}) or MN-MAJOR (the contraction runs down its rows: 64 x 64 boxes, one
// per 64 elements of M / N, 8 KB apart = the descriptor's leading byte offset).  The three FC GEMMs:
//   forward        y[b][o]  = x[b][:] . w[o][:]      A = x  K-major (MA = 2: the whole batch), B = w  K-major, split over k
//   data gradient  dx[b][i] = dy[b][:] . w[:][i]     A = dy K-major (MA = 2),                  B = w  MN-major
//   weight grad.   dw[o][i] = dy[:][o] . x[:][i]     A = dy MN-major (MA = 1),                 B = x  MN-major
// so no operand is ever transposed in memory.  Rows / columns beyond a matrix's extent are zero-filled by TMA and
// masked in the epilogue: any extent that keeps rows 16-byte aligned (a multiple of 8 elements) is accepted.
//
// Roles as in conv3x3_igemm_kernel: warp 0 = producer A, warp 2 = producer B, warp 1 = MMA issuer + TMEM, warps 4-7 =
// epilogue (thread = accumulator row: half rows, or float rows when the k range is split or D is float, staged in
// shared memory and written by TMA).  MA = 2 keeps two 128 x 256 accumulators (512 TMEM columns) that share every B
// tile; MA = 1 double-buffers one so that the epilogue of a tile overlaps the next tile's MMAs.
//
// This file is included by conv_igemm_sm100.cu inside its anonymous namespace.
#pragma once

struct SkinnyParams {
    int m_real, n_real;       // extents of D
    int k_steps;              // ceil(K / 64)
    int m_tiles, n_tiles, splits;
    int64_t ldd;              // D row stride in elements
    void* d;                  // half D, or float partials [split][m_real][ldd]
    int64_t split_stride;     // elements between two splits' partials
    int bf16;
};

constexpr int kSkN = 256;
constexpr int kSkBBytes = kSkN * 128;

template <int MA>
struct SkinnyCfg {
    static constexpr int kABytes = MA * kATileBytes;
    static constexpr int kStageBytes = kABytes + kSkBBytes;
    static constexpr int kEpiBytes = 2 * kATileBytes;                        // two 128 x 64 half staging tiles
    static constexpr int kStages = (kSmemBudget - 2048 - kEpiBytes) / kStageBytes;      // 4 (MA = 1) or 3 (MA = 2)
    static constexpr int kTotal = kStages * kStageBytes + kEpiBytes + 2048;
    static constexpr int kBufs = MA == 1 ? 2 : 1;
};

template <bool A_MN, bool B_MN, int MA, bool F32OUT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_d, const SkinnyParams p, int* status) {
    using L = SkinnyCfg<MA>;
    constexpr int kStages = L::kStages, kBufs = L::kBufs;
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_base = base, b_base = base + kStages * L::kABytes;
    const uint32_t epi_base = b_base + kStages * kSkBBytes;
    const uint32_t bar_base = epi_base + L::kEpiBytes;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_epi_fail;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_epi_fail = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, 2); mbar_init(empty0 + 8u * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpiThreads); }
        fence_barrier_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        if (!F32OUT) prefetch_tmap(&tm_d);
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

    const int items = p.splits * p.m_tiles * p.n_tiles;
    // item -> (split, m tile, n tile), n fastest: neighbouring CTAs share their A rows in L2
    auto k_range = [&](int split, int& k0, int& k1) {
        k0 = (int)((long)p.k_steps * split / p.splits);
        k1 = (int)((long)p.k_steps * (split + 1) / p.splits);
    };

    if (warp == 0) {
        // producer A
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int nt = item % p.n_tiles, mt = (item / p.n_tiles) % p.m_tiles, split = item / (p.n_tiles * p.m_tiles);
            (void)nt;
            int k0, k1;
            k_range(split, k0, k1);
            const int m0 = mt * (MA * 128);
            for (int ks = k0; ks < k1; ++ks) {
                ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t fb = full0 + 8u * stage;
                    const uint32_t dst = a_base + stage * L::kABytes;
                    mbar_expect_tx(fb, L::kABytes);
                    if (A_MN) {
#pragma unroll
                        for (int blk = 0; blk < MA * 2; ++blk)
                            tma_load_2d(dst + blk * kStageTileBytes, &tm_a, fb, m0 + blk * 64, ks * 64);
                    } else {
#pragma unroll
                        for (int a = 0; a < MA; ++a)
                            tma_load_2d(dst + a * kATileBytes, &tm_a, fb, ks * 64, m0 + a * 128);
                    }
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 2) {
        // producer B
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int nt = item % p.n_tiles, split = item / (p.n_tiles * p.m_tiles);
            int k0, k1;
            k_range(split, k0, k1);
            const int n0 = nt * kSkN;
            for (int ks = k0; ks < k1; ++ks) {
                ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t fb = full0 + 8u * stage;
                    const uint32_t dst = b_base + stage * kSkBBytes;
                    mbar_expect_tx(fb, kSkBBytes);
                    if (B_MN) {
#pragma unroll
                        for (int blk = 0; blk < 4; ++blk)
                            tma_load_2d(dst + blk * kStageTileBytes, &tm_b, fb, n0 + blk * 64, ks * 64);
                    } else {
                        tma_load_2d(dst, &tm_b, fb, ks * 64, n0);
                    }
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // MMA issuer
        const uint32_t idesc = idesc_f16(128, kSkN, A_MN, B_MN) | (p.bf16 ? idesc_ab_bf16() : 0u);
        constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
        constexpr uint32_t kAAdv = A_MN ? 128u : 2u, kBAdv = B_MN ? 128u : 2u;     // address-field step per 16 of k
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        int iter = 0;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++iter) {
            const int split = item / (p.n_tiles * p.m_tiles);
            int k0, k1;
            k_range(split, k0, k1);
            const int buf = kBufs == 2 ? (iter & 1) : 0;
            const uint32_t use = kBufs == 2 ? ((uint32_t)iter >> 1) : (uint32_t)iter;
            ok = mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, status, kStatusMmaTimeout);
            if (!ok) break;
            tc_fence_after();
            uint32_t accumulate = 0;
            for (int ks = k0; ks < k1; ++ks) {
                ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t b_lo = smem_desc_lo(b_base + stage * kSkBBytes, B_MN ? kStageTileBytes : 16);
#pragma unroll
                    for (int a = 0; a < MA; ++a) {
                        const uint32_t a_lo = smem_desc_lo(a_base + stage * L::kABytes + (A_MN ? 0 : a * kATileBytes),
                                                           A_MN ? kStageTileBytes : 16);
                        const uint32_t d_tmem = tmem_base + (uint32_t)((kBufs == 2 ? buf : a) * kSkN);
#pragma unroll
                        for (int kq = 0; kq < 4; ++kq)
                            umma_f16_lohi(d_tmem, a_lo + kq * kAAdv, desc_hi, b_lo + kq * kBAdv, desc_hi, idesc,
                                          kq ? 1u : accumulate);
                    }
                    umma_commit(empty0 + 8u * stage);
                }
                __syncwarp();
                accumulate = 1u;
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok && lane == 0) umma_commit(tfull_bar(buf));
            __syncwarp();
        }
    } else if (warp >= 4) {
        // epilogue: thread = accumulator row.  Half output: 64-column chunks are rounded, staged in shared memory in
        // the 128-byte swizzle and written by TMA (whole 128-byte rows; the copy clips what hangs over the matrix).
        // Float output (partials of a split, or a float D): the same in 32-column chunks, through a tensor map that
        // views the float matrix as rows of twice as many 16-bit elements, with the split as third coordinate.
        const int q = warp & 3;
        const int trow = q * 32 + lane;
        const bool leader = threadIdx.x == 128;
        int iter = 0, chunk_count = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++iter) {
            const int nt = item % p.n_tiles, mt = (item / p.n_tiles) % p.m_tiles, split = item / (p.n_tiles * p.m_tiles);
            const int buf = kBufs == 2 ? (iter & 1) : 0;
            const uint32_t use = kBufs == 2 ? ((uint32_t)iter >> 1) : (uint32_t)iter;
            if (!mbar_wait_relaxed(tfull_bar(buf), use & 1u, abort_flag, status, kStatusEpilogueTimeout)) s_epi_fail = 1;
            named_barrier(2, kEpiThreads);
            if (*(volatile int*)&s_epi_fail) break;
            tc_fence_after();
            const int n0 = nt * kSkN;
#pragma unroll
            for (int a = 0; a < MA; ++a) {
                const int row0 = mt * (MA * 128) + a * 128;
                const int row = row0 + trow;
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((kBufs == 2 ? buf : a) * kSkN);
                if (F32OUT) {
                    // 32 float columns of the thread's row are one 128-byte row of the staging tile
#pragma unroll 1
                    for (int chunk = 0; chunk < kSkN / 32; ++chunk) {
                        if (n0 + chunk * 32 >= p.n_real || row0 >= p.m_real) continue;      // block-uniform
                        const uint32_t sbuf = epi_base + (uint32_t)(chunk_count & 1) * kATileBytes;
                        if (leader) tma_store_wait_read<1>();
                        named_barrier(1, kEpiThreads);
                        uint32_t v[32];
                        tmem_ld_32x32(t0 + (uint32_t)(chunk * 32), v);
                        tmem_ld_wait();
                        const uint32_t row_addr = sbuf + (uint32_t)trow * 128u;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t dst = row_addr + (uint32_t)((j ^ (trow & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * j]),
                                         "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        named_barrier(1, kEpiThreads);
                        if (leader) {
                            tma_store_3d(&tm_d, sbuf, (n0 + chunk * 32) * 2, row0, split);
                            tma_store_commit();
                        }
                        ++chunk_count;          // the staging buffers alternate per store, not per chunk
                    }
                } else {
#pragma unroll 1
                    for (int chunk = 0; chunk < kSkN / 64; ++chunk) {
                        if (n0 + chunk * 64 >= p.n_real || row0 >= p.m_real) continue;      // block-uniform
                        const uint32_t sbuf = epi_base + (uint32_t)(chunk_count & 1) * kATileBytes;
                        if (leader) tma_store_wait_read<1>();
                        named_barrier(1, kEpiThreads);
                        uint32_t v0[32], v1[32];
                        tmem_ld_32x32(t0 + (uint32_t)(chunk * 64), v0);
                        tmem_ld_32x32(t0 + (uint32_t)(chunk * 64 + 32), v1);
                        tmem_ld_wait();
                        const uint32_t row_addr = sbuf + (uint32_t)trow * 128u;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t* src = j < 4 ? &v0[j * 8] : &v1[(j - 4) * 8];
                            uint32_t pk[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                pk[e] = p.bf16 ? pack2_t<true>(__uint_as_float(src[2 * e]), __uint_as_float(src[2 * e + 1]))
                                               : pack2_t<false>(__uint_as_float(src[2 * e]), __uint_as_float(src[2 * e + 1]));
                            const uint32_t dst = row_addr + (uint32_t)((j ^ (trow & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]),
                                         "r"(pk[2]), "r"(pk[3])
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        named_barrier(1, kEpiThreads);
                        if (leader) {
                            tma_store_2d(&tm_d, sbuf, n0 + chunk * 64, row0);
                            tma_store_commit();
                        }
                        ++chunk_count;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(buf));
        }
        if (leader) tma_store_wait_all();
    }

    abort_drain(abort_flag);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// row-major half matrix [rows][cols]; K-major operand: box {64, box_rows}; MN-major operand: box {64, 64}
int make_matrix_tmap(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows,
                     const char* what) {
    const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    const uint64_t str[2] = {2, (uint64_t)ld * 2};
    const uint32_t box[2] = {64, (uint32_t)box_rows};
    return make_tmap(m, base, 2, dims, str, box, what);
}

template <bool A_MN, bool B_MN, int MA, bool F32OUT>
int launch_skinny(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const SkinnyParams& p,
                  cudaStream_t st) {
    using L = SkinnyCfg<MA>;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(gemm_skinny_kernel<A_MN, B_MN, MA, F32OUT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int items = p.splits * p.m_tiles * p.n_tiles;
    const int grid = items < sm_count() ? items : sm_count();
    CUtensorMap tdf;
    if (F32OUT) {
        // float D [split][m_real][ldd] as 16-bit elements: box = 32 floats x 128 rows of one split
        const int64_t plane = p.split_stride ? p.split_stride : (int64_t)p.m_real * p.ldd;
        const uint64_t dims[3] = {(uint64_t)p.n_real * 2, (uint64_t)p.m_real, (uint64_t)p.splits};
        const uint64_t str[3] = {2, (uint64_t)p.ldd * 4, (uint64_t)plane * 4};
        const uint32_t box[3] = {64, 128, 1};
        const int rc = make_tmap(&tdf, p.d, 3, dims, str, box, "float D");
        if (rc) return rc;
    }
    gemm_skinny_kernel<A_MN, B_MN, MA, F32OUT><<<grid, kThreads, L::kTotal, st>>>(ta, tb, F32OUT ? tdf : td, p, status);
    TRB_LAUNCH_CHECK("gemm_skinny_kernel");
    return TRB200_OK;
}
