// 3x3 / stride 1 / pad 1 convolution (forward and data gradient) with the output PIXELS on
// the MMA's N dimension, for layers with 64 or 128 output channels.
//
// A tcgen05.mma of shape M x N x 16 occupies the tensor pipe for max(N / 2, operand bytes / 128) clocks whatever
// M is, and the thread that issues it pays about 55 clocks per MMA, commit or barrier probe: a K step of four MMAs
// costs its issuer ~460 clocks inside a kernel, which only N = 256 (512 pipe clocks) hides.  The kernels in
// conv_igemm_sm100.cu put the output channels on N and reach 28 % / 60 % of peak at 64 / 128 channels.  Here the
// GEMM is transposed:
//
//   D[co][pixel] = sum_{tap} sum_{ci} Wv[tap][co][ci] * in[pixel + tap offset][ci]
//   M = MT output channels (A operand = filters, K-major rows of 64 input channels),
//   N = 256 output pixels (B operand = a bw x bh x bn box of the image, bw*bh*bn = 256,
//       fetched as two 128-pixel boxes moved by the tap; out-of-image pixels zero-filled),
//   K loop = 9 taps x (Cin / 64) slices.
//
// The accumulator has one output channel per TMEM lane and one pixel per column, so an
// epilogue thread owns a channel: it rounds its 256 values to half, writes them into NHWC
// staging rows (2-byte stores; a warp's 32 channels fill 64 contiguous bytes of a pixel's
// row) for TMA stores of 64 pixels x 64 channels, and - for the forward pass - keeps the
// channel's running sum and sum of squares in two registers: the batch statistics need no
// second look at the tile and no reduction between threads.
//
// This file is included by conv_igemm_sm100.cu inside its anonymous namespace.
#pragma once

struct PixnParams {
    int taps, cin_slices;
    int c_tiles;            // ceil(cout / MT)
    int p_tiles;            // pixel tiles
    int tw, th;             // tiles along w and h
    int bw, bh, bn;         // tile box, bw * bh * bn = 256
    int lbw, lbh;           // log2 of bw, bh
    int b_tap_is_dim1;      // filter view is (ci, tap, co) instead of (ci, co, tap)
    int cout;
    int ext_w, ext_h, ext_n;
    int has_padding;
    float* stats_partial;   // [strip][2][cout], strip = block / c_tiles
};

constexpr int kPixN = 256;                      // pixels per tile
constexpr int kPixBTileBytes = kPixN * 128;     // 256 pixels x 64 halfs
constexpr int kPixATileBytes = 128 * 128;       // up to 128 channels x 64 halfs
constexpr int kPixStageBytes = kPixATileBytes + kPixBTileBytes;
constexpr int kPixStages = 4;
constexpr int kPixChunk = 64;                   // pixels per TMA store
constexpr int kPixEpiBufBytes = 2 * kPixChunk * 128;   // 64 pixels x (2 x 64 channels)
constexpr int kPixSmemTotal = kPixStages * kPixStageBytes + 2 * kPixEpiBufBytes + 2048;
static_assert(kPixSmemTotal <= kSmemBudget, "shared memory budget");

// rows [r0, r0 + span) of a tile (w fastest): origin offset of that sub-box inside the tile's box
__device__ __forceinline__ void pixn_sub_origin(const PixnParams& p, int r0, int& ow, int& oh, int& on) {
    ow = r0 & (p.bw - 1);
    oh = (r0 >> p.lbw) & (p.bh - 1);
    on = r0 >> (p.lbw + p.lbh);
}

// One 64-pixel chunk of the epilogue: this thread's channel, 64 accumulator columns -> half ->
// staging rows; MASKED applies the pixel validity bits (m0: pixels 0-31, m1: 32-63) to the sums.
// The TMEM loads are warp-wide (every lane of the warp must run them); `keep` says whether this lane's row
// is a channel at all (at M = 64 only lanes 0-15 of a warp hold one).
template <bool STATS, bool MASKED, bool BF16>
__device__ __forceinline__ void pixn_epi_chunk(uint32_t taddr, uint32_t dst0, int sw_base, uint32_t m0, uint32_t m1,
                                               bool keep, float& sum, float& sumsq) {
    // dst0 = staging address of (pixel 0, this channel) without the swizzle term; the 16-byte piece
    // index of the channel is sw_base, pixel j moves it to sw_base ^ (j & 7)
    uint32_t rowbase[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) rowbase[k] = dst0 + (uint32_t)((sw_base ^ k) << 4);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)(half * 32), v);
        tmem_ld_wait();
        const uint32_t m = half == 0 ? m0 : m1;
        if (keep) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const uint32_t hb = pack2_t<BF16>(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            const int pj = half * 32 + j;
            asm volatile("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\t"
                         "st.shared.b16 [%0], lo;\n\tst.shared.b16 [%1], hi;\n\t}"
                         ::"r"(rowbase[pj & 7] + (uint32_t)pj * 128u),
                           "r"(rowbase[(pj + 1) & 7] + (uint32_t)(pj + 1) * 128u), "r"(hb)
                         : "memory");
            if (STATS) {
                float2 f = unpack2_t<BF16>(hb);
                if (MASKED) {
                    if (!((m >> j) & 1u)) f.x = 0.f;
                    if (!((m >> (j + 1)) & 1u)) f.y = 0.f;
                }
                sum += f.x;
                sumsq = fmaf(f.x, f.x, sumsq);
                sum += f.y;
                sumsq = fmaf(f.y, f.y, sumsq);
            }
        }
        }
    }
}

template <int MT, bool STATS, bool BF16>
__device__ __forceinline__ void
conv3x3_pixn_body(const CUtensorMap& tm_in, const CUtensorMap& tm_w, const CUtensorMap& tm_out, const PixnParams& p,
                  int* status) {
    constexpr int kStages = kPixStages;
    constexpr uint32_t kTmemCols = 512;                    // two accumulators of 256 pixels
    constexpr uint32_t kATxBytes = MT * 128;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_base = base;
    const uint32_t b_base = base + kStages * kPixATileBytes;
    const uint32_t epi_base = b_base + kStages * kPixBTileBytes;
    const uint32_t bar_base = epi_base + 2 * kPixEpiBufBytes;
    // barriers: full[kStages] (filters + two pixel halves), empty[kStages], tmem_full[2], tmem_empty[2]
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
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, 3); mbar_init(empty0 + 8u * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpiThreads); }
        fence_barrier_init();
        prefetch_tmap(&tm_in);
        prefetch_tmap(&tm_w);
        prefetch_tmap(&tm_out);
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

    const int total_tiles = p.p_tiles * p.c_tiles;
    const int ksteps = p.taps * p.cin_slices;
    const int t_lo = p.taps == 9 ? 0 : 1, t_hi = p.taps == 9 ? 3 : 2;

    if (warp == 0) {
        // filter producer: MT rows of 64 input channels per K step
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int c_off = (tile % p.c_tiles) * MT;
            for (int tap = 0; tap < p.taps && ok; ++tap)
                for (int slice = 0; slice < p.cin_slices; ++slice) {
                    ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                    if (!ok) break;
                    const uint32_t fb = full0 + 8u * stage;
                    if (lane == 0) {
                        mbar_expect_tx(fb, kATxBytes);
                        if (p.b_tap_is_dim1)
                            tma_load_3d(a_base + stage * kPixATileBytes, &tm_w, fb, slice * 64, tap, c_off);
                        else
                            tma_load_3d(a_base + stage * kPixATileBytes, &tm_w, fb, slice * 64, c_off, tap);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
        }
    } else if (warp == 2 || warp == 3) {
        // pixel producers: warp 2 fetches rows 0-127 of the tile, warp 3 rows 128-255, moved by the tap
        const int hb = warp - 2;
        int ow, oh, on;
        pixn_sub_origin(p, hb * 128, ow, oh, on);
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        RT_DECL;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int pt = tile / p.c_tiles;
            const int w0 = (pt % p.tw) * p.bw + ow, h0 = ((pt / p.tw) % p.th) * p.bh + oh;
            const int n0 = (pt / (p.tw * p.th)) * p.bn + on;
            for (int r = t_lo; r < t_hi && ok; ++r)
                for (int s = t_lo; s < t_hi && ok; ++s)
                    for (int slice = 0; slice < p.cin_slices; ++slice) {
                        RT_ADD(1);
                        ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                        RT_ADD(0);
                        if (!ok) break;
                        const uint32_t fb = full0 + 8u * stage;
                        if (lane == 0) {
                            mbar_expect_tx(fb, kPixBTileBytes / 2);
                            tma_load_4d(b_base + stage * kPixBTileBytes + hb * (kPixBTileBytes / 2), &tm_in, fb,
                                        slice * 64, w0 + s - 1, h0 + r - 1, n0);
                        }
                        __syncwarp();
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
        }
        RT_ADD(1);
        if (lane == 0 && warp == 2) RT_STORE(0);
    } else if (warp == 1) {
        // MMA issuer
        constexpr uint32_t idesc = idesc_f16(MT, kPixN, false, false) | (BF16 ? idesc_ab_bf16() : 0u);
        constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
        const uint32_t a_lo0 = smem_desc_lo(a_base, 16), b_lo0 = smem_desc_lo(b_base, 16);
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        int iter = 0;
        RT_DECL;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++iter) {
            const int acc = iter & 1;
            RT_ADD(2);
            ok = mbar_wait(tempty_bar(acc), (((uint32_t)iter >> 1) & 1u) ^ 1u, abort_flag, status, kStatusMmaTimeout);
            RT_ADD(0);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kPixN);
            uint32_t accumulate = 0;
            for (int ks = 0; ks < ksteps; ++ks) {
                RT_ADD(2);
                ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
                RT_ADD(1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + stage * (kPixATileBytes >> 4);
                const uint32_t b_lo = b_lo0 + stage * (kPixBTileBytes >> 4);
                if (lane == 0) {
                    umma_f16_lohi(d_tmem, a_lo, desc_hi, b_lo, desc_hi, idesc, accumulate);
                    umma_f16_lohi(d_tmem, a_lo + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                    umma_f16_lohi(d_tmem, a_lo + 4, desc_hi, b_lo + 4, desc_hi, idesc, 1u);
                    umma_f16_lohi(d_tmem, a_lo + 6, desc_hi, b_lo + 6, desc_hi, idesc, 1u);
                    umma_commit(empty0 + 8u * stage);
                }
                __syncwarp();
                accumulate = 1u;
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok && lane == 0) umma_commit(tfull_bar(acc));
            __syncwarp();
        }
        RT_ADD(2);
        if (lane == 0) RT_STORE(1);
    } else if (warp >= 4) {
        // epilogue: warp w owns TMEM lanes [32*(w%4), +32) = 32 output channels of the tile
        // (M = 64: the accumulator's 64 rows sit in lanes 0-15 of each 32-lane quarter)
        const int q = warp & 3;
        const int ch = MT == 64 ? q * 16 + (lane & 15) : q * 32 + lane;   // channel inside the MT tile
        const bool leader = threadIdx.x == 128;
        float run_s = 0.f, run_q = 0.f;
        int iter = 0, chunk_count = 0;
        RT_DECL;
        // staging: [64-channel half][pixel][128 bytes], 16-byte pieces swizzled by (pixel & 7)
        const uint32_t ch_off = (uint32_t)((ch >> 6) * (kPixChunk * 128) + (ch & 7) * 2);
        const int sw_base = (ch & 63) >> 3;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++iter) {
            const int acc = iter & 1;
            const int ct = tile % p.c_tiles, pt = tile / p.c_tiles;
            const int c_off = ct * MT;
            const int w0 = (pt % p.tw) * p.bw, h0 = ((pt / p.tw) % p.th) * p.bh;
            const int n0 = (pt / (p.tw * p.th)) * p.bn;
            // channel halves of 64 that exist (the last tile of a 64-channel output has one)
            const int halves = (p.cout - c_off) >= MT ? MT / 64 : (p.cout - c_off + 63) / 64;
            const bool live = (MT == 64 ? q * 16 : q * 32) < halves * 64;   // warp-uniform
            const bool keep = MT == 128 || lane < 16;
            RT_ADD(2);
            if (!mbar_wait_relaxed(tfull_bar(acc), ((uint32_t)iter >> 1) & 1u, abort_flag, status, kStatusEpilogueTimeout))
                s_epi_fail = 1;
            named_barrier(2, kEpiThreads);
            RT_ADD(0);
            if (*(volatile int*)&s_epi_fail) break;
            tc_fence_after();
#pragma unroll 1
            for (int chunk = 0; chunk < kPixN / kPixChunk; ++chunk, ++chunk_count) {
                const uint32_t buf = epi_base + (uint32_t)(chunk_count & 1) * kPixEpiBufBytes;
                int ow, oh, on;
                pixn_sub_origin(p, chunk * kPixChunk, ow, oh, on);
                uint32_t m0 = 0xffffffffu, m1 = 0xffffffffu;
                if (STATS && p.has_padding) {
                    int x0, y0, i0, x1, y1, i1;
                    pixn_sub_origin(p, chunk * kPixChunk + lane, x0, y0, i0);
                    pixn_sub_origin(p, chunk * kPixChunk + 32 + lane, x1, y1, i1);
                    m0 = __ballot_sync(0xffffffffu, w0 + x0 < p.ext_w && h0 + y0 < p.ext_h && n0 + i0 < p.ext_n);
                    m1 = __ballot_sync(0xffffffffu, w0 + x1 < p.ext_w && h0 + y1 < p.ext_h && n0 + i1 < p.ext_n);
                }
                RT_ADD(2);
                if (leader) tma_store_wait_read<1>();     // the stores that last read this buffer are done
                named_barrier(1, kEpiThreads);
                RT_ADD(1);
                if (live) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) +
                                           (uint32_t)(acc * kPixN + chunk * kPixChunk);
                    if (STATS && p.has_padding)
                        pixn_epi_chunk<STATS, true, BF16>(taddr, buf + ch_off, sw_base, m0, m1, keep, run_s, run_q);
                    else
                        pixn_epi_chunk<STATS, false, BF16>(taddr, buf + ch_off, sw_base, m0, m1, keep, run_s, run_q);
                }
                RT_ADD(3);
                fence_proxy_async_smem();
                named_barrier(1, kEpiThreads);
                if (leader) {
                    for (int hf = 0; hf < halves; ++hf)
                        tma_store_4d(&tm_out, buf + (uint32_t)hf * (kPixChunk * 128), c_off + hf * 64, w0 + ow, h0 + oh,
                                     n0 + on);
                    tma_store_commit();
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
        }
        if (leader) tma_store_wait_all();
        RT_ADD(2);
        if (leader) RT_STORE(2);
        if (STATS && !*(volatile int*)&s_epi_fail) {
            // this block only ever sees one channel tile (the grid is a multiple of c_tiles)
            const int strip = blockIdx.x / p.c_tiles;
            const int c = (blockIdx.x % p.c_tiles) * MT + ch;
            if (c < p.cout && (MT == 128 || lane < 16)) {
                p.stats_partial[((size_t)strip * 2) * p.cout + c] = run_s;
                p.stats_partial[((size_t)strip * 2 + 1) * p.cout + c] = run_q;
            }
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

// sub-box of `span` consecutive rows (a power of two) of a tile box
inline TileShape pixn_sub_box(const TileShape& t, int span) {
    TileShape s = t;
    s.bw = span < t.bw ? span : t.bw;
    const int rest = span / s.bw;
    s.bh = rest < t.bh ? (rest < 1 ? 1 : rest) : t.bh;
    const int rest2 = span / (s.bw * s.bh);
    s.bn = rest2 < 1 ? 1 : rest2;
    return s;
}

// The kernels proper: one instantiation of the body per storage type, the half one under the plain name.
template <int MT, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_pixn_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_out, const PixnParams p, int* status) {
    conv3x3_pixn_body<MT, STATS, false>(tm_in, tm_w, tm_out, p, status);
}

template <int MT, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_pixn_kernel_bf16(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_out, const PixnParams p, int* status) {
    conv3x3_pixn_body<MT, STATS, true>(tm_in, tm_w, tm_out, p, status);
}

template <int MT, bool STATS>
int launch_pixn(const CUtensorMap& tin, const CUtensorMap& tw, const CUtensorMap& tout, const PixnParams& p,
                cudaStream_t st, bool bf16) {
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_pixn_kernel<MT, STATS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kPixSmemTotal));
        TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_pixn_kernel_bf16<MT, STATS>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kPixSmemTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = conv3x3_grid(p.p_tiles, p.c_tiles);
    if (bf16) conv3x3_pixn_kernel_bf16<MT, STATS><<<grid, kThreads, kPixSmemTotal, st>>>(tin, tw, tout, p, status);
    else conv3x3_pixn_kernel<MT, STATS><<<grid, kThreads, kPixSmemTotal, st>>>(tin, tw, tout, p, status);
    TRB_LAUNCH_CHECK("conv3x3_pixn_kernel");
    return TRB200_OK;
}

// whether the pixel-N kernel is the better one for `cout` output channels
inline bool pixn_preferred(int cin, int cout) { return cin % 64 == 0 && (cout == 64 || cout == 128); }

// Same contract as conv3x3_run (taps = 9 or 1, cin a multiple of 64).
int conv3x3_pixn_run(const void* in, const void* wv, int tap_is_dim1, void* out, int n, int h, int w, int cin,
                     int cout, cudaStream_t st, float* stats_partial, int* stats_strips, bool bf16, int taps) {
    const int MT = cout == 64 ? 64 : 128;
    const TileShape t = pick_tile(n, h, w, kPixN);
    const TileShape th = pixn_sub_box(t, 128), tc = pixn_sub_box(t, kPixChunk);
    CUtensorMap tin, tw, tout;
    int rc = make_act_tmap(&tin, in, n, h, w, cin, th, "conv input");
    if (rc) return rc;
    rc = make_act_tmap(&tout, out, n, h, w, cout, tc, "conv output");
    if (rc) return rc;
    if (tap_is_dim1) {
        const uint64_t dims[3] = {(uint64_t)cin, (uint64_t)taps, (uint64_t)cout};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)taps * cin * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)MT};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,tap,co)");
    } else {
        const uint64_t dims[3] = {(uint64_t)cin, (uint64_t)cout, (uint64_t)taps};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)cout * cin * 2};
        const uint32_t box[3] = {64, (uint32_t)MT, 1};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,co,tap)");
    }
    if (rc) return rc;
    PixnParams p;
    p.taps = taps;
    p.cin_slices = cin / 64;
    p.c_tiles = (cout + MT - 1) / MT;
    p.p_tiles = t.tw * t.th * t.tn;
    p.tw = t.tw; p.th = t.th;
    p.bw = t.bw; p.bh = t.bh; p.bn = t.bn;
    p.lbw = 0; p.lbh = 0;
    while ((1 << p.lbw) < t.bw) ++p.lbw;
    while ((1 << p.lbh) < t.bh) ++p.lbh;
    p.b_tap_is_dim1 = tap_is_dim1;
    p.cout = cout;
    p.ext_w = w; p.ext_h = h; p.ext_n = n;
    p.has_padding = (t.tw * t.bw != w) || (t.th * t.bh != h) || (t.tn * t.bn != n);
    p.stats_partial = stats_partial;
    if (stats_partial && stats_strips) *stats_strips = conv3x3_grid(p.p_tiles, p.c_tiles) / p.c_tiles;
    if (MT == 64) {
        if (stats_partial) return launch_pixn<64, true>(tin, tw, tout, p, st, bf16);
        return launch_pixn<64, false>(tin, tw, tout, p, st, bf16);
    }
    if (stats_partial) return launch_pixn<128, true>(tin, tw, tout, p, st, bf16);
    return launch_pixn<128, false>(tin, tw, tout, p, st, bf16);
}
