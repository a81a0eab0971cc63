// 3x3 / stride 1 / pad 1 convolution gradients as implicit GEMMs on the sm_100a
// tensor cores: tcgen05.mma with accumulators in tensor memory, operands staged
// in shared memory by TMA (tile mode, no cluster multicast), one output tile per
// loop iteration of a persistent CTA.
//
// Reference counterparts: the cuDNN-FE conv_dgrad / conv_wgrad graphs that
// launch_cbr_amp_bwd_cuda executes, src/backend/ops/dtensor/cbr_op.cpp:763-917,
// 1431-1508.
//
// ---------------------------------------------------------------------------
// dgrad (and forward conv: same kernel, other filter view)
//   out[n,y,x,co] = sum_{tap=(r,s)} sum_{ci} in[n, y+r-1, x+s-1, ci] * Wv[tap][co][ci]
//   GEMM: M = 128 output pixels (a bw x bh x bn box of the image, bw*bh*bn = 128),
//         N = NT output channels, K loop = 9 taps x (Cin/64) slices of 64 channels.
//   A (pixels x 64 channels) is K-major: one pixel = one 128-byte row; the TMA box
//   of a tap is the tile's box moved by (s-1, r-1), and out-of-image pixels are
//   zero-filled by TMA, which is the padding.  B (NT x 64) is K-major too.
//   For dgrad, in = dconv, Wv[tap'][c][k] = W[k][2-r'][2-s'][c] (a small kernel
//   writes that view into the workspace first).
// wgrad
//   dW[k][tap][c] = sum_pixels dconv[p][k] * X[p + tap offset][c]
//   GEMM: M = 128 = two (tap, 64-channel block of c) units, N = NT channels of k,
//   K loop = pixels, 64 per stage.  Both operands have the reduction dimension
//   (pixels) strided and the M/N dimension contiguous: MN-major descriptors.
//   Work = (M tile, N tile, split of the pixel range); every split writes a float
//   partial tile and a second kernel adds the splits in split order (bitwise
//   reproducible) and writes half KRSC.
//
// Warp roles (256 threads and up): warp 0 (and 3, 8, 9) = TMA producers for the activation operand, warp 1 = MMA
// issuer + TMEM allocation, warp 2 (and 3 / 8) = TMA producers for the filter / dconv operand, warps 4-7 =
// epilogue (TMEM -> registers -> half -> shared -> TMA store, or float partial -> global).  One thread pays about
// 55 clocks for every tcgen05.mma, commit or barrier probe it issues and a few hundred for a TMA box, so the loads
// of a stage are spread over several threads that all arrive on the stage's "full" barrier, K steps are dealt to
// producer warps in turn, and the MMA issuer probes the barrier of its next stage before it issues the MMAs of the
// current one.  A stage of a ring keeps the same producers and the same consumer for the whole kernel (the rings
// have a length their parties divide): a parity wait is only safe for a party that saw the previous use of that
// stage complete.  Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
// A tcgen05.mma occupies the tensor pipe for max(N / 2, operand bytes / 128) clocks whatever M is, and the issuer's
// ~460 clocks per K step of four MMAs hide behind it only at N = 256.  The kernels of this file therefore serve the
// layers with 256 channels or more on N; conv_pixn_sm100.cuh (pixels on N) and wgrad_unitn_sm100.cuh ((tap,
// channel-block) units on N) serve the layers with 64 or 128.
#include "common.cuh"
#include "conv.cuh"
#include "sm100_ptx.cuh"

#include <cuda.h>

#include <mutex>

namespace trb {

__device__ int g_device_status = 0;   // first device-side failure code, 0 = none

// Optional per-role cycle counters (development builds only, -DTRB200_ROLE_TIMERS):
// [block][role 0 producer / 1 MMA / 2 epilogue][4 slots], see the RT_ADD sites.
#ifdef TRB200_ROLE_TIMERS
__device__ long long g_role_timers[256 * 3 * 4];
#define RT_DECL long long rt_t0 = clock64(), rt_acc[4] = {0, 0, 0, 0}
#define RT_ADD(i) do { const long long rt_t = clock64(); rt_acc[i] += rt_t - rt_t0; rt_t0 = rt_t; } while (0)
#define RT_STORE(role) do { if (blockIdx.x < 256) for (int rt_i = 0; rt_i < 4; ++rt_i) \
        g_role_timers[(blockIdx.x * 3 + (role)) * 4 + rt_i] = rt_acc[rt_i]; } while (0)
#else
#define RT_DECL do { } while (0)
#define RT_ADD(i) do { } while (0)
#define RT_STORE(role) do { } while (0)
#endif

namespace {

using namespace ptx;

constexpr int kThreads = 256;
// IM2COL kernels add 256 builder threads (warps 8-15).  One global-load round trip per stage is
// longer than the MMAs of a stage, so the builders work in groups that take stages in turn.
constexpr int kBuilderThreads = 256;
// The builders' source is a ring of raw image tiles (the tile's pixels plus a halo, 8 bytes per
// pixel) that a TMA producer keeps filled several tiles ahead; shapes whose halo tile does not
// fit a ring slot, or whose width is odd, are read with plain global loads instead.
constexpr int kRawStages = 8;
constexpr int kRawStageBytes = 4096;      // warp 0: TMA producer A, 1: MMA, 2 (and 3): TMA producer B, 4-7: epilogue
constexpr int kEpiThreads = 128;
constexpr int kATileBytes = 128 * 128;    // 128 pixels x 64 halfs
constexpr int kStageTileBytes = 64 * 128; // wgrad: 64 pixels x 64 halfs
constexpr int kSmemBudget = 227 * 1024;

enum StatusCode {
    kStatusProducerTimeout = 1,
    kStatusMmaTimeout = 2,
    kStatusEpilogueTimeout = 3,
};

struct TileShape {
    int bw, bh, bn;       // box extents along w, h, n (product = pixels per tile)
    int tw, th, tn;       // tiles along w, h, n
};

// Box of `pixels` image positions with the least padding; ties go to the widest box.
TileShape pick_tile(int n, int h, int w, int pixels) {
    TileShape best{};
    long best_cost = -1;
    for (int bw = pixels; bw >= 1; bw >>= 1)
        for (int bh = pixels / bw; bh >= 1; bh >>= 1) {
            const int bn = pixels / (bw * bh);
            if (bw > 256 || bh > 256 || bn > 256) continue;
            const int tw = (w + bw - 1) / bw, th = (h + bh - 1) / bh, tn = (n + bn - 1) / bn;
            const long cost = (long)tw * bw * th * bh * tn * bn;
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                best = TileShape{bw, bh, bn, tw, th, tn};
            }
        }
    return best;
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Half tensor, `rank` dims (innermost first), 128-byte swizzle, zero fill.
int make_tmap(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
              const uint32_t* box, const char* what, const uint32_t* elem_strides = nullptr) {
    EncodeTiledFn fn = encode_fn();
    TRB_REQUIRE(fn, TRB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t gdim[5];
    cuuint64_t gstr[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = elem_strides ? elem_strides[i] : 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i];
    }
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim,
                          gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TRB_REQUIRE(r == CUDA_SUCCESS, TRB200_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what,
                (int)r);
    return TRB200_OK;
}

// NHWC half activation [n,h,w,c] viewed as (c, w, h, n) with a {64, bw, bh, bn} box.
int make_act_tmap(CUtensorMap* m, const void* base, int n, int h, int w, int c, const TileShape& t,
                  const char* what) {
    const uint64_t dims[4] = {(uint64_t)c, (uint64_t)w, (uint64_t)h, (uint64_t)n};
    const uint64_t str[4] = {2, (uint64_t)c * 2, (uint64_t)w * c * 2, (uint64_t)h * w * c * 2};
    const uint32_t box[4] = {64, (uint32_t)t.bw, (uint32_t)t.bh, (uint32_t)t.bn};
    return make_tmap(m, base, 4, dims, str, box, what);
}

// The same tensor read with a step of `step` pixels along w and h (a stride-2 convolution's input): the box spans
// bw * step x bh * step pixels and holds every step-th of them, so the tile in shared memory is the bw x bh x bn pixels
// of the stride-1 case.  Box coordinates stay in the tensor's own pixel grid.
int make_act_tmap_stepped(CUtensorMap* m, const void* base, int n, int h, int w, int c, const TileShape& t, int step,
                          const char* what) {
    const uint64_t dims[4] = {(uint64_t)c, (uint64_t)w, (uint64_t)h, (uint64_t)n};
    const uint64_t str[4] = {2, (uint64_t)c * 2, (uint64_t)w * c * 2, (uint64_t)h * w * c * 2};
    const uint32_t box[4] = {64, (uint32_t)(t.bw * step), (uint32_t)(t.bh * step), (uint32_t)t.bn};
    const uint32_t es[4] = {1, (uint32_t)step, (uint32_t)step, 1};
    TRB_REQUIRE(box[1] <= 256 && box[2] <= 256, TRB200_ERR_UNSUPPORTED, "%s: a stepped box of %u x %u pixels", what, box[1],
                box[2]);
    return make_tmap(m, base, 4, dims, str, box, what, es);
}

// Every second pixel of an [n,h,w,c] tensor, starting at pixel (py, px): a plain tensor map over the pixels of one
// parity (the outputs one class of a stride-2 data gradient writes).
int make_act_tmap_parity(CUtensorMap* m, const void* base, int n, int h, int w, int c, int py, int px, const TileShape& t,
                         const char* what) {
    const int hc = (h - py + 1) / 2, wc = (w - px + 1) / 2;
    const uint64_t dims[4] = {(uint64_t)c, (uint64_t)wc, (uint64_t)hc, (uint64_t)n};
    const uint64_t str[4] = {2, (uint64_t)c * 4, (uint64_t)w * c * 4, (uint64_t)h * w * c * 2};
    const uint32_t box[4] = {64, (uint32_t)t.bw, (uint32_t)t.bh, (uint32_t)t.bn};
    const unsigned char* b = static_cast<const unsigned char*>(base) + ((int64_t)py * w + px) * c * 2;
    return make_tmap(m, b, 4, dims, str, box, what);
}

// 4-channel half image [n,h,w] of 8-byte pixels viewed as (w, h, n) with a {bw + 4, bh + 2, bn} box,
// no swizzle.  The box starts two pixels left of the tile so that its first byte is 16-byte aligned.
int make_raw_x4_tmap(CUtensorMap* m, const void* base, int n, int h, int w, const TileShape& t) {
    EncodeTiledFn fn = encode_fn();
    TRB_REQUIRE(fn, TRB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[3] = {(cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
    const cuuint64_t gstr[2] = {(cuuint64_t)w * 8, (cuuint64_t)h * w * 8};
    const cuuint32_t bx[3] = {(cuuint32_t)t.bw + 4, (cuuint32_t)t.bh + 2, (cuuint32_t)t.bn};
    const cuuint32_t es[3] = {1, 1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(base), gdim, gstr, bx, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TRB_REQUIRE(r == CUDA_SUCCESS, TRB200_ERR_CUDA, "cuTensorMapEncodeTiled(4-channel image) failed with CUresult %d",
                (int)r);
    return TRB200_OK;
}

// whether the halo tile of shape t can go through the raw ring
bool raw_ring_fits(const TileShape& t, int w, const void* x4) {
    return (w % 2 == 0) && t.bw >= 2 && (t.bw + 4) * (t.bh + 2) * t.bn * 8 <= kRawStageBytes &&
           (reinterpret_cast<uintptr_t>(x4) & 15u) == 0;
}

// ------------------------------------------------------------------ shared helpers
__device__ __forceinline__ void abort_drain(volatile int* abort_flag) {
    // after a failed wait: give copies already in flight time to land before the
    // block gives its shared memory back
    if (*abort_flag) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
}

// First layer (4 input channels): the 3x3 neighbourhood of a pixel is 36 halfs, written as one
// 128-byte operand row (9 taps x 8 bytes + zeros) straight into the swizzled shared-memory
// tile, so that the im2col matrix never exists in HBM.  `row` is the row's index in the tile
// (it decides the swizzle phase), (y, x, img) the pixel; a pixel outside the image gives zeros.
__device__ __forceinline__ void store_im2col_row_c4(const uint2 (&t)[10], uint32_t tile, int row) {
    const uint32_t row_addr = tile + (uint32_t)row * 128u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint2 a = j < 5 ? t[2 * j] : make_uint2(0u, 0u);
        const uint2 b = j < 5 ? t[2 * j + 1] : make_uint2(0u, 0u);
        const uint32_t dst = row_addr + (uint32_t)((j ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a.x), "r"(a.y), "r"(b.x), "r"(b.y)
                     : "memory");
    }
}

__device__ __forceinline__ void load_neighbourhood_global(uint2 (&t)[10], const uint2* __restrict__ x4, int img, int y,
                                                          int x, int ext_n, int ext_h, int ext_w) {
#pragma unroll
    for (int k = 0; k < 10; ++k) t[k] = make_uint2(0u, 0u);
    if (img < ext_n && y < ext_h && x < ext_w) {
        const uint2* base = x4 + ((int64_t)img * ext_h) * ext_w;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int yy = y + r - 1;
            if (yy < 0 || yy >= ext_h) continue;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const int xx = x + c - 1;
                if (xx >= 0 && xx < ext_w) t[r * 3 + c] = __ldg(base + (int64_t)yy * ext_w + xx);
            }
        }
    }
}

// `centre` = shared-memory address of the pixel in a raw halo tile whose rows are `pitch` pixels long;
// pixels outside the image were zero-filled by the copy
__device__ __forceinline__ void load_neighbourhood_raw(uint2 (&t)[10], uint32_t centre, int pitch) {
    t[9] = make_uint2(0u, 0u);
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            const uint32_t a = centre + (uint32_t)(((r - 1) * pitch + (c - 1)) * 8);
            asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(t[r * 3 + c].x), "=r"(t[r * 3 + c].y) : "r"(a));
        }
}

__device__ __forceinline__ void build_im2col_row_c4(const uint2* __restrict__ x4, uint32_t tile, int row, int img,
                                                    int y, int x, int ext_n, int ext_h, int ext_w) {
    uint2 t[10];
    load_neighbourhood_global(t, x4, img, y, x, ext_n, ext_h, ext_w);
    store_im2col_row_c4(t, tile, row);
}

// ------------------------------------------------------------------ dgrad / fprop kernel
struct FpropParams {
    int taps;            // 9 (3x3, pad 1) or 1 (1x1, pad 0)
    int tap_base;        // 0 for 3x3; 4 for 1x1 (the centre tap: offset (0, 0))
    int step;            // input pixels per output pixel (1, or 2 for a stride-2 convolution)
    unsigned long long tap_offsets;   // 4 bits per tap: input offset of the tap, (dw + 1) | (dh + 1) << 2
    int cin_slices;      // Cin / 64
    int n_tiles;         // Cout / NT
    int m_tiles;         // tw * th * tn
    int tw, th;          // tiles along w, h
    int bw, bh, bn;
    int b_tap_is_dim1;   // 1: filter view dims (ci, tap, co) [KRSC as is]; 0: (ci, co, tap)
    // batch statistics of the output (STATS kernels only)
    const uint2* x4;        // IM2COL kernels: the 4-channel input image [n,h,w] of 8-byte pixels
    int raw_ring;           // IM2COL kernels: tm_in describes x4 and halo tiles go through the raw ring
    float* stats_partial;   // [strip][2][cout], strip = block / n_tiles
    int cout;
    int lbw, lbh;           // log2 of bw, bh
    int ext_w, ext_h, ext_n;   // image extents: rows of a tile beyond them are padding
    int has_padding;        // some tile hangs over an image edge
};

template <int NT, bool IM2COL = false>
struct FpropSmem {
    static constexpr int kBTileBytes = NT * 128;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kEpiBytes = 2 * kATileBytes;
    static constexpr int kRawBytes = IM2COL ? kRawStages * kRawStageBytes : 0;
    // parties that take stages in turn (builder groups, producers dealt K steps) need a ring they divide, so that a
    // stage always has the same owner: a parity wait is only safe for a party that has seen the previous use of the
    // same stage complete.  The ring is 8 stages, or the largest even count that fits.
    static constexpr int kStagesFit = (kSmemBudget - 2048 - kEpiBytes - kRawBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit >= 8 ? 8 : (kStagesFit >= 2 ? kStagesFit / 2 * 2 : kStagesFit);
    static constexpr int kTotal = kStages * kStageBytes + kEpiBytes + kRawBytes + 2048;   // + alignment slack and barriers
};

// Issuing one TMA box costs its thread a few hundred clocks, which is more than the MMAs of a K step take when
// the tile is narrow: the activation boxes of consecutive K steps are then issued by several warps in turn
// (warps 0 and 3, and for NT = 64 two more warps behind the epilogue).
template <int NT> __host__ __device__ constexpr int conv3x3_a_producers() { return NT == 64 ? 4 : 2; }
// the 256-row filter tile is fetched as two 128-row boxes by two warps (warp 2 and warp 8)
template <int NT, bool IM2COL> __host__ __device__ constexpr int conv3x3_b_split() { return (NT == 256 && !IM2COL) ? 2 : 1; }
template <int NT, bool IM2COL> __host__ __device__ constexpr int conv3x3_threads() {
    // IM2COL: 8 builder warps and, for 64 filters, a second group of 4 epilogue warps
    return IM2COL ? kThreads + kBuilderThreads + (NT == 64 ? 128 : 0) : (NT == 64 ? kThreads + 64 : (NT == 256 ? kThreads + 32 : kThreads));
}

// IM2COL: 8 more warps (two groups of 128 threads) build the A tiles from the 4-channel image instead of TMA.
template <int NT, bool STATS, bool IM2COL, bool BF16>
__device__ __forceinline__ void
conv3x3_igemm_body(const CUtensorMap& tm_in, const CUtensorMap& tm_w, const CUtensorMap& tm_out, const FpropParams& p,
                   int* status) {
    using L = FpropSmem<NT, IM2COL>;
    constexpr int kStages = L::kStages;
    constexpr uint32_t kTmemCols = 2 * NT;
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_base = base;
    const uint32_t b_base = base + kStages * kATileBytes;
    const uint32_t epi_base = b_base + kStages * L::kBTileBytes;
    const uint32_t raw_base = epi_base + L::kEpiBytes;
    const uint32_t bar_base = raw_base + L::kRawBytes;
    // barriers: full[kStages] (2 producers), empty[kStages], tmem_full[2], tmem_empty[2],
    // raw_full[kRawStages], raw_empty[kRawStages]
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    const uint32_t rfull0 = bar_base + 8u * (2 * kStages + 4), rempty0 = rfull0 + 8u * kRawStages;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    // First-layer variant: a tile is one K step, so the kernel runs at the pace of its epilogue (~1300 clocks per
    // 128-pixel tile for TMEM -> half -> staging -> TMA store and the channel sums).  Two epilogue groups of four warps
    // take alternate tiles, each with its own accumulator, staging buffer and named barriers.
    constexpr int kEpiGroups = (IM2COL && NT == 64) ? 2 : 1;
    __shared__ int s_epi_fail[2];
    __shared__ uint32_t s_valid[2][4];   // STATS: which of the tile's 128 rows are real pixels

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_epi_fail[0] = 0; s_epi_fail[1] = 0;
        // a stage is full once its B tile has landed and its A tile has (one TMA box, or 128 built rows)
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8u * s, IM2COL ? 129 : 1 + conv3x3_b_split<NT, IM2COL>()); mbar_init(empty0 + 8u * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpiThreads); }
        if (IM2COL)
            for (int s = 0; s < kRawStages; ++s) { mbar_init(rfull0 + 8u * s, 1); mbar_init(rempty0 + 8u * s, 128); }
        fence_barrier_init();
        if (!IM2COL || p.raw_ring) prefetch_tmap(&tm_in);
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

    static_assert(IM2COL || kStages % conv3x3_a_producers<NT>() == 0, "a stage keeps its A producer");
    static_assert(!IM2COL || kStages % (kBuilderThreads / 128) == 0, "a stage keeps its builder group");
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int ksteps = p.taps * p.cin_slices;

    // The single-thread roles below are paced by their own instruction count (a lone
    // thread issues roughly one dependent instruction every few clocks), so their inner
    // loops carry running addresses and counters instead of divisions and multiplies.
    // Each of these roles is run by a whole (converged) warp with warp-uniform values, and
    // only the instructions that must come from one thread are predicated on lane 0: the
    // compiler can then keep addresses, coordinates and descriptors in uniform registers,
    // which is where the TMA and MMA instructions take them from.
    if (IM2COL && warp >= 8 && warp < 8 + kBuilderThreads / 32) {
        // A-tile builders: thread = one pixel row of the tile, one K step (= one stage) per tile;
        // group g takes the block's tiles g, g + 2, ...
        constexpr int kGroups = kBuilderThreads / 128;
        const int row = (threadIdx.x - kThreads) & 127, group = (threadIdx.x - kThreads) >> 7;
        const int bx = row & (p.bw - 1), by = (row >> p.lbw) & (p.bh - 1), bi = row >> (p.lbw + p.lbh);
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            if (it % kGroups != group) continue;
            const uint32_t stage = (uint32_t)(it % kStages), phase = (uint32_t)((it / kStages) & 1);
            uint2 t[10];
            if (p.raw_ring) {
                const uint32_t rs = (uint32_t)(it % kRawStages), rphase = (uint32_t)((it / kRawStages) & 1);
                const int pitch = p.bw + 4;
                if (!mbar_wait_relaxed(rfull0 + 8u * rs, rphase, abort_flag, status, kStatusProducerTimeout)) break;
                load_neighbourhood_raw(t, raw_base + rs * kRawStageBytes +
                                              (uint32_t)((((bi * (p.bh + 2)) + by + 1) * pitch + bx + 2) * 8), pitch);
                if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                store_im2col_row_c4(t, a_base + stage * kATileBytes, row);
                mbar_arrive(rempty0 + 8u * rs);   // after the stores: the loads above have all returned
            } else {
                const int mt = tile / p.n_tiles;
                const int w0 = (mt % p.tw) * p.bw, h0 = ((mt / p.tw) % p.th) * p.bh;
                const int n0 = (mt / (p.tw * p.th)) * p.bn;
                load_neighbourhood_global(t, p.x4, n0 + bi, h0 + by, w0 + bx, p.ext_n, p.ext_h, p.ext_w);
                if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                store_im2col_row_c4(t, a_base + stage * kATileBytes, row);
            }
            fence_proxy_async_smem();             // generic-proxy stores -> visible to the MMA's async proxy
            mbar_arrive(full0 + 8u * stage);
        }
    } else if (IM2COL && warp == 0) {
        if (p.raw_ring) {                                  // raw producer: the tile's pixels plus halo, one box per tile
            const uint32_t raw_bytes = (uint32_t)((p.bw + 4) * (p.bh + 2) * p.bn * 8);
            uint32_t rs = 0, rphase = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int mt = tile / p.n_tiles;
                const int w0 = (mt % p.tw) * p.bw, h0 = ((mt / p.tw) % p.th) * p.bh;
                const int n0 = (mt / (p.tw * p.th)) * p.bn;
                if (!mbar_wait_relaxed(rempty0 + 8u * rs, rphase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                if (lane == 0) {
                    mbar_expect_tx(rfull0 + 8u * rs, raw_bytes);
                    tma_load_3d(raw_base + rs * kRawStageBytes, &tm_in, rfull0 + 8u * rs, w0 - 2, h0 - 1, n0);
                }
                __syncwarp();
                if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
            }
        }
    } else if (!IM2COL && (warp == 0 || (warp == 3 && conv3x3_a_producers<NT>() >= 2) ||
                           (warp >= 8 && conv3x3_a_producers<NT>() >= 4))) {
        {                                                  // producers A: one shifted activation box per K step,
            constexpr int kAProd = conv3x3_a_producers<NT>();      // K steps dealt out to the producer warps in turn
            const int pidx = warp == 0 ? 0 : (warp == 3 ? 1 : warp - 6);
            uint32_t stage = 0, phase = 0;
            int turn = 0;                                  // index of the producer whose K step this is
            bool ok = true;
            RT_DECL;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int mt = tile / p.n_tiles;
                const int w0 = (mt % p.tw) * p.bw, h0 = ((mt / p.tw) % p.th) * p.bh;
                const int n0 = (mt / (p.tw * p.th)) * p.bn;
                const int wi0 = w0 * p.step - 1, hi0 = h0 * p.step - 1;
                for (int tap = 0; tap < p.taps && ok; ++tap) {
                        const int s = (int)((p.tap_offsets >> (4 * tap)) & 3ull), r = (int)((p.tap_offsets >> (4 * tap + 2)) & 3ull);
                        for (int slice = 0; slice < p.cin_slices; ++slice) {
                            if (kAProd == 1 || turn == pidx) {
                                RT_ADD(1);
                                ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status,
                                               kStatusProducerTimeout);
                                RT_ADD(0);
                                if (!ok) break;
                                const uint32_t fb = full0 + 8u * stage;
                                if (lane == 0) {
                                    mbar_expect_tx(fb, kATileBytes);
                                    tma_load_4d(a_base + stage * kATileBytes, &tm_in, fb, slice * 64, wi0 + s, hi0 + r, n0);
                                }
                                __syncwarp();
                            }
                            if (kAProd > 1 && ++turn == kAProd) turn = 0;
                            if (++stage == kStages) { stage = 0; phase ^= 1u; }
                        }
                }
            }
            RT_ADD(1);
            if (lane == 0 && warp == 0) RT_STORE(0);
        }
    } else if (warp == 2 || (conv3x3_b_split<NT, IM2COL>() == 2 && warp == 8)) {
        {                                                  // producer(s) B: one filter tile per K step; the 256-row
            constexpr int kSplit = conv3x3_b_split<NT, IM2COL>();   // tile is fetched as two boxes by two warps
            constexpr uint32_t kBoxBytes = L::kBTileBytes / kSplit;
            const int half = warp == 2 ? 0 : 1;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int n_off = (tile % p.n_tiles) * NT + half * (NT / kSplit);
                for (int tap = 0; tap < p.taps && ok; ++tap)
                    for (int slice = 0; slice < p.cin_slices; ++slice) {
                        ok = mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout);
                        if (!ok) break;
                        const uint32_t fb = full0 + 8u * stage;
                        if (lane == 0) {
                            mbar_expect_tx(fb, kBoxBytes);
                            const uint32_t dst = b_base + stage * L::kBTileBytes + (uint32_t)half * kBoxBytes;
                            if (p.b_tap_is_dim1)
                                tma_load_3d(dst, &tm_w, fb, slice * 64, tap, n_off);
                            else
                                tma_load_3d(dst, &tm_w, fb, slice * 64, n_off, tap);
                        }
                        __syncwarp();
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
            }
        }
    } else if (warp == 1) {
        {                                                  // MMA issuer
            constexpr uint32_t idesc = idesc_f16(128, NT, false, false) | (BF16 ? idesc_ab_bf16() : 0u);
            // one thread runs the whole loop; per K step: wait, fence, two descriptor adds, four MMAs, commit
            if (lane == 0) {
                const uint64_t a_desc0 = smem_desc_sw128(a_base, 16, 1024), b_desc0 = smem_desc_sw128(b_base, 16, 1024);
                uint32_t stage = 0, phase = 0;
                uint64_t a_desc = a_desc0, b_desc = b_desc0;           // descriptors of the current stage
                bool ok = true;
                int iter = 0;
                // the barrier of the next K step is probed before the MMAs of the current one are issued
                bool ready = false;
                RT_DECL;
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++iter) {
                    const int acc = iter & 1;
                    RT_ADD(2);
                    ok = mbar_wait(tempty_bar(acc), (((uint32_t)iter >> 1) & 1u) ^ 1u, abort_flag, status,
                                   kStatusMmaTimeout);
                    RT_ADD(0);
                    if (!ok) break;
                    const uint32_t d_tmem = tmem_base + (uint32_t)(acc * NT);
                    uint32_t accumulate = 0;
                    for (int ks = 0; ks < ksteps; ++ks) {
                        RT_ADD(2);
                        if (!ready) {
                            ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
                            if (!ok) break;
                        }
                        RT_ADD(1);
                        const uint32_t cur = stage;
                        const uint64_t a_cur = a_desc, b_cur = b_desc;
                        if (++stage == kStages) {
                            stage = 0; phase ^= 1u; a_desc = a_desc0; b_desc = b_desc0;
                        } else {
                            a_desc += (uint64_t)(kATileBytes >> 4); b_desc += (uint64_t)(L::kBTileBytes >> 4);
                        }
                        ready = mbar_test_wait(full0 + 8u * stage, phase);
                        tc_fence_after();
                        umma_f16_x4<2>(d_tmem, a_cur, b_cur, idesc, accumulate);
                        umma_commit(empty0 + 8u * cur);
                        accumulate = 1u;
                    }
                    if (ok) umma_commit(tfull_bar(acc));
                }
                RT_ADD(2);
                RT_STORE(1);
            }
            __syncwarp();
        }
    } else if ((warp >= 4 && warp < 8) || (kEpiGroups == 2 && warp >= 16)) {
        // epilogue: warp w may touch TMEM lanes [32*(w%4), +32).  Group eg takes the block's tiles eg, eg + kEpiGroups, ...
        const int eg = (kEpiGroups == 2 && warp >= 16) ? 1 : 0;
        const int et = (int)threadIdx.x - (eg ? 512 : 128);     // thread of the group
        const int bar_a = 1 + 2 * eg, bar_b = 2 + 2 * eg;        // the group's named barriers
        const int q = warp & 3;
        const int row = q * 32 + lane;             // pixel of the tile = TMEM lane
        const bool leader = et == 0;               // first thread of the group issues its TMA stores
        int iter = eg;
        int chunk_count = 0;
        // STATS: thread (16-byte column st_cc, row group st_rg) adds its 8 channels of every 64-channel
        // chunk over 8 rows of the half-rounded tile in shared memory; the sums run over all tiles of
        // this block and meet once, in row-group order, when the block is done
        const int st_cc = et & 7, st_rg = et >> 3;
        float run_s[NT / 64][8], run_q[NT / 64][8];
#pragma unroll
        for (int i = 0; i < NT / 64; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) { run_s[i][e] = 0.f; run_q[i][e] = 0.f; }
        RT_DECL;
        for (int tile = blockIdx.x + eg * gridDim.x; tile < total_tiles; tile += kEpiGroups * gridDim.x, iter += kEpiGroups) {
            const int acc = iter & 1;
            const int nt = tile % p.n_tiles, mt = tile / p.n_tiles;
            const int w0 = (mt % p.tw) * p.bw, h0 = ((mt / p.tw) % p.th) * p.bh;
            const int n0 = (mt / (p.tw * p.th)) * p.bn;
            RT_ADD(2);
            if (STATS && p.has_padding) {
                // row = ((image * bh) + y) * bw + x inside the tile's box
                const int bx = row & (p.bw - 1), by = (row >> p.lbw) & (p.bh - 1), bi = row >> (p.lbw + p.lbh);
                const bool real = (w0 + bx < p.ext_w) && (h0 + by < p.ext_h) && (n0 + bi < p.ext_n);
                const uint32_t m = __ballot_sync(0xffffffffu, real);
                if (lane == 0) s_valid[eg][q] = m;
            }
            if (!mbar_wait_relaxed(tfull_bar(acc), ((uint32_t)iter >> 1) & 1u, abort_flag, status, kStatusEpilogueTimeout))
                s_epi_fail[eg] = 1;
            // the 128 threads of the group must take the same decision: they meet at named barriers below
            named_barrier(bar_b, kEpiThreads);
            RT_ADD(0);
            if (*(volatile int*)&s_epi_fail[eg]) break;
            tc_fence_after();
            uint32_t vm = 0xffu;      // which of this thread's 8 rows are real pixels
            if (STATS && p.has_padding) vm = (s_valid[eg][st_rg >> 2] >> ((st_rg & 3) * 8)) & 0xffu;
#pragma unroll
            for (int chunk = 0; chunk < NT / 64; ++chunk, ++chunk_count) {
                // one group: two staging buffers in turn; two groups: one buffer each
                const uint32_t buf = epi_base + (uint32_t)(kEpiGroups == 2 ? eg : (chunk_count & 1)) * kATileBytes;
                RT_ADD(2);
                if (leader) {                              // the store that last read this buffer is done
                    if (kEpiGroups == 2) tma_store_wait_read<0>();
                    else tma_store_wait_read<1>();
                }
                named_barrier(bar_a, kEpiThreads);
                RT_ADD(1);
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * NT + chunk * 64);
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(taddr, v0);
                tmem_ld_32x32(taddr + 32, v1);
                tmem_ld_wait();
                // 64 floats -> 64 halfs = eight 16-byte pieces of this pixel's 128-byte row,
                // stored with the 128-byte swizzle the output tensor map expects
                const uint32_t row_addr = buf + (uint32_t)row * 128u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t* src = j < 4 ? &v0[j * 8] : &v1[(j - 4) * 8];
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pk[e] = pack2_t<BF16>(__uint_as_float(src[2 * e]), __uint_as_float(src[2 * e + 1]));
                    }
                    const uint32_t dst = row_addr + (uint32_t)((j ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]),
                                 "r"(pk[2]), "r"(pk[3])
                                 : "memory");
                }
                fence_proxy_async_smem();
                named_barrier(bar_a, kEpiThreads);
                if (leader) {
                    tma_store_4d(&tm_out, buf, nt * NT + chunk * 64, w0, h0, n0);
                    tma_store_commit();
                }
                if (STATS) {
                    RT_ADD(2);
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
                    RT_ADD(3);
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
        }
        if (leader) tma_store_wait_all();
        if (STATS) {
            // the row groups meet through the (now idle) output staging buffers: red[rg][sum | sumsq][NT], one buffer
            // per epilogue group.  Every epilogue thread reaches these barriers, also after a failed wait.
            named_barrier(bar_a, kEpiThreads);
            float* red = reinterpret_cast<float*>(smem_dyn + (epi_base - smem_u32(smem_dyn))) +
                         (kEpiGroups == 2 ? (size_t)eg * (kATileBytes / 4) : 0);
            static_assert(kEpiGroups == 1 || 16 * 2 * NT * 4 <= kATileBytes, "a group's sums fit its staging buffer");
#pragma unroll
            for (int i = 0; i < NT / 64; ++i) {
                float4* ds = reinterpret_cast<float4*>(red + (st_rg * 2) * NT + i * 64 + st_cc * 8);
                float4* dq = reinterpret_cast<float4*>(red + (st_rg * 2 + 1) * NT + i * 64 + st_cc * 8);
                ds[0] = make_float4(run_s[i][0], run_s[i][1], run_s[i][2], run_s[i][3]);
                ds[1] = make_float4(run_s[i][4], run_s[i][5], run_s[i][6], run_s[i][7]);
                dq[0] = make_float4(run_q[i][0], run_q[i][1], run_q[i][2], run_q[i][3]);
                dq[1] = make_float4(run_q[i][4], run_q[i][5], run_q[i][6], run_q[i][7]);
            }
            if (kEpiGroups == 2) named_barrier(5, 2 * kEpiThreads);     // both groups' sums are in place
            else named_barrier(bar_a, kEpiThreads);
            const bool failed = *(volatile int*)&s_epi_fail[0] || *(volatile int*)&s_epi_fail[1];
            // this block only ever sees one N tile (the grid is a multiple of n_tiles)
            const int strip = blockIdx.x / p.n_tiles;
            const int ch0 = (blockIdx.x % p.n_tiles) * NT;
            if (eg == 0 && !failed) {
                const float* red0 = reinterpret_cast<const float*>(smem_dyn + (epi_base - smem_u32(smem_dyn)));
                for (int ch = et; ch < NT; ch += kEpiThreads) {
                    float s1 = 0.f, s2 = 0.f;
#pragma unroll
                    for (int gq = 0; gq < kEpiGroups; ++gq) {
                        const float* rg = red0 + (size_t)gq * (kATileBytes / 4);
#pragma unroll
                        for (int g = 0; g < 16; ++g) {
                            s1 += rg[(g * 2) * NT + ch];
                            s2 += rg[(g * 2 + 1) * NT + ch];
                        }
                    }
                    p.stats_partial[((size_t)strip * 2) * p.cout + ch0 + ch] = s1;
                    p.stats_partial[((size_t)strip * 2 + 1) * p.cout + ch0 + ch] = s2;
                }
            }
        }
        RT_ADD(2);
        if (leader) RT_STORE(2);
    }

    abort_drain(abort_flag);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// The kernels proper: one instantiation of the body per storage type, the half one under the plain name.  The
// 4-channel first-layer variant (IM2COL) is built for half only.
template <int NT, bool STATS, bool IM2COL>
__global__ void __launch_bounds__(conv3x3_threads<NT, IM2COL>(), 1)
conv3x3_igemm_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                     const __grid_constant__ CUtensorMap tm_out, const FpropParams p, int* status) {
    conv3x3_igemm_body<NT, STATS, IM2COL, false>(tm_in, tm_w, tm_out, p, status);
}

template <int NT, bool STATS>
__global__ void __launch_bounds__(conv3x3_threads<NT, false>(), 1)
conv3x3_igemm_kernel_bf16(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_w,
                          const __grid_constant__ CUtensorMap tm_out, const FpropParams p, int* status) {
    conv3x3_igemm_body<NT, STATS, false, true>(tm_in, tm_w, tm_out, p, status);
}

// Filter view for dgrad: out[tap'][c][k] = W[k][taps - 1 - tap'][c], i.e. the filter turned by 180 degrees
// (3x3: W[k][2 - tap'/3][2 - tap'%3][c]; 1x1: the transpose).
__global__ void __launch_bounds__(256)
dgrad_filter_view_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ out, int kk, int cc, int taps) {
    const int total = taps * kk * cc;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % kk, c = (i / kk) % cc, tap = i / (kk * cc);
        out[i] = w[((int64_t)k * taps + (taps - 1 - tap)) * cc + c];
    }
}

// persistent grid: one block per SM, a multiple of n_tiles so that a block keeps its N tile
int conv3x3_grid(int m_tiles, int n_tiles) {
    const int total = m_tiles * n_tiles;
    int grid = total < sm_count() ? total : sm_count();
    if (grid > n_tiles) grid = grid / n_tiles * n_tiles;
    return grid;
}

template <int NT, bool STATS, bool IM2COL>
int launch_conv3x3(const CUtensorMap& tin, const CUtensorMap& tw, const CUtensorMap& tout, const FpropParams& p,
                   cudaStream_t st, bool bf16) {
    using L = FpropSmem<NT, IM2COL>;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_igemm_kernel<NT, STATS, IM2COL>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        if constexpr (!IM2COL)
            TRB_CUDA_TRY(cudaFuncSetAttribute(conv3x3_igemm_kernel_bf16<NT, STATS>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = conv3x3_grid(p.m_tiles, p.n_tiles);
    if constexpr (!IM2COL) {
        if (bf16) {
            conv3x3_igemm_kernel_bf16<NT, STATS><<<grid, conv3x3_threads<NT, false>(), L::kTotal, st>>>(tin, tw, tout, p,
                                                                                                      status);
            TRB_LAUNCH_CHECK("conv3x3_igemm_kernel_bf16");
            return TRB200_OK;
        }
    }
    TRB_REQUIRE(!bf16, TRB200_ERR_UNSUPPORTED, "conv3x3 igemm: the 4-channel variant is built for half tensors only");
    conv3x3_igemm_kernel<NT, STATS, IM2COL><<<grid, conv3x3_threads<NT, IM2COL>(), L::kTotal, st>>>(tin, tw, tout,
                                                                                                       p, status);
    TRB_LAUNCH_CHECK("conv3x3_igemm_kernel");
    return TRB200_OK;
}

template <int NT>
int launch_conv3x3_any(const CUtensorMap& tin, const CUtensorMap& tw, const CUtensorMap& tout, const FpropParams& p,
                       cudaStream_t st, bool bf16) {
    const bool stats = p.stats_partial != nullptr, im2col = p.x4 != nullptr;
    if (stats && im2col) return launch_conv3x3<NT, true, true>(tin, tw, tout, p, st, bf16);
    if (stats) return launch_conv3x3<NT, true, false>(tin, tw, tout, p, st, bf16);
    if (im2col) return launch_conv3x3<NT, false, true>(tin, tw, tout, p, st, bf16);
    return launch_conv3x3<NT, false, false>(tin, tw, tout, p, st, bf16);
}

int pick_nt(int cout) {
    if (cout % 256 == 0) return 256;
    if (cout == 128) return 128;
    if (cout == 64) return 64;
    return 0;
}

// in: [n,h,w,cin] half; filter view described by (wv, tap_is_dim1); out: [n,h,w,cout] half.
// stats_partial != nullptr: also leave per-strip sums / sums of squares of the (half) output there and report
// the number of strips through *stats_strips.
// x4 != nullptr: `in` is ignored, the A tiles are built in the kernel from the 4-channel image x4 (taps must be 1,
// cin 64: the 36 neighbourhood values + 28 zeros).
// What a convolution that is not the plain stride-1 case adds (h, w of conv3x3_run are then the output grid):
struct ConvRunEx {
    int step = 1;                          // input pixels per output pixel; the input is [n, in_h, in_w, cin]
    int in_h = 0, in_w = 0;
    unsigned long long tap_offsets = 0;    // 0: the 3x3 window (or the centre tap) around the output pixel
    int parity = -1;                       // py * 2 + px: the output grid is that parity class of [n, full_h, full_w, cout]
    int full_h = 0, full_w = 0;
};

constexpr unsigned long long kTapOffsets3x3 = 0xa98654210ull;     // tap = r * 3 + s: nibble s | r << 2
constexpr unsigned long long kTapOffsets1x1 = 0x5ull;

int conv3x3_run(const void* in, const void* wv, int tap_is_dim1, void* out, int n, int h, int w, int cin, int cout,
                cudaStream_t st, int taps = 9, float* stats_partial = nullptr, int* stats_strips = nullptr,
                const void* x4 = nullptr, bool bf16 = false, const ConvRunEx* ex = nullptr) {
    const int nt = pick_nt(cout);
    TRB_REQUIRE(nt != 0 && cin % 64 == 0, TRB200_ERR_UNSUPPORTED, "conv3x3 igemm: cin=%d cout=%d not covered", cin,
                cout);
    const TileShape t = pick_tile(n, h, w, 128);
    CUtensorMap tin, tw, tout;
    int rc;
    if (ex && ex->parity >= 0)
        rc = make_act_tmap_parity(&tout, out, n, ex->full_h, ex->full_w, cout, ex->parity >> 1, ex->parity & 1, t,
                                  "conv output (parity class)");
    else
        rc = make_act_tmap(&tout, out, n, h, w, cout, t, "conv output");
    if (rc) return rc;
    const bool raw_ring = x4 && raw_ring_fits(t, w, x4);
    if (raw_ring) rc = make_raw_x4_tmap(&tin, x4, n, h, w, t);
    else if (x4) tin = tout;      // not used by the kernel
    else if (ex && ex->in_h) rc = make_act_tmap_stepped(&tin, in, n, ex->in_h, ex->in_w, cin, t, ex->step, "conv input");
    else rc = make_act_tmap(&tin, in, n, h, w, cin, t, "conv input");
    if (rc) return rc;
    const int b_rows = (nt == 256 && !x4) ? 128 : nt;      // rows of one filter box (the 256-row tile takes two)
    if (tap_is_dim1) {
        // KRSC as stored: (ci, tap, co)
        const uint64_t dims[3] = {(uint64_t)cin, (uint64_t)taps, (uint64_t)cout};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)taps * cin * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)b_rows};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,tap,co)");
    } else {
        const uint64_t dims[3] = {(uint64_t)cin, (uint64_t)cout, (uint64_t)taps};
        const uint64_t str[3] = {2, (uint64_t)cin * 2, (uint64_t)cout * cin * 2};
        const uint32_t box[3] = {64, (uint32_t)b_rows, 1};
        rc = make_tmap(&tw, wv, 3, dims, str, box, "filters (ci,co,tap)");
    }
    if (rc) return rc;
    FpropParams p;
    p.taps = taps;
    p.tap_base = taps == 1 ? 4 : 0;
    p.step = ex ? ex->step : 1;
    p.tap_offsets = (ex && ex->tap_offsets) ? ex->tap_offsets : (taps == 9 ? kTapOffsets3x3 : kTapOffsets1x1);
    p.cin_slices = cin / 64;
    p.n_tiles = cout / nt;
    p.m_tiles = t.tw * t.th * t.tn;
    p.tw = t.tw; p.th = t.th;
    p.bw = t.bw; p.bh = t.bh; p.bn = t.bn;
    p.b_tap_is_dim1 = tap_is_dim1;
    p.stats_partial = stats_partial;
    p.x4 = static_cast<const uint2*>(x4);
    p.raw_ring = raw_ring ? 1 : 0;
    p.cout = cout;
    p.lbw = 0; p.lbh = 0;
    while ((1 << p.lbw) < t.bw) ++p.lbw;
    while ((1 << p.lbh) < t.bh) ++p.lbh;
    p.ext_w = w; p.ext_h = h; p.ext_n = n;
    p.has_padding = (t.tw * t.bw != w) || (t.th * t.bh != h) || (t.tn * t.bn != n);
    if (stats_partial && stats_strips) *stats_strips = conv3x3_grid(p.m_tiles, p.n_tiles) / p.n_tiles;
    if (nt == 256) return launch_conv3x3_any<256>(tin, tw, tout, p, st, bf16);
    if (nt == 128) return launch_conv3x3_any<128>(tin, tw, tout, p, st, bf16);
    return launch_conv3x3_any<64>(tin, tw, tout, p, st, bf16);
}

// upper bound of the strips the STATS kernels write for an output of `cout` channels
int conv3x3_stats_max_strips() { return sm_count(); }

#include "conv_pixn_sm100.cuh"
#include "conv_halo_pair_sm100.cuh"

// 64 / 128 channels on both sides go to the CTA-pair kernel with the resident filters, other layers with 64 / 128
// output channels to the kernel with the pixels on N (development builds can switch either off)
int conv3x3_any_run(const void* in, const void* wv, int tap_is_dim1, void* out, int n, int h, int w, int cin, int cout,
                    cudaStream_t st, float* stats_partial = nullptr, int* stats_strips = nullptr, bool bf16 = false,
                    int taps = 9) {
#ifndef TRB200_NO_HALO_PAIR
    if (halo_pair_preferred(cin, cout, taps))
        return conv3x3_halo_pair_run(in, wv, tap_is_dim1, out, n, h, w, cin, cout, st, stats_partial, stats_strips, bf16);
#endif
#ifndef TRB200_NO_PIXN
    // 1x1: the channels-on-N kernel (TMA-store epilogue) is the faster one: 0.043 against 0.060 ms at 256x56x56, 64 -> 64
    if (pixn_preferred(cin, cout) && taps != 1)
        return conv3x3_pixn_run(in, wv, tap_is_dim1, out, n, h, w, cin, cout, st, stats_partial, stats_strips, bf16,
                                taps);
#endif
    return conv3x3_run(in, wv, tap_is_dim1, out, n, h, w, cin, cout, st, taps, stats_partial, stats_strips, nullptr,
                       bf16);
}

// ------------------------------------------------------------------ wgrad kernel
struct WgradParams {
    int taps;           // 9 (3x3, pad 1) or 1 (1x1)
    int tap_base;       // 0 for 3x3; 4 for 1x1 (centre tap)
    int step;           // pixels of x per pixel of dy (1, or 2 for a stride-2 convolution)
    int cblocks;        // C / 64
    int units;          // taps * cblocks  (unit u: tap = u / cblocks, cblock = u % cblocks)
    int m_tiles;        // ceil(units / 2)
    int n_tiles;        // K / NT
    int splits;
    int pix_tiles;      // tw * th * tn
    int tw, th;
    int bw, bh, bn;
    const uint2* x4;    // IM2COL kernels: the 4-channel input image; A tiles are built in the kernel
    int raw_ring;       // IM2COL kernels: tm_x describes x4 and halo tiles go through the raw ring
    int lbw, lbh;       // log2 of bw, bh
    int ext_w, ext_h, ext_n;
    int bf16;           // operands and dW are bfloat16 instead of half
};

template <int NT, bool IM2COL = false>
struct WgradSmem {
    // two units; the first-layer variant has a single unit, stored once: the descriptor's block offset of 0 makes the
    // second 64-row block of the M = 128 operand read the same tile
    static constexpr int kABytes = (IM2COL ? 1 : 2) * kStageTileBytes;
    static constexpr int kBBytes = (NT / 64) * kStageTileBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kRawBytes = IM2COL ? kRawStages * kRawStageBytes : 0;
    static constexpr int kStagesRaw = (kSmemBudget - 2048 - kRawBytes) / kStageBytes;
    // the first-layer builder groups take stages in turn: a ring of 8 or 4 keeps every stage with one group
    static constexpr int kStages = (IM2COL && kStagesRaw >= 12) ? 12 : (kStagesRaw >= 8 ? 8 : (IM2COL && kStagesRaw >= 4 ? 4 : kStagesRaw));
    static constexpr int kTotal = kStages * kStageBytes + kRawBytes + 2048;
};

// IM2COL: 8 more warps (four groups of 64 threads) build the A tiles (one unit, read twice by the MMA) from the 4-channel image.
template <int NT, bool IM2COL>
__global__ void __launch_bounds__(IM2COL ? kThreads + kBuilderThreads : kThreads, 1)
wgrad_igemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                   float* __restrict__ partial, const WgradParams p, int* status) {
    using L = WgradSmem<NT, IM2COL>;
    constexpr int kStages = L::kStages;
    constexpr int kBBlocks = NT / 64;                       // 64-channel boxes of dy per stage
    constexpr int kBProducers = kBBlocks >= 2 ? 2 : 1;
    // first-layer variant: a stage is only 64 pixels x 128 bytes of dy, and one thread issues four MMAs, a commit and a
    // wait per stage at about the rate HBM delivers the stages; two issuing warps on alternate stages, each with its
    // own accumulator (added up in the epilogue), lift that ceiling
    constexpr int kIssuers = (IM2COL && kBProducers == 1) ? 2 : 1;      // warp 3 is free when one warp loads dy
    static_assert(kStages % kIssuers == 0, "a stage keeps its issuer");
    constexpr uint32_t kTmemCols = (NT < 32 ? 32 : NT) * kIssuers;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_base = base;
    const uint32_t b_base = base + kStages * L::kABytes;
    const uint32_t raw_base = b_base + kStages * L::kBBytes;
    const uint32_t bar_base = raw_base + L::kRawBytes;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * kStages;
    const uint32_t done_bar = bar_base + 8u * (2 * kStages);
    const uint32_t rfull0 = done_bar + 8u, rempty0 = rfull0 + 8u * kRawStages;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8u * s, (IM2COL ? 64 : 1) + kBProducers);
            mbar_init(empty0 + 8u * s, 1);
        }
        mbar_init(done_bar, kIssuers);
        if (IM2COL)
            for (int s = 0; s < kRawStages; ++s) { mbar_init(rfull0 + 8u * s, 1); mbar_init(rempty0 + 8u * s, 64); }
        fence_barrier_init();
        if (!IM2COL || p.raw_ring) prefetch_tmap(&tm_x);
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

    // work item -> (split, m tile, n tile)
    const int item = blockIdx.x;
    const int nt = item % p.n_tiles;
    const int mt = (item / p.n_tiles) % p.m_tiles;
    const int split = item / (p.n_tiles * p.m_tiles);
    const int pt0 = (int)((long)p.pix_tiles * split / p.splits);
    const int pt1 = (int)((long)p.pix_tiles * (split + 1) / p.splits);
    // pixel tiles are walked with running box origins (w fastest, then h, then n)
    const int w_first = (pt0 % p.tw) * p.bw, h_first = ((pt0 / p.tw) % p.th) * p.bh;
    const int n_first = (pt0 / (p.tw * p.th)) * p.bn;
    const int w_end = p.tw * p.bw, h_end = p.th * p.bh;

    if (IM2COL && warp >= 8) {
        // A-tile builders: thread = one of the stage's 64 pixels; both 64-row halves of the M = 128
        // operand read the same rows (there is a single (tap, channel) unit)
        // group g takes the block's stages g, g + 4, ...
        constexpr int kGroups = kBuilderThreads / 64;
        static_assert(!IM2COL || kStages % kGroups == 0, "a stage keeps its builder group");
        const int row = (threadIdx.x - kThreads) & 63, group = (threadIdx.x - kThreads) >> 6;
        const int bx = row & (p.bw - 1), by = (row >> p.lbw) & (p.bh - 1), bi = row >> (p.lbw + p.lbh);
        int w0 = w_first, h0 = h_first, n0 = n_first;
        for (int pt = pt0; pt < pt1; ++pt) {
            const int it = pt - pt0;
            if (it % kGroups == group) {
                const uint32_t stage = (uint32_t)(it % kStages), phase = (uint32_t)((it / kStages) & 1);
                const uint32_t a_dst = a_base + stage * L::kABytes;
                uint2 t[10];
                if (p.raw_ring) {
                    const uint32_t rs = (uint32_t)(it % kRawStages), rphase = (uint32_t)((it / kRawStages) & 1);
                    const int pitch = p.bw + 4;
                    if (!mbar_wait_relaxed(rfull0 + 8u * rs, rphase, abort_flag, status, kStatusProducerTimeout)) break;
                    load_neighbourhood_raw(t, raw_base + rs * kRawStageBytes +
                                                  (uint32_t)((((bi * (p.bh + 2)) + by + 1) * pitch + bx + 2) * 8), pitch);
                } else {
                    load_neighbourhood_global(t, p.x4, n0 + bi, h0 + by, w0 + bx, p.ext_n, p.ext_h, p.ext_w);
                }
                if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                store_im2col_row_c4(t, a_dst, row);
                if (p.raw_ring) mbar_arrive(rempty0 + 8u * (uint32_t)(it % kRawStages));
                fence_proxy_async_smem();
                mbar_arrive(full0 + 8u * stage);
            }
            w0 += p.bw;
            if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
        }
    } else if (IM2COL && warp == 0) {
        if (p.raw_ring) {                                  // raw producer: the stage's pixels plus halo, one box per stage
            const uint32_t raw_bytes = (uint32_t)((p.bw + 4) * (p.bh + 2) * p.bn * 8);
            uint32_t rs = 0, rphase = 0;
            int w0 = w_first, h0 = h_first, n0 = n_first;
            for (int pt = pt0; pt < pt1; ++pt) {
                if (!mbar_wait_relaxed(rempty0 + 8u * rs, rphase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                if (lane == 0) {
                    mbar_expect_tx(rfull0 + 8u * rs, raw_bytes);
                    tma_load_3d(raw_base + rs * kRawStageBytes, &tm_x, rfull0 + 8u * rs, w0 - 2, h0 - 1, n0);
                }
                __syncwarp();
                if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
                w0 += p.bw;
                if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
            }
        }
    } else if (warp == 0 && !IM2COL) {
        {                                                  // producer A: two tap-shifted boxes of x per stage
            const int u0 = mt * 2;
            const int u1 = (u0 + 1 < p.units) ? u0 + 1 : u0;   // odd unit count: the last tile repeats its unit
            const int tap0 = u0 / p.cblocks + p.tap_base, c0 = (u0 % p.cblocks) * 64;
            const int tap1 = u1 / p.cblocks + p.tap_base, c1 = (u1 % p.cblocks) * 64;
            const int dw0 = tap0 % 3 - 1, dh0 = tap0 / 3 - 1, dw1 = tap1 % 3 - 1, dh1 = tap1 / 3 - 1;
            uint32_t stage = 0, phase = 0;
            int w0 = w_first, h0 = h_first, n0 = n_first;
            for (int pt = pt0; pt < pt1; ++pt) {
                if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                const uint32_t fb = full0 + 8u * stage;
                const uint32_t a_dst = a_base + stage * L::kABytes;
                if (lane == 0) {
                    mbar_expect_tx(fb, L::kABytes);
                    tma_load_4d(a_dst, &tm_x, fb, c0, w0 * p.step + dw0, h0 * p.step + dh0, n0);
                    tma_load_4d(a_dst + kStageTileBytes, &tm_x, fb, c1, w0 * p.step + dw1, h0 * p.step + dh1, n0);
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                w0 += p.bw;
                if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
            }
        }
    } else if (warp == 2 || (warp == 3 && kBProducers == 2)) {
        {                                                  // producers B: the stage's boxes of dy, split over two warps
            constexpr int kPer = kBBlocks / kBProducers;
            const int j0 = (warp - 2) * kPer;
            const int k_off = nt * NT + j0 * 64;
            uint32_t stage = 0, phase = 0;
            int w0 = w_first, h0 = h_first, n0 = n_first;
            for (int pt = pt0; pt < pt1; ++pt) {
                if (!mbar_wait_relaxed(empty0 + 8u * stage, phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) break;
                const uint32_t fb = full0 + 8u * stage;
                const uint32_t b_dst = b_base + stage * L::kBBytes + j0 * kStageTileBytes;
                if (lane == 0) {
                    mbar_expect_tx(fb, kPer * kStageTileBytes);
#pragma unroll
                    for (int j = 0; j < kPer; ++j)
                        tma_load_4d(b_dst + j * kStageTileBytes, &tm_dy, fb, k_off + j * 64, w0, h0, n0);
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                w0 += p.bw;
                if (w0 >= w_end) { w0 = 0; h0 += p.bh; if (h0 >= h_end) { h0 = 0; n0 += p.bn; } }
            }
        }
    } else if (warp == 1 || (kIssuers == 2 && warp == 3)) {
        {                                                  // MMA issuer(s): issuer i takes stages i, i + kIssuers, ...
            const int issuer = warp == 1 ? 0 : 1;
            const uint32_t idesc = idesc_f16(128, NT, true, true) | (p.bf16 ? idesc_ab_bf16() : 0u);
            // MN-major: 64-element blocks of M/N are one 8 KB tile apart, 8 pixels are 1024 bytes apart
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(a_base, IM2COL ? 0 : kStageTileBytes), b_lo0 = smem_desc_lo(b_base, kStageTileBytes);
            const uint32_t d_tmem = tmem_base + (uint32_t)(issuer * NT);
            uint32_t stage = (uint32_t)issuer, phase = 0;
            uint32_t accumulate = 0;
            bool ok = true;
            for (int pt = pt0 + issuer; pt < pt1; pt += kIssuers) {
                ok = mbar_wait(full0 + 8u * stage, phase, abort_flag, status, kStatusMmaTimeout);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + stage * (L::kABytes >> 4);
                const uint32_t b_lo = b_lo0 + stage * (L::kBBytes >> 4);
                // 4 x (K = 16 pixels = 2048 bytes: +128 in the address field)
                if (lane == 0) {
                    umma_f16_lohi(d_tmem, a_lo, desc_hi, b_lo, desc_hi, idesc, accumulate);
                    umma_f16_lohi(d_tmem, a_lo + 128, desc_hi, b_lo + 128, desc_hi, idesc, 1u);
                    umma_f16_lohi(d_tmem, a_lo + 256, desc_hi, b_lo + 256, desc_hi, idesc, 1u);
                    umma_f16_lohi(d_tmem, a_lo + 384, desc_hi, b_lo + 384, desc_hi, idesc, 1u);
                    umma_commit(empty0 + 8u * stage);
                }
                __syncwarp();
                accumulate = 1u;
                stage += kIssuers;
                if (stage >= (uint32_t)kStages) { stage -= kStages; phase ^= 1u; }
            }
            if (ok && lane == 0) umma_commit(done_bar);
            __syncwarp();
        }
    } else if (warp >= 4 && warp < 8) {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        float* dst = partial + ((size_t)item * 128 + row) * NT;
        if (pt1 > pt0) {
            if (mbar_wait_relaxed(done_bar, 0, abort_flag, status, kStatusEpilogueTimeout)) {
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < NT; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (kIssuers == 2 && pt1 - pt0 >= 2) {     // the second issuer's accumulator (it has seen a stage)
                        uint32_t v2[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(NT + c0), v2);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(dst + c0)[j] =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                }
            }
        } else {
            for (int c0 = 0; c0 < NT; c0 += 4) *reinterpret_cast<float4*>(dst + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
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

// dW[k][tap][c] = half(sum over splits, in split order, of partial[split][mt][nt][row][col]).
// One block = 32 rows (c) x 32 cols (k) of one partial tile, transposed through
// shared memory so that both the reads (along k) and the writes (along c) coalesce.
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ dw, WgradParams p, int nt_cols, int kk,
                    int cc) {
    __shared__ float tile[32][33];
    const int mt = blockIdx.z / p.n_tiles, nt = blockIdx.z % p.n_tiles;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const size_t tile_elems = (size_t)128 * nt_cols;
    const size_t split_stride = (size_t)p.m_tiles * p.n_tiles * tile_elems;
    const size_t tile_off = ((size_t)mt * p.n_tiles + nt) * tile_elems;
    for (int rr = ty; rr < 32; rr += 8) {
        float acc = 0.f;
        const size_t off = tile_off + (size_t)(r0 + rr) * nt_cols + c0 + tx;
        for (int s = 0; s < p.splits; ++s) acc += partial[(size_t)s * split_stride + off];
        tile[rr][tx] = acc;
    }
    __syncthreads();
    const int unit = mt * 2 + r0 / 64;
    if (unit >= p.units) return;
    const int tap = unit / p.cblocks, cb = unit % p.cblocks;
    for (int cj = ty; cj < 32; cj += 8) {
        const int k = nt * nt_cols + c0 + cj;
        const int c = cb * 64 + (r0 % 64) + tx;
        dw[((size_t)k * p.taps + tap) * cc + c] = p.bf16 ? round16_t<true>(tile[tx][cj]) : round16_t<false>(tile[tx][cj]);
    }
    (void)kk;
}

template <int NT, bool IM2COL>
int launch_wgrad_t(const CUtensorMap& tx, const CUtensorMap& tdy, float* partial, const WgradParams& p, cudaStream_t st) {
    using L = WgradSmem<NT, IM2COL>;
    static bool attr_done[64] = {false};
    int dev = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        TRB_CUDA_TRY(cudaFuncSetAttribute(wgrad_igemm_kernel<NT, IM2COL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          L::kTotal));
        attr_done[dev] = true;
    }
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    const int grid = p.m_tiles * p.n_tiles * p.splits;
    wgrad_igemm_kernel<NT, IM2COL><<<grid, IM2COL ? kThreads + kBuilderThreads : kThreads, L::kTotal, st>>>(tx, tdy, partial, p, status);
    TRB_LAUNCH_CHECK("wgrad_igemm_kernel");
    return TRB200_OK;
}

template <int NT>
int launch_wgrad(const CUtensorMap& tx, const CUtensorMap& tdy, float* partial, const WgradParams& p, cudaStream_t st) {
    return p.x4 ? launch_wgrad_t<NT, true>(tx, tdy, partial, p, st) : launch_wgrad_t<NT, false>(tx, tdy, partial, p, st);
}

WgradParams wgrad_plan(const trb200_conv_desc& d, int nt, const TileShape& t, int taps = 9) {
    WgradParams p;
    p.taps = taps;
    p.tap_base = taps == 1 ? 4 : 0;
    p.step = 1;
    p.cblocks = d.c / 64;
    p.units = taps * p.cblocks;
    p.m_tiles = (p.units + 1) / 2;
    p.n_tiles = d.k / nt;
    p.pix_tiles = t.tw * t.th * t.tn;
    const int tiles = p.m_tiles * p.n_tiles;
    int splits = sm_count() / tiles;
    if (splits < 1) splits = 1;
    if (splits > p.pix_tiles) splits = p.pix_tiles;
    p.splits = splits;
    p.tw = t.tw; p.th = t.th;
    p.bw = t.bw; p.bh = t.bh; p.bn = t.bn;
    p.x4 = nullptr;
    p.raw_ring = 0;
    p.lbw = 0; p.lbh = 0;
    while ((1 << p.lbw) < t.bw) ++p.lbw;
    while ((1 << p.lbh) < t.bh) ++p.lbh;
    p.ext_w = d.w; p.ext_h = d.h; p.ext_n = d.n;
    p.bf16 = d.dtype == TRB200_DTYPE_BF16 ? 1 : 0;
    return p;
}

#include "wgrad_unitn_sm100.cuh"
#include "wgrad_halo_sm100.cuh"

// which weight-gradient kernel a layer gets: up to 128 filters the one with the units on N
// (development builds can move the limit)
#ifndef TRB200_UNITN_MAX_K
#define TRB200_UNITN_MAX_K 128
#endif
inline bool wgrad_use_unitn(const trb200_conv_desc& d) {
    return d.r == 3 && wgrad_unitn_supports(d) && d.k <= TRB200_UNITN_MAX_K;
}

#include "gemm_skinny_sm100.cuh"

// 64 -> 64 channels: the kernel that reads all nine taps from one halo copy (development builds can switch it off)
inline bool wgrad_use_halo(const trb200_conv_desc& d) {
#ifdef TRB200_NO_WGRAD_HALO
    (void)d;
    return false;
#else
    return wgrad_halo_supports(d) && d.s == 3 && d.pad_h == 1 && d.pad_w == 1 && d.stride_h == 1 && d.stride_w == 1;
#endif
}

// ------------------------------------------------------------------ first layer (C = 4)
// A 3x3 / pad 1 convolution over 4 input channels is a 1x1 convolution over the 36
// values of each pixel's 3x3 neighbourhood.  The IM2COL variants of the kernels above
// build that neighbourhood as one 128-byte operand row per pixel (36 halfs + 28 zeros)
// in shared memory, after which the forward conv and the weight gradient are plain GEMMs
// (taps = 1, 64 input channels) against filters packed to 64 columns; the zero columns
// contribute exact zeros.
// wp[k][j] = j < 36 ? w[k][j] : 0   (KRSC with c = 4 is already [k][36])
__global__ void pack_w_c4_kernel(const __half* __restrict__ w, __half* __restrict__ wp, int kk) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kk * 64) return;
    const int k = i >> 6, j = i & 63;
    wp[i] = j < 36 ? w[k * 36 + j] : __float2half_rn(0.f);
}

__global__ void unpack_dw_c4_kernel(const __half* __restrict__ dwp, __half* __restrict__ dw, int kk) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kk * 36) return;
    dw[i] = dwp[(i / 36) * 64 + i % 36];
}

}  // namespace

// ------------------------------------------------------------------ entry points of this file
static bool is_3x3_s1_p1(const trb200_conv_desc& d) {
    return d.r == 3 && d.s == 3 && d.pad_h == 1 && d.pad_w == 1 && d.stride_h == 1 && d.stride_w == 1;
}

// first-layer shape: 4 input channels, handled as a 1x1 convolution over 36 (+28 zero) values
bool igemm_small_c(const trb200_conv_desc& d) {
    return d.dtype == TRB200_DTYPE_F16 && is_3x3_s1_p1(d) && d.c == 4 && d.k % 64 == 0 && pick_nt(d.k) != 0 && d.n >= 1 && d.h >= 1 && d.w >= 1;
}

static bool is_1x1_s1_p0(const trb200_conv_desc& d) {
    return d.r == 1 && d.s == 1 && d.pad_h == 0 && d.pad_w == 0 && d.stride_h == 1 && d.stride_w == 1;
}

// filter taps of a geometry the tensor-core kernels take: 9 or 1
static int igemm_taps(const trb200_conv_desc& d) { return is_1x1_s1_p0(d) ? 1 : 9; }

bool igemm_supports(const trb200_conv_desc& d, int which) {
    if (!is_3x3_s1_p1(d) && !is_1x1_s1_p0(d)) return false;
    if (d.n < 1 || d.h < 1 || d.w < 1) return false;
    if (igemm_small_c(d)) return which != 1;      // wgrad and fprop; a first layer has no dgrad
    if (d.c % 64 != 0 || d.k % 64 != 0) return false;
    if (which == 0) return pick_nt(d.k) != 0;     // wgrad: N dimension = k
    if (which == 1) return pick_nt(d.c) != 0;     // dgrad: N dimension = c
    return pick_nt(d.k) != 0;                     // fprop: N dimension = k
}

size_t igemm_dgrad_workspace(const trb200_conv_desc& d) {
    return (size_t)align_up((int64_t)igemm_taps(d) * d.c * d.k * 2, 256);
}

static size_t wgrad_partial_bytes(const trb200_conv_desc& d, int taps) {
    const int nt = pick_nt(d.k);
    const TileShape t = pick_tile(d.n, d.h, d.w, 64);
    const WgradParams p = wgrad_plan(d, nt, t, taps);
    return (size_t)p.splits * p.m_tiles * p.n_tiles * 128 * nt * sizeof(float);
}

// small C: [packed dW (k x 64 half)][partials]
bool conv1x1_wgrad_gemm_supports(const trb200_conv_desc& d);
size_t conv1x1_wgrad_gemm_workspace(const trb200_conv_desc& d);
int conv1x1_wgrad_gemm(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, float* partial, cudaStream_t st);

size_t igemm_wgrad_workspace(const trb200_conv_desc& d) {
    if (igemm_small_c(d)) {
        trb200_conv_desc e = d;
        e.c = 64;
        return (size_t)align_up((int64_t)d.k * 64 * 2, 256) + wgrad_partial_bytes(e, 1);
    }
    if (conv1x1_wgrad_gemm_supports(d)) return conv1x1_wgrad_gemm_workspace(d);
    if (wgrad_use_halo(d)) return wgrad_halo_partial_bytes(d);
    if (wgrad_use_unitn(d)) return wgrad_unitn_partial_bytes(d);
    return wgrad_partial_bytes(d, igemm_taps(d));
}

// small C: the filters packed to 64 columns
size_t igemm_fprop_workspace(const trb200_conv_desc& d) {
    if (igemm_small_c(d)) return (size_t)align_up((int64_t)d.k * 64 * 2, 256);
    return 0;
}

int igemm_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes,
                cudaStream_t st) {
    const size_t need = igemm_dgrad_workspace(d);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, "conv_dgrad: workspace of %zu bytes needed, %zu given",
                need, ws_bytes);
    TRB_REQUIRE(aligned16(ws), TRB200_ERR_INVALID_ARGUMENT, "conv_dgrad: workspace must be 16-byte aligned");
    const int taps = igemm_taps(d);
    const int total = taps * d.k * d.c;
    int blocks = (total + 255) / 256;
    if (blocks > sm_count() * 4) blocks = sm_count() * 4;
    dgrad_filter_view_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(w), static_cast<uint16_t*>(ws), d.k,
                                                     d.c, taps);
    TRB_LAUNCH_CHECK("dgrad_filter_view_kernel");
    // in = dY [n,h,w,k], filter view (ci = k, co = c, tap), out = dX [n,h,w,c]
    return conv3x3_any_run(dy, ws, 0, dx, d.n, d.h, d.w, d.k, d.c, st, nullptr, nullptr, d.dtype == TRB200_DTYPE_BF16,
                           taps);
}

size_t igemm_fprop_stats_bytes(const trb200_conv_desc& d) {
    return (size_t)align_up((int64_t)conv3x3_stats_max_strips() * 2 * d.k * (int64_t)sizeof(float), 256);
}

// stats_partial: optional float scratch of igemm_fprop_stats_bytes(); *stats_strips receives the strip count
int igemm_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
                cudaStream_t st, float* stats_partial, int* stats_strips) {
    if (!igemm_small_c(d))
        return conv3x3_any_run(x, w, 1, y, d.n, d.h, d.w, d.c, d.k, st, stats_partial, stats_strips,
                               d.dtype == TRB200_DTYPE_BF16, igemm_taps(d));
    const size_t need = igemm_fprop_workspace(d);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, "conv_fprop: workspace of %zu bytes needed, %zu given",
                need, ws_bytes);
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv_fprop: workspace must be 256-byte aligned");
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 7u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv_fprop: a 4-channel input must be 8-byte aligned");
    __half* wp = static_cast<__half*>(ws);
    pack_w_c4_kernel<<<(d.k * 64 + 255) / 256, 256, 0, st>>>(static_cast<const __half*>(w), wp, d.k);
    TRB_LAUNCH_CHECK("pack_w_c4_kernel");
    // 1x1 convolution: filter view (ci = 64, tap = 1, co = k), operand rows built from x in the kernel
    return conv3x3_run(nullptr, wp, 1, y, d.n, d.h, d.w, 64, d.k, st, 1, stats_partial, stats_strips, x);
}

// x4 != nullptr: `x` is ignored and the operand rows are built in the kernel from the 4-channel image x4
// step > 1: d.h, d.w are the extents of dy and x is [n, x_h, x_w, c], read every step-th pixel
static int wgrad_run(const trb200_conv_desc& d, int taps, const void* dy, const void* x, void* dw, float* partial,
                     cudaStream_t st, const void* x4 = nullptr, int step = 1, int x_h = 0, int x_w = 0) {
    const int nt = pick_nt(d.k);
    const TileShape t = pick_tile(d.n, d.h, d.w, 64);
    WgradParams p = wgrad_plan(d, nt, t, taps);
    p.step = step;
    p.x4 = static_cast<const uint2*>(x4);
    p.raw_ring = (x4 && raw_ring_fits(t, d.w, x4)) ? 1 : 0;
    CUtensorMap tx, tdy;
    int rc = make_act_tmap(&tdy, dy, d.n, d.h, d.w, d.k, t, "wgrad dy");
    if (rc) return rc;
    if (p.raw_ring) rc = make_raw_x4_tmap(&tx, x4, d.n, d.h, d.w, t);
    else if (x4) tx = tdy;      // not used by the kernel
    else if (step > 1) rc = make_act_tmap_stepped(&tx, x, d.n, x_h, x_w, d.c, t, step, "wgrad x");
    else rc = make_act_tmap(&tx, x, d.n, d.h, d.w, d.c, t, "wgrad x");
    if (rc) return rc;
    if (nt == 256) rc = launch_wgrad<256>(tx, tdy, partial, p, st);
    else if (nt == 128) rc = launch_wgrad<128>(tx, tdy, partial, p, st);
    else rc = launch_wgrad<64>(tx, tdy, partial, p, st);
    if (rc) return rc;
    dim3 grid(nt / 32, 4, p.m_tiles * p.n_tiles);
    wgrad_reduce_kernel<<<grid, 256, 0, st>>>(partial, static_cast<uint16_t*>(dw), p, nt, d.k, d.c);
    TRB_LAUNCH_CHECK("wgrad_reduce_kernel");
    return TRB200_OK;
}

// Small-C weight gradient.  ws: [packed dW (k x 64 half)][partials].
static int igemm_wgrad_small_c(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws,
                               cudaStream_t st) {
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 7u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv_wgrad: a 4-channel input must be 8-byte aligned");
    unsigned char* base = static_cast<unsigned char*>(ws);
    __half* dwp = reinterpret_cast<__half*>(base);
    float* partial = reinterpret_cast<float*>(base + align_up((int64_t)d.k * 64 * 2, 256));
    trb200_conv_desc e = d;
    e.c = 64;
    const int rc = wgrad_run(e, 1, dy, nullptr, dwp, partial, st, x);
    if (rc) return rc;
    unpack_dw_c4_kernel<<<(d.k * 36 + 255) / 256, 256, 0, st>>>(dwp, static_cast<__half*>(dw), d.k);
    TRB_LAUNCH_CHECK("unpack_dw_c4_kernel");
    return TRB200_OK;
}

int igemm_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
                cudaStream_t st) {
    const int nt = pick_nt(d.k);
    TRB_REQUIRE(nt != 0, TRB200_ERR_UNSUPPORTED, "conv_wgrad igemm: k=%d not covered", d.k);
    const size_t need = igemm_wgrad_workspace(d);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, "conv_wgrad: workspace of %zu bytes needed, %zu given",
                need, ws_bytes);
    TRB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0, TRB200_ERR_INVALID_ARGUMENT,
                "conv_wgrad: workspace must be 256-byte aligned");
    if (igemm_small_c(d)) return igemm_wgrad_small_c(d, dy, x, dw, ws, st);
    if (conv1x1_wgrad_gemm_supports(d)) return conv1x1_wgrad_gemm(d, dy, x, dw, static_cast<float*>(ws), st);
    if (wgrad_use_halo(d)) return wgrad_halo_run(d, dy, x, dw, static_cast<float*>(ws), st);
    if (wgrad_use_unitn(d)) return wgrad_unitn_run(d, dy, x, dw, static_cast<float*>(ws), st);
    return wgrad_run(d, igemm_taps(d), dy, x, dw, static_cast<float*>(ws), st);
}

// ------------------------------------------------------------------ stride 2 (3x3 pad 1, 1x1 pad 0) without resampling
// d describes the strided convolution: x is [n, h, w, c], y / dy [n, oh, ow, k] with oh = (h - 1) / 2 + 1.
// Forward and weight gradient read x through a tensor map that steps two pixels (the tile in shared memory is the
// stride-1 tile).  The data gradient of the 3x3 case is four stride-1 convolutions of dy, one per parity class of
// the dx pixel (iy, ix) = (2 ty + py, 2 tx + px): a row tap r contributes when iy + 1 - r is even, i.e. r = 1 for
// even rows (dy row ty) and r = 0 (dy row ty + 1), r = 2 (dy row ty) for odd rows; the same along w.  The classes
// use 1, 2, 2 and 4 of the nine taps, so the flop count is that of the forward convolution.
static bool native_s2_shape(const trb200_conv_desc& d) {
    const bool k3 = d.r == 3 && d.s == 3 && d.pad_h == 1 && d.pad_w == 1;
    const bool k1 = d.r == 1 && d.s == 1 && d.pad_h == 0 && d.pad_w == 0;
    return (k3 || k1) && d.stride_h == 2 && d.stride_w == 2 && d.c % 64 == 0 && d.k % 64 == 0;
}

bool igemm_s2_supports(const trb200_conv_desc& d, int which) {
    if (!native_s2_shape(d) || !valid_dtype(d.dtype)) return false;
    if (which == 1) return pick_nt(d.c) != 0;
    return pick_nt(d.k) != 0;
}

size_t igemm_s2_workspace(const trb200_conv_desc& d, int which) {
    if (which == 1) return (size_t)align_up((int64_t)d.r * d.s * d.k * d.c * 2, 256);
    if (which == 0) {
        trb200_conv_desc e = d;
        e.h = (d.h - 1) / 2 + 1; e.w = (d.w - 1) / 2 + 1; e.stride_h = e.stride_w = 1;
        return wgrad_partial_bytes(e, d.r * d.s);
    }
    return 0;
}

// stats_partial / stats_strips as in igemm_fprop: the BN batch statistics of y from the epilogue
int igemm_s2_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, cudaStream_t st, float* stats_partial,
                   int* stats_strips) {
    ConvRunEx ex;
    ex.step = 2; ex.in_h = d.h; ex.in_w = d.w;
    const int oh = (d.h - 1) / 2 + 1, ow = (d.w - 1) / 2 + 1;
    return conv3x3_run(x, w, 1, y, d.n, oh, ow, d.c, d.k, st, d.r * d.s, stats_partial, stats_strips, nullptr,
                       d.dtype == TRB200_DTYPE_BF16, &ex);
}

int igemm_s2_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
                   cudaStream_t st) {
    const size_t need = igemm_s2_workspace(d, 0);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, "conv_wgrad: workspace of %zu bytes needed, %zu given", need,
                ws_bytes);
    trb200_conv_desc e = d;
    e.h = (d.h - 1) / 2 + 1; e.w = (d.w - 1) / 2 + 1; e.stride_h = e.stride_w = 1;
    return wgrad_run(e, d.r * d.s, dy, x, dw, static_cast<float*>(ws), st, nullptr, 2, d.h, d.w);
}

// out[j][c][k] = W[k][tap_j][c] for the nine taps in class order
__global__ void __launch_bounds__(256)
dgrad_s2_filter_view_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ out, int kk, int cc) {
    // class (py, px) = (0,0): tap 4; (0,1): taps 3, 5; (1,0): taps 1, 7; (1,1): taps 0, 2, 6, 8
    const int order[9] = {4, 3, 5, 1, 7, 0, 2, 6, 8};
    const int total = 9 * kk * cc;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % kk, c = (i / kk) % cc, j = i / (kk * cc);
        out[i] = w[((int64_t)k * 9 + order[j]) * cc + c];
    }
}

// zeros in every pixel of [n,h,w,c] that has an odd row or column (what a 1x1 stride-2 data gradient leaves untouched)
__global__ void __launch_bounds__(256)
zero_odd_pixels_kernel(uint4* __restrict__ dx, int64_t vectors, int h, int w, int tpr) {
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vectors; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pix = v / tpr;
        const int x = (int)(pix % w), y = (int)((pix / w) % h);
        if ((x | y) & 1) dx[v] = make_uint4(0u, 0u, 0u, 0u);
    }
}

int igemm_s2_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes,
                   cudaStream_t st) {
    const size_t need = igemm_s2_workspace(d, 1);
    TRB_REQUIRE(ws && ws_bytes >= need, TRB200_ERR_WORKSPACE, "conv_dgrad: workspace of %zu bytes needed, %zu given", need,
                ws_bytes);
    if (d.r == 1) {
        // 1x1: dx at the even pixels is the 1x1 data gradient of dy, everything else is zero
        const int total1 = d.k * d.c;
        int blocks1 = (total1 + 255) / 256;
        if (blocks1 > sm_count() * 4) blocks1 = sm_count() * 4;
        dgrad_filter_view_kernel<<<blocks1, 256, 0, st>>>(static_cast<const uint16_t*>(w), static_cast<uint16_t*>(ws), d.k,
                                                          d.c, 1);
        TRB_LAUNCH_CHECK("dgrad_filter_view_kernel");
        const int64_t vectors = (int64_t)d.n * d.h * d.w * (d.c / 8);
        int zb = (int)((vectors + 1023) / 1024);
        if (zb > sm_count() * 16) zb = sm_count() * 16;
        zero_odd_pixels_kernel<<<zb, 256, 0, st>>>(static_cast<uint4*>(dx), vectors, d.h, d.w, d.c / 8);
        TRB_LAUNCH_CHECK("zero_odd_pixels_kernel");
        ConvRunEx ex;
        ex.step = 1; ex.in_h = (d.h - 1) / 2 + 1; ex.in_w = (d.w - 1) / 2 + 1;
        ex.parity = 0; ex.full_h = d.h; ex.full_w = d.w;
        return conv3x3_run(dy, ws, 0, dx, d.n, ex.in_h, ex.in_w, d.k, d.c, st, 1, nullptr, nullptr, nullptr,
                           d.dtype == TRB200_DTYPE_BF16, &ex);
    }
    const int total = 9 * d.k * d.c;
    int blocks = (total + 255) / 256;
    if (blocks > sm_count() * 4) blocks = sm_count() * 4;
    dgrad_s2_filter_view_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(w), static_cast<uint16_t*>(ws), d.k, d.c);
    TRB_LAUNCH_CHECK("dgrad_s2_filter_view_kernel");
    const int oh = (d.h - 1) / 2 + 1, ow = (d.w - 1) / 2 + 1;
    // a tap's dy offset: r (or s) = 1 -> 0 on the even class; r = 0 -> +1, r = 2 -> 0 on the odd class; nibble = (dw+1) | (dh+1) << 2
    auto nib = [](int dh, int dw) { return (unsigned long long)((dw + 1) | ((dh + 1) << 2)); };
    const int first[4] = {0, 1, 3, 5}, count[4] = {1, 2, 2, 4};
    const unsigned long long offs[4] = {
        nib(0, 0),                                                             // tap (1,1)
        nib(0, 1) | nib(0, 0) << 4,                                            // taps (1,0), (1,2)
        nib(1, 0) | nib(0, 0) << 4,                                            // taps (0,1), (2,1)
        nib(1, 1) | nib(1, 0) << 4 | nib(0, 1) << 8 | nib(0, 0) << 12};        // taps (0,0), (0,2), (2,0), (2,2)
    for (int cls = 0; cls < 4; ++cls) {
        const int py = cls >> 1, px = cls & 1;
        const int hc = (d.h - py + 1) / 2, wc = (d.w - px + 1) / 2;
        if (hc <= 0 || wc <= 0) continue;
        ConvRunEx ex;
        ex.step = 1; ex.in_h = oh; ex.in_w = ow;
        ex.tap_offsets = offs[cls];
        ex.parity = cls; ex.full_h = d.h; ex.full_w = d.w;
        const uint16_t* view = static_cast<const uint16_t*>(ws) + (size_t)first[cls] * d.k * d.c;
        // in = dY [n, oh, ow, k], filter view (ci = k, co = c, tap), out = the class's pixels of dX
        const int rc = conv3x3_run(dy, view, 0, dx, d.n, hc, wc, d.k, d.c, st, count[cls], nullptr, nullptr, nullptr,
                                   d.dtype == TRB200_DTYPE_BF16, &ex);
        if (rc) return rc;
    }
    return TRB200_OK;
}

// ------------------------------------------------------------------ classifier GEMMs (gemm_skinny_sm100.cuh)
static bool fc_dims_ok(int batch, int in_f, int out_f) {
    return batch > 0 && in_f > 0 && out_f > 0 && in_f % 8 == 0 && out_f % 8 == 0;
}

bool fc_gemm_supports(int batch, int in_f, int out_f) { return fc_dims_ok(batch, in_f, out_f); }

// k splits of a GEMM with `tiles` output tiles and `k_steps` stages of k: enough work items to fill the GPU, at
// least 8 stages each
static int fc_splits(int tiles, int k_steps) {
    int splits = sm_count() / tiles;
    if (splits > k_steps / 8) splits = k_steps / 8;
    return splits < 1 ? 1 : splits;
}

static int fc_fwd_splits(int batch, int in_f, int out_f) {
    return fc_splits(((batch + 255) / 256) * ((out_f + kSkN - 1) / kSkN), (in_f + 63) / 64);
}

static int fc_dgrad_splits(int batch, int in_f, int out_f) {
    return fc_splits(((batch + 255) / 256) * ((in_f + kSkN - 1) / kSkN), (out_f + 63) / 64);
}

size_t fc_gemm_fwd_partial_bytes(int batch, int in_f, int out_f) {
    return (size_t)fc_fwd_splits(batch, in_f, out_f) * (size_t)batch * (size_t)out_f * sizeof(float);
}

// 0 when the data-gradient GEMM writes its half output directly
size_t fc_gemm_dgrad_partial_bytes(int batch, int in_f, int out_f) {
    const int splits = fc_dgrad_splits(batch, in_f, out_f);
    return splits == 1 ? 0 : (size_t)splits * (size_t)batch * (size_t)in_f * sizeof(float);
}

// partial[split][b][o] (float) = x[b][k range of the split] . w[o][same]; *splits receives the split count
int fc_gemm_fwd(const void* x, const void* w, float* partial, int batch, int in_f, int out_f, int* splits,
                cudaStream_t st, bool bf16) {
    TRB_REQUIRE(fc_dims_ok(batch, in_f, out_f), TRB200_ERR_UNSUPPORTED, "fc: in_features=%d, out_features=%d must be multiples of 8", in_f, out_f);
    CUtensorMap ta, tb;
    int rc = make_matrix_tmap(&ta, x, batch, in_f, in_f, 128, "fc x");
    if (rc) return rc;
    rc = make_matrix_tmap(&tb, w, out_f, in_f, in_f, 256, "fc w");
    if (rc) return rc;
    SkinnyParams p;
    p.m_real = batch; p.n_real = out_f;
    p.k_steps = (in_f + 63) / 64;
    p.m_tiles = (batch + 255) / 256; p.n_tiles = (out_f + kSkN - 1) / kSkN;
    p.splits = fc_fwd_splits(batch, in_f, out_f);
    p.ldd = out_f; p.d = partial; p.split_stride = (int64_t)batch * out_f; p.bf16 = bf16 ? 1 : 0;
    *splits = p.splits;
    return launch_skinny<false, false, 2, true>(ta, tb, ta, p, st);
}

// dx[b][i] = dy[b][:] . w[:][i]: half into dx when *splits comes back 1, else float partials [split][b][i]
int fc_gemm_dgrad(const void* dy, const void* w, void* dx, float* partial, int batch, int in_f, int out_f, int* splits,
                  cudaStream_t st, bool bf16) {
    TRB_REQUIRE(fc_dims_ok(batch, in_f, out_f), TRB200_ERR_UNSUPPORTED, "fc: in_features=%d, out_features=%d must be multiples of 8", in_f, out_f);
    CUtensorMap ta, tb, td;
    int rc = make_matrix_tmap(&ta, dy, batch, out_f, out_f, 128, "fc dy");
    if (rc) return rc;
    rc = make_matrix_tmap(&tb, w, out_f, in_f, in_f, 64, "fc w (columns)");
    if (rc) return rc;
    rc = make_matrix_tmap(&td, dx, batch, in_f, in_f, 128, "fc dx");
    if (rc) return rc;
    SkinnyParams p;
    p.m_real = batch; p.n_real = in_f;
    p.k_steps = (out_f + 63) / 64;
    p.m_tiles = (batch + 255) / 256; p.n_tiles = (in_f + kSkN - 1) / kSkN;
    p.splits = fc_dgrad_splits(batch, in_f, out_f);
    p.ldd = in_f; p.bf16 = bf16 ? 1 : 0;
    *splits = p.splits;
    if (p.splits == 1) {
        p.d = dx; p.split_stride = 0;
        return launch_skinny<false, true, 2, false>(ta, tb, td, p, st);
    }
    p.d = partial; p.split_stride = (int64_t)batch * in_f;
    return launch_skinny<false, true, 2, true>(ta, tb, td, p, st);
}

// dw[o][i] = dy[:][o] . x[:][i], half or (dw_float) float as the reference's FC_AMP_BWD writes it
int fc_gemm_wgrad(const void* dy, const void* x, void* dw, int dw_float, int batch, int in_f, int out_f, cudaStream_t st,
                  bool bf16) {
    TRB_REQUIRE(fc_dims_ok(batch, in_f, out_f), TRB200_ERR_UNSUPPORTED, "fc: in_features=%d, out_features=%d must be multiples of 8", in_f, out_f);
    CUtensorMap ta, tb, td;
    int rc = make_matrix_tmap(&ta, dy, batch, out_f, out_f, 64, "fc dy (columns)");
    if (rc) return rc;
    rc = make_matrix_tmap(&tb, x, batch, in_f, in_f, 64, "fc x (columns)");
    if (rc) return rc;
    if (!dw_float) rc = make_matrix_tmap(&td, dw, out_f, in_f, in_f, 128, "fc dw");
    if (rc) return rc;
    SkinnyParams p;
    p.m_real = out_f; p.n_real = in_f;
    p.k_steps = (batch + 63) / 64;
    p.m_tiles = (out_f + 127) / 128; p.n_tiles = (in_f + kSkN - 1) / kSkN;
    p.splits = 1;
    p.ldd = in_f; p.d = dw; p.split_stride = 0; p.bf16 = bf16 ? 1 : 0;
    if (dw_float) return launch_skinny<true, true, 1, true>(ta, tb, ta, p, st);
    return launch_skinny<true, true, 1, false>(ta, tb, td, p, st);
}

// ------------------------------------------------------------------ 1x1 stride-1 weight gradient as a split-K GEMM
// dW[k][c] = sum over pixels of dy[pixel][k] * x[pixel][c]: both operands MN-major, the pixels are the reduction,
// split over about one CTA per SM; float partials [split][k][c], added in split order.
namespace {
__global__ void __launch_bounds__(256)
conv1x1_wgrad_reduce(const float* __restrict__ partial, uint16_t* __restrict__ dw, int splits, int64_t total, int bf16) {
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += (int64_t)gridDim.x * blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < splits; ++sp) {
            const float4 v = *reinterpret_cast<const float4*>(partial + (int64_t)sp * total + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint2 o;
        o.x = bf16 ? pack2_t<true>(acc.x, acc.y) : pack2_t<false>(acc.x, acc.y);
        o.y = bf16 ? pack2_t<true>(acc.z, acc.w) : pack2_t<false>(acc.z, acc.w);
        *reinterpret_cast<uint2*>(dw + i) = o;
    }
}

int conv1x1_wgrad_splits(const trb200_conv_desc& d) {
    const int64_t pixels = (int64_t)d.n * d.h * d.w;
    const int tiles = ((d.k + 127) / 128) * ((d.c + kSkN - 1) / kSkN);
    return fc_splits(tiles, (int)((pixels + 63) / 64));
}
}  // namespace

bool conv1x1_wgrad_gemm_supports(const trb200_conv_desc& d) {
    return d.r == 1 && d.s == 1 && d.pad_h == 0 && d.pad_w == 0 && d.stride_h == 1 && d.stride_w == 1 && d.c % 8 == 0 &&
           d.k % 8 == 0 && ((int64_t)d.k * d.c) % 4 == 0 && (int64_t)d.n * d.h * d.w < (1ll << 31);
}

size_t conv1x1_wgrad_gemm_workspace(const trb200_conv_desc& d) {
    return (size_t)align_up((int64_t)conv1x1_wgrad_splits(d) * d.k * d.c * 4, 256);
}

int conv1x1_wgrad_gemm(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, float* partial, cudaStream_t st) {
    const int64_t pixels = (int64_t)d.n * d.h * d.w;
    CUtensorMap ta, tb;
    int rc = make_matrix_tmap(&ta, dy, pixels, d.k, d.k, 64, "1x1 wgrad dy (columns)");
    if (rc) return rc;
    rc = make_matrix_tmap(&tb, x, pixels, d.c, d.c, 64, "1x1 wgrad x (columns)");
    if (rc) return rc;
    SkinnyParams p;
    p.m_real = d.k; p.n_real = d.c;
    p.k_steps = (int)((pixels + 63) / 64);
    p.m_tiles = (d.k + 127) / 128; p.n_tiles = (d.c + kSkN - 1) / kSkN;
    p.splits = conv1x1_wgrad_splits(d);
    p.ldd = d.c; p.d = partial; p.split_stride = (int64_t)d.k * d.c;
    p.bf16 = d.dtype == TRB200_DTYPE_BF16 ? 1 : 0;
    rc = launch_skinny<true, true, 1, true>(ta, tb, ta, p, st);
    if (rc) return rc;
    const int64_t total = (int64_t)d.k * d.c;
    int blocks = (int)((total / 4 + 255) / 256);
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    conv1x1_wgrad_reduce<<<blocks, 256, 0, st>>>(partial, static_cast<uint16_t*>(dw), p.splits, total, p.bf16);
    TRB_LAUNCH_CHECK("conv1x1_wgrad_reduce");
    return TRB200_OK;
}

// ------------------------------------------------------------------ self-test of the give-up path
// One warp initialises an mbarrier that nothing ever arrives on and waits for it with the kernels' own bounded wait
// and a short limit.  The wait runs out, the status word gets kStatusSelfTest, the block's abort flag is raised
// (which the second warp's wait then sees) and the kernel returns: nothing faults and the context stays usable.
namespace {
constexpr int kStatusSelfTest = 99;

__global__ void __launch_bounds__(64, 1) wait_timeout_selftest_kernel(unsigned long long limit_ns, int* status, int* out) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
    }
    __syncthreads();
    const unsigned long long t0 = global_ns();
    bool ok;
    if (threadIdx.x < 32) {
        ok = mbar_wait_limit(smem_u32(&bar), 0, &s_abort, status, kStatusSelfTest, limit_ns);
    } else {
        // a role that would wait a full second on its own: it must leave when the first one raises the abort flag
        ok = mbar_wait(smem_u32(&bar), 0, &s_abort, status, kStatusSelfTest);
    }
    const unsigned long long waited = global_ns() - t0;
    if ((threadIdx.x & 31) == 0) {
        out[(threadIdx.x >> 5) * 2] = ok ? 1 : 0;
        out[(threadIdx.x >> 5) * 2 + 1] = (int)(waited > 0x7fffffffull ? 0x7fffffffull : waited);
    }
}
}  // namespace

// out4: device array of four ints: {warp 0 returned true?, ns it waited, warp 1 returned true?, ns it waited}
int wait_timeout_selftest(unsigned long long limit_ns, int* out4, cudaStream_t st) {
    TRB_REQUIRE(out4 != nullptr, TRB200_ERR_INVALID_ARGUMENT, "selftest_wait_timeout: null output");
    TRB_REQUIRE(limit_ns >= 1000ull && limit_ns <= 100ull * 1000ull * 1000ull, TRB200_ERR_INVALID_ARGUMENT,
                "selftest_wait_timeout: limit of %llu ns outside [1 us, 100 ms]", limit_ns);
    int* status = nullptr;
    TRB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_device_status));
    wait_timeout_selftest_kernel<<<1, 64, 0, st>>>(limit_ns, status, out4);
    TRB_LAUNCH_CHECK("wait_timeout_selftest_kernel");
    return TRB200_OK;
}

#ifdef TRB200_ROLE_TIMERS
extern "C" int trb200_debug_read_role_timers(long long* host_out, int count) {
    TRB_CUDA_TRY(cudaMemcpyFromSymbol(host_out, g_role_timers, sizeof(long long) * (size_t)count));
    return TRB200_OK;
}
#endif

int device_status_read_and_clear(int* out) {
    int v = 0;
    TRB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        TRB_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    *out = v;
    return TRB200_OK;
}

}  // namespace trb
