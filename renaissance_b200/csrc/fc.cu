// Classifier layers of the AMP step: FC forward / backward (the reference's FC_AMP_FWD / FC_AMP_BWD,
// src/backend/ops/dtensor/fc_op.cpp:259-480 with the bias kernels of fc_op.cu:20-101) with the ReLU
// (relu_op.cu:101-126) and the dropout (dropout_op.cu:50-274) that follow an FC layer in VGG folded into the
// bias pass.
//
// The three GEMMs (y = x W^T: forward; dx = dy W: data gradient; dW = dy^T x: weight gradient) run on this library's
// own tcgen05 kernel for GEMMs with one batch-sized dimension (gemm_skinny_sm100.cuh), which reads every operand in
// place, K-major or MN-major as it lies in memory.  The forward GEMM is split over the input features so that it
// fills the GPU; its float partial sums are added, in split order, by the bias / ReLU / dropout pass.  No cuBLAS.
//
// Dropout draws its bits from Philox4x32-10 (the counter-based generator the reference uses, src/core/rng.cpp)
// keyed by (seed, offset) and indexed by the element: no mask is stored.  An element that was dropped, or that the
// ReLU zeroed, is zero in the layer's output, so the backward needs only that output:
//   dz = out > 0 ? da / (1 - p) : 0.
#include "common.cuh"
#include "conv.cuh"

namespace trb {
namespace {

// ---------------------------------------------------------------- Philox4x32-10
struct Philox4 { uint32_t v[4]; };

__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                 uint32_t k1) {
    constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u, kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(kM0, c0), lo0 = kM0 * c0;
        const uint32_t hi1 = __umulhi(kM1, c2), lo1 = kM1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += kW0; k1 += kW1;
    }
    return Philox4{{c0, c1, c2, c3}};
}

// a float rounded to the layer's 16-bit type and back
template <bool BF16>
__device__ __forceinline__ float round_trip16(float f) {
    if constexpr (BF16) return __uint_as_float((uint32_t)round16_t<true>(f) << 16);
    else return __half2float(__float2half_rn(f));
}

// y[b][o] = dropout(relu(half(sum over splits of partial[s][b][o]) + bias[o])); one thread = 8 consecutive outputs
template <bool BF16>
__global__ void __launch_bounds__(256)
fc_bias_act_kernel(const float* __restrict__ partial, int splits, int64_t split_stride, uint16_t* __restrict__ y,
                   const float* __restrict__ bias, int64_t vecs, int out_vecs, int relu, uint32_t drop_threshold,
                   float keep_scale, uint32_t seed_lo, uint32_t seed_hi, uint32_t off_lo, uint32_t off_hi) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        const int col = (int)(v % out_vecs) * 8;
        float f[8];
        *reinterpret_cast<float4*>(f) = reinterpret_cast<const float4*>(partial + v * 8)[0];
        *reinterpret_cast<float4*>(f + 4) = reinterpret_cast<const float4*>(partial + v * 8)[1];
        for (int s = 1; s < splits; ++s) {                   // split order: reproducible
            const float4 a = reinterpret_cast<const float4*>(partial + (int64_t)s * split_stride + v * 8)[0];
            const float4 b = reinterpret_cast<const float4*>(partial + (int64_t)s * split_stride + v * 8)[1];
            f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
            f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
        }
        float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (bias) {
            *reinterpret_cast<float4*>(b) = __ldg(reinterpret_cast<const float4*>(bias + col));
            *reinterpret_cast<float4*>(b + 4) = __ldg(reinterpret_cast<const float4*>(bias + col + 4));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // the GEMM's output rounded to half, plus the float bias, rounded to half again
            // (cublasGemmEx writes half, then fc_fwd_bias_add_amp_kernel, fc_op.cu:88-99)
            f[j] = round_trip16<BF16>(f[j]);
            if (bias) f[j] = round_trip16<BF16>(f[j] + b[j]);
            if (relu) f[j] = fmaxf(f[j], 0.f);
        }
        if (drop_threshold != 0u) {
            const Philox4 r0 = philox4x32_10((uint32_t)(2 * v), (uint32_t)((2 * v) >> 32), off_lo, off_hi, seed_lo, seed_hi);
            const Philox4 r1 = philox4x32_10((uint32_t)(2 * v + 1), (uint32_t)((2 * v + 1) >> 32), off_lo, off_hi, seed_lo, seed_hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[j] = r0.v[j] >= drop_threshold ? f[j] * keep_scale : 0.f;
                f[4 + j] = r1.v[j] >= drop_threshold ? f[4 + j] * keep_scale : 0.f;
            }
        }
        uint4 o;
        o.x = pack2_t<BF16>(f[0], f[1]); o.y = pack2_t<BF16>(f[2], f[3]);
        o.z = pack2_t<BF16>(f[4], f[5]); o.w = pack2_t<BF16>(f[6], f[7]);
        reinterpret_cast<uint4*>(y)[v] = o;
    }
}

// dz = act > 0 ? da * scale : 0 (ReLU and dropout backward in one select); dz may be da
template <bool BF16>
__global__ void __launch_bounds__(256)
fc_act_bwd_kernel(const uint4* da, const uint4* __restrict__ act, uint4* dz, int64_t vecs, float scale) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        float g[8], a[8];
        unpack8_t<BF16>(da[v], g);
        unpack8_t<BF16>(act[v], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = a[j] > 0.f ? g[j] * scale : 0.f;
        uint4 o;
        o.x = pack2_t<BF16>(g[0], g[1]); o.y = pack2_t<BF16>(g[2], g[3]);
        o.z = pack2_t<BF16>(g[4], g[5]); o.w = pack2_t<BF16>(g[6], g[7]);
        dz[v] = o;
    }
}

// dx = half(sum over splits of partial[s]) [then, with act: act > 0 ? . * scale : 0]; one thread = 8 elements
template <bool BF16>
__global__ void __launch_bounds__(256)
fc_reduce_act_bwd_kernel(const float* __restrict__ partial, int splits, int64_t split_stride, const uint4* __restrict__ act,
                         uint4* __restrict__ dx, int64_t vecs, float scale) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += stride) {
        float f[8];
        *reinterpret_cast<float4*>(f) = reinterpret_cast<const float4*>(partial + v * 8)[0];
        *reinterpret_cast<float4*>(f + 4) = reinterpret_cast<const float4*>(partial + v * 8)[1];
        for (int s = 1; s < splits; ++s) {                   // split order: reproducible
            const float4 a = reinterpret_cast<const float4*>(partial + (int64_t)s * split_stride + v * 8)[0];
            const float4 b = reinterpret_cast<const float4*>(partial + (int64_t)s * split_stride + v * 8)[1];
            f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
            f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
        }
        if (act) {
            float a[8];
            unpack8_t<BF16>(act[v], a);
            // the GEMM's 16-bit result first, as when the two steps run apart
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = a[j] > 0.f ? round_trip16<BF16>(f[j]) * scale : 0.f;
        }
        uint4 o;
        o.x = pack2_t<BF16>(f[0], f[1]); o.y = pack2_t<BF16>(f[2], f[3]);
        o.z = pack2_t<BF16>(f[4], f[5]); o.w = pack2_t<BF16>(f[6], f[7]);
        dx[v] = o;
    }
}

// db[o] = sum over the batch of dy[b][o], rows added in order (fc_bwd_db_amp_kernel, fc_op.cu:33-47, with eight
// row groups per column block that meet in shared memory in group order: reproducible)
template <bool BF16>
__global__ void __launch_bounds__(256)
fc_bias_grad_kernel(const uint16_t* __restrict__ dy, float* __restrict__ db, int batch, int out_f) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int o = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (o < out_f)
        for (int b = grp; b < batch; b += 8) s += load16_t<BF16>(dy + (int64_t)b * out_f + o);
    part[grp][lane] = s;
    __syncthreads();
    if (grp == 0 && o < out_f) {
        float t = part[0][lane];
#pragma unroll
        for (int g = 1; g < 8; ++g) t += part[g][lane];
        db[o] = t;
    }
}

int grid_for(int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

int check_dims(int batch, int in_f, int out_f, const char* who) {
    TRB_REQUIRE(batch > 0 && in_f > 0 && out_f > 0, TRB200_ERR_INVALID_ARGUMENT, "%s: sizes must be positive", who);
    TRB_REQUIRE(fc_gemm_supports(batch, in_f, out_f), TRB200_ERR_UNSUPPORTED,
                "%s: in_features=%d and out_features=%d must be multiples of 8 (rows of 16-byte vectors)", who, in_f, out_f);
    return TRB200_OK;
}

}  // namespace
}  // namespace trb

// the float partial sums of the forward GEMM, or of the data-gradient GEMM when that one is split (the larger)
extern "C" size_t trb200_fc_amp_workspace_bytes(int32_t batch, int32_t in_features, int32_t out_features) {
    if (!trb::fc_gemm_supports(batch, in_features, out_features)) return 0;
    const size_t f = trb::fc_gemm_fwd_partial_bytes(batch, in_features, out_features);
    const size_t d = trb::fc_gemm_dgrad_partial_bytes(batch, in_features, out_features);
    return (size_t)trb::align_up((int64_t)(f > d ? f : d), 256);
}

static int fc_amp_fwd_any(const void* x, const void* w, const float* bias, void* y, int32_t batch, int32_t in_features,
                          int32_t out_features, int32_t relu, float dropout_p, uint64_t seed, uint64_t offset,
                          void* workspace, size_t workspace_bytes, void* stream, int32_t dtype) {
    int rc = trb::check_dims(batch, in_features, out_features, "fc_amp_fwd");
    if (rc) return rc;
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "fc_amp_fwd: unknown dtype %d", dtype);
    TRB_REQUIRE(x && w && y, TRB200_ERR_INVALID_ARGUMENT, "fc_amp_fwd: null pointer");
    TRB_REQUIRE(dropout_p >= 0.f && dropout_p < 1.f, TRB200_ERR_INVALID_ARGUMENT, "fc_amp_fwd: dropout_p=%f outside [0, 1)",
                (double)dropout_p);
    TRB_REQUIRE(trb::aligned16(x) && trb::aligned16(w) && trb::aligned16(y) && (!bias || trb::aligned16(bias)),
                TRB200_ERR_INVALID_ARGUMENT, "fc_amp_fwd: tensors must be 16-byte aligned");
    const size_t need = trb200_fc_amp_workspace_bytes(batch, in_features, out_features);
    TRB_REQUIRE(workspace && workspace_bytes >= need, TRB200_ERR_WORKSPACE,
                "fc_amp_fwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    TRB_REQUIRE(trb::aligned16(workspace), TRB200_ERR_INVALID_ARGUMENT, "fc_amp_fwd: workspace must be 16-byte aligned");
    cudaStream_t st = trb::as_stream(stream);
    const bool bf16 = dtype == TRB200_DTYPE_BF16;
    int splits = 1;
    rc = trb::fc_gemm_fwd(x, w, static_cast<float*>(workspace), batch, in_features, out_features, &splits, st, bf16);
    if (rc) return rc;
    const int64_t vecs = (int64_t)batch * out_features / 8;
    const uint32_t thr = dropout_p > 0.f ? (uint32_t)((double)dropout_p * 4294967296.0) : 0u;
    (bf16 ? trb::fc_bias_act_kernel<true> : trb::fc_bias_act_kernel<false>)<<<trb::grid_for(vecs), 256, 0, st>>>(
        static_cast<const float*>(workspace), splits, (int64_t)batch * out_features, static_cast<uint16_t*>(y), bias, vecs,
        out_features / 8, relu ? 1 : 0, thr, 1.0f / (1.0f - dropout_p), (uint32_t)seed, (uint32_t)(seed >> 32),
        (uint32_t)offset, (uint32_t)(offset >> 32));
    TRB_LAUNCH_CHECK("fc_bias_act_kernel");
    return TRB200_OK;
}

extern "C" int trb200_fc_amp_fwd(const void* x, const void* w, const float* bias, void* y, int32_t batch,
                                 int32_t in_features, int32_t out_features, int32_t relu, float dropout_p,
                                 uint64_t seed, uint64_t offset, void* workspace, size_t workspace_bytes, void* stream) {
    return fc_amp_fwd_any(x, w, bias, y, batch, in_features, out_features, relu, dropout_p, seed, offset, workspace,
                          workspace_bytes, stream, TRB200_DTYPE_F16);
}

extern "C" int trb200_fc_amp_fwd_dtype(const void* x, const void* w, const float* bias, void* y, int32_t batch,
                                       int32_t in_features, int32_t out_features, int32_t relu, float dropout_p,
                                       uint64_t seed, uint64_t offset, int32_t dtype, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    return fc_amp_fwd_any(x, w, bias, y, batch, in_features, out_features, relu, dropout_p, seed, offset, workspace,
                          workspace_bytes, stream, dtype);
}

static int fc_act_bwd_any(const void* da, const void* act, void* dz, int64_t n, float scale, void* stream, int32_t dtype) {
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "fc_act_bwd: unknown dtype %d", dtype);
    TRB_REQUIRE(n >= 0 && n % 8 == 0, TRB200_ERR_INVALID_ARGUMENT, "fc_act_bwd: the element count must be a multiple of 8");
    if (n == 0) return TRB200_OK;
    TRB_REQUIRE(da && act && dz, TRB200_ERR_INVALID_ARGUMENT, "fc_act_bwd: null pointer");
    TRB_REQUIRE(trb::aligned16(da) && trb::aligned16(act) && trb::aligned16(dz), TRB200_ERR_INVALID_ARGUMENT,
                "fc_act_bwd: tensors must be 16-byte aligned");
    (dtype == TRB200_DTYPE_BF16 ? trb::fc_act_bwd_kernel<true> : trb::fc_act_bwd_kernel<false>)
        <<<trb::grid_for(n / 8), 256, 0, trb::as_stream(stream)>>>(static_cast<const uint4*>(da), static_cast<const uint4*>(act),
                                                                    static_cast<uint4*>(dz), n / 8, scale);
    TRB_LAUNCH_CHECK("fc_act_bwd_kernel");
    return TRB200_OK;
}

extern "C" int trb200_fc_act_bwd(const void* da, const void* act, void* dz, int64_t n, float scale, void* stream) {
    return fc_act_bwd_any(da, act, dz, n, scale, stream, TRB200_DTYPE_F16);
}

static int fc_amp_bwd_any(const void* dy, const void* w, const void* x, void* dx, void* dw, int32_t dw_float, float* db,
                          const void* act, float act_scale, int32_t batch, int32_t in_features, int32_t out_features,
                          void* workspace, size_t workspace_bytes, void* stream, int32_t dtype) {
    int rc = trb::check_dims(batch, in_features, out_features, "fc_amp_bwd");
    if (rc) return rc;
    TRB_REQUIRE(trb::valid_dtype(dtype), TRB200_ERR_INVALID_ARGUMENT, "fc_amp_bwd: unknown dtype %d", dtype);
    TRB_REQUIRE(dy && w && x && dw, TRB200_ERR_INVALID_ARGUMENT, "fc_amp_bwd: null pointer");
    TRB_REQUIRE(trb::aligned16(dy) && trb::aligned16(w) && trb::aligned16(x) && trb::aligned16(dw) &&
                    (!dx || trb::aligned16(dx)) && (!act || trb::aligned16(act)),
                TRB200_ERR_INVALID_ARGUMENT, "fc_amp_bwd: tensors must be 16-byte aligned");
    cudaStream_t st = trb::as_stream(stream);
    const bool bf16 = dtype == TRB200_DTYPE_BF16;
    if (db) {
        (bf16 ? trb::fc_bias_grad_kernel<true> : trb::fc_bias_grad_kernel<false>)<<<(out_features + 31) / 32, 256, 0, st>>>(
            static_cast<const uint16_t*>(dy), db, batch, out_features);
        TRB_LAUNCH_CHECK("fc_bias_grad_kernel");
    }
    rc = trb::fc_gemm_wgrad(dy, x, dw, dw_float, batch, in_features, out_features, st, bf16);
    if (rc || !dx) return rc;
    const size_t need = trb::fc_gemm_dgrad_partial_bytes(batch, in_features, out_features);
    TRB_REQUIRE(need == 0 || (workspace && workspace_bytes >= need && trb::aligned16(workspace)), TRB200_ERR_WORKSPACE,
                "fc_amp_bwd: 16-byte aligned workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    int splits = 1;
    rc = trb::fc_gemm_dgrad(dy, w, dx, static_cast<float*>(workspace), batch, in_features, out_features, &splits, st, bf16);
    if (rc) return rc;
    const int64_t vecs = (int64_t)batch * in_features / 8;
    if (splits > 1) {
        (bf16 ? trb::fc_reduce_act_bwd_kernel<true> : trb::fc_reduce_act_bwd_kernel<false>)<<<trb::grid_for(vecs), 256, 0, st>>>(
            static_cast<const float*>(workspace), splits, (int64_t)batch * in_features, static_cast<const uint4*>(act),
            static_cast<uint4*>(dx), vecs, act_scale);
        TRB_LAUNCH_CHECK("fc_reduce_act_bwd_kernel");
    } else if (act) {
        (bf16 ? trb::fc_act_bwd_kernel<true> : trb::fc_act_bwd_kernel<false>)<<<trb::grid_for(vecs), 256, 0, st>>>(
            static_cast<const uint4*>(dx), static_cast<const uint4*>(act), static_cast<uint4*>(dx), vecs, act_scale);
        TRB_LAUNCH_CHECK("fc_act_bwd_kernel");
    }
    return TRB200_OK;
}

extern "C" int trb200_fc_amp_bwd(const void* dy, const void* w, const void* x, void* dx, void* dw, int32_t dw_float,
                                 float* db, const void* act, float act_scale, int32_t batch, int32_t in_features,
                                 int32_t out_features, void* workspace, size_t workspace_bytes, void* stream) {
    return fc_amp_bwd_any(dy, w, x, dx, dw, dw_float, db, act, act_scale, batch, in_features, out_features, workspace,
                          workspace_bytes, stream, TRB200_DTYPE_F16);
}

extern "C" int trb200_fc_amp_bwd_dtype(const void* dy, const void* w, const void* x, void* dx, void* dw, int32_t dw_float,
                                       float* db, const void* act, float act_scale, int32_t batch, int32_t in_features,
                                       int32_t out_features, int32_t dtype, void* workspace, size_t workspace_bytes,
                                       void* stream) {
    return fc_amp_bwd_any(dy, w, x, dx, dw, dw_float, db, act, act_scale, batch, in_features, out_features, workspace,
                          workspace_bytes, stream, dtype);
}
