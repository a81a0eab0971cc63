// Shared host/device helpers of the trb200 library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "trb200.h"

namespace trb {

// Thread-local text of the last failure, returned by trb200_last_error().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
inline cudaEvent_t as_event(void* e) { return static_cast<cudaEvent_t>(e); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Number of SMs of the current device (cached per device).
int sm_count();
int ring_status_ptr(int** out);     // status word of the bulk-copy ring kernels (bounded waits)

// Counts kernel launches made by this library (every launch site goes through
// TRB_LAUNCH_CHECK); read by trb200_kernel_launch_count().
void note_launch();

#define TRB_CUDA_TRY(expr)                                                                  \
    do {                                                                                    \
        cudaError_t err__ = (expr);                                                         \
        if (err__ != cudaSuccess)                                                           \
            return ::trb::fail(TRB200_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

#define TRB_LAUNCH_CHECK(what)                                                               \
    do {                                                                                     \
        ::trb::note_launch();                                                                \
        cudaError_t err__ = cudaGetLastError();                                              \
        if (err__ != cudaSuccess)                                                            \
            return ::trb::fail(TRB200_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(err__)); \
    } while (0)

#define TRB_REQUIRE(cond, code, ...)                   \
    do {                                               \
        if (!(cond)) return ::trb::fail(code, __VA_ARGS__); \
    } while (0)

// 16-bit storage types.  The kernels are written once over these helpers: BF16 = false is IEEE half (the
// reference's AMP dtype), BF16 = true is bfloat16.  All arithmetic is float either way.
#ifdef __CUDACC__
template <bool BF16>
__device__ __forceinline__ float2 unpack2_t(uint32_t v) {
    if constexpr (BF16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
    else return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2_t(float a, float b) {
    if constexpr (BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

template <bool BF16>
__device__ __forceinline__ float load16_t(const uint16_t* p) {
    if constexpr (BF16) return __uint_as_float((uint32_t)*p << 16);
    else return __half2float(*reinterpret_cast<const __half*>(p));
}

template <bool BF16>
__device__ __forceinline__ uint16_t round16_t(float v) {
    if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

template <bool BF16>
__device__ __forceinline__ void unpack8_t(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = unpack2_t<BF16>(w[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
#endif

inline bool valid_dtype(int dtype) { return dtype == TRB200_DTYPE_F16 || dtype == TRB200_DTYPE_BF16; }

// Output extent of a convolution along one axis.
inline int conv_out(int in, int pad, int k, int stride) { return (in + 2 * pad - k) / stride + 1; }

}  // namespace trb
