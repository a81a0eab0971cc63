// Shared host/device helpers of the trb200 library.
#pragma once

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

// Output extent of a convolution along one axis.
inline int conv_out(int in, int pad, int k, int stride) { return (in + 2 * pad - k) / stride + 1; }

}  // namespace trb
