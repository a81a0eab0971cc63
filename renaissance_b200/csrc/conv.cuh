// Internal interface between the convolution entry points and their kernels.
#pragma once

#include "common.cuh"

namespace trb {

// Direct CUDA-core kernels (conv_direct.cu): any geometry.
size_t wgrad_direct_workspace(const trb200_conv_desc& d);
int wgrad_direct(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws,
                 size_t ws_bytes, cudaStream_t st);
int dgrad_direct(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, cudaStream_t st);

// tcgen05 / TMEM implicit-GEMM kernels (conv_igemm_sm100.cu): 3x3, stride 1,
// pad 1, channel counts that are multiples of 64; plus the 4-input-channel first
// layer (as a 1x1 convolution over 3x3 neighbourhoods built in shared memory).
bool igemm_supports(const trb200_conv_desc& d, int which);   // 0 wgrad, 1 dgrad, 2 fprop
bool igemm_small_c(const trb200_conv_desc& d);
size_t igemm_wgrad_workspace(const trb200_conv_desc& d);
size_t igemm_dgrad_workspace(const trb200_conv_desc& d);
// stride 2 (3x3 pad 1, 1x1 pad 0) on the tensor-core kernels without a resampling pass: forward and weight gradient
// read x through a tensor map that steps two pixels, the 3x3 data gradient runs as four parity classes
bool igemm_s2_supports(const trb200_conv_desc& d, int which);
size_t igemm_s2_workspace(const trb200_conv_desc& d, int which);
int igemm_s2_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, cudaStream_t st,
                   float* stats_partial = nullptr, int* stats_strips = nullptr);
int igemm_s2_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
                   cudaStream_t st);
int igemm_s2_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes,
                   cudaStream_t st);
size_t igemm_fprop_workspace(const trb200_conv_desc& d);
size_t igemm_fprop_stats_bytes(const trb200_conv_desc& d);
int igemm_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
                cudaStream_t st, float* stats_partial = nullptr, int* stats_strips = nullptr);

// block_fwd.cu: adds [strips][2][c] partial sums in strip order and finalizes the batch statistics
int bn_finalize_from_partials(const float* partial, int strips, int c, int64_t m, const float* gamma,
                              const float* beta, float eps, float momentum, float* ch_sum, float* ch_sqsum,
                              float* saved_mean, float* saved_inv_std, float* eq_scale, float* eq_bias,
                              float* running_mean, float* running_var, cudaStream_t st);
int igemm_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws,
                size_t ws_bytes, cudaStream_t st);
int igemm_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws,
                size_t ws_bytes, cudaStream_t st);

// conv_strided.cu: 3x3 pad 1 and 1x1 pad 0 with stride 2, through the stride-1 tensor-core kernels and one
// resampling pass (workspace: the resampled tensor, then the inner kernel's workspace).
bool strided_supports(const trb200_conv_desc& d, int which);   // 0 wgrad, 1 dgrad, 2 fprop
size_t strided_workspace(const trb200_conv_desc& d, int which);
int strided_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
                  cudaStream_t st);
int strided_dgrad(const trb200_conv_desc& d, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes,
                  cudaStream_t st);
int strided_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
                  cudaStream_t st);

// conv_strided.cu: a first layer (4 input channels, any filter / stride / padding) lowered to rows of r*s*4 values
// and run as a 1x1 convolution; forward and weight gradient.
bool stem_supports(const trb200_conv_desc& d, int which);
size_t stem_workspace(const trb200_conv_desc& d, int which);
int stem_wgrad(const trb200_conv_desc& d, const void* dy, const void* x, void* dw, void* ws, size_t ws_bytes,
               cudaStream_t st);
int stem_fprop(const trb200_conv_desc& d, const void* x, const void* w, void* y, void* ws, size_t ws_bytes,
               cudaStream_t st);

// conv_igemm_sm100.cu (gemm_skinny_sm100.cuh): the three GEMMs of a fully connected layer, operands read in place
bool fc_gemm_supports(int batch, int in_f, int out_f);
size_t fc_gemm_fwd_partial_bytes(int batch, int in_f, int out_f);
int fc_gemm_fwd(const void* x, const void* w, float* partial, int batch, int in_f, int out_f, int* splits,
                cudaStream_t st, bool bf16 = false);
size_t fc_gemm_dgrad_partial_bytes(int batch, int in_f, int out_f);
int fc_gemm_dgrad(const void* dy, const void* w, void* dx, float* partial, int batch, int in_f, int out_f, int* splits,
                  cudaStream_t st, bool bf16 = false);
int fc_gemm_wgrad(const void* dy, const void* x, void* dw, int dw_float, int batch, int in_f, int out_f,
                  cudaStream_t st, bool bf16 = false);

int validate_conv_desc(const trb200_conv_desc* d, const char* who);

}  // namespace trb
