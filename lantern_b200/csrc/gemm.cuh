// Internal declarations shared by the contraction translation units.
#pragma once
#include "common.cuh"

namespace ltb {

struct ConvDims { int N, C, H, W, K, R, S, sh, sw, ph, pw, oH, oW; };

// FP32 CUDA-core path (gemm_fp32.cu)
int gemm_fp32(const float* a, int64_t sam, int64_t sak, const float* b, int64_t sbk, int64_t sbn, float* c, int64_t scm, int64_t scn,
              int M, int N, int K, float alpha, bool accumulate);
int conv_fwd_fp32(const float* x, const float* w, const float* bias, float* y, const ConvDims& d);
int conv_dgrad_fp32(const float* dy, const float* w, float* dx, const ConvDims& d);
int conv_wgrad_fp32(const float* x, const float* dy, float* dw, const ConvDims& d);
int conv_bias_grad(const float* dy, float* dbias, const ConvDims& d);

// TF32 tensor-core path (gemm_tc.cu). Each returns 1 when it took the problem, 0 when the shape is not eligible
// (the caller then uses the FP32 path), or a negative LTB_E_* code.
int gemm_tc(const float* a, bool a_kmajor, const float* b, bool b_kmajor, float* c, bool c_row_major,
            int M, int N, int K, float alpha, bool accumulate);
int conv_fwd_tc(const float* x, const float* w, const float* bias, float* y, const ConvDims& d);
int conv_dgrad_tc(const float* dy, const float* w, float* dx, const ConvDims& d, bool* fresh);
int conv_wgrad_tc(const float* x, const float* dy, float* dw, const ConvDims& d);
// Before the two halves of a convolution's backward call are issued: stages what both will read (one channels-last copy of dy).
int conv_bwd_prestage(const float* dy, const ConvDims& d, bool both_halves);

}  // namespace ltb
