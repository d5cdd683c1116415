// C-ABI entry points of the contraction family: they validate shapes, then route each problem to the TF32
// tensor-core engine (gemm_tc.cu) when the math mode allows it and the shape is eligible, else to the FP32
// CUDA-core path (gemm_fp32.cu).  There is no library (cuBLAS/cuDNN) and no CPU path behind either.
#include "gemm.cuh"

using namespace ltb;

namespace {

// C[M,N] (op)= alpha * op(A) op(B); A stored [M,K] (ta=0) or [K,M]; B stored [K,N] (tb=0) or [N,K].
int gemm_any(const float* a, bool ta, const float* b, bool tb, float* c, int M, int N, int K, float alpha, bool acc) {
  if (g.math == LTB_MATH_TF32) {
    int r = gemm_tc(a, /*a_kmajor=*/!ta, b, /*b_kmajor=*/tb, c, true, M, N, K, alpha, acc);
    if (r != 0) return r < 0 ? r : LTB_OK;
  }
  return gemm_fp32(a, ta ? 1 : K, ta ? M : 1, b, tb ? 1 : N, tb ? K : 1, c, N, 1, M, N, K, alpha, acc);
}

bool conv_dims(ConvDims& d, int N, int C, int H, int W, int K, int R, int S, int sh, int sw, int ph, int pw) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || K <= 0 || R <= 0 || S <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0) return false;
  d = ConvDims{N, C, H, W, K, R, S, sh, sw, ph, pw, (H + 2 * ph - R) / sh + 1, (W + 2 * pw - S) / sw + 1};
  if (H + 2 * ph < R || W + 2 * pw < S) return false;
  return (int64_t)N * d.oH * d.oW < (1ll << 31) && (int64_t)N * H * W < (1ll << 31) && (int64_t)C * R * S < (1ll << 31);
}

// A convolution whose filter covers the whole unpadded image has one output pixel per image and is a plain matrix
// product over (channel, row, column): y[N][K] = x[N][CHW] w[K][CHW]^T (the last layer of the reference's SqueezeNet, a 4x4
// filter on 4x4 maps).  The gemm paths split a long reduction over the machine; the convolution paths would give it to one tile.
bool covers_image(const ConvDims& d) { return d.R == d.H && d.S == d.W && d.ph == 0 && d.pw == 0 && d.oH == 1 && d.oW == 1; }

}  // namespace

extern "C" {

// matrixMatrixDot and the (2,2) case of dot_grad: TensorDslCPU.scala:158-169, 208-225.
int ltb_mm_dot(const float* a, const float* b, float* out, int m, int k, int n) {
  LTB_INITED(); LTB_REQUIRE(a && b && out && m > 0 && k > 0 && n > 0, "ltb_mm_dot: bad argument");
  return gemm_any(a, false, b, false, out, m, n, k, 1.0f, false);
}
int ltb_add_dot_trans1(float* db, const float* a, const float* dc, int m, int k, int n) {   // dB[k,n] += A^T[k,m] dC[m,n]
  LTB_INITED(); LTB_SETTLE(db); LTB_SETTLE(dc); LTB_REQUIRE(db && a && dc && m > 0 && k > 0 && n > 0, "ltb_add_dot_trans1: bad argument");
  return gemm_any(a, true, dc, false, db, k, n, m, 1.0f, true);
}
int ltb_add_dot_trans2(float* da, const float* dc, const float* b, int m, int k, int n) {   // dA[m,k] += dC[m,n] B^T[n,k]
  LTB_INITED(); LTB_SETTLE(da); LTB_SETTLE(dc); LTB_REQUIRE(da && dc && b && m > 0 && k > 0 && n > 0, "ltb_add_dot_trans2: bad argument");
  return gemm_any(dc, false, b, true, da, m, k, n, 1.0f, true);
}

// gemm: TensorDslCPU.scala:379-426.
int ltb_gemm(const float* a, int ta, const float* b, int tb, float alpha, float* c, int M, int N, int K) {
  LTB_INITED(); LTB_REQUIRE(a && b && c && M > 0 && N > 0 && K > 0, "ltb_gemm: bad argument");
  return gemm_any(a, ta != 0, b, tb != 0, c, M, N, K, alpha, false);
}
// gemm_grad: the eight cblas_sgemm calls of TensorDslCPU.scala:428-472, all with beta = 1.
int ltb_gemm_grad(const float* a, float* da, int ta, const float* b, float* db, int tb, float alpha, const float* dc, int M, int N, int K) {
  LTB_INITED(); LTB_SETTLE(da); LTB_SETTLE(db); LTB_SETTLE(dc); LTB_REQUIRE(a && b && dc && M > 0 && N > 0 && K > 0, "ltb_gemm_grad: bad argument");
  int rc = LTB_OK;
  if (!ta && !tb) {
    if (da) rc = gemm_any(dc, false, b, true, da, M, K, N, alpha, true);             // dA[M,K] += dC B^T
    if (!rc && db) rc = gemm_any(a, true, dc, false, db, K, N, M, alpha, true);      // dB[K,N] += A^T dC
  } else if (!ta && tb) {
    if (da) rc = gemm_any(dc, false, b, false, da, M, K, N, alpha, true);            // dA[M,K] += dC B      (B is [N,K])
    if (!rc && db) rc = gemm_any(dc, true, a, false, db, N, K, M, alpha, true);      // dB[N,K] += dC^T A
  } else if (ta && !tb) {
    if (da) rc = gemm_any(b, false, dc, true, da, K, M, N, alpha, true);             // dA[K,M] += B dC^T
    if (!rc && db) rc = gemm_any(a, false, dc, false, db, K, N, M, alpha, true);     // dB[K,N] += A dC      (A is [K,M])
  } else {
    if (da) rc = gemm_any(b, true, dc, true, da, K, M, N, alpha, true);              // dA[K,M] += B^T dC^T  (B is [N,K])
    if (!rc && db) rc = gemm_any(dc, true, a, true, db, N, K, M, alpha, true);       // dB[N,K] += dC^T A^T
  }
  return rc;
}

// conv2D_batch: TensorDslCPU.scala:532-571.
int ltb_conv2d_fwd(const float* x, const float* w, const float* bias, float* y, int N, int C, int H, int W, int K, int R, int S,
                   int sh, int sw, int ph, int pw) {
  LTB_INITED(); ConvDims d;
  LTB_REQUIRE(x && w && y && conv_dims(d, N, C, H, W, K, R, S, sh, sw, ph, pw), "ltb_conv2d_fwd: bad argument");
  if (covers_image(d) && d.R * d.S > 1) {
    if (bias) { int rc = ltb_fill_with_bias(y, bias, N, K, 1); if (rc) return rc; }
    return gemm_any(x, false, w, true, y, N, K, C * R * S, 1.0f, bias != nullptr);
  }
  if (g.math == LTB_MATH_TF32) { int r = conv_fwd_tc(x, w, bias, y, d); if (r != 0) return r < 0 ? r : LTB_OK; }
  return conv_fwd_fp32(x, w, bias, y, d);
}
// conv2D_batch_grad: TensorDslCPU.scala:575-692. dx, dw, dbias accumulate; dx is NULL for a leaf input.
int ltb_conv2d_bwd(const float* x, float* dx, const float* w, float* dw, float* dbias, const float* dy, int N, int C, int H, int W,
                   int K, int R, int S, int sh, int sw, int ph, int pw) {
  LTB_INITED(); ConvDims d;
  LTB_REQUIRE(x && w && dy && conv_dims(d, N, C, H, W, K, R, S, sh, sw, ph, pw), "ltb_conv2d_bwd: bad argument");
  int rc = LTB_OK;
  LTB_SETTLE(dy);
  if (covers_image(d) && d.R * d.S > 1) {
    LTB_SETTLE(dx);
    const int crs = C * R * S;
    if (dw) rc = gemm_any(dy, true, x, false, dw, K, crs, N, 1.0f, true);           // dw[K][CHW] += dy^T x
    if (!rc && dx) rc = gemm_any(dy, false, w, false, dx, N, crs, K, 1.0f, true);   // dx[N][CHW] += dy w
    if (!rc && dbias) rc = conv_bias_grad(dy, dbias, d);
    return rc;
  }
  // The two halves are independent (dx needs dy and w; dw needs dy and x). When both are asked for, the weight-gradient
  // half is issued on the side stream and the data-gradient half on the caller's, and the caller's stream waits for both
  // before the call returns: program order at the boundary is unchanged, and inside a recorded step the two become
  // parallel branches of the graph. Per-launch profiling keeps them serial so that each kernel is timed alone.
  // dx declared unset (ltb_grad_unset): the engine's data-grad writes instead of adding; any other path starts from zeros
  bool fresh = dx && g.math == LTB_MATH_TF32 && grad_take_unset(dx, (size_t)N * C * H * W * 4);
  if (!fresh) LTB_SETTLE(dx);
  if (g.math == LTB_MATH_TF32) { rc = conv_bwd_prestage(dy, d, dx && dw); if (rc) return rc; }
  const bool overlap = dx && dw && !g.profiling && g.side != nullptr;
  const size_t arena_base = g.used;
  cudaStream_t main_stream = g.stream;
  if (overlap) {
    LTB_CUDA(cudaEventRecord(g.fork_ev, main_stream));
    LTB_CUDA(cudaStreamWaitEvent(g.side, g.fork_ev, 0));
    g.hold_workspace = true;
    g.stream = g.side;
  }
  if (dw) {
    int r = g.math == LTB_MATH_TF32 ? conv_wgrad_tc(x, dy, dw, d) : 0;
    if (r == 0) rc = conv_wgrad_fp32(x, dy, dw, d); else if (r < 0) rc = r;
  }
  if (overlap) g.stream = main_stream;
  if (dx && rc == LTB_OK) {
    int r = g.math == LTB_MATH_TF32 ? conv_dgrad_tc(dy, w, dx, d, &fresh) : 0;
    if (r == 0 && fresh) { fresh = false; if (cudaMemsetAsync(dx, 0, (size_t)N * C * H * W * 4, g.stream) != cudaSuccess) rc = fail(LTB_E_CUDA, "ltb_conv2d_bwd: zero fill failed"); }
    if (r == 0 && !rc) rc = conv_dgrad_fp32(dy, w, dx, d); else if (r < 0) rc = r;
  }
  if (overlap) {                                   // join, also on the error path: nothing may stay forked
    g.hold_workspace = false;
    if (!g.branch_marked) g.used = arena_base;
    cudaError_t e1 = cudaEventRecord(g.join_ev, g.side);
    cudaError_t e2 = cudaStreamWaitEvent(main_stream, g.join_ev, 0);
    if (rc == LTB_OK && (e1 != cudaSuccess || e2 != cudaSuccess)) return fail(LTB_E_CUDA, "ltb_conv2d_bwd: joining the side stream failed");
  }
  if (rc) return rc;
  if (dbias) rc = conv_bias_grad(dy, dbias, d);
  return rc;
}

}  // extern "C"
