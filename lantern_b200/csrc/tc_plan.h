// Host-side plans for the TF32 tensor-core engine (pure C++, no CUDA: also compiled into the CPU layout test).
//
// The engine kernel (gemm_tc.cu) is generic: for every operand it is told how to turn (output tile, k-iteration) into
// TMA box coordinates, how many bytes a stage holds, and the UMMA shared-memory descriptors of the MMA steps of a stage.
// Everything that depends on the tensor layout (NCHW activations with pixels contiguous, OIHW filters, row-major
// matrices, tiny images) is decided here and expressed in those numbers.
//
// Shared-memory layouts are the canonical UMMA layouts for 32-bit operands:
//   K-major,  swizzle span X bytes : rows of X bytes (X/4 floats of K), 8-row groups SBO apart; an MMA step covers 32 B of K
//   MN-major (32-bit operands)     : the only layout the tensor core accepts is the 128-byte swizzle with 32-byte atoms:
//                                    chunks of 32 elements of M (or N) contiguous (128 B), one row per k, 4 k-rows per group
//                                    (512 B), groups SBO apart, chunks LBO apart; an MMA step (K = 8) spans two groups.
//   no swizzle (K-major only)      : 16-byte rows, 8-row groups SBO apart, the second 16-byte k-chunk LBO apart.
// A TMA box whose inner extent is X bytes, loaded with the matching swizzle mode, lands in exactly that layout.
// Operands whose contiguous axis is shorter than 128 bytes cannot be fed MN-major; the callers hand those in as K-major
// row matrices instead (`a_rows`), produced by a small transposing copy.
#pragma once
#include <cstdint>

namespace ltb {

enum TcSwizzle { TC_SW_NONE = 0, TC_SW_32 = 1, TC_SW_64 = 2, TC_SW_128 = 3, TC_SW_128_32B = 4 };

struct TcTensorMap {          // arguments of cuTensorMapEncodeTiled for one FP32 operand
  const void* base;
  int rank;
  uint64_t dims[5];           // innermost first
  uint64_t strides[5];        // bytes; strides[0] is implied (4) and unused
  uint32_t box[5];
  int swizzle;                // TcSwizzle
};

struct TcOperand {
  TcTensorMap map;
  // box coordinate d = c_off[d] + ((tile / t_div[d]) % t_mod[d]) * t_mul[d] + ((kiter / k_div[d]) % k_mod[d]) * k_mul[d]
  // (c_off and k_mul may be negative: the taps of a convolution window start left of / above the image, where TMA fills zeros)
  int t_div[5], t_mod[5], t_mul[5];
  int k_div[5], k_mod[5], k_mul[5];
  int c_off[5];
  uint32_t stage_bytes;       // bytes one stage of this operand occupies (== bytes the TMA box delivers)
  int mn_major;               // 0: K-major, 1: M/N-major (instruction descriptor transpose bit)
  uint32_t lbo, sbo;          // bytes
  int nk;                     // MMA steps (K = 8 each) per stage
  uint32_t kstep_off[8];      // start-address offset of each step within the stage
};

// The k part of the coordinates as a mixed-radix counter, so that the single producer thread advances them with additions
// only: level 0 steps n0 times, then level 1 steps once (and level 0 returns to its start), after n1 of those level 2
// steps.  inc[j][d] is what reaching level j adds to coordinate d (returns of the lower levels included).
struct TcWalk { int n0, n1; int inc[3][5]; };
bool tc_walk_of(const TcOperand& o, TcWalk& w);

enum TcEpilogue {
  TC_EPI_PIXEL = 0,   // D row = pixel, D column = channel: out[img][chan][pix]   (conv forward / data-grad)
  TC_EPI_ROWMAJOR = 1 // D row = row, D column contiguous:   out[row*ld + col]      (gemm, weight-grad)
};

struct TcPlan {
  TcOperand a, b;             // a: the M-side operand (128 rows per tile), b: the N-side operand (bn columns per tile)
  int M, N;                   // logical extents of D
  int bn;                     // tile width: 64, 128 or 256
  int m_tiles, n_tiles, k_iters, splits;
  int epilogue;
  float* out;
  const float* bias;          // per D column, or null
  float alpha;
  int accumulate;             // 1: out += ..., 0: out = ...   (split-K > 1 forces atomic accumulation)
  int64_t pix_per_img, img_stride, chan_stride;   // TC_EPI_PIXEL
  int64_t ld;                                     // TC_EPI_ROWMAJOR
  int col_mod, col_mul;                           // TC_EPI_ROWMAJOR, when col_mul != 0: D column n is stored at column (n % col_mod) * col_mul + n / col_mod
  // Gather mode (tc_plan_gather): operand a keeps its K-major row descriptors but is not loaded by TMA; the kernel's
  // epilogue warps collect it from gather_src[img][chan][pix] (pix = 4 or 16), warp g filling rows 16 g .. 16 g + 15 of
  // the tile, lane = channel within the 32-channel block, 128-byte swizzle.
  const float* gather_src;
  int g_pix, g_chan, g_imgs;
};

// "Flat" convolution view: activations X[n][k][p] with p contiguous (k = channels, or channels*kh*kw after unfolding),
// weights W[co][k] row-major with ldw >= k floats per row (zeros beyond k: the caller pads a copy when the engine needs a
// wider row -- forward: ldw a multiple of 4, dgrad: a multiple of 32), outputs Y[n][co][p].  P is the number of pixels per image.
//   forward : Y[n][co][p]  = sum_k  W[co][k] X[n][k][p] (+ bias[co])         D = pixels x co
//   dgrad   : dX[n][k][p] (+)= sum_co W[co][k] dY[n][co][p]                   D = pixels x k
//   wgrad   : dW[co][k]  += sum_{n,p} dY[n][co][p] X[n][k][p]                 D = co x k
// Each returns false when the shape is not eligible (the caller then uses the FP32 path).
// a_rows: the activation operand (x for forward, dy for dgrad) is given as a K-major row matrix [n_img*pix][channels]
// instead of [n_img][channels][pix]; tc_conv_needs_rows says when that form is required.
bool tc_conv_needs_rows(int pix);
// Whether an activation [n_img][chan][pix] that needs the row form can be gathered by the kernel itself instead of being
// copied into a row matrix first; tc_plan_gather switches a plan made with a_rows = true (x = src as base) to that mode.
bool tc_gather_possible(const float* src, int chan, int pix);
void tc_plan_gather(TcPlan& p, const float* src, int n_img, int chan, int pix);
bool tc_plan_conv_fwd(TcPlan& p, const float* x, bool a_rows, const float* w, int ldw, const float* bias, float* y, int n_img, int ck, int co, int pix, int sm_count);
bool tc_plan_conv_dgrad(TcPlan& p, const float* dy, bool a_rows, const float* w, int ldw, float* dx, int n_img, int ck, int co, int pix, bool accumulate, int sm_count);
bool tc_plan_conv_wgrad(TcPlan& p, const float* x, const float* dy, float* dw, int n_img, int ck, int co, int pix, int sm_count);
// Implicit ("tap loop") forms for R x S convolutions with stride 1.  The activations are channels-last copies
// xr[n][h][w][c] and dyr[n][oh][ow][k] (made by a transposing copy); a TMA box then is a window of whole image rows
// with 32 channels, and the tap (r, s) only shifts the box coordinates -- the nine-fold unfolded matrix never exists.
//   forward : rows = output pixels, K loop = (r, s, channel block); weights permuted to wt[r*S+s][k][c]
//   dgrad   : rows = input pixels,  K loop = (r, s, k block);       weights permuted to wd[r*S+s][c][k]
//   wgrad   : D = k x (tap, c), K loop = blocks of 32 pixels, both operands M/N-major; stored to OIHW through col_mod/col_mul
struct TcConvGeom { int n_img, C, H, W, K, R, S, ph, pw, oH, oW; };
bool tc_plan_conv_taps_fwd(TcPlan& p, const float* xr, const float* wt, const float* bias, float* y, const TcConvGeom& g, int sm_count);
bool tc_plan_conv_taps_dgrad(TcPlan& p, const float* dyr, const float* wd, float* dx, const TcConvGeom& g, bool accumulate, int sm_count);
bool tc_plan_conv_taps_wgrad(TcPlan& p, const float* dyr, const float* xr, float* dw, const TcConvGeom& g, int sm_count);
// C[M,N] (op)= alpha * A B; a_kmajor: A stored [M,K] (else [K,M]); b_kmajor: B stored [N,K] (else [K,N]).
bool tc_plan_gemm(TcPlan& p, const float* a, bool a_kmajor, const float* b, bool b_kmajor, float* c, int M, int N, int K, float alpha,
                  bool accumulate, int sm_count);

}  // namespace ltb
