// CPU check of the tensor-core engine's bookkeeping (test infrastructure).
//
// Emulates, for every plan the planner produces, (1) what a tiled TMA load writes to shared memory (box order, out-of-
// bounds zero fill, 32/64/128-byte swizzle as an XOR of address bits [4,7) with bits [7,10)), (2) which element the
// tensor core reads for (row, k) of an MMA step from the canonical UMMA layout described by the step's descriptor
// (start offset, LBO, SBO, swizzle, major-ness), and (3) the epilogue's output indexing.  The result of the emulated
// engine is compared with a direct evaluation of the convolution / GEMM.  This pins coordinates, strides, descriptors
// and tile/split arithmetic without a GPU; it does not prove that the hardware follows the emulated conventions.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../lantern_b200/csrc/tc_plan.h"

using namespace ltb;

static uint32_t swz(uint32_t off, int mode) {
  if (mode == TC_SW_128_32B) return off ^ (((off >> 7) & 3u) << 5);       // 32-byte atoms: bits [5,7) ^= bits [7,9)
  int bits = mode == TC_SW_128 ? 3 : mode == TC_SW_64 ? 2 : mode == TC_SW_32 ? 1 : 0;
  return off ^ (((off >> 7) & ((1u << bits) - 1)) << 4);
}
static int span(int mode) { return (mode == TC_SW_128 || mode == TC_SW_128_32B) ? 128 : mode == TC_SW_64 ? 64 : mode == TC_SW_32 ? 32 : 16; }

static void coords_of(const TcOperand& o, int tile, int kiter, int64_t* c) {
  for (int d = 0; d < 5; ++d) c[d] = (int64_t)o.c_off[d] + (int64_t)((tile / o.t_div[d]) % o.t_mod[d]) * o.t_mul[d] + (int64_t)((kiter / o.k_div[d]) % o.k_mod[d]) * o.k_mul[d];
}
static bool tma_load(const TcOperand& o, int tile, int kiter, std::vector<float>& smem) {
  const TcTensorMap& m = o.map;
  int64_t c[5]; coords_of(o, tile, kiter, c);
  if ((c[0] * 4) % 16) { printf("unaligned innermost TMA coordinate %lld\n", (long long)c[0]); return false; }
  for (int d = 1; d < m.rank; ++d) if (m.strides[d] % 16) { printf("stride %d not a multiple of 16 bytes\n", d); return false; }
  if ((m.box[0] * 4) % 16 || (int)m.box[0] * 4 > span(m.swizzle) && m.swizzle != TC_SW_NONE) { printf("bad inner box\n"); return false; }
  int64_t total = 1; for (int d = 0; d < m.rank; ++d) { if (m.box[d] > 256) { printf("box > 256\n"); return false; } total *= m.box[d]; }
  if (total * 4 != o.stage_bytes) { printf("stage_bytes %u != box bytes %lld\n", o.stage_bytes, (long long)total * 4); return false; }
  smem.assign(o.stage_bytes / 4, 0.0f);
  for (int64_t lin = 0; lin < total; ++lin) {
    int64_t r = lin, goff = 0; bool inb = true;
    for (int d = 0; d < m.rank; ++d) {
      int64_t i = r % m.box[d]; r /= m.box[d];
      int64_t g = c[d] + i;
      if (g < 0 || g >= (int64_t)m.dims[d]) inb = false;
      goff += g * (d == 0 ? 4 : (int64_t)m.strides[d]);
    }
    float v = inb ? *(const float*)((const char*)m.base + goff) : 0.0f;
    smem[swz((uint32_t)lin * 4, m.swizzle) / 4] = v;
  }
  return true;
}
// What the kernel's gathering warps store for operand a of a plan in gather mode (gemm_tc.cu): warp g, lane l, run j, element
// i write row 16 g + 4 j + i, channel l of the 32-channel block, at 16-byte chunk (l >> 2) ^ (row & 7) of the 128-byte row.
static bool gather_load(const TcPlan& p, int tile, int kiter, std::vector<float>& smem) {
  if (p.a.stage_bytes != 128 * 128 || p.a.mn_major || p.a.map.swizzle != TC_SW_128) { printf("gather mode needs a K-major 128-byte-swizzled operand\n"); return false; }
  smem.assign(p.a.stage_bytes / 4, 0.0f);
  const int pix = p.g_pix, chan = p.g_chan, runs = 16 / pix;
  for (int gw = 0; gw < 8; ++gw) for (int lane = 0; lane < 32; ++lane) {
    const int64_t row0 = (int64_t)tile * 128 + gw * 16, img0 = row0 / pix;
    const int c = kiter * 32 + lane;
    for (int j = 0; j < 4; ++j) for (int i = 0; i < 4; ++i) {
      const int64_t img = runs == 1 ? img0 : img0 + j;
      const int q = runs == 1 ? j * 4 + i : i;
      const float v = (c < chan && img < p.g_imgs) ? p.gather_src[(img * chan + c) * pix + q] : 0.0f;
      const uint32_t r = (uint32_t)(j * 4 + i);
      const uint32_t off = (uint32_t)gw * 16 * 128 + r * 128 + (((((uint32_t)lane >> 2) ^ (r & 7u)) << 4) | (((uint32_t)lane & 3u) << 2));
      smem[off / 4] = v;
    }
  }
  return true;
}
// Element (r, kk) of MMA step `ks`: r = row (M or N index within the tile), kk in [0,8).
static float umma_fetch(const TcOperand& o, const std::vector<float>& smem, int ks, int r, int kk) {
  const int X = span(o.map.swizzle); uint32_t off = o.kstep_off[ks];
  if (!o.mn_major) {
    if (o.map.swizzle != TC_SW_NONE) off += (uint32_t)(r / 8) * o.sbo + (uint32_t)(r % 8) * X + (uint32_t)kk * 4;
    else off += (uint32_t)(r / 8) * o.sbo + (uint32_t)(r % 8) * 16 + (uint32_t)(kk / 4) * o.lbo + (uint32_t)(kk % 4) * 4;
  } else {
    // 32-bit operands: only the 128-byte swizzle with 32-byte atoms exists (chunks of 32 elements, 4 k-rows per group)
    if (o.map.swizzle != TC_SW_128_32B) { printf("MN-major operand with an unsupported swizzle mode\n"); exit(1); }
    off += (uint32_t)(r / 32) * o.lbo + (uint32_t)(kk / 4) * o.sbo + (uint32_t)(kk % 4) * 128 + (uint32_t)(r % 32) * 4;
  }
  off = swz(off, o.map.swizzle);
  if (off / 4 >= smem.size()) { printf("MMA read beyond the stage (%u >= %zu)\n", off, smem.size() * 4); exit(1); }
  return smem[off / 4];
}

// The producer's incremental walk (TcWalk) must visit the coordinates the closed formula gives, from any starting iteration.
static bool walk_matches(const TcOperand& o, int tile, int k_iters) {
  TcWalk w;
  if (!tc_walk_of(o, w)) { printf("operand has no walk\n"); return false; }
  for (int k0 = 0; k0 < k_iters; k0 += (k_iters > 7 ? k_iters / 7 : 1)) {
    int64_t c[5]; coords_of(o, tile, k0, c);
    int i0 = k0 % w.n0, i1 = (k0 / w.n0) % w.n1;
    for (int it = k0; it < k_iters; ++it) {
      int64_t want[5]; coords_of(o, tile, it, want);
      for (int d = 0; d < 5; ++d) if (c[d] != want[d]) { printf("walk: coordinate %d at iteration %d (start %d): %lld, formula %lld\n", d, it, k0, (long long)c[d], (long long)want[d]); return false; }
      int lvl = 0;
      if (++i0 == w.n0) { i0 = 0; lvl = 1; if (++i1 == w.n1) { i1 = 0; lvl = 2; } }
      for (int d = 0; d < 5; ++d) c[d] += w.inc[lvl][d];
    }
  }
  return true;
}

static bool run_plan(const TcPlan& p, size_t out_count) {
  if (p.a.nk != p.b.nk) { printf("nk mismatch\n"); return false; }
  if (!walk_matches(p.a, p.m_tiles - 1, p.k_iters) || !walk_matches(p.b, p.n_tiles - 1, p.k_iters)) return false;
  // overwrite semantics under split-K: the partial results of the splits are summed and then stored; emulated by zeroing first
  if (p.splits > 1 && !p.accumulate) for (size_t i = 0; i < out_count; ++i) p.out[i] = 0.0f;
  std::vector<float> sa, sb;
  for (int mt = 0; mt < p.m_tiles; ++mt) for (int nt = 0; nt < p.n_tiles; ++nt) for (int z = 0; z < p.splits; ++z) {
    int per = (p.k_iters + p.splits - 1) / p.splits, k0 = z * per, k1 = k0 + per < p.k_iters ? k0 + per : p.k_iters;
    if (k0 >= k1) continue;
    std::vector<double> D((size_t)128 * p.bn, 0.0);
    for (int it = k0; it < k1; ++it) {
      if (!(p.gather_src ? gather_load(p, mt, it, sa) : tma_load(p.a, mt, it, sa)) || !tma_load(p.b, nt, it, sb)) return false;
      for (int ks = 0; ks < p.a.nk; ++ks) for (int r = 0; r < 128; ++r) for (int c = 0; c < p.bn; ++c) {
        double s = 0; for (int kk = 0; kk < 8; ++kk) s += (double)umma_fetch(p.a, sa, ks, r, kk) * umma_fetch(p.b, sb, ks, c, kk);
        D[(size_t)r * p.bn + c] += s;
      }
    }
    bool atomic = p.splits > 1;
    for (int r = 0; r < 128; ++r) for (int c = 0; c < p.bn; ++c) {
      int64_t m = (int64_t)mt * 128 + r, n = (int64_t)nt * p.bn + c;
      if (m >= p.M || n >= p.N) continue;
      int64_t idx = p.epilogue == TC_EPI_PIXEL ? (m / p.pix_per_img) * p.img_stride + n * p.chan_stride + (m % p.pix_per_img)
                                                : m * p.ld + (p.col_mul ? (n % p.col_mod) * p.col_mul + n / p.col_mod : n);
      if ((size_t)idx >= out_count) { printf("epilogue index out of range\n"); return false; }
      float v = p.alpha * (float)D[(size_t)r * p.bn + c] + ((p.bias && z == 0) ? p.bias[n] : 0.0f);
      if (p.accumulate || atomic) p.out[idx] += v; else p.out[idx] = v;
    }
  }
  return true;
}

static std::vector<float> rnd(size_t n, unsigned seed) { std::vector<float> v(n); srand(seed); for (auto& x : v) x = (float)(rand() % 17 - 8) / 4.0f; return v; }
static bool close(const std::vector<float>& a, const std::vector<float>& b, const char* what) {
  for (size_t i = 0; i < a.size(); ++i) if (std::fabs(a[i] - b[i]) > 1e-3f * (1.0f + std::fabs(a[i]))) { printf("%s: mismatch at %zu: %f vs %f\n", what, i, a[i], b[i]); return false; }
  return true;
}

static int conv_case(int n_img, int ck, int co, int pix) {
  auto x = rnd((size_t)n_img * ck * pix, 1), w = rnd((size_t)co * ck, 2), dy = rnd((size_t)n_img * co * pix, 3), bias = rnd(co, 4);
  // TMA bases must be 16-byte aligned: std::vector<float> storage from operator new is.
  std::vector<float> y((size_t)n_img * co * pix, 7.0f), yr(y.size()), dx((size_t)n_img * ck * pix, 0.5f), dxr(dx), dw((size_t)co * ck, -1.0f), dwr(dw);
  for (int n = 0; n < n_img; ++n) for (int c = 0; c < co; ++c) for (int q = 0; q < pix; ++q) {
    double s = bias[c]; for (int k = 0; k < ck; ++k) s += (double)w[(size_t)c * ck + k] * x[((size_t)n * ck + k) * pix + q];
    yr[((size_t)n * co + c) * pix + q] = (float)s;
  }
  for (int n = 0; n < n_img; ++n) for (int k = 0; k < ck; ++k) for (int q = 0; q < pix; ++q) {
    double s = 0; for (int c = 0; c < co; ++c) s += (double)w[(size_t)c * ck + k] * dy[((size_t)n * co + c) * pix + q];
    dxr[((size_t)n * ck + k) * pix + q] += (float)s;
  }
  for (int c = 0; c < co; ++c) for (int k = 0; k < ck; ++k) {
    double s = 0; for (int n = 0; n < n_img; ++n) for (int q = 0; q < pix; ++q) s += (double)dy[((size_t)n * co + c) * pix + q] * x[((size_t)n * ck + k) * pix + q];
    dwr[(size_t)c * ck + k] += (float)s;
  }
  int taken = 0; TcPlan p;
  const bool rows = tc_conv_needs_rows(pix);
  std::vector<float> xt, dyt;           // K-major row copies [n*pix + q][channel], what the library's transposing copy produces
  if (rows) {
    xt.resize(x.size()); dyt.resize(dy.size());
    for (int n = 0; n < n_img; ++n) for (int q = 0; q < pix; ++q) {
      for (int k = 0; k < ck; ++k) xt[((size_t)n * pix + q) * ck + k] = x[((size_t)n * ck + k) * pix + q];
      for (int c = 0; c < co; ++c) dyt[((size_t)n * pix + q) * co + c] = dy[((size_t)n * co + c) * pix + q];
    }
  }
  // filter rows padded with zeros the way the library stages them: to 4 floats for forward, to 32 for data-grad
  auto padded = [&](int ld) { std::vector<float> o((size_t)co * ld, 0.0f); for (int c = 0; c < co; ++c) for (int k = 0; k < ck; ++k) o[(size_t)c * ld + k] = w[(size_t)c * ck + k]; return o; };
  const int ld4 = (ck + 3) / 4 * 4, ld32 = (ck + 31) / 32 * 32;
  const std::vector<float> w4 = padded(ld4), w32 = padded(ld32);
  if (tc_plan_conv_fwd(p, rows ? xt.data() : x.data(), rows, w4.data(), ld4, bias.data(), y.data(), n_img, ck, co, pix, 148)) { ++taken; if (!run_plan(p, y.size()) || !close(yr, y, "fwd")) return -1; }
  if (tc_plan_conv_dgrad(p, rows ? dyt.data() : dy.data(), rows, w32.data(), ld32, dx.data(), n_img, ck, co, pix, true, 148)) { ++taken; if (!run_plan(p, dx.size()) || !close(dxr, dx, "dgrad")) return -1; }
  // the same two contractions with the kernel gathering the activation itself (small images: 4 or 16 pixels)
  if (rows && tc_gather_possible(x.data(), ck, pix) && tc_gather_possible(dy.data(), co, pix)) {
    std::fill(y.begin(), y.end(), 7.0f); std::fill(dx.begin(), dx.end(), 0.5f);
    if (tc_plan_conv_fwd(p, x.data(), true, w4.data(), ld4, bias.data(), y.data(), n_img, ck, co, pix, 148)) {
      tc_plan_gather(p, x.data(), n_img, ck, pix); ++taken; if (!run_plan(p, y.size()) || !close(yr, y, "fwd (gather)")) return -1; }
    if (tc_plan_conv_dgrad(p, dy.data(), true, w32.data(), ld32, dx.data(), n_img, ck, co, pix, true, 148)) {
      tc_plan_gather(p, dy.data(), n_img, co, pix); ++taken; if (!run_plan(p, dx.size()) || !close(dxr, dx, "dgrad (gather)")) return -1; }
  }
  if (tc_plan_conv_wgrad(p, x.data(), dy.data(), dw.data(), n_img, ck, co, pix, 148)) { ++taken; if (!run_plan(p, dw.size()) || !close(dwr, dw, "wgrad")) return -1; }
  printf("conv n=%d ck=%d co=%d pix=%d: %d of 3 plans taken, all match\n", n_img, ck, co, pix, taken);
  return taken;
}

// R x S convolution with stride 1 through the tap-loop plans, against a direct evaluation.
static int taps_case(int n_img, int C, int K, int H, int W, int R, int S, int ph, int pw) {
  const int oH = H + 2 * ph - R + 1, oW = W + 2 * pw - S + 1, taps = R * S;
  TcConvGeom g{n_img, C, H, W, K, R, S, ph, pw, oH, oW};
  auto x = rnd((size_t)n_img * C * H * W, 11), w = rnd((size_t)K * C * taps, 12), dy = rnd((size_t)n_img * K * oH * oW, 13), bias = rnd(K, 14);
  std::vector<float> y((size_t)n_img * K * oH * oW, 7.0f), yr(y.size()), dx(x.size(), 0.5f), dxr(dx), dw(w.size(), -1.0f), dwr(dw);
  auto X = [&](int n, int c, int h, int ww) -> double { return (h < 0 || h >= H || ww < 0 || ww >= W) ? 0.0 : x[(((size_t)n * C + c) * H + h) * W + ww]; };
  for (int n = 0; n < n_img; ++n) for (int k = 0; k < K; ++k) for (int oh = 0; oh < oH; ++oh) for (int ow = 0; ow < oW; ++ow) {
    double s = bias[k];
    for (int c = 0; c < C; ++c) for (int r = 0; r < R; ++r) for (int q = 0; q < S; ++q) s += X(n, c, oh - ph + r, ow - pw + q) * w[(((size_t)k * C + c) * R + r) * S + q];
    yr[(((size_t)n * K + k) * oH + oh) * oW + ow] = (float)s;
    const double d = dy[(((size_t)n * K + k) * oH + oh) * oW + ow];
    for (int c = 0; c < C; ++c) for (int r = 0; r < R; ++r) for (int q = 0; q < S; ++q) {
      const int h = oh - ph + r, ww = ow - pw + q;
      if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
      dxr[(((size_t)n * C + c) * H + h) * W + ww] += (float)(d * w[(((size_t)k * C + c) * R + r) * S + q]);
      dwr[(((size_t)k * C + c) * R + r) * S + q] += (float)(d * x[(((size_t)n * C + c) * H + h) * W + ww]);
    }
  }
  // what the library's staging kernels produce: channels-last copies and per-tap weight matrices
  std::vector<float> xr(x.size()), dyr(dy.size()), wt(w.size()), wd(w.size());
  for (int n = 0; n < n_img; ++n) for (int c = 0; c < C; ++c) for (int i = 0; i < H * W; ++i) xr[((size_t)n * H * W + i) * C + c] = x[((size_t)n * C + c) * H * W + i];
  for (int n = 0; n < n_img; ++n) for (int k = 0; k < K; ++k) for (int i = 0; i < oH * oW; ++i) dyr[((size_t)n * oH * oW + i) * K + k] = dy[((size_t)n * K + k) * oH * oW + i];
  for (int k = 0; k < K; ++k) for (int c = 0; c < C; ++c) for (int t = 0; t < taps; ++t) {
    wt[((size_t)t * K + k) * C + c] = w[((size_t)k * C + c) * taps + t];
    wd[((size_t)t * C + c) * K + k] = w[((size_t)k * C + c) * taps + t];
  }
  int taken = 0; TcPlan p;
  if (tc_plan_conv_taps_fwd(p, xr.data(), wt.data(), bias.data(), y.data(), g, 148)) { ++taken; if (!run_plan(p, y.size()) || !close(yr, y, "taps fwd")) return -1; }
  if (tc_plan_conv_taps_dgrad(p, dyr.data(), wd.data(), dx.data(), g, true, 148)) { ++taken; if (!run_plan(p, dx.size()) || !close(dxr, dx, "taps dgrad")) return -1; }
  if (tc_plan_conv_taps_wgrad(p, dyr.data(), xr.data(), dw.data(), g, 148)) { ++taken; if (!run_plan(p, dw.size()) || !close(dwr, dw, "taps wgrad")) return -1; }
  printf("taps conv n=%d C=%d K=%d %dx%d k%dx%d pad %d,%d: %d of 3 plans taken, all match\n", n_img, C, K, H, W, R, S, ph, pw, taken);
  return taken;
}

static int gemm_case(int M, int N, int K, bool ak, bool bk, bool acc) {
  auto a = rnd((size_t)M * K, 5), b = rnd((size_t)N * K, 6);
  std::vector<float> c((size_t)M * N, 2.0f), cr(c);
  for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) {
    double s = 0; for (int k = 0; k < K; ++k) s += (double)(ak ? a[(size_t)m * K + k] : a[(size_t)k * M + m]) * (bk ? b[(size_t)n * K + k] : b[(size_t)k * N + n]);
    cr[(size_t)m * N + n] = (acc ? cr[(size_t)m * N + n] : 0.0f) + 0.5f * (float)s;
  }
  TcPlan p;
  if (!tc_plan_gemm(p, a.data(), ak, b.data(), bk, c.data(), M, N, K, 0.5f, acc, 148)) { printf("gemm %dx%dx%d ak=%d bk=%d: not eligible\n", M, N, K, ak, bk); return 0; }
  if (!run_plan(p, c.size()) || !close(cr, c, "gemm")) return -1;
  printf("gemm %dx%dx%d ak=%d bk=%d acc=%d: bn=%d splits=%d match\n", M, N, K, ak, bk, acc, p.bn, p.splits);
  return 1;
}

int main() {
  int bad = 0, taken = 0;
  const int convs[][4] = {{2, 64, 64, 256}, {3, 64, 256, 256}, {4, 128, 96, 64}, {5, 256, 128, 64}, {11, 256, 128, 16}, {35, 512, 64, 4}, {1, 32, 48, 1024},
                          {8, 576, 64, 256}, {2, 40, 64, 32}, {3, 64, 64, 36}, {2, 2048, 512, 4}, {9, 1024, 256, 16}, {70, 512, 32, 1},
                          // filter rows that need padding (3x3 over 3, 16 and 48 channels; 1x1 over 16 and 48) and few output channels
                          {2, 27, 96, 1024}, {3, 144, 64, 256}, {4, 16, 64, 256}, {2, 48, 192, 64}, {2, 432, 192, 64}, {3, 128, 12, 64}, {5, 48, 192, 16},
                          // small images of a 3x3 or strided convolution: the kernel gathers from the unfolded matrix [n][(c, r, s)][p]
                          {3, 2304, 256, 16}, {5, 4608, 128, 4}, {2, 72, 64, 16}};
  for (auto& c : convs) { int r = conv_case(c[0], c[1], c[2], c[3]); if (r < 0) ++bad; else taken += r; }
  const int taps[][9] = {{3, 64, 64, 16, 16, 3, 3, 1, 1}, {5, 128, 128, 8, 8, 3, 3, 1, 1}, {9, 64, 128, 4, 4, 3, 3, 1, 1}, {35, 64, 64, 2, 2, 3, 3, 1, 1},
                         {1, 32, 64, 32, 32, 3, 3, 1, 1}, {2, 64, 32, 16, 16, 3, 3, 0, 0}, {2, 64, 64, 8, 8, 5, 5, 2, 2}, {3, 96, 64, 8, 8, 1, 3, 0, 1},
                         {3, 64, 128, 16, 16, 1, 1, 0, 0}};
  int taps_taken = 0;
  for (auto& c : taps) { int r = taps_case(c[0], c[1], c[2], c[3], c[4], c[5], c[6], c[7], c[8]); if (r < 0) ++bad; else { taken += r; taps_taken += r; } }
  if (taps_taken < 17) { printf("too few tap-loop plans taken (%d)\n", taps_taken); ++bad; }
  for (int ak = 0; ak < 2; ++ak) for (int bk = 0; bk < 2; ++bk) for (int acc = 0; acc < 2; ++acc) {
    int r = gemm_case(160, 96, 72, ak, bk, acc); if (r < 0) ++bad; else taken += r;
    r = gemm_case(128, 256, 2048, ak, bk, acc); if (r < 0) ++bad; else taken += r;
  }
  printf("%d plans emulated, %d failures\n", taken, bad);
  return bad ? 1 : (taken >= 40 ? 0 : 2);
}
