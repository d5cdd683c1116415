// Planner of the TF32 tensor-core engine: see tc_plan.h.  Pure host code.
#include "tc_plan.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace ltb {

namespace {

constexpr int kBK = 32;          // K elements per pipeline stage (4 MMA steps of K = 8)
constexpr int kTileM = 128;      // UMMA M with one CTA

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
int cdiv(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

void clear(TcOperand& o) {
  std::memset(&o, 0, sizeof o);
  for (int d = 0; d < 5; ++d) {
    o.map.dims[d] = 1; o.map.strides[d] = 0; o.map.box[d] = 1;
    o.t_div[d] = 1; o.t_mod[d] = 1 << 30; o.t_mul[d] = 0;
    o.k_div[d] = 1; o.k_mod[d] = 1 << 30; o.k_mul[d] = 0;
  }
}

// Operand indexed [img][k][pix] (pix contiguous) whose M/N index is the pixel (img, pix) and whose K index is k.
// One tile = `kTileM` pixels.  Returns the number of k-iterations through *k_iters.
bool operand_mn_pixels(TcOperand& o, const float* base, int n_img, int kdim, int pix, int* k_iters) {
  clear(o);
  if (!aligned16(base) || kdim < 1 || n_img < 1) return false;
  o.map.base = base; o.mn_major = 1; o.nk = 4; o.stage_bytes = kTileM * kBK * 4;
  *k_iters = cdiv(kdim, kBK);
  if (pix >= 32 && pix % 32 == 0) {
    int cpt, ipt, tpi;
    if (pix >= kTileM) { if (pix % kTileM) return false; cpt = kTileM / 32; ipt = 1; tpi = pix / kTileM; }
    else { if (kTileM % pix) return false; cpt = pix / 32; ipt = kTileM / pix; tpi = 1; }
    o.map.rank = 4; o.map.swizzle = TC_SW_128_32B;
    o.map.dims[0] = 32; o.map.dims[1] = (uint64_t)kdim; o.map.dims[2] = (uint64_t)pix / 32; o.map.dims[3] = (uint64_t)n_img;
    o.map.strides[1] = (uint64_t)pix * 4; o.map.strides[2] = 128; o.map.strides[3] = (uint64_t)kdim * pix * 4;
    o.map.box[0] = 32; o.map.box[1] = kBK; o.map.box[2] = (uint32_t)cpt; o.map.box[3] = (uint32_t)ipt;
    o.k_mul[1] = kBK;
    o.t_div[2] = 1; o.t_mod[2] = tpi; o.t_mul[2] = cpt;          // chunk coordinate inside the image
    o.t_div[3] = tpi; o.t_mul[3] = ipt;                          // image coordinate
    o.lbo = kBK * 128; o.sbo = 512;                              // chunk stride; stride between the 4-row groups
    for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 1024;
    return true;
  }
  return false;
}

// Row-major matrix [rows][kdim] used K-major (rows = M or N index). One tile = tile_rows rows.
bool operand_k_rows(TcOperand& o, const float* base, int rows, int kdim, int tile_rows, int* k_iters) {
  clear(o);
  if (!aligned16(base) || kdim % 4 || rows < 1) return false;
  o.map.base = base; o.mn_major = 0; o.nk = 4; o.stage_bytes = (uint32_t)tile_rows * 128;
  o.map.rank = 2; o.map.swizzle = TC_SW_128;
  o.map.dims[0] = (uint64_t)kdim; o.map.dims[1] = (uint64_t)rows;
  o.map.strides[1] = (uint64_t)kdim * 4;
  o.map.box[0] = kBK; o.map.box[1] = (uint32_t)tile_rows;
  o.k_mul[0] = kBK; o.t_mul[1] = tile_rows;
  o.lbo = 16; o.sbo = 1024;
  for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 32;
  *k_iters = cdiv(kdim, kBK);
  return true;
}

// Row-major matrix [kdim][cols] used M/N-major (cols = M or N index, contiguous). One tile = tile_cols columns.
bool operand_mn_cols(TcOperand& o, const float* base, int kdim, int cols, int tile_cols, int* k_iters) {
  clear(o);
  if (!aligned16(base) || cols % 32 || kdim < 1) return false;
  o.map.base = base; o.mn_major = 1; o.nk = 4; o.stage_bytes = (uint32_t)tile_cols * 128;
  o.map.rank = 3; o.map.swizzle = TC_SW_128_32B;
  o.map.dims[0] = 32; o.map.dims[1] = (uint64_t)kdim; o.map.dims[2] = (uint64_t)cols / 32;
  o.map.strides[1] = (uint64_t)cols * 4; o.map.strides[2] = 128;
  o.map.box[0] = 32; o.map.box[1] = kBK; o.map.box[2] = (uint32_t)tile_cols / 32;
  o.k_mul[1] = kBK; o.t_mul[2] = tile_cols / 32;
  o.lbo = kBK * 128; o.sbo = 512;
  for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 1024;
  *k_iters = cdiv(kdim, kBK);
  return true;
}

// Operand indexed [img][row][pix] used K-major with the reduction running over (img, pix). One tile = tile_rows rows.
bool operand_k_pixels(TcOperand& o, const float* base, int n_img, int rows, int pix, int tile_rows, int* k_iters) {
  clear(o);
  if (!aligned16(base) || rows < 1 || n_img < 1) return false;
  o.map.base = base; o.mn_major = 0; o.nk = 4; o.stage_bytes = (uint32_t)tile_rows * 128;
  o.map.rank = 3;
  o.map.dims[0] = (uint64_t)pix; o.map.dims[1] = (uint64_t)rows; o.map.dims[2] = (uint64_t)n_img;
  o.map.strides[1] = (uint64_t)pix * 4; o.map.strides[2] = (uint64_t)rows * pix * 4;
  o.map.box[1] = (uint32_t)tile_rows; o.t_mul[1] = tile_rows;
  if (pix >= 32 && pix % 32 == 0) {
    const int cpi = pix / 32;
    o.map.swizzle = TC_SW_128; o.map.box[0] = 32; o.map.box[2] = 1;
    o.k_div[0] = 1; o.k_mod[0] = cpi; o.k_mul[0] = 32;
    o.k_div[2] = cpi; o.k_mul[2] = 1;
    o.lbo = 16; o.sbo = 1024;
    for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 32;
    *k_iters = n_img * cpi;
    return true;
  }
  if (pix == 16) {            // two images per stage, each a 64-byte row: 2 MMA steps per image
    o.map.swizzle = TC_SW_64; o.map.box[0] = 16; o.map.box[2] = 2;
    o.k_mul[2] = 2;
    o.lbo = 16; o.sbo = 512;
    const uint32_t img = (uint32_t)tile_rows * 64;
    o.kstep_off[0] = 0; o.kstep_off[1] = 32; o.kstep_off[2] = img; o.kstep_off[3] = img + 32;
    *k_iters = cdiv(n_img, 2);
    return true;
  }
  if (pix == 4) {             // eight images per stage, 16 bytes each: an MMA step spans two images
    o.map.swizzle = TC_SW_NONE; o.map.box[0] = 4; o.map.box[2] = 8;
    o.k_mul[2] = 8;
    const uint32_t img = (uint32_t)tile_rows * 16;
    o.sbo = 128; o.lbo = img;                                    // interleaved K-major: LBO = stride between the two 16-byte k-chunks
    for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 2 * img;
    *k_iters = cdiv(n_img, 8);
    return true;
  }
  return false;
}

// ---- operands of the tap-loop convolutions: channels-last activations act[n][h][w][ch] -------------------------------

// How a run of `want` consecutive pixels (row-major over h, w, then images) is cut out of images of eh x ew pixels as
// a box of whole rows: bw x bh x bi with bw*bh*bi == want.  blocks_per_img > 1 when an image holds several boxes.
struct PixelBox { int bw, bh, bi, per_img; };
bool pixel_box(int want, int eh, int ew, PixelBox& b) {
  if (ew < 1 || eh < 1 || ew > want || want % ew) return false;
  const int rows = want / ew;
  b.bw = ew;
  if (rows <= eh) { if (eh % rows) return false; b.bh = rows; b.bi = 1; b.per_img = eh / rows; }
  else { if (rows % eh) return false; b.bh = eh; b.bi = rows / eh; b.per_img = 1; }
  return b.bw <= 256 && b.bh <= 256 && b.bi <= 256;
}

// K-major activation window.  Rows of D = pixels (n, h, w) of a th x tw grid (the output grid for forward, the input grid
// for data-grad); row pixel (h, w) reads act[n][h*1 + off_h + dir*r][w + off_w + dir*s][ch] at tap (r, s).  K loop:
// kiter = (r*S + s)*chunks + chunk, 32 channels per iteration.  act has eh x ew pixels per image and `ch` channels.
bool operand_k_window(TcOperand& o, const float* act, int n_img, int eh, int ew, int ch, int th, int tw, int R, int S, int off_h, int off_w,
                      int dir, int* k_iters) {
  clear(o);
  PixelBox b;
  if (!aligned16(act) || ch % 4 || !pixel_box(kTileM, th, tw, b)) return false;
  const int chunks = cdiv(ch, kBK);
  o.map.base = act; o.mn_major = 0; o.nk = 4; o.stage_bytes = kTileM * 128;
  o.map.rank = 4; o.map.swizzle = TC_SW_128;
  o.map.dims[0] = (uint64_t)ch; o.map.dims[1] = (uint64_t)ew; o.map.dims[2] = (uint64_t)eh; o.map.dims[3] = (uint64_t)n_img;
  o.map.strides[1] = (uint64_t)ch * 4; o.map.strides[2] = (uint64_t)ew * ch * 4; o.map.strides[3] = (uint64_t)eh * ew * ch * 4;
  o.map.box[0] = kBK; o.map.box[1] = (uint32_t)b.bw; o.map.box[2] = (uint32_t)b.bh; o.map.box[3] = (uint32_t)b.bi;
  if (chunks > 1) { o.k_div[0] = 1; o.k_mod[0] = chunks; o.k_mul[0] = kBK; }
  if (S > 1) { o.k_div[1] = chunks; o.k_mod[1] = S; o.k_mul[1] = dir; }
  if (R > 1) { o.k_div[2] = chunks * S; o.k_mod[2] = R; o.k_mul[2] = dir; }
  o.c_off[1] = off_w; o.c_off[2] = off_h;
  if (b.per_img > 1) { o.t_div[2] = 1; o.t_mod[2] = b.per_img; o.t_mul[2] = b.bh; }
  o.t_div[3] = b.per_img; o.t_mul[3] = b.bi;
  o.lbo = 16; o.sbo = 1024;
  for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 32;
  *k_iters = R * S * chunks;
  return true;
}

// Per-tap weight matrices wp[tap][rows][kdim] used K-major: box (32 of kdim, tile_rows rows, 1 tap); kiter as above.
bool operand_k_taps(TcOperand& o, const float* wp, int taps, int rows, int kdim, int tile_rows, int* k_iters) {
  clear(o);
  if (!aligned16(wp) || kdim % 4 || rows < 1) return false;
  const int chunks = cdiv(kdim, kBK);
  o.map.base = wp; o.mn_major = 0; o.nk = 4; o.stage_bytes = (uint32_t)tile_rows * 128;
  o.map.rank = 3; o.map.swizzle = TC_SW_128;
  o.map.dims[0] = (uint64_t)kdim; o.map.dims[1] = (uint64_t)rows; o.map.dims[2] = (uint64_t)taps;
  o.map.strides[1] = (uint64_t)kdim * 4; o.map.strides[2] = (uint64_t)rows * kdim * 4;
  o.map.box[0] = kBK; o.map.box[1] = (uint32_t)tile_rows; o.map.box[2] = 1;
  if (chunks > 1) { o.k_div[0] = 1; o.k_mod[0] = chunks; o.k_mul[0] = kBK; }
  o.k_div[2] = chunks; o.k_mul[2] = 1;
  o.t_mul[1] = tile_rows;
  o.lbo = 16; o.sbo = 1024;
  for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 32;
  *k_iters = taps * chunks;
  return true;
}

// M/N-major activation for weight-grad: the M (or N) index is the channel, the K index the pixel.  One stage = 32
// pixels (a box of whole rows of the th x tw pixel grid the reduction runs over) x tile_ch channels, stored as
// tile_ch/32 chunks of [32 pixels][32 channels].  The tile index selects the channel block and, when taps > 1, the tap
// whose shift (r + off_h, s + off_w) is added to the pixel coordinates: tile = (r*S + s)*ch_blocks + block.
bool operand_mn_window(TcOperand& o, const float* act, int n_img, int eh, int ew, int ch, int th, int tw, int tile_ch, int R, int S, int off_h, int off_w,
                       int* k_iters) {
  clear(o);
  PixelBox b;
  if (!aligned16(act) || ch % 32 || tile_ch % 32 || !pixel_box(kBK, th, tw, b)) return false;
  const int blocks = cdiv(ch, tile_ch);
  o.map.base = act; o.mn_major = 1; o.nk = 4; o.stage_bytes = (uint32_t)tile_ch * 128;
  o.map.rank = 5; o.map.swizzle = TC_SW_128_32B;
  o.map.dims[0] = 32; o.map.dims[1] = (uint64_t)ew; o.map.dims[2] = (uint64_t)eh; o.map.dims[3] = (uint64_t)n_img; o.map.dims[4] = (uint64_t)ch / 32;
  o.map.strides[1] = (uint64_t)ch * 4; o.map.strides[2] = (uint64_t)ew * ch * 4; o.map.strides[3] = (uint64_t)eh * ew * ch * 4; o.map.strides[4] = 128;
  o.map.box[0] = 32; o.map.box[1] = (uint32_t)b.bw; o.map.box[2] = (uint32_t)b.bh; o.map.box[3] = (uint32_t)b.bi; o.map.box[4] = (uint32_t)tile_ch / 32;
  // reduction: pixel blocks of the th x tw grid, image after image
  if (b.per_img > 1) { o.k_div[2] = 1; o.k_mod[2] = b.per_img; o.k_mul[2] = b.bh; }
  o.k_div[3] = b.per_img; o.k_mul[3] = b.bi;
  // tile: channel block, then tap
  o.t_div[4] = 1; o.t_mod[4] = blocks; o.t_mul[4] = tile_ch / 32;
  if (S > 1) { o.t_div[1] = blocks; o.t_mod[1] = S; o.t_mul[1] = 1; }
  if (R > 1) { o.t_div[2] = blocks * S; o.t_mod[2] = R; o.t_mul[2] = 1; }
  o.c_off[1] = off_w; o.c_off[2] = off_h;
  o.lbo = kBK * 128; o.sbo = 512;
  for (int i = 0; i < 4; ++i) o.kstep_off[i] = (uint32_t)i * 1024;
  *k_iters = b.per_img > 1 ? n_img * b.per_img : cdiv(n_img, b.bi);
  return true;
}

// Tile width.  The MMA-issuing thread spends a few hundred cycles per k-iteration whatever the width, so narrow tiles
// leave the tensor core idle; 128 columns with three stages lets two CTAs share an SM (one's epilogue and issue gaps
// overlap the other's main loop).  Parallelism for small outputs comes from split-K, not from narrower tiles.
// Split policy knobs, read once from LTB_SPLIT="fill,min_iters,prefer64" (a sweep aid; the defaults are the measured optimum):
// fill = CTAs per SM that split-K aims for (x 100), min_iters = fewest k-iterations a split may have, prefer64 = 64-wide tiles
// whenever 128-wide ones would not cover the SMs.
struct SplitKnobs { int fill100 = 100, min_iters = 8, prefer64 = 0; };
const SplitKnobs& split_knobs() {
  static SplitKnobs k = [] {
    SplitKnobs v;
    if (const char* e = std::getenv("LTB_SPLIT")) std::sscanf(e, "%d,%d,%d", &v.fill100, &v.min_iters, &v.prefer64);
    if (v.fill100 < 10) v.fill100 = 10;
    if (v.min_iters < 1) v.min_iters = 1;
    return v;
  }();
  return k;
}
int pick_bn(int n_extent, int m_tiles, int sm_count) {
  if (n_extent <= 64) return 64;
  if (split_knobs().prefer64 && (int64_t)m_tiles * cdiv(n_extent, 128) * 10 < (int64_t)8 * sm_count) return 64;
  return 128;
}

void finish(TcPlan& p, int M, int N, int k_iters, int sm_count, bool may_split) {
  p.M = M; p.N = N; p.k_iters = k_iters;
  p.m_tiles = cdiv(M, kTileM); p.n_tiles = cdiv(N, p.bn);
  p.splits = 1;
  if (may_split) {
    const int tiles = p.m_tiles * p.n_tiles;
    // Split-K pays with atomic traffic (splits x the output) and a zero-fill, so it is used sparingly: measured on the
    // ResNet-50 layer set, the best step time comes from about one CTA per SM, at least eight k-iterations per split, and
    // no split at all once the tiles alone cover 80 % of the SMs (two CTAs per SM with four iterations each was 6 % slower).
    int s = cdiv(sm_count * split_knobs().fill100 / 100, tiles);
    int mx = k_iters / split_knobs().min_iters; if (mx < 1) mx = 1;
    if (s > mx) s = mx;
    if ((int64_t)tiles * 10 >= (int64_t)8 * sm_count) s = 1;
    p.splits = s < 1 ? 1 : s;
  }
}

}  // namespace

bool tc_walk_of(const TcOperand& o, TcWalk& w) {
  std::memset(&w, 0, sizeof w);
  w.n0 = w.n1 = 1 << 30;
  int D[5], nd = 0;
  auto moves = [&](int d) { return o.k_mul[d] != 0 && o.k_mod[d] > 1; };     // a modulus of 1 pins the coordinate
  for (int d = 0; d < 5; ++d) {
    if (!moves(d)) continue;
    bool seen = false;
    for (int i = 0; i < nd; ++i) seen = seen || D[i] == o.k_div[d];
    if (!seen) D[nd++] = o.k_div[d];
  }
  if (nd == 0) return true;
  for (int i = 0; i < nd; ++i) for (int j = i + 1; j < nd; ++j) if (D[j] < D[i]) { int t = D[i]; D[i] = D[j]; D[j] = t; }
  if (D[0] != 1) { if (nd == 5) return false; for (int i = nd; i > 0; --i) D[i] = D[i - 1]; D[0] = 1; ++nd; }
  if (nd > 3) return false;
  int n[3] = {1 << 30, 1 << 30, 1 << 30};
  for (int j = 0; j + 1 < nd; ++j) { if (D[j + 1] % D[j]) return false; n[j] = D[j + 1] / D[j]; }
  w.n0 = n[0]; w.n1 = n[1];
  for (int j = 0; j < nd; ++j) for (int d = 0; d < 5; ++d) {
    if (!moves(d)) continue;
    int v = o.k_div[d] == D[j] ? o.k_mul[d] : 0;
    for (int i = 0; i < j; ++i) if (o.k_div[d] == D[i]) v -= o.k_mul[d] * (n[i] - 1);
    w.inc[j][d] = v;
  }
  return true;
}

bool tc_conv_needs_rows(int pix) { return !(pix >= 32 && pix % 32 == 0 && (pix >= kTileM ? pix % kTileM == 0 : kTileM % pix == 0)); }

bool tc_gather_possible(const float* src, int chan, int pix) { return aligned16(src) && (pix == 4 || pix == 16) && chan % 4 == 0 && chan >= 8; }
void tc_plan_gather(TcPlan& p, const float* src, int n_img, int chan, int pix) { p.gather_src = src; p.g_pix = pix; p.g_chan = chan; p.g_imgs = n_img; }

bool tc_plan_conv_fwd(TcPlan& p, const float* x, bool a_rows, const float* w, int ldw, const float* bias, float* y, int n_img, int ck, int co, int pix, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (co < 8 || ck < 8 || ldw < ck || (a_rows && ldw != ck) || (int64_t)n_img * pix > (1ll << 30)) return false;
  int ka = 0, kb = 0;
  const int M = n_img * pix;
  if (!(a_rows ? operand_k_rows(p.a, x, M, ck, kTileM, &ka) : operand_mn_pixels(p.a, x, n_img, ck, pix, &ka))) return false;
  p.bn = pick_bn(co, cdiv(M, kTileM), sm_count);
  if (!operand_k_rows(p.b, w, co, ldw, p.bn, &kb) || ka != kb) return false;      // columns ck..ldw of w are zero padding
  finish(p, M, co, ka, sm_count, true);             // split-K for small outputs: the launcher zeroes y first
  p.epilogue = TC_EPI_PIXEL; p.out = y; p.bias = bias; p.alpha = 1.0f; p.accumulate = 0;
  p.pix_per_img = pix; p.img_stride = (int64_t)co * pix; p.chan_stride = pix;
  return true;
}

bool tc_plan_conv_dgrad(TcPlan& p, const float* dy, bool a_rows, const float* w, int ldw, float* dx, int n_img, int ck, int co, int pix, bool accumulate, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (ck < 8 || co < 8 || ldw < ck || (int64_t)n_img * pix > (1ll << 30)) return false;
  int ka = 0, kb = 0;
  const int M = n_img * pix;
  if (!(a_rows ? operand_k_rows(p.a, dy, M, co, kTileM, &ka) : operand_mn_pixels(p.a, dy, n_img, co, pix, &ka))) return false;
  p.bn = pick_bn(ck, cdiv(M, kTileM), sm_count);
  if (!operand_mn_cols(p.b, w, co, ldw, p.bn, &kb) || ka != kb) return false;      // w is stored with ldw (a multiple of 32) columns
  finish(p, M, ck, ka, sm_count, true);
  p.epilogue = TC_EPI_PIXEL; p.out = dx; p.bias = nullptr; p.alpha = 1.0f; p.accumulate = accumulate ? 1 : 0;
  p.pix_per_img = pix; p.img_stride = (int64_t)ck * pix; p.chan_stride = pix;
  return true;
}

bool tc_plan_conv_wgrad(TcPlan& p, const float* x, const float* dy, float* dw, int n_img, int ck, int co, int pix, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (co < 8 || ck < 16) return false;
  int ka = 0, kb = 0;
  if (!operand_k_pixels(p.a, dy, n_img, co, pix, kTileM, &ka)) return false;
  p.bn = pick_bn(ck, cdiv(co, kTileM), sm_count);     // narrower tiles before more split-K: fewer atomic partial sums
  if (!operand_k_pixels(p.b, x, n_img, ck, pix, p.bn, &kb) || ka != kb) return false;
  finish(p, co, ck, ka, sm_count, true);
  p.epilogue = TC_EPI_ROWMAJOR; p.out = dw; p.bias = nullptr; p.alpha = 1.0f; p.accumulate = 1; p.ld = ck;
  return true;
}

static bool taps_geometry_ok(const TcConvGeom& g) {
  return g.n_img >= 1 && g.R * g.S >= 1 && g.R <= 7 && g.S <= 7 && g.oH == g.H + 2 * g.ph - g.R + 1 && g.oW == g.W + 2 * g.pw - g.S + 1 &&
         g.oH >= 1 && g.oW >= 1 && g.C % 32 == 0 && g.K % 32 == 0 && (int64_t)g.n_img * g.H * g.W < (1ll << 30);
}

bool tc_plan_conv_taps_fwd(TcPlan& p, const float* xr, const float* wt, const float* bias, float* y, const TcConvGeom& g, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (!taps_geometry_ok(g)) return false;
  int ka = 0, kb = 0;
  const int M = g.n_img * g.oH * g.oW;
  // output pixel (oh, ow) reads input (oh - ph + r, ow - pw + s)
  if (!operand_k_window(p.a, xr, g.n_img, g.H, g.W, g.C, g.oH, g.oW, g.R, g.S, -g.ph, -g.pw, +1, &ka)) return false;
  p.bn = pick_bn(g.K, cdiv(M, kTileM), sm_count);
  if (!operand_k_taps(p.b, wt, g.R * g.S, g.K, g.C, p.bn, &kb) || ka != kb) return false;
  finish(p, M, g.K, ka, sm_count, true);
  p.epilogue = TC_EPI_PIXEL; p.out = y; p.bias = bias; p.alpha = 1.0f; p.accumulate = 0;
  p.pix_per_img = (int64_t)g.oH * g.oW; p.img_stride = (int64_t)g.K * g.oH * g.oW; p.chan_stride = (int64_t)g.oH * g.oW;
  return true;
}

bool tc_plan_conv_taps_dgrad(TcPlan& p, const float* dyr, const float* wd, float* dx, const TcConvGeom& g, bool accumulate, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (!taps_geometry_ok(g)) return false;
  int ka = 0, kb = 0;
  const int M = g.n_img * g.H * g.W;
  // input pixel (h, w) receives dy(h + ph - r, w + pw - s) * w[k][c][r][s]
  if (!operand_k_window(p.a, dyr, g.n_img, g.oH, g.oW, g.K, g.H, g.W, g.R, g.S, g.ph, g.pw, -1, &ka)) return false;
  p.bn = pick_bn(g.C, cdiv(M, kTileM), sm_count);
  if (!operand_k_taps(p.b, wd, g.R * g.S, g.C, g.K, p.bn, &kb) || ka != kb) return false;
  finish(p, M, g.C, ka, sm_count, true);
  p.epilogue = TC_EPI_PIXEL; p.out = dx; p.bias = nullptr; p.alpha = 1.0f; p.accumulate = accumulate ? 1 : 0;
  p.pix_per_img = (int64_t)g.H * g.W; p.img_stride = (int64_t)g.C * g.H * g.W; p.chan_stride = (int64_t)g.H * g.W;
  return true;
}

bool tc_plan_conv_taps_wgrad(TcPlan& p, const float* dyr, const float* xr, float* dw, const TcConvGeom& g, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (!taps_geometry_ok(g) || g.C % 64) return false;
  int ka = 0, kb = 0;
  const int taps = g.R * g.S;
  // dw[k][c][r][s] += sum over output pixels dy[n][k][oh][ow] * x[n][c][oh - ph + r][ow - pw + s]
  if (!operand_mn_window(p.a, dyr, g.n_img, g.oH, g.oW, g.K, g.oH, g.oW, kTileM, 1, 1, 0, 0, &ka)) return false;
  p.bn = g.C % 128 == 0 ? 128 : 64;
  if (!operand_mn_window(p.b, xr, g.n_img, g.H, g.W, g.C, g.oH, g.oW, p.bn, g.R, g.S, -g.ph, -g.pw, &kb) || ka != kb) return false;
  finish(p, g.K, taps * g.C, ka, sm_count, true);
  p.epilogue = TC_EPI_ROWMAJOR; p.out = dw; p.bias = nullptr; p.alpha = 1.0f; p.accumulate = 1; p.ld = (int64_t)taps * g.C;
  p.col_mod = g.C; p.col_mul = taps;
  return true;
}

bool tc_plan_gemm(TcPlan& p, const float* a, bool a_kmajor, const float* b, bool b_kmajor, float* c, int M, int N, int K, float alpha,
                  bool accumulate, int sm_count) {
  std::memset(&p, 0, sizeof p);
  if (M < 64 || N < 32 || K < 32 || !aligned16(c)) return false;
  int ka = 0, kb = 0;
  bool ok = a_kmajor ? operand_k_rows(p.a, a, M, K, kTileM, &ka) : operand_mn_cols(p.a, a, K, M, kTileM, &ka);
  if (!ok) return false;
  p.bn = pick_bn(N, cdiv(M, kTileM), sm_count);
  ok = b_kmajor ? operand_k_rows(p.b, b, N, K, p.bn, &kb) : operand_mn_cols(p.b, b, K, N, p.bn, &kb);
  if (!ok || ka != kb) return false;
  finish(p, M, N, ka, sm_count, true);
  p.epilogue = TC_EPI_ROWMAJOR; p.out = c; p.bias = nullptr; p.alpha = alpha; p.accumulate = accumulate ? 1 : 0; p.ld = N;
  return true;
}

}  // namespace ltb
