// FP32 CUDA-core contraction path: GEMM family and implicit-GEMM convolution (forward, data-grad, weight-grad).
//
// This is the 1e-4 path (LTB_MATH_FP32) and the path for shapes the tensor-core engine does not take
// (strides not multiples of 16 bytes, tiny K such as the 1->10 5x5 MNIST convolution or the 3->64 stem).
// Replaces cublasSgemm call sites (TensorDslCublas.scala:204-282, 589-688) and the cuDNN convolution calls
// (TensorDslCudnn.scala:515-831).  Semantics follow TensorDslCPU.scala:379-472 (gemm) and 484-692 (conv).
//
// One kernel template: C[m,n] (op)= sum_k A(m,k) * B(k,n) with A, B and the store given as functors, so that the
// convolution variants never materialise the reference's `finput` (im2col) buffer.  64x64x16 tiles, 256 threads,
// 4x4 outputs per thread, optional split-K over gridDim.z with atomic accumulation.
#include "gemm.cuh"

namespace ltb {

constexpr int BM = 64, BN = 64, BKK = 16;

// AFAST / BFAST: which index of the operand is contiguous in memory (0: the k index, 1: the m resp. n index);
// decides how the 256 threads sweep the tile so that global loads coalesce.
template <int AFAST, int BFAST, class LA, class LB, class ST>
__global__ void __launch_bounds__(256) igemm_kernel(int M, int N, int K, int k_per_split, LA la, LB lb, ST st) {
  __shared__ float As[BKK][BM + 4];
  __shared__ float Bs[BKK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int k_begin = blockIdx.z * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int tm = tid & 15, tn = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = k_begin; k0 < k_end; k0 += BKK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + 256 * e;
      int mm = AFAST ? (idx & 63) : (idx >> 4), kk = AFAST ? (idx >> 6) : (idx & 15);
      int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < k_end) ? la(gm, gk) : 0.0f;
      int nn = BFAST ? (idx & 63) : (idx >> 4), kb = BFAST ? (idx >> 6) : (idx & 15);
      int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < k_end) ? lb(gkb, gn) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BKK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + 16 * i];
      float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tn * 4]);
      b[0] = bv.x; b[1] = bv.y; b[2] = bv.z; b[3] = bv.w;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + tm + 16 * i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tn * 4 + j;
      if (gn < N) st(gm, gn, acc[i][j]);
    }
  }
}

// ---- plain matrices ------------------------------------------------------------------------------------------
struct MatLoadA { const float* p; int64_t sm, sk; __device__ float operator()(int m, int k) const { return p[m * sm + k * sk]; } };
struct MatLoadB { const float* p; int64_t sk, sn; __device__ float operator()(int k, int n) const { return p[k * sk + n * sn]; } };
// C[m*ldm + n*ldn] = alpha*v (MODE 0), += alpha*v (MODE 1), atomic += (MODE 2, split-K)
template <int MODE>
struct MatStore {
  float* p; int64_t sm, sn; float alpha;
  __device__ void operator()(int m, int n, float v) const {
    float* q = p + m * sm + n * sn;
    if (MODE == 0) *q = alpha * v; else if (MODE == 1) *q += alpha * v; else atomicAdd(q, alpha * v);
  }
};

// ---- skinny products: one extent of 16 or less (a 10-way classifier and its gradients) -----------------------------------
// The 64 x 64 tiles above leave such products to one or two CTAs walking a long K; these three kernels give every output
// (or every output column) its own thread or warp instead.
// N <= 16, A and B both contiguous along k: a block of sixteen warps per row m, each warp a sixteenth of K, lanes stride over
// k (at K = 2048 a lane makes four independent iterations: the loads of a row are all in flight at once).  The warps' sums are
// added in warp order by one thread per column: the same bits on every run.
constexpr int kSkinnyNWarps = 16;
template <bool ACC>
__global__ void __launch_bounds__(kSkinnyNWarps * 32) skinny_n_kernel(const float* __restrict__ a, int64_t sam, const float* __restrict__ b, int64_t sbn, float* c,
                                                                      int64_t scm, int64_t scn, int N, int K, float alpha) {
  __shared__ float part[kSkinnyNWarps][16];
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = (int)((int64_t)K * warp / kSkinnyNWarps), k1 = (int)((int64_t)K * (warp + 1) / kSkinnyNWarps);
  float acc[16];
#pragma unroll
  for (int n = 0; n < 16; ++n) acc[n] = 0.0f;
  const float* ar = a + (int64_t)m * sam;
#pragma unroll 4
  for (int k = k0 + lane; k < k1; k += 32) {
    const float av = ar[k];
#pragma unroll
    for (int n = 0; n < 16; ++n) if (n < N) acc[n] += av * b[(int64_t)n * sbn + k];
  }
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    float v = acc[n];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) part[warp][n] = v;
  }
  __syncthreads();
  if (threadIdx.x < N) {
    const int n = threadIdx.x;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kSkinnyNWarps; ++w) v += part[w][n];
    v *= alpha;
    float* q = c + (int64_t)m * scm + (int64_t)n * scn;
    *q = ACC ? *q + v : v;
  }
}
// K <= 16: a thread per output element.
template <bool ACC>
__global__ void skinny_k_kernel(const float* __restrict__ a, int64_t sam, int64_t sak, const float* __restrict__ b, int64_t sbk, int64_t sbn,
                                float* c, int64_t scm, int64_t scn, int M, int N, int K, float alpha) {
  const int64_t total = (int64_t)M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(i % N); const int64_t m = i / N;
    float v = 0.0f;
    for (int k = 0; k < K; ++k) v += a[m * sam + k * sak] * b[k * sbk + n * sbn];
    float* q = c + m * scm + n * scn;
    *q = ACC ? *q + alpha * v : alpha * v;
  }
}
// M <= 16: a block is 32 output columns x 8 slices of K (blockIdx.y splits K further when it is long); a thread keeps all
// rows of its column in registers over its slice, B is read once, coalesced when contiguous along n.  The slices of a block
// are added in slice order through shared memory (a lane's loop over k is a chain of dependent steps: the classifier's weight
// gradient, 10 x 2048 over a batch of 128, took 89 us as sixteen blocks walking all of K, 19 us as sixteen slabs and a second
// launch).  With blockIdx.y > 1 a block's sum goes to its own slab and skinny_sum_kernel adds the slabs in order.
constexpr int kSkinnyMSlices = 8;
template <bool ACC>
__global__ void __launch_bounds__(32 * kSkinnyMSlices) skinny_m_kernel(const float* __restrict__ a, int64_t sam, int64_t sak, const float* __restrict__ b, int64_t sbk,
                                                                       int64_t sbn, float* c, int64_t scm, int64_t scn, int M, int N, int K, float alpha, float* part) {
  __shared__ float sums[kSkinnyMSlices][16][33];
  const int n = blockIdx.x * 32 + threadIdx.x, slice = threadIdx.y;
  const int q0 = (int)((int64_t)K * blockIdx.y / gridDim.y), q1 = (int)((int64_t)K * (blockIdx.y + 1) / gridDim.y);
  const int k0 = q0 + (int)((int64_t)(q1 - q0) * slice / kSkinnyMSlices), k1 = q0 + (int)((int64_t)(q1 - q0) * (slice + 1) / kSkinnyMSlices);
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.0f;
  if (n < N) {
#pragma unroll 4
    for (int k = k0; k < k1; ++k) {
      const float bv = b[(int64_t)k * sbk + (int64_t)n * sbn];
#pragma unroll
      for (int m = 0; m < 16; ++m) if (m < M) acc[m] += a[(int64_t)m * sam + (int64_t)k * sak] * bv;
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) sums[slice][m][threadIdx.x] = acc[m];
  __syncthreads();
  if (n >= N) return;
  for (int m = slice; m < M; m += kSkinnyMSlices) {                              // the rows are dealt out to the slices' threads
    float v = 0.0f;
#pragma unroll
    for (int z = 0; z < kSkinnyMSlices; ++z) v += sums[z][m][threadIdx.x];
    float* q = c + (int64_t)m * scm + (int64_t)n * scn;
    if (part) part[((int64_t)blockIdx.y * M + m) * N + n] = v;                   // K was split over blocks too: this block's share goes to its own slab
    else *q = ACC ? *q + alpha * v : alpha * v;
  }
}
// c[m][n] (+)= alpha * (part[0][m][n] + part[1][m][n] + ...), in that order: the second half of skinny_m_kernel when K is split.
template <bool ACC>
__global__ void skinny_sum_kernel(const float* __restrict__ part, int slabs, float* c, int64_t scm, int64_t scn, int M, int N, float alpha) {
  const int64_t total = (int64_t)M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float v = 0.0f;
    for (int z = 0; z < slabs; ++z) v += part[(int64_t)z * total + i];
    float* q = c + (i / N) * scm + (i % N) * scn;
    *q = ACC ? *q + alpha * v : alpha * v;
  }
}
static int skinny_gemm(const float* a, int64_t sam, int64_t sak, const float* b, int64_t sbk, int64_t sbn, float* c, int64_t scm, int64_t scn,
                       int M, int N, int K, float alpha, bool accumulate, bool* taken) {
  *taken = true;
  if (N <= 16 && sak == 1 && sbk == 1 && K >= 128 && M <= 65535) {
    // one block per row, its warps share K and are added in a fixed order: the same bits on every run (splitting K over
    // more blocks would need atomics, whose order changes from run to run)
    if (accumulate) LTB_LAUNCH(skinny_n_kernel<true>, dim3(M), kSkinnyNWarps * 32, 0, a, sam, b, sbn, c, scm, scn, N, K, alpha);
    else LTB_LAUNCH(skinny_n_kernel<false>, dim3(M), kSkinnyNWarps * 32, 0, a, sam, b, sbn, c, scm, scn, N, K, alpha);
  } else if (K <= 16) {
    const unsigned grid = (unsigned)grid_for((int64_t)M * N, 256);
    if (accumulate) LTB_LAUNCH(skinny_k_kernel<true>, grid, 256, 0, a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha);
    else LTB_LAUNCH(skinny_k_kernel<false>, grid, 256, 0, a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha);
  } else if (M <= 16 && N >= 256 && K <= 4096) {
    const unsigned gx = (unsigned)ceil_div(N, 32);
    // a thread's loop over k is a chain of dependent steps: beyond 64 steps per in-block slice K is also split over blockIdx.y,
    // every such split writes its share into a slab of the library's workspace and a second small launch adds the slabs in
    // order (no atomics: same bits every run)
    int ks = (int)ceil_div(K, 64 * kSkinnyMSlices);
    const size_t room = g.cur_scratch_bytes() / ((size_t)M * N * sizeof(float));
    if ((size_t)ks > room) ks = (int)room;
    if (ks < 1) ks = 1;
    float* part = ks > 1 ? g.cur_scratch() : nullptr;
    if (accumulate) LTB_LAUNCH(skinny_m_kernel<true>, dim3(gx, ks), dim3(32, kSkinnyMSlices), 0, a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha, part);
    else LTB_LAUNCH(skinny_m_kernel<false>, dim3(gx, ks), dim3(32, kSkinnyMSlices), 0, a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha, part);
    if (part) {
      const unsigned gr = (unsigned)grid_for((int64_t)M * N, 256);
      if (accumulate) LTB_LAUNCH(skinny_sum_kernel<true>, gr, 256, 0, (const float*)part, ks, c, scm, scn, M, N, alpha);
      else LTB_LAUNCH(skinny_sum_kernel<false>, gr, 256, 0, (const float*)part, ks, c, scm, scn, M, N, alpha);
    }
  } else *taken = false;
  return LTB_OK;
}

// C[M,N] (op)= alpha * A B with arbitrary strides; accumulate selects += (gradients) over = (forward).
static int strided_gemm(const float* a, int64_t sam, int64_t sak, const float* b, int64_t sbk, int64_t sbn, float* c, int64_t scm,
                        int64_t scn, int M, int N, int K, float alpha, bool accumulate) {
  { bool taken = false; int rc = skinny_gemm(a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha, accumulate, &taken); if (rc || taken) return rc; }
  dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN, 1);
  int tiles = grid.x * grid.y;
  int splits = 1;
  // A forward product with few output tiles and a long K (the 2048 -> 10 classifier: two tiles) would leave the machine to two
  // CTAs; when the output is a dense matrix it is zeroed and the product accumulated from K-splits like a gradient.
  const bool dense_c = (scn == 1 && scm == N) || (scm == 1 && scn == M);
  // deterministic mode (ltb_set_deterministic): no split over K on the CUDA-core paths either -- their splits add atomically
  if (!g.deterministic && !accumulate && K >= 1024 && tiles < g.sm_count && dense_c) {
    LTB_CUDA(cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(float), g.stream));
    accumulate = true;
  }
  if (!g.deterministic && accumulate && K >= 1024 && tiles < g.sm_count) { splits = (2 * g.sm_count + tiles - 1) / tiles; int mx = K / 256; if (splits > mx) splits = mx; if (splits < 1) splits = 1; }
  int kps = (int)ceil_div(ceil_div(K, splits), BKK) * BKK;
  grid.z = (unsigned)ceil_div(K, kps);
  MatLoadA la{a, sam, sak}; MatLoadB lb{b, sbk, sbn};
  const int af = sam == 1 ? 1 : 0, bf = sbn == 1 ? 1 : 0;
#define LTB_GEMM_DISPATCH(AF, BF)                                                                                              \
  do {                                                                                                                          \
    if (!accumulate) LTB_LAUNCH((igemm_kernel<AF, BF, MatLoadA, MatLoadB, MatStore<0>>), grid, 256, 0, M, N, K, kps, la, lb, (MatStore<0>{c, scm, scn, alpha})); \
    else if (grid.z == 1) LTB_LAUNCH((igemm_kernel<AF, BF, MatLoadA, MatLoadB, MatStore<1>>), grid, 256, 0, M, N, K, kps, la, lb, (MatStore<1>{c, scm, scn, alpha})); \
    else LTB_LAUNCH((igemm_kernel<AF, BF, MatLoadA, MatLoadB, MatStore<2>>), grid, 256, 0, M, N, K, kps, la, lb, (MatStore<2>{c, scm, scn, alpha})); \
  } while (0)
  if (af && bf) LTB_GEMM_DISPATCH(1, 1); else if (af) LTB_GEMM_DISPATCH(1, 0); else if (bf) LTB_GEMM_DISPATCH(0, 1); else LTB_GEMM_DISPATCH(0, 0);
#undef LTB_GEMM_DISPATCH
  return LTB_OK;
}

// ---- convolution as implicit GEMM -----------------------------------------------------------------------------
// forward: m = (n, ho, wo), k = (ci, kh, kw), n = co
struct ConvFwdA {
  const float* x; ConvDims d;
  __device__ float operator()(int m, int k) const {
    int wo = m % d.oW, t = m / d.oW, ho = t % d.oH, n = t / d.oH;
    int kw = k % d.S, t2 = k / d.S, kh = t2 % d.R, ci = t2 / d.R;
    int ih = ho * d.sh - d.ph + kh, iw = wo * d.sw - d.pw + kw;
    if (ih < 0 || ih >= d.H || iw < 0 || iw >= d.W) return 0.0f;
    return x[(((int64_t)n * d.C + ci) * d.H + ih) * d.W + iw];
  }
};
struct ConvFwdB { const float* w; int ckk; __device__ float operator()(int k, int co) const { return w[(int64_t)co * ckk + k]; } };
struct ConvFwdStore {
  float* y; const float* bias; ConvDims d;
  __device__ void operator()(int m, int co, float v) const {
    int hw = d.oH * d.oW, n = m / hw, p = m % hw;
    y[((int64_t)n * d.K + co) * hw + p] = v + (bias ? bias[co] : 0.0f);
  }
};
// data gradient: m = (n, h, w), k = (co, kh, kw), n = ci; dX += ...
struct ConvDgradA {
  const float* dy; ConvDims d;
  __device__ float operator()(int m, int k) const {
    int w = m % d.W, t = m / d.W, h = t % d.H, n = t / d.H;
    int kw = k % d.S, t2 = k / d.S, kh = t2 % d.R, co = t2 / d.R;
    int hs = h + d.ph - kh, ws = w + d.pw - kw;
    if (hs < 0 || ws < 0 || hs % d.sh || ws % d.sw) return 0.0f;
    int ho = hs / d.sh, wo = ws / d.sw;
    if (ho >= d.oH || wo >= d.oW) return 0.0f;
    return dy[(((int64_t)n * d.K + co) * d.oH + ho) * d.oW + wo];
  }
};
struct ConvDgradB {
  const float* w; ConvDims d;
  __device__ float operator()(int k, int ci) const { int rs = d.R * d.S, co = k / rs, r = k % rs; return w[((int64_t)co * d.C + ci) * rs + r]; }
};
struct ConvDgradStore {
  float* dx; ConvDims d;
  __device__ void operator()(int m, int ci, float v) const { int hw = d.H * d.W, n = m / hw, p = m % hw; dx[((int64_t)n * d.C + ci) * hw + p] += v; }
};
// weight gradient: m = co, n = (ci, kh, kw), k = (n, ho, wo); dW += ...
struct ConvWgradA {
  const float* dy; ConvDims d;
  __device__ float operator()(int co, int k) const { int hw = d.oH * d.oW, n = k / hw, p = k % hw; return dy[((int64_t)n * d.K + co) * hw + p]; }
};
struct ConvWgradB {
  const float* x; ConvDims d;
  __device__ float operator()(int k, int j) const {
    int wo = k % d.oW, t = k / d.oW, ho = t % d.oH, n = t / d.oH;
    int kw = j % d.S, t2 = j / d.S, kh = t2 % d.R, ci = t2 / d.R;
    int ih = ho * d.sh - d.ph + kh, iw = wo * d.sw - d.pw + kw;
    if (ih < 0 || ih >= d.H || iw < 0 || iw >= d.W) return 0.0f;
    return x[(((int64_t)n * d.C + ci) * d.H + ih) * d.W + iw];
  }
};

// dbias[co] += sum over n, ho, wo of dy (TensorDslCPU.scala:607-617).  grid (channel, image split): with one block per
// channel a 16-channel squeeze layer would read its 4 MB gradient with 16 blocks; the splits each add their partial sum
// atomically.  VEC: hw is a multiple of 4 and dy is 16-byte aligned.
template <bool VEC>
__global__ void conv_bias_grad_kernel(const float* __restrict__ dy, float* dbias, int N, int K, int hw, int img_per_split) {
  const int co = blockIdx.x;
  const int n0 = blockIdx.y * img_per_split, n1 = min(N, n0 + img_per_split);
  float s = 0.0f;
  const int per = VEC ? hw / 4 : hw;                       // the threads run over (image, element) pairs: small maps keep every lane busy
  for (int j = threadIdx.x; j < (n1 - n0) * per; j += blockDim.x) {
    const int n = j / per, i = j - n * per;
    const float* p = dy + ((int64_t)(n0 + n) * K + co) * hw;
    if (VEC) { const float4 v = reinterpret_cast<const float4*>(p)[i]; s += (v.x + v.y) + (v.z + v.w); }
    else s += p[i];
  }
  __shared__ float sh[32];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.0f;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) { if (gridDim.y == 1) dbias[co] += s; else atomicAdd(dbias + co, s); }
  }
}

int conv_fwd_fp32(const float* x, const float* w, const float* bias, float* y, const ConvDims& d) {
  int M = d.N * d.oH * d.oW, Kd = d.C * d.R * d.S;
  dim3 grid((M + BM - 1) / BM, (d.K + BN - 1) / BN, 1);
  int kps = (int)ceil_div(Kd, BKK) * BKK;
  LTB_LAUNCH((igemm_kernel<1, 0, ConvFwdA, ConvFwdB, ConvFwdStore>), grid, 256, 0, M, d.K, Kd, kps, (ConvFwdA{x, d}), (ConvFwdB{w, Kd}), (ConvFwdStore{y, bias, d}));
  return LTB_OK;
}
int conv_dgrad_fp32(const float* dy, const float* w, float* dx, const ConvDims& d) {
  int M = d.N * d.H * d.W, Kd = d.K * d.R * d.S;
  dim3 grid((M + BM - 1) / BM, (d.C + BN - 1) / BN, 1);
  int kps = (int)ceil_div(Kd, BKK) * BKK;
  LTB_LAUNCH((igemm_kernel<1, 1, ConvDgradA, ConvDgradB, ConvDgradStore>), grid, 256, 0, M, d.C, Kd, kps, (ConvDgradA{dy, d}), (ConvDgradB{w, d}), (ConvDgradStore{dx, d}));
  return LTB_OK;
}
int conv_wgrad_fp32(const float* x, const float* dy, float* dw, const ConvDims& d) {
  int M = d.K, Nn = d.C * d.R * d.S, Kd = d.N * d.oH * d.oW;
  dim3 grid((M + BM - 1) / BM, (Nn + BN - 1) / BN, 1);
  int tiles = grid.x * grid.y;
  int splits = (2 * g.sm_count + tiles - 1) / tiles; int mx = Kd / 128; if (splits > mx) splits = mx; if (splits < 1 || g.deterministic) splits = 1;
  int kps = (int)ceil_div(ceil_div(Kd, splits), BKK) * BKK;
  grid.z = (unsigned)ceil_div(Kd, kps);
  if (grid.z == 1) LTB_LAUNCH((igemm_kernel<0, 0, ConvWgradA, ConvWgradB, MatStore<1>>), grid, 256, 0, M, Nn, Kd, kps, (ConvWgradA{dy, d}), (ConvWgradB{x, d}), (MatStore<1>{dw, (int64_t)Nn, 1, 1.0f}));
  else LTB_LAUNCH((igemm_kernel<0, 0, ConvWgradA, ConvWgradB, MatStore<2>>), grid, 256, 0, M, Nn, Kd, kps, (ConvWgradA{dy, d}), (ConvWgradB{x, d}), (MatStore<2>{dw, (int64_t)Nn, 1, 1.0f}));
  return LTB_OK;
}
int conv_bias_grad(const float* dy, float* dbias, const ConvDims& d) {
  const int hw = d.oH * d.oW;
  int splits = (int)ceil_div(2 * g.sm_count, d.K);                      // about two blocks per SM in all
  if (splits > d.N) splits = d.N;
  if ((int64_t)d.N * hw < 4096 || g.deterministic) splits = 1;           // a few KB per channel: one block reads it at once (deterministic mode: no atomics)
  const int ips = (int)ceil_div(d.N, splits);
  splits = (int)ceil_div(d.N, ips);
  const int threads = 256;
  const bool vec = hw % 4 == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0;
  if (vec) LTB_LAUNCH(conv_bias_grad_kernel<true>, dim3(d.K, splits), threads, 0, dy, dbias, d.N, d.K, hw, ips);
  else LTB_LAUNCH(conv_bias_grad_kernel<false>, dim3(d.K, splits), threads, 0, dy, dbias, d.N, d.K, hw, ips);
  return LTB_OK;
}

// Entry used by the other translation units (declared in gemm.cuh).
int gemm_fp32(const float* a, int64_t sam, int64_t sak, const float* b, int64_t sbk, int64_t sbn, float* c, int64_t scm, int64_t scn,
              int M, int N, int K, float alpha, bool accumulate) {
  return strided_gemm(a, sam, sak, b, sbk, sbn, c, scm, scn, M, N, K, alpha, accumulate);
}

}  // namespace ltb
