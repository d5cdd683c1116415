// Pooling and batch normalisation: HBM-streaming kernels.
//
// Replaces cudnnPooling* (TensorDslCudnn.scala:882-982) and cudnnBatchNormalization* (TensorDslCudnn.scala:984-1131).
// Max pooling emits the int32 arg-max indices the reference's CPU backend saves (TensorDslCPU.scala:889-923),
// which the reference's GPU backend does not produce at all (it returns None, TensorDslCudnn.scala:930).
#include <cfloat>

#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ltb {

// ------------------------------------------------------------------------------------------------ max pool
// One thread per output; window scanned row-major with strict '>' from -FLT_MAX so the first maximum wins.
__global__ void maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ idx, int64_t n_out,
                                   int H, int W, int oH, int oW, int kh, int kw, int sh, int sw, int pad) {
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n_out; o += (int64_t)gridDim.x * blockDim.x) {
    int q = (int)(o % oW); int64_t t = o / oW; int r = (int)(t % oH); int64_t plane = t / oH;
    const int64_t base = plane * H * W;
    float best = -FLT_MAX; int32_t bi = 0;
    for (int a = 0; a < kh; ++a) {
      int ir = r * sh - pad + a;
      if (ir < 0 || ir >= H) continue;
      for (int b = 0; b < kw; ++b) {
        int ic = q * sw - pad + b;
        if (ic < 0 || ic >= W) continue;
        int64_t ii = base + (int64_t)ir * W + ic;
        float v = x[ii];
        if (v > best) { best = v; bi = (int32_t)ii; }
      }
    }
    y[o] = best; idx[o] = bi;
  }
}
// 2x2 stride 2, no padding, even W: each thread produces two adjacent outputs from two float4 loads
// (4 B read per input element, 1+1 B written: the compulsory traffic).
__global__ void maxpool2x2_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ idx, int64_t n_pairs,
                                      int H, int W, int oH, int oW2) {
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += (int64_t)gridDim.x * blockDim.x) {
    int q2 = (int)(p % oW2); int64_t t = p / oW2; int r = (int)(t % oH); int64_t plane = t / oH;
    int64_t i0 = plane * H * W + (int64_t)(2 * r) * W + 4 * q2;
    float4 top = *reinterpret_cast<const float4*>(x + i0), bot = *reinterpret_cast<const float4*>(x + i0 + W);
    float b0 = -FLT_MAX, b1 = -FLT_MAX; int32_t k0 = 0, k1 = 0;
    if (top.x > b0) { b0 = top.x; k0 = (int32_t)i0; }
    if (top.y > b0) { b0 = top.y; k0 = (int32_t)i0 + 1; }
    if (bot.x > b0) { b0 = bot.x; k0 = (int32_t)(i0 + W); }
    if (bot.y > b0) { b0 = bot.y; k0 = (int32_t)(i0 + W) + 1; }
    if (top.z > b1) { b1 = top.z; k1 = (int32_t)i0 + 2; }
    if (top.w > b1) { b1 = top.w; k1 = (int32_t)i0 + 3; }
    if (bot.z > b1) { b1 = bot.z; k1 = (int32_t)(i0 + W) + 2; }
    if (bot.w > b1) { b1 = bot.w; k1 = (int32_t)(i0 + W) + 3; }
    int64_t o = (plane * oH + r) * (int64_t)(2 * oW2) + 2 * q2;
    *reinterpret_cast<float2*>(y + o) = make_float2(b0, b1);
    *reinterpret_cast<int2*>(idx + o) = make_int2(k0, k1);
  }
}
// dx[idx[i]] += dy[i] (TensorDslCPU.scala:955-957); windows may overlap, so the add is atomic.
__global__ void maxpool_bwd_kernel(float* dx, const float* __restrict__ dy, const int32_t* __restrict__ idx, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) atomicAdd(dx + idx[i], dy[i]);
}

// ------------------------------------------------------------------------------------------------ average pool
__global__ void avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n_out, int H, int W, int oH, int oW,
                                   int kh, int kw, int sh, int sw) {
  float ksz = (float)(kh * kw);
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n_out; o += (int64_t)gridDim.x * blockDim.x) {
    int q = (int)(o % oW); int64_t t = o / oW; int r = (int)(t % oH); int64_t plane = t / oH;
    const float* p = x + plane * H * W + (int64_t)(r * sh) * W + q * sw;
    float s = 0.0f;
    for (int a = 0; a < kh; ++a) for (int b = 0; b < kw; ++b) s += p[a * W + b];
    y[o] = s / ksz;
  }
}
// One thread per INPUT element gathers dy/k over the windows that cover it (no atomics, deterministic).
__global__ void avgpool_bwd_kernel(float* dx, const float* __restrict__ dy, int64_t n_in, int H, int W, int oH, int oW,
                                   int kh, int kw, int sh, int sw) {
  float ksz = (float)(kh * kw);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_in; i += (int64_t)gridDim.x * blockDim.x) {
    int c = (int)(i % W); int64_t t = i / W; int r = (int)(t % H); int64_t plane = t / H;
    float s = 0.0f;
    int r_lo = r - kh + 1 > 0 ? (r - kh + 1 + sh - 1) / sh : 0, c_lo = c - kw + 1 > 0 ? (c - kw + 1 + sw - 1) / sw : 0;
    for (int orow = r_lo; orow < oH && orow * sh <= r; ++orow)
      for (int ocol = c_lo; ocol < oW && ocol * sw <= c; ++ocol) s += dy[(plane * oH + orow) * oW + ocol] / ksz;
    dx[i] += s;
  }
}

// ------------------------------------------------------------------------------------------------ batch norm
__device__ __forceinline__ float wsum(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }
__device__ void block_sum2(float& a, float& b) {
  __shared__ float sa[32], sb[32];
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = wsum(a); b = wsum(b);
  __syncthreads();
  if (lane == 0) { sa[w] = a; sb[w] = b; }
  __syncthreads();
  a = threadIdx.x < nw ? sa[threadIdx.x] : 0.0f; b = threadIdx.x < nw ? sb[threadIdx.x] : 0.0f;
  if (w == 0) { a = wsum(a); b = wsum(b); }
}

// Pass 1 of the forward: per (channel, split) shifted sums  S1 = sum(x-K), S2 = sum((x-K)^2), K = x[0,c,0]
// (shifting by a sample of the data keeps E[x^2]-E[x]^2 well conditioned).  grid = (C, S); split s takes images
// s, s+S, ...  MODE 1 (backward): S1 = sum(dy), S2 = sum(dy * xhat).
template <int MODE>
__global__ void bn_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ mean,
                                 const float* __restrict__ istd, float* __restrict__ partial, int N, int C, int HW) {
  int c = blockIdx.x, s = blockIdx.y, S = gridDim.y;
  float k = MODE == 0 ? x[(int64_t)c * HW] : mean[c];
  float is = MODE == 0 ? 1.0f : istd[c];
  float a = 0.0f, b = 0.0f;
  // The split's images are walked as one flat index space so that all threads stay busy when HW is small.
  const int n_imgs = (N - s + S - 1) / S;
  if ((HW & 3) == 0) {
    const int hw4 = HW >> 2;
    const int64_t total = (int64_t)n_imgs * hw4;
    for (int64_t t = threadIdx.x; t < total; t += blockDim.x) {
      int n = s + (int)(t / hw4) * S, i = (int)(t % hw4);
      const int64_t off = ((int64_t)n * C + c) * HW;
      float4 v = reinterpret_cast<const float4*>(x + off)[i];
      if (MODE == 0) {
        float d0 = v.x - k, d1 = v.y - k, d2 = v.z - k, d3 = v.w - k;
        a += (d0 + d1) + (d2 + d3); b += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      } else {
        float4 d = reinterpret_cast<const float4*>(dy + off)[i];
        a += (d.x + d.y) + (d.z + d.w);
        b += (d.x * ((v.x - k) * is) + d.y * ((v.y - k) * is)) + (d.z * ((v.z - k) * is) + d.w * ((v.w - k) * is));
      }
    }
  } else {
    const int64_t total = (int64_t)n_imgs * HW;
    for (int64_t t = threadIdx.x; t < total; t += blockDim.x) {
      int n = s + (int)(t / HW) * S, i = (int)(t % HW);
      const int64_t off = ((int64_t)n * C + c) * HW + i;
      float v = x[off] - k;
      if (MODE == 0) { a += v; b += v * v; } else { a += dy[off]; b += dy[off] * (v * is); }
    }
  }
  block_sum2(a, b);
  if (threadIdx.x == 0) { partial[((int64_t)c * S + s) * 2] = a; partial[((int64_t)c * S + s) * 2 + 1] = b; }
}
// Forward finalize: mean, biased variance (TensorDslCPU.scala:1047-1056), saved mean / inverse std and the running
// statistics update the reference gets from cuDNN (factor `momentum`, unbiased variance; TensorDslCudnn.scala:1025-1056).
__global__ void bn_fwd_finalize_kernel(const float* __restrict__ x, const float* __restrict__ partial, int S, int C, int HW, double m,
                                       float eps, float momentum, float* save_mean, float* save_istd, float* run_mean, float* run_var) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s1 = 0, s2 = 0;
  for (int s = 0; s < S; ++s) { s1 += partial[((int64_t)c * S + s) * 2]; s2 += partial[((int64_t)c * S + s) * 2 + 1]; }
  double k = x[(int64_t)c * HW];
  double dm = s1 / m, var = s2 / m - dm * dm;
  if (var < 0) var = 0;
  float mean = (float)(k + dm);
  save_mean[c] = mean;
  save_istd[c] = 1.0f / sqrtf((float)var + eps);
  if (run_mean) run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mean;
  if (run_var) run_var[c] = (1.0f - momentum) * run_var[c] + momentum * (float)(var * (m > 1 ? m / (m - 1) : 1.0));
}
// y = (x - mean) * istd * gamma + beta, 8 B per element.
__global__ void bn_apply_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ mean,
                                const float* __restrict__ istd, const float* __restrict__ gamma, const float* __restrict__ beta,
                                int C, int HW, int64_t n, bool vec) {
  if (vec) {
    int hw4 = HW >> 2; int64_t n4 = n >> 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
      int c = (int)((i / hw4) % C);
      float mu = mean[c], sc = istd[c] * gamma[c], sh = beta[c];
      float4 v = reinterpret_cast<const float4*>(x)[i];
      v.x = (v.x - mu) * sc + sh; v.y = (v.y - mu) * sc + sh; v.z = (v.z - mu) * sc + sh; v.w = (v.w - mu) * sc + sh;
      reinterpret_cast<float4*>(y)[i] = v;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
      int c = (int)((i / HW) % C);
      y[i] = (x[i] - mean[c]) * (istd[c] * gamma[c]) + beta[c];
    }
  }
}
// Backward finalize: dbeta += sum dy, dgamma += sum dy*xhat; coef[c] = {gamma*istd, sum dy / m, sum dy*xhat / m}.
__global__ void bn_bwd_finalize_kernel(const float* __restrict__ partial, int S, int C, double m, const float* __restrict__ gamma,
                                       const float* __restrict__ istd, float* dgamma, float* dbeta, float* __restrict__ coef) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s1 = 0, s2 = 0;
  for (int s = 0; s < S; ++s) { s1 += partial[((int64_t)c * S + s) * 2]; s2 += partial[((int64_t)c * S + s) * 2 + 1]; }
  if (dbeta) dbeta[c] += (float)s1;
  if (dgamma) dgamma[c] += (float)s2;
  coef[c * 3] = gamma[c] * istd[c]; coef[c * 3 + 1] = (float)(s1 / m); coef[c * 3 + 2] = (float)(s2 / m);
}
// dx += gamma*istd * (dy - mean(dy) - xhat * mean(dy*xhat)): reads x, dy, dx and writes dx, 16 B per element.
__global__ void bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* dx, const float* __restrict__ mean,
                                    const float* __restrict__ istd, const float* __restrict__ coef, int C, int HW, int64_t n, bool vec) {
  if (vec) {
    int hw4 = HW >> 2; int64_t n4 = n >> 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
      int c = (int)((i / hw4) % C);
      float mu = mean[c], is = istd[c], a = coef[c * 3], b = coef[c * 3 + 1], c2 = coef[c * 3 + 2];
      float4 v = reinterpret_cast<const float4*>(x)[i], d = reinterpret_cast<const float4*>(dy)[i], o = reinterpret_cast<float4*>(dx)[i];
      o.x += a * (d.x - b - (v.x - mu) * is * c2); o.y += a * (d.y - b - (v.y - mu) * is * c2);
      o.z += a * (d.z - b - (v.z - mu) * is * c2); o.w += a * (d.w - b - (v.w - mu) * is * c2);
      reinterpret_cast<float4*>(dx)[i] = o;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
      int c = (int)((i / HW) % C);
      dx[i] += coef[c * 3] * (dy[i] - coef[c * 3 + 1] - (x[i] - mean[c]) * istd[c] * coef[c * 3 + 2]);
    }
  }
}
__global__ void bn_inference_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ gamma, const float* __restrict__ beta,
                                    const float* __restrict__ rm, const float* __restrict__ rv, int C, int HW, int64_t n, float eps) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int c = (int)((i / HW) % C);
    y[i] = (x[i] - rm[c]) / sqrtf(rv[c] + eps) * gamma[c] + beta[c];   // TensorDslCPU.scala:1040-1045
  }
}

// ---- One launch per batch norm: a thread-block cluster of K CTAs owns one channel.
// Every CTA sums its contiguous slice of the channel's (image, pixel) items, the K partial pairs are exchanged through
// distributed shared memory, every CTA derives the same statistics from them in the same order (double), and the
// second sweep re-reads the slice (at most a few tens of KB per CTA, still in L2) to write the result. DRAM sees the
// compulsory traffic only: x once and y once forward (8 B per element); x, dy, dx in and dx out backward (16 B).
// cluster.sync() is the hardware cluster barrier (all CTAs of a cluster are co-scheduled), not a spin on memory.
struct BnClusterPlan { int K; int threads; int per_cta; };
static BnClusterPlan bn_cluster_plan(int N, int C, int HW) {
  const int64_t items = (int64_t)N * (HW >> 2);                   // float4 items per channel
  int K = 1;
  while (K < 8 && (int64_t)C * K < 2 * (int64_t)g.sm_count && items / (K * 2) >= 512) K *= 2;
  BnClusterPlan p;
  p.K = K; p.per_cta = (int)ceil_div(items, K);
  int t = 64; while (t < 512 && t * 4 < p.per_cta) t <<= 1;    // about four float4 per thread: small slices get small CTAs, many per SM
  p.threads = t;
  return p;
}

// add != null in the forward kernels below (fusion level 3, a residual block's last layer): the normalised value is not
// written to y; `add` is added to it, the ReLU applied, and the sum goes where the held add would have put it (the
// launcher passes that destination as y).  The value is rounded to a float before the addition exactly as the separate
// kernels would have rounded it on its way through memory, so the result is the same bit for bit.
__device__ __forceinline__ float4 add4(float4 v, float4 s) { v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w; return v; }

// VPT > 0: the CTA's slice is at most VPT float4 per thread and stays in registers between the two sweeps (all loads of a
// thread are issued back to back); VPT == 0: any slice length, the second sweep re-reads it.
constexpr int kBnVpt = 8;          // forward: x
constexpr int kBnVptBwd = 4;       // backward keeps x, dy and dx: half the slice per thread for the same register budget

template <int VPT>
__global__ void __launch_bounds__(512, 2) bn_fwd_cluster_kernel(const float* x, float* y, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                             float* run_mean, float* run_var, float* save_mean, float* save_istd,
                                                             int N, int C, int HW, int per_cta, float eps, float momentum, int relu, const float* __restrict__ add) {
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned K = cluster.num_blocks(), r = cluster.block_rank();
  const int c = blockIdx.x / K;
  const int hw4 = HW >> 2;
  const int total = N * hw4, begin = (int)r * per_cta;              // the launcher keeps N * hw4 below 2^31
  const int end = begin + per_cta < total ? begin + per_cta : total;
  __shared__ float part[2];
  __shared__ float stat[2];
  const float k = x[(int64_t)c * HW];                               // shift: a sample of the channel (see bn_reduce_kernel)
  float a = 0.0f, b = 0.0f;
  float4 keep[VPT > 0 ? VPT : 1];
  if (VPT > 0) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) { const int n = t / hw4, i = t - n * hw4; keep[j] = reinterpret_cast<const float4*>(x + ((int64_t)n * C + c) * HW)[i]; }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) {
        const float d0 = keep[j].x - k, d1 = keep[j].y - k, d2 = keep[j].z - k, d3 = keep[j].w - k;
        a += (d0 + d1) + (d2 + d3); b += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
    }
  } else {
#pragma unroll 4
    for (int t = begin + (int)threadIdx.x; t < end; t += (int)blockDim.x) {
      const int n = t / hw4, i = t - n * hw4;
      const float4 v = reinterpret_cast<const float4*>(x + ((int64_t)n * C + c) * HW)[i];
      const float d0 = v.x - k, d1 = v.y - k, d2 = v.z - k, d3 = v.w - k;
      a += (d0 + d1) + (d2 + d3); b += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  block_sum2(a, b);
  if (threadIdx.x == 0) { part[0] = a; part[1] = b; }
  cluster.sync();
  if (threadIdx.x == 0) {
    double s1 = 0, s2 = 0;
    for (unsigned q = 0; q < K; ++q) { const float* p = cluster.map_shared_rank(part, q); s1 += p[0]; s2 += p[1]; }
    const double m = (double)N * HW;
    const double dm = s1 / m;
    double var = s2 / m - dm * dm;
    if (var < 0) var = 0;
    const float mean = (float)((double)k + dm), is = 1.0f / sqrtf((float)var + eps);
    stat[0] = mean; stat[1] = is;
    if (r == 0) {
      save_mean[c] = mean; save_istd[c] = is;
      if (run_mean) run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mean;
      if (run_var) run_var[c] = (1.0f - momentum) * run_var[c] + momentum * (float)(var * (m > 1 ? m / (m - 1) : 1.0));
    }
  }
  cluster.sync();                // every remote read of part[] is over before a CTA may leave; stat[] is visible to the block
  const float mu = stat[0], sc = stat[1] * gamma[c], sh = beta[c];
  if (VPT > 0) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) {
        const int n = t / hw4, i = t - n * hw4;
        float4 v = keep[j];
        v.x = (v.x - mu) * sc + sh; v.y = (v.y - mu) * sc + sh; v.z = (v.z - mu) * sc + sh; v.w = (v.w - mu) * sc + sh;
        if (add) v = add4(v, reinterpret_cast<const float4*>(add + ((int64_t)n * C + c) * HW)[i]);
        if (relu) { v.x = v.x < 0.0f ? 0.0f : v.x; v.y = v.y < 0.0f ? 0.0f : v.y; v.z = v.z < 0.0f ? 0.0f : v.z; v.w = v.w < 0.0f ? 0.0f : v.w; }
        reinterpret_cast<float4*>(y + ((int64_t)n * C + c) * HW)[i] = v;
      }
    }
  } else {
#pragma unroll 4
    for (int t = begin + (int)threadIdx.x; t < end; t += (int)blockDim.x) {
      const int n = t / hw4, i = t - n * hw4;
      const int64_t off = ((int64_t)n * C + c) * HW;
      float4 v = reinterpret_cast<const float4*>(x + off)[i];
      v.x = (v.x - mu) * sc + sh; v.y = (v.y - mu) * sc + sh; v.z = (v.z - mu) * sc + sh; v.w = (v.w - mu) * sc + sh;
      if (add) v = add4(v, reinterpret_cast<const float4*>(add + off)[i]);
      if (relu) { v.x = v.x < 0.0f ? 0.0f : v.x; v.y = v.y < 0.0f ? 0.0f : v.y; v.z = v.z < 0.0f ? 0.0f : v.z; v.w = v.w < 0.0f ? 0.0f : v.w; }
      reinterpret_cast<float4*>(y + off)[i] = v;
    }
  }
}

// mask_y != null: the ReLU gradient held back by the look-ahead fusion is applied to dy on the way in (dy = mask_y > 0 ? dy : 0)
// and the masked values are written back, so that dy ends up as the separate ReLU-gradient kernel would have left it.
__device__ __forceinline__ float4 relu_mask(float4 d, float4 m) {
  d.x = m.x > 0.0f ? d.x : 0.0f; d.y = m.y > 0.0f ? d.y : 0.0f; d.z = m.z > 0.0f ? d.z : 0.0f; d.w = m.w > 0.0f ? d.w : 0.0f;
  return d;
}

template <int VPT>
__global__ void __launch_bounds__(512, 2) bn_bwd_cluster_kernel(const float* __restrict__ x, float* dy, float* dx, const float* __restrict__ gamma,
                                                             float* dgamma, float* dbeta, const float* __restrict__ mean, const float* __restrict__ istd,
                                                             int N, int C, int HW, int per_cta, const float* mask_y, int fresh, float* extra) {
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned K = cluster.num_blocks(), r = cluster.block_rank();
  const int c = blockIdx.x / K;
  const int hw4 = HW >> 2;
  const int total = N * hw4, begin = (int)r * per_cta;
  const int end = begin + per_cta < total ? begin + per_cta : total;
  __shared__ float part[2];
  __shared__ float stat[3];
  const float mu = mean[c], is = istd[c];
  float a = 0.0f, b = 0.0f;
  float4 kx[VPT > 0 ? VPT : 1], kd[VPT > 0 ? VPT : 1];
  if (VPT > 0) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) {
        const int n = t / hw4, i = t - n * hw4;
        const int64_t off = ((int64_t)n * C + c) * HW;
        kx[j] = reinterpret_cast<const float4*>(x + off)[i]; kd[j] = reinterpret_cast<const float4*>(dy + off)[i];
        if (mask_y) { kd[j] = relu_mask(kd[j], reinterpret_cast<const float4*>(mask_y + off)[i]); if (!(fresh & 2)) reinterpret_cast<float4*>(dy + off)[i] = kd[j]; }
        if (extra) {                       // the absorbed add gradient's other destination: extra (+)= masked dy (bit 2 of fresh: it holds nothing yet)
          float4 e = (fresh & 4) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(extra + off)[i];
          e.x += kd[j].x; e.y += kd[j].y; e.z += kd[j].z; e.w += kd[j].w;
          reinterpret_cast<float4*>(extra + off)[i] = e;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) {
        const float4 v = kx[j], d = kd[j];
        a += (d.x + d.y) + (d.z + d.w);
        b += (d.x * ((v.x - mu) * is) + d.y * ((v.y - mu) * is)) + (d.z * ((v.z - mu) * is) + d.w * ((v.w - mu) * is));
      }
    }
  } else {
#pragma unroll 4
    for (int t = begin + (int)threadIdx.x; t < end; t += (int)blockDim.x) {
      const int n = t / hw4, i = t - n * hw4;
      const int64_t off = ((int64_t)n * C + c) * HW;
      const float4 v = reinterpret_cast<const float4*>(x + off)[i];
      float4 d = reinterpret_cast<const float4*>(dy + off)[i];
      if (mask_y) { d = relu_mask(d, reinterpret_cast<const float4*>(mask_y + off)[i]); reinterpret_cast<float4*>(dy + off)[i] = d; }   // always written: the second sweep below reads dy again
      if (extra) {
        float4 e = (fresh & 4) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(extra + off)[i];
        e.x += d.x; e.y += d.y; e.z += d.z; e.w += d.w;
        reinterpret_cast<float4*>(extra + off)[i] = e;
      }
      a += (d.x + d.y) + (d.z + d.w);
      b += (d.x * ((v.x - mu) * is) + d.y * ((v.y - mu) * is)) + (d.z * ((v.z - mu) * is) + d.w * ((v.w - mu) * is));
    }
  }
  block_sum2(a, b);
  if (threadIdx.x == 0) { part[0] = a; part[1] = b; }
  cluster.sync();
  if (threadIdx.x == 0) {
    double s1 = 0, s2 = 0;
    for (unsigned q = 0; q < K; ++q) { const float* p = cluster.map_shared_rank(part, q); s1 += p[0]; s2 += p[1]; }
    const double m = (double)N * HW;
    stat[0] = gamma[c] * is; stat[1] = (float)(s1 / m); stat[2] = (float)(s2 / m);
    if (r == 0) { if (dbeta) dbeta[c] += (float)s1; if (dgamma) dgamma[c] += (float)s2; }
  }
  cluster.sync();
  if (dx == nullptr) return;                                        // uniform over the cluster, after its last barrier
  const float ca = stat[0], cb = stat[1], cc = stat[2];
  if (VPT > 0) {
    float4 o[VPT > 0 ? VPT : 1];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) { const int n = t / hw4, i = t - n * hw4; o[j] = (fresh & 1) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(dx + ((int64_t)n * C + c) * HW)[i]; }   // bit 0 of fresh: dx holds nothing yet, the result is written (bit 1: an absorbed ReLU gradient is not written back)
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int t = begin + j * (int)blockDim.x + (int)threadIdx.x;
      if (t < end) {
        const int n = t / hw4, i = t - n * hw4;
        const float4 v = kx[j], d = kd[j];
        float4 w = o[j];
        w.x += ca * (d.x - cb - (v.x - mu) * is * cc); w.y += ca * (d.y - cb - (v.y - mu) * is * cc);
        w.z += ca * (d.z - cb - (v.z - mu) * is * cc); w.w += ca * (d.w - cb - (v.w - mu) * is * cc);
        reinterpret_cast<float4*>(dx + ((int64_t)n * C + c) * HW)[i] = w;
      }
    }
  } else {
#pragma unroll 4
    for (int t = begin + (int)threadIdx.x; t < end; t += (int)blockDim.x) {
      const int n = t / hw4, i = t - n * hw4;
      const int64_t off = ((int64_t)n * C + c) * HW;
      const float4 v = reinterpret_cast<const float4*>(x + off)[i], d = reinterpret_cast<const float4*>(dy + off)[i];
      float4 o = (fresh & 1) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(dx + off)[i];
      o.x += ca * (d.x - cb - (v.x - mu) * is * cc); o.y += ca * (d.y - cb - (v.y - mu) * is * cc);
      o.z += ca * (d.z - cb - (v.z - mu) * is * cc); o.w += ca * (d.w - cb - (v.w - mu) * is * cc);
      reinterpret_cast<float4*>(dx + off)[i] = o;
    }
  }
}


// ---- channels that one CTA row can hold: no cluster, several channels per CTA -------------------------------------------
// When a channel's N*HW/4 items fit the registers of at most 512 threads (every layer of the last three ResNet stages at
// batch 128) the cluster machinery buys nothing: a plain launch is cheaper than a cluster launch, two __syncthreads are
// cheaper than two cluster barriers, and with 1024 or 2048 channels of a few hundred values each the launch is bound by
// the rate at which CTAs can be dispatched (measured: 9.5 us at 512 CTAs, 18 us at 2048 CTAs for the same 4 MB).  Here a
// CTA is G rows of T threads (T a multiple of 32: warps never straddle rows), row g owns channel blockIdx.x * G + g.
struct BnPackedPlan { int T, G; };
static bool bn_packed_plan(int N, int C, int HW, int vpt, BnPackedPlan& p) {
  const int64_t items = (int64_t)N * (HW >> 2);
  if (items > (int64_t)vpt * 512) return false;
  int T = 32; while (T < 512 && (int64_t)T * 4 < items) T <<= 1;      // about four float4 per thread
  while ((int64_t)T * vpt < items) T <<= 1;
  if (T > 512) return false;
  int G = 512 / T;
  while (G > 1 && (C + G - 1) / G < 128) G >>= 1;                       // keep at least 128 CTAs when there are channels for them
  p.T = T; p.G = G;
  return true;
}
// Sums of a and b over the T threads of this thread's row; every thread of the row returns the totals.  red: 2 x 16 floats.
__device__ __forceinline__ void row_sum2(float& a, float& b, float* red) {
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, lane = tid & 31, warp = tid >> 5;
  a = wsum(a); b = wsum(b);
  if (lane == 0) { red[warp] = a; red[16 + warp] = b; }
  __syncthreads();
  const int w0 = (threadIdx.y * blockDim.x) >> 5, nw = blockDim.x >> 5;
  float s1 = 0.0f, s2 = 0.0f;
  for (int w = 0; w < nw; ++w) { s1 += red[w0 + w]; s2 += red[16 + w0 + w]; }
  a = s1; b = s2;
}

template <int VPT>
__global__ void __launch_bounds__(512, 2) bn_fwd_packed_kernel(const float* x, float* y, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            float* run_mean, float* run_var, float* save_mean, float* save_istd,
                                                            int N, int C, int HW, float eps, float momentum, int relu, const float* __restrict__ add) {
  __shared__ float red[32];
  __shared__ float stat[16][2];
  const int g = threadIdx.y, T = blockDim.x;
  const int c = blockIdx.x * blockDim.y + g;
  const bool live = c < C;                                              // idle rows of the last CTA still meet the barriers
  const int hw4 = HW >> 2, total = N * hw4;
  const float k = live ? x[(int64_t)c * HW] : 0.0f;                     // shift: a sample of the channel (see bn_reduce_kernel)
  float a = 0.0f, b = 0.0f;
  float4 keep[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (live && t < total) { const int n = t / hw4, i = t - n * hw4; keep[j] = reinterpret_cast<const float4*>(x + ((int64_t)n * C + c) * HW)[i]; }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (live && t < total) {
      const float d0 = keep[j].x - k, d1 = keep[j].y - k, d2 = keep[j].z - k, d3 = keep[j].w - k;
      a += (d0 + d1) + (d2 + d3); b += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  row_sum2(a, b, red);
  if (threadIdx.x == 0 && live) {
    const double m = (double)N * HW;
    const double dm = (double)a / m;
    double var = (double)b / m - dm * dm;
    if (var < 0) var = 0;
    const float mean = (float)((double)k + dm), is = 1.0f / sqrtf((float)var + eps);
    stat[g][0] = mean; stat[g][1] = is;
    save_mean[c] = mean; save_istd[c] = is;
    if (run_mean) run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mean;
    if (run_var) run_var[c] = (1.0f - momentum) * run_var[c] + momentum * (float)(var * (m > 1 ? m / (m - 1) : 1.0));
  }
  __syncthreads();
  if (!live) return;
  const float mu = stat[g][0], sc = stat[g][1] * gamma[c], sh = beta[c];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (t < total) {
      const int n = t / hw4, i = t - n * hw4;
      float4 v = keep[j];
      v.x = (v.x - mu) * sc + sh; v.y = (v.y - mu) * sc + sh; v.z = (v.z - mu) * sc + sh; v.w = (v.w - mu) * sc + sh;
      if (add) v = add4(v, reinterpret_cast<const float4*>(add + ((int64_t)n * C + c) * HW)[i]);
      if (relu) { v.x = v.x < 0.0f ? 0.0f : v.x; v.y = v.y < 0.0f ? 0.0f : v.y; v.z = v.z < 0.0f ? 0.0f : v.z; v.w = v.w < 0.0f ? 0.0f : v.w; }
      reinterpret_cast<float4*>(y + ((int64_t)n * C + c) * HW)[i] = v;
    }
  }
}

template <int VPT>
__global__ void __launch_bounds__(512, 2) bn_bwd_packed_kernel(const float* __restrict__ x, float* dy, float* dx, const float* __restrict__ gamma,
                                                            float* dgamma, float* dbeta, const float* __restrict__ mean, const float* __restrict__ istd,
                                                            int N, int C, int HW, const float* mask_y, int fresh, float* extra) {
  __shared__ float red[32];
  const int g = threadIdx.y, T = blockDim.x;
  const int c = blockIdx.x * blockDim.y + g;
  const bool live = c < C;
  const int hw4 = HW >> 2, total = N * hw4;
  const float mu = live ? mean[c] : 0.0f, is = live ? istd[c] : 0.0f;
  float a = 0.0f, b = 0.0f;
  float4 kx[VPT], kd[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (live && t < total) {
      const int n = t / hw4, i = t - n * hw4;
      const int64_t off = ((int64_t)n * C + c) * HW;
      kx[j] = reinterpret_cast<const float4*>(x + off)[i]; kd[j] = reinterpret_cast<const float4*>(dy + off)[i];
      if (mask_y) { kd[j] = relu_mask(kd[j], reinterpret_cast<const float4*>(mask_y + off)[i]); if (!(fresh & 2)) reinterpret_cast<float4*>(dy + off)[i] = kd[j]; }
      if (extra) {
        float4 e = (fresh & 4) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(extra + off)[i];
        e.x += kd[j].x; e.y += kd[j].y; e.z += kd[j].z; e.w += kd[j].w;
        reinterpret_cast<float4*>(extra + off)[i] = e;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (live && t < total) {
      const float4 v = kx[j], d = kd[j];
      a += (d.x + d.y) + (d.z + d.w);
      b += (d.x * ((v.x - mu) * is) + d.y * ((v.y - mu) * is)) + (d.z * ((v.z - mu) * is) + d.w * ((v.w - mu) * is));
    }
  }
  row_sum2(a, b, red);                                                  // every thread of the row holds both totals: no second barrier
  if (!live) return;
  if (threadIdx.x == 0) { if (dbeta) dbeta[c] += a; if (dgamma) dgamma[c] += b; }
  if (dx == nullptr) return;
  const float m = (float)N * (float)HW;
  const float ca = gamma[c] * is, cb = a / m, cc = b / m;
  float4 o[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (t < total) { const int n = t / hw4, i = t - n * hw4; o[j] = (fresh & 1) ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(dx + ((int64_t)n * C + c) * HW)[i]; }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int t = j * T + (int)threadIdx.x;
    if (t < total) {
      const int n = t / hw4, i = t - n * hw4;
      const float4 v = kx[j], d = kd[j];
      float4 w = o[j];
      w.x += ca * (d.x - cb - (v.x - mu) * is * cc); w.y += ca * (d.y - cb - (v.y - mu) * is * cc);
      w.z += ca * (d.z - cb - (v.z - mu) * is * cc); w.w += ca * (d.w - cb - (v.w - mu) * is * cc);
      reinterpret_cast<float4*>(dx + ((int64_t)n * C + c) * HW)[i] = w;
    }
  }
}

static int bn_splits(int N, int C) {
  int s = (int)ceil_div(2 * (int64_t)g.sm_count, C);
  if (s > N) s = N;
  if (s > 64) s = 64;
  return s < 1 ? 1 : s;
}

// Issues a BN forward described by `p` (the cluster path), optionally with the ReLU of its result; a PEND_BN_ADD also adds
// p.a and writes p.out instead of p.y.
int bn_fwd_issue(const Pending& p, bool relu) {
  const BnClusterPlan c = bn_cluster_plan(p.N, p.C, p.HW);
  const int r = relu ? 1 : 0;
  const float* add = p.kind == PEND_BN_ADD ? p.a : nullptr;
  float* y = p.kind == PEND_BN_ADD ? p.out : p.y;
  BnPackedPlan pk;
  if ((c.K == 1 || p.C >= 96) && bn_packed_plan(p.N, p.C, p.HW, kBnVpt, pk)) {
    LTB_LAUNCH(bn_fwd_packed_kernel<kBnVpt>, (unsigned)ceil_div(p.C, pk.G), dim3(pk.T, pk.G), 0, p.x, y, p.gamma, p.beta, p.run_mean, p.run_var,
               p.save_mean, p.save_istd, p.N, p.C, p.HW, p.eps, p.momentum, r, add);
    return LTB_OK;
  }
  if (c.per_cta <= kBnVpt * c.threads)
    LTB_LAUNCH_CLUSTER(bn_fwd_cluster_kernel<kBnVpt>, dim3((unsigned)p.C * c.K), dim3(c.threads), c.K, p.x, y, p.gamma, p.beta, p.run_mean, p.run_var,
                       p.save_mean, p.save_istd, p.N, p.C, p.HW, c.per_cta, p.eps, p.momentum, r, add);
  else
    LTB_LAUNCH_CLUSTER(bn_fwd_cluster_kernel<0>, dim3((unsigned)p.C * c.K), dim3(c.threads), c.K, p.x, y, p.gamma, p.beta, p.run_mean, p.run_var,
                       p.save_mean, p.save_istd, p.N, p.C, p.HW, c.per_cta, p.eps, p.momentum, r, add);
  return LTB_OK;
}

}  // namespace ltb

using namespace ltb;

extern "C" {

int ltb_maxpool_fwd(const float* x, float* y, int32_t* idx, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int pad) {
  LTB_INITED();
  LTB_REQUIRE(x && y && idx && N > 0 && C > 0 && kh >= 1 && kw >= 1 && sh >= 1 && sw >= 1 && pad >= 0, "ltb_maxpool_fwd: bad argument");
  LTB_REQUIRE(H + 2 * pad >= kh && W + 2 * pad >= kw, "ltb_maxpool_fwd: image too small for the window");
  LTB_REQUIRE((int64_t)N * C * H * W < ((int64_t)1 << 31), "ltb_maxpool_fwd: tensor too large for int32 indices");
  int oH = (H + 2 * pad - kh) / sh + 1, oW = (W + 2 * pad - kw) / sw + 1;
  int64_t n_out = (int64_t)N * C * oH * oW;
  if (kh == 2 && kw == 2 && sh == 2 && sw == 2 && pad == 0 && (W & 3) == 0 && (H & 1) == 0 && aligned16(x) && aligned16(y) && aligned16(idx)) {
    int64_t pairs = n_out / 2;
    LTB_LAUNCH(maxpool2x2_fwd_kernel, grid_for(pairs, 256), 256, 0, x, y, idx, pairs, H, W, oH, oW / 2);
  } else {
    LTB_LAUNCH(maxpool_fwd_kernel, grid_for(n_out, 256), 256, 0, x, y, idx, n_out, H, W, oH, oW, kh, kw, sh, sw, pad);
  }
  return LTB_OK;
}
int ltb_maxpool_bwd(float* dx, const float* dy, const int32_t* idx, int64_t n_out) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_REQUIRE(dx && dy && idx && n_out >= 0, "ltb_maxpool_bwd: bad argument");
  if (n_out) LTB_LAUNCH(maxpool_bwd_kernel, grid_for(n_out, 256), 256, 0, dx, dy, idx, n_out);
  return LTB_OK;
}
int ltb_avgpool_fwd(const float* x, float* y, int N, int C, int H, int W, int kh, int kw, int sh, int sw) {
  LTB_INITED();
  LTB_REQUIRE(x && y && N > 0 && C > 0 && kh >= 1 && kw >= 1 && sh >= 1 && sw >= 1 && H >= kh && W >= kw, "ltb_avgpool_fwd: bad argument");
  int oH = (H - kh) / sh + 1, oW = (W - kw) / sw + 1;
  int64_t n_out = (int64_t)N * C * oH * oW;
  LTB_LAUNCH(avgpool_fwd_kernel, grid_for(n_out, 256), 256, 0, x, y, n_out, H, W, oH, oW, kh, kw, sh, sw);
  return LTB_OK;
}
int ltb_avgpool_bwd(float* dx, const float* dy, int N, int C, int H, int W, int kh, int kw, int sh, int sw) {
  LTB_INITED(); { int rc_ = grad_settle(dx, 0); if (!rc_) rc_ = grad_settle(dy, 0); if (rc_) return rc_; }
  LTB_REQUIRE(dx && dy && N > 0 && C > 0 && kh >= 1 && kw >= 1 && sh >= 1 && sw >= 1 && H >= kh && W >= kw, "ltb_avgpool_bwd: bad argument");
  int oH = (H - kh) / sh + 1, oW = (W - kw) / sw + 1;
  int64_t n_in = (int64_t)N * C * H * W;
  LTB_LAUNCH(avgpool_bwd_kernel, grid_for(n_in, 256), 256, 0, dx, dy, n_in, H, W, oH, oW, kh, kw, sh, sw);
  return LTB_OK;
}

int ltb_bn_train_fwd(const float* x, float* y, const float* gamma, const float* beta, float* run_mean, float* run_var,
                     float* save_mean, float* save_istd, int N, int C, int HW, float eps, float momentum) {
  LTB_INITED();
  LTB_REQUIRE(x && y && gamma && beta && save_mean && save_istd && N > 0 && C > 0 && HW > 0, "ltb_bn_train_fwd: bad argument");
  int S = bn_splits(N, C);
  LTB_REQUIRE((size_t)C * S * 2 * 4 <= g.cur_scratch_bytes(), "ltb_bn_train_fwd: too many channels");
  int64_t n = (int64_t)N * C * HW;
  bool vec = (HW & 3) == 0 && aligned16(x) && aligned16(y);
  if (vec && (int64_t)N * (HW >> 2) < ((int64_t)1 << 30)) {      // one cluster launch: statistics and result in the same kernel
    Pending p;
    p.kind = PEND_BN_FWD; p.n = n; p.x = x; p.y = y; p.gamma = gamma; p.beta = beta; p.run_mean = run_mean; p.run_var = run_var;
    p.save_mean = save_mean; p.save_istd = save_istd; p.N = N; p.C = C; p.HW = HW; p.eps = eps; p.momentum = momentum;
    if (g.fusion) { g.pending = p; return LTB_OK; }              // held for one call: an in-place ReLU of y may join it
    return bn_fwd_issue(p, false);
  }
  LTB_LAUNCH(bn_reduce_kernel<0>, dim3(C, S), 256, 0, x, nullptr, nullptr, nullptr, g.cur_scratch(), N, C, HW);
  LTB_LAUNCH(bn_fwd_finalize_kernel, (C + 127) / 128, 128, 0, x, (const float*)g.cur_scratch(), S, C, HW, (double)N * HW, eps, momentum,
             save_mean, save_istd, run_mean, run_var);
  LTB_LAUNCH(bn_apply_kernel, grid_for(vec ? n / 4 : n, 256), 256, 0, x, y, (const float*)save_mean, (const float*)save_istd, gamma, beta, C, HW, n, vec);
  return LTB_OK;
}
int ltb_bn_bwd(const float* x, float* dx, const float* dy, const float* gamma, float* dgamma, float* dbeta,
               const float* save_mean, const float* save_istd, int N, int C, int HW) {
  LTB_INITED_NOFLUSH();
  LTB_REQUIRE(x && dy && gamma && save_mean && save_istd && N > 0 && C > 0 && HW > 0, "ltb_bn_bwd: bad argument");
  int S = bn_splits(N, C);
  LTB_REQUIRE((size_t)C * (S * 2 + 3) * 4 <= g.cur_scratch_bytes(), "ltb_bn_bwd: too many channels");
  float* coef = g.cur_scratch() + (size_t)C * S * 2;
  int64_t n = (int64_t)N * C * HW;
  bool vec = (HW & 3) == 0 && aligned16(x) && aligned16(dy) && aligned16(dx);
  const bool cluster_path = vec && (int64_t)N * (HW >> 2) < ((int64_t)1 << 30);
  // a held in-place ReLU gradient on exactly this dy is applied by the kernel itself
  const float* mask_y = nullptr;
  float* extra = nullptr; int extra_fresh = 0;
  if (g.pending.kind == PEND_RELU_GRAD && cluster_path && g.pending.d == dy && g.pending.n == n && aligned16(g.pending.relu_y)) {
    mask_y = g.pending.relu_y; g.pending.kind = PEND_NONE;
  } else if (g.pending.kind == PEND_RELU_ADD_GRAD && cluster_path && g.pending.n == n && aligned16(g.pending.relu_y) && aligned16(g.pending.d) &&
             aligned16(g.pending.da) && aligned16(g.pending.db) &&
             ((g.pending.da == dy && g.pending.fa) || (g.pending.db == dy && g.pending.fb))) {
    // The held ReLU + add gradient would write m = (y > 0 ? d : 0) into this dy, which nothing else has written: read m straight
    // from d instead, and write the add's other destination here.  dy itself stays unwritten (its owner declared it dead after
    // this call: fusion level 2).
    const bool first = g.pending.da == dy;
    extra = first ? g.pending.db : g.pending.da; extra_fresh = first ? g.pending.fb : g.pending.fa;
    mask_y = g.pending.relu_y; dy = g.pending.d;
    g.pending.kind = PEND_NONE;
  } else if (g.pending.kind) { int rc = flush_pending(); if (rc) return rc; }
  // dx declared unset (ltb_grad_unset): the one-launch kernels write their result instead of adding; the three-kernel path
  // fills it with zeros first.  dy itself is someone's gradient buffer too: it must hold data by now.
  { int rc = grad_settle(dy, (size_t)n * 4); if (rc) return rc; }
  const int fresh = (dx && cluster_path && grad_take_unset(dx, (size_t)n * 4) ? 1 : 0) | (mask_y && g.fusion_no_writeback ? 2 : 0) | (extra_fresh ? 4 : 0);
  if (dx && !(fresh & 1)) { int rc = grad_settle(dx, (size_t)n * 4); if (rc) return rc; }
  if (cluster_path) {
    const BnClusterPlan p = bn_cluster_plan(N, C, HW);
    float* dyw = const_cast<float*>(dy);                           // written only when the held ReLU gradient is applied to it
    BnPackedPlan pk;
    if ((p.K == 1 || C >= 96) && bn_packed_plan(N, C, HW, kBnVptBwd, pk)) {
      LTB_LAUNCH(bn_bwd_packed_kernel<kBnVptBwd>, (unsigned)ceil_div(C, pk.G), dim3(pk.T, pk.G), 0, x, dyw, dx, gamma, dgamma, dbeta,
                 save_mean, save_istd, N, C, HW, mask_y, fresh, extra);
      return LTB_OK;
    }
    if (p.per_cta <= kBnVptBwd * p.threads)
      LTB_LAUNCH_CLUSTER(bn_bwd_cluster_kernel<kBnVptBwd>, dim3((unsigned)C * p.K), dim3(p.threads), p.K, x, dyw, dx, gamma, dgamma, dbeta,
                         save_mean, save_istd, N, C, HW, p.per_cta, mask_y, fresh, extra);
    else
      LTB_LAUNCH_CLUSTER(bn_bwd_cluster_kernel<0>, dim3((unsigned)C * p.K), dim3(p.threads), p.K, x, dyw, dx, gamma, dgamma, dbeta,
                         save_mean, save_istd, N, C, HW, p.per_cta, mask_y, fresh, extra);
    return LTB_OK;
  }
  LTB_LAUNCH(bn_reduce_kernel<1>, dim3(C, S), 256, 0, x, dy, save_mean, save_istd, g.cur_scratch(), N, C, HW);
  LTB_LAUNCH(bn_bwd_finalize_kernel, (C + 127) / 128, 128, 0, (const float*)g.cur_scratch(), S, C, (double)N * HW, gamma, save_istd, dgamma, dbeta, coef);
  if (dx) LTB_LAUNCH(bn_bwd_apply_kernel, grid_for(vec ? n / 4 : n, 256), 256, 0, x, dy, dx, save_mean, save_istd, (const float*)coef, C, HW, n, vec);
  return LTB_OK;
}
int ltb_bn_inference(const float* x, float* y, const float* gamma, const float* beta, const float* rm, const float* rv,
                     int N, int C, int HW, float eps) {
  LTB_INITED(); LTB_REQUIRE(x && y && gamma && beta && rm && rv && N > 0 && C > 0 && HW > 0, "ltb_bn_inference: bad argument");
  int64_t n = (int64_t)N * C * HW;
  LTB_LAUNCH(bn_inference_kernel, grid_for(n, 256), 256, 0, x, y, gamma, beta, rm, rv, C, HW, n, eps);
  return LTB_OK;
}

}  // extern "C"
