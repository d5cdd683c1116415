// Reductions, softmax family, NLL loss and the vector/matrix-vector dot family.
//
// Replaces cudnnReduceTensor / cudnnSoftmax* (TensorDslCudnn.scala:1431-1576), the one-thread-per-block nllLoss
// kernels (DslAPI.scala:506-516) and cublasSdot/Sgemv (TensorDslCublas.scala:173-201, 257-264).  Semantics follow
// TensorDslCPU.scala (cited per entry point).  Rows are reduced by one warp each with shuffles; full reductions
// use a block tree in shared memory and, for large inputs, a second pass over per-block partials.
#include <cfloat>

#include "common.cuh"

namespace ltb {

__device__ __forceinline__ float warp_sum(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }
__device__ __forceinline__ float warp_max(float v) { for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }

__device__ float block_sum(float v) {
  __shared__ float sh[32];
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  v = threadIdx.x < nw ? sh[threadIdx.x] : 0.0f;
  if (w == 0) v = warp_sum(v);
  return v;   // valid in warp 0
}

// out[0] = scale * sum(x) (single block) or partial[b] = sum of the block's slice.
__global__ void sum_kernel(const float* __restrict__ x, float* out, int64_t n, float scale, bool partial) {
  float s = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s += x[i];
  s = block_sum(s);
  if (threadIdx.x == 0) out[partial ? blockIdx.x : 0] = partial ? s : s * scale;
}
__global__ void add_scalar_from_kernel(float* dx, const float* __restrict__ dout, float scale, int64_t n) {
  float v = dout[0] * scale;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dx[i] += v;
}
// out[o, l] = sum_s x[o, s, l]
__global__ void sum_dim_kernel(const float* __restrict__ x, float* out, int outer, int d, int inner) {
  int64_t n = (int64_t)outer * inner;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t o = i / inner, l = i % inner;
    const float* p = x + o * d * inner + l;
    float s = 0.0f;
    for (int k = 0; k < d; ++k) s += p[(int64_t)k * inner];
    out[i] = s;
  }
}
// inner == 1: one warp per output
__global__ void sum_lastdim_kernel(const float* __restrict__ x, float* out, int outer, int d) {
  int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; int lane = threadIdx.x & 31;
  if (w >= outer) return;
  float s = 0.0f;
  for (int k = lane; k < d; k += 32) s += x[w * d + k];
  s = warp_sum(s);
  if (lane == 0) out[w] = s;
}
__global__ void sum_dim_grad_kernel(float* dx, const float* __restrict__ dout, int outer, int d, int inner) {
  int64_t n = (int64_t)outer * d * inner;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t l = i % inner, o = i / ((int64_t)d * inner);
    dx[i] += dout[o * inner + l];
  }
}

// One warp per row. MODE 0 softmax, 1 logSoftmax (TensorDslCPU.scala:783-832).
template <int MODE>
__global__ void softmax_kernel(const float* __restrict__ x, float* y, int rows, int cols) {
  int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* p = x + r * cols; float* q = y + r * cols;
  float mx = -FLT_MAX;
  for (int i = lane; i < cols; i += 32) mx = fmaxf(mx, p[i]);
  mx = warp_max(mx);
  float s = 0.0f;
  for (int i = lane; i < cols; i += 32) s += expf(p[i] - mx);
  s = warp_sum(s);
  if (MODE == 0) { for (int i = lane; i < cols; i += 32) q[i] = expf(p[i] - mx) / s; }
  else { float logsum = mx + logf(s); for (int i = lane; i < cols; i += 32) q[i] = p[i] - logsum; }
}
// MODE 0: dx += y*(dy - sum dy*y) (cudnnSoftmaxBackward ACCURATE, TensorDslCudnn.scala:1465-1504);
// MODE 1: dx += dy - exp(y)*sum dy (TensorDslCPU.scala:837-846).
template <int MODE>
__global__ void softmax_grad_kernel(float* dx, const float* __restrict__ y, const float* __restrict__ dy, int rows, int cols) {
  int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* yy = y + r * cols; const float* d = dy + r * cols; float* o = dx + r * cols;
  float s = 0.0f;
  for (int i = lane; i < cols; i += 32) s += MODE == 0 ? d[i] * yy[i] : d[i];
  s = warp_sum(s);
  for (int i = lane; i < cols; i += 32) o[i] += MODE == 0 ? yy[i] * (d[i] - s) : d[i] - expf(yy[i]) * s;
}
__global__ void nll_kernel(const float* __restrict__ x, const int32_t* __restrict__ t, float* out, int rows, int cols) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < rows) { int k = t[b]; out[b] = (k >= 0 && k < cols) ? -1.0f * x[(int64_t)b * cols + k] : 0.0f; }
}
__global__ void nll_grad_kernel(float* dx, const float* __restrict__ dout, const int32_t* __restrict__ t, int rows, int cols) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < rows) { int k = t[b]; if (k >= 0 && k < cols) dx[(int64_t)b * cols + k] += -1.0f * dout[b]; }
}

// y[m] (+)= A[m,k] x[k]: one warp per row, float4 when k % 4 == 0 (memory-bound: A is read once).
template <bool ACC>
__global__ void gemv_rows_kernel(const float* __restrict__ a, const float* __restrict__ x, float* y, int m, int k) {
  int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; int lane = threadIdx.x & 31;
  if (r >= m) return;
  const float* row = a + r * k;
  float s = 0.0f;
  if ((k & 3) == 0 && ((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
    for (int i = lane * 4; i < k; i += 128) {
      float4 av = *reinterpret_cast<const float4*>(row + i), xv = *reinterpret_cast<const float4*>(x + i);
      s += av.x * xv.x + av.y * xv.y + av.z * xv.z + av.w * xv.w;
    }
  } else for (int i = lane; i < k; i += 32) s += row[i] * x[i];
  s = warp_sum(s);
  if (lane == 0) y[r] = ACC ? y[r] + s : s;
}
// dx[k] += sum_i A[i,k] dout[i]: threads along k (coalesced), loop over rows.
__global__ void gemv_cols_kernel(const float* __restrict__ a, const float* __restrict__ dout, float* dx, int m, int k) {
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= k) return;
  float s = 0.0f;
  for (int i = 0; i < m; ++i) s += a[(int64_t)i * k + j] * dout[i];
  dx[j] += s;
}
__global__ void outer_acc_kernel(float* da, const float* __restrict__ y, const float* __restrict__ dout, int m, int k) {
  int64_t n = (int64_t)m * k;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) da[i] += y[i % k] * dout[i / k];
}
__global__ void dot_kernel(const float* __restrict__ x, const float* __restrict__ y, float* out, int n) {
  float s = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i] * y[i];
  s = block_sum(s);
  if (threadIdx.x == 0) out[0] = s;
}
__global__ void axpy_from_scalar_kernel(float* dx, const float* __restrict__ y, const float* __restrict__ a, int n) {
  float av = a[0];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dx[i] += av * y[i];
}

static int full_sum(const float* x, float* out, int64_t n, float scale) {
  if (n <= (1 << 16)) { LTB_LAUNCH(sum_kernel, 1, 1024, 0, x, out, n, scale, false); return LTB_OK; }
  int blocks = grid_for(n, 1024, 2);
  LTB_LAUNCH(sum_kernel, blocks, 1024, 0, x, g.cur_scratch(), n, 1.0f, true);
  LTB_LAUNCH(sum_kernel, 1, 1024, 0, (const float*)g.cur_scratch(), out, (int64_t)blocks, scale, false);
  return LTB_OK;
}

}  // namespace ltb

using namespace ltb;

extern "C" {

// sum / mean and their grads: TensorDslCPU.scala:1115-1124.
int ltb_sum(const float* x, float* out, int64_t n) { LTB_INITED(); LTB_REQUIRE(x && out && n >= 0, "ltb_sum: bad argument"); return full_sum(x, out, n, 1.0f); }
int ltb_mean(const float* x, float* out, int64_t n) { LTB_INITED(); LTB_REQUIRE(x && out && n > 0, "ltb_mean: bad argument"); return full_sum(x, out, n, 1.0f / (float)n); }
int ltb_sum_grad(float* dx, const float* dout, int64_t n) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dout); LTB_REQUIRE(dx && dout && n >= 0, "ltb_sum_grad: bad argument");
  if (n) LTB_LAUNCH(add_scalar_from_kernel, grid_for(n, 256), 256, 0, dx, dout, 1.0f, n);
  return LTB_OK;
}
int ltb_mean_grad(float* dx, const float* dout, int64_t n) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dout); LTB_REQUIRE(dx && dout && n > 0, "ltb_mean_grad: bad argument");
  LTB_LAUNCH(add_scalar_from_kernel, grid_for(n, 256), 256, 0, dx, dout, 1.0f / (float)n, n);
  return LTB_OK;
}
// sum(dim) / sum_grad(dim): TensorDslCPU.scala:1125-1164.
int ltb_sum_dim(const float* x, float* out, int outer, int d, int inner) {
  LTB_INITED(); LTB_REQUIRE(x && out && outer > 0 && d > 0 && inner > 0, "ltb_sum_dim: bad argument");
  if (inner == 1) LTB_LAUNCH(sum_lastdim_kernel, (unsigned)ceil_div((int64_t)outer * 32, 256), 256, 0, x, out, outer, d);
  else LTB_LAUNCH(sum_dim_kernel, grid_for((int64_t)outer * inner, 256), 256, 0, x, out, outer, d, inner);
  return LTB_OK;
}
int ltb_sum_dim_grad(float* dx, const float* dout, int outer, int d, int inner) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dout); LTB_REQUIRE(dx && dout && outer > 0 && d > 0 && inner > 0, "ltb_sum_dim_grad: bad argument");
  LTB_LAUNCH(sum_dim_grad_kernel, grid_for((int64_t)outer * d * inner, 256), 256, 0, dx, dout, outer, d, inner);
  return LTB_OK;
}

// ---- the full sum with its partials in a file-scope device array: nothing is allocated, at set-up or per call.
// ltb_sum takes its partials from the workspace that ltb_init obtains with cudaMalloc. This variant is for callers
// for whom an allocation is not acceptable at all: cudaMalloc and cudaFree synchronise the whole device, which
// stalls every other stream of a process that serves requests while it computes, and a process that runs under a
// memory budget fixed at start-up cannot let a library grow its footprint afterwards. No counterpart in the reference.
//   * The first call on a device looks the array's address up (cudaGetSymbolAddress, with that device current); that
//     is set-up work and belongs before any stream capture. Later calls only launch.
//   * Limit: n <= kStaticSumMaxN elements; beyond it the call fails with LTB_E_LIMIT and launches nothing.
//   * Nothing has to start at zero: stage one writes one partial per CTA into slots [0, CTAs), stage two reads exactly
//     those slots, so stale contents of the array are never read.
//   * The array is one per device and process: two calls in flight at once (different streams or threads) race on it.
//     Calls on one stream are ordered and safe.
constexpr int kStaticSumSlots = 2048;
constexpr int64_t kStaticSumMaxN = (int64_t)1 << 30;
constexpr int kStaticSumMaxDevices = 64;
static __device__ __align__(256) float static_sum_scratch[kStaticSumSlots];
static float* static_sum_ptr[kStaticSumMaxDevices] = {};
}  // extern "C"
namespace ltb { void static_sum_forget() { for (auto& p : static_sum_ptr) p = nullptr; } }   // ltb_shutdown: a later context looks the address up again
extern "C" {

int ltb_sum_static_scratch(const float* x, float* out, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(x && out && n >= 0, "ltb_sum_static_scratch: bad argument");
  if (n > kStaticSumMaxN)
    return fail(LTB_E_LIMIT, "ltb_sum_static_scratch: %lld elements exceed the limit of %lld", (long long)n, (long long)kStaticSumMaxN);
  LTB_REQUIRE(g.device >= 0 && g.device < kStaticSumMaxDevices, "ltb_sum_static_scratch: device index out of range");
  if (!static_sum_ptr[g.device]) {                        // set-up, once per device
    // A symbol's address belongs to the device that is current in the calling thread, which need not be the context's
    // (another thread of the host may have selected a different GPU): select ours for the look-up and put the caller's back.
    LTB_REQUIRE(!g.capturing, "ltb_sum_static_scratch: the first call on a device does its set-up and must come before a step is recorded");
    int prev = -1;
    LTB_CUDA(cudaGetDevice(&prev));
    if (prev != g.device) LTB_CUDA(cudaSetDevice(g.device));
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, static_sum_scratch);
    if (prev != g.device) cudaSetDevice(prev);
    if (e != cudaSuccess || !p) return fail(LTB_E_CUDA, "ltb_sum_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    static_sum_ptr[g.device] = p;
  }
  float* partial = static_sum_ptr[g.device];
  if (n <= (1 << 16)) { LTB_LAUNCH(sum_kernel, 1, 1024, 0, x, out, n, 1.0f, false); return LTB_OK; }
  int blocks = grid_for(n, 1024, 2);                      // the same grid as ltb_sum: the two agree bit for bit
  if (blocks > kStaticSumSlots) blocks = kStaticSumSlots;
  LTB_LAUNCH(sum_kernel, blocks, 1024, 0, x, partial, n, 1.0f, true);
  LTB_LAUNCH(sum_kernel, 1, 1024, 0, (const float*)partial, out, (int64_t)blocks, 1.0f, false);
  return LTB_OK;
}

// softmax / logSoftmax and grads: TensorDslCPU.scala:783-846.
int ltb_softmax(const float* x, float* y, int rows, int cols) {
  LTB_INITED(); LTB_REQUIRE(x && y && rows > 0 && cols > 0, "ltb_softmax: bad argument");
  LTB_LAUNCH(softmax_kernel<0>, (unsigned)ceil_div((int64_t)rows * 32, 256), 256, 0, x, y, rows, cols); return LTB_OK;
}
int ltb_log_softmax(const float* x, float* y, int rows, int cols) {
  LTB_INITED(); LTB_REQUIRE(x && y && rows > 0 && cols > 0, "ltb_log_softmax: bad argument");
  LTB_LAUNCH(softmax_kernel<1>, (unsigned)ceil_div((int64_t)rows * 32, 256), 256, 0, x, y, rows, cols); return LTB_OK;
}
int ltb_softmax_grad(float* dx, const float* y, const float* dy, int rows, int cols) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_REQUIRE(dx && y && dy && rows > 0 && cols > 0, "ltb_softmax_grad: bad argument");
  LTB_LAUNCH(softmax_grad_kernel<0>, (unsigned)ceil_div((int64_t)rows * 32, 256), 256, 0, dx, y, dy, rows, cols); return LTB_OK;
}
int ltb_log_softmax_grad(float* dx, const float* y, const float* dy, int rows, int cols) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_REQUIRE(dx && y && dy && rows > 0 && cols > 0, "ltb_log_softmax_grad: bad argument");
  LTB_LAUNCH(softmax_grad_kernel<1>, (unsigned)ceil_div((int64_t)rows * 32, 256), 256, 0, dx, y, dy, rows, cols); return LTB_OK;
}
// nllLoss / nllLoss_grad: TensorDslCPU.scala:1090-1110.
int ltb_nll(const float* x, const int32_t* t, float* out, int rows, int cols) {
  LTB_INITED(); LTB_REQUIRE(x && t && out && rows > 0 && cols > 0, "ltb_nll: bad argument");
  LTB_LAUNCH(nll_kernel, (rows + 127) / 128, 128, 0, x, t, out, rows, cols); return LTB_OK;
}
int ltb_nll_grad(float* dx, const float* dout, const int32_t* t, int rows, int cols) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dout); LTB_REQUIRE(dx && dout && t && rows > 0 && cols > 0, "ltb_nll_grad: bad argument");
  LTB_LAUNCH(nll_grad_kernel, (rows + 127) / 128, 128, 0, dx, dout, t, rows, cols); return LTB_OK;
}

// vectorVectorDot / matrixVectorDot and the (1,1), (2,1) cases of dot_grad: TensorDslCPU.scala:135-206.
int ltb_vv_dot(const float* x, const float* y, float* out, int n) {
  LTB_INITED(); LTB_REQUIRE(x && y && out && n > 0, "ltb_vv_dot: bad argument");
  LTB_LAUNCH(dot_kernel, 1, 1024, 0, x, y, out, n); return LTB_OK;
}
int ltb_vv_dot_grad(float* dx, float* dy, const float* x, const float* y, const float* dout, int n) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_SETTLE(dout); LTB_REQUIRE(x && y && dout && n > 0, "ltb_vv_dot_grad: bad argument");
  if (dx) LTB_LAUNCH(axpy_from_scalar_kernel, grid_for(n, 256), 256, 0, dx, y, dout, n);
  if (dy) LTB_LAUNCH(axpy_from_scalar_kernel, grid_for(n, 256), 256, 0, dy, x, dout, n);
  return LTB_OK;
}
}  // extern "C"
namespace ltb {
// One warp per output row: lanes stride over the columns of W0 (and W1), shuffle reduction, lane 0 adds the bias and
// applies the activation.  150 x 150 gates of a TreeLSTM node: 38 blocks of four warps.
__global__ void affine_act_kernel(const float* __restrict__ W0, const float* __restrict__ a, int cols0, const float* __restrict__ W1,
                                  const float* __restrict__ b, int cols1, const float* __restrict__ bias, int act, float* out, int rows) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  float s0 = 0.0f, s1 = 0.0f;
  const float* w = W0 + (int64_t)r * cols0;
  for (int j = lane; j < cols0; j += 32) s0 += w[j] * a[j];
  if (W1) { w = W1 + (int64_t)r * cols1; for (int j = lane; j < cols1; j += 32) s1 += w[j] * b[j]; }
  for (int o = 16; o > 0; o >>= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o); }
  if (lane == 0) {
    float v = (s0 + s1) + bias[r];
    if (act == LTB_TANH) v = tanhf(v); else if (act == LTB_SIGMOID) v = 1.0f / (expf(-v) + 1.0f);
    out[r] = v;
  }
}
// The gradient of the same row: dpre from the saved output, the row of dW0 (dW1) updated in place, the row's share of
// W0^T dpre added atomically to da (db): rows x cols atomic additions on cols addresses, a few microseconds at these sizes.
__global__ void affine_act_grad_kernel(const float* __restrict__ W0, float* dW0, const float* __restrict__ a, float* da, int cols0,
                                       const float* __restrict__ W1, float* dW1, const float* __restrict__ b, float* db, int cols1,
                                       float* dbias, int act, const float* __restrict__ out, const float* __restrict__ dout, int rows) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float y = out[r];
  float dpre = dout[r];
  if (act == LTB_TANH) dpre *= 1.0f - y * y; else if (act == LTB_SIGMOID) dpre *= (1.0f - y) * y;     // TD.scala:789-809
  if (lane == 0) dbias[r] += dpre;
  {
    const float* w = W0 + (int64_t)r * cols0; float* dw = dW0 + (int64_t)r * cols0;
    for (int j = lane; j < cols0; j += 32) { dw[j] += dpre * a[j]; if (da) atomicAdd(da + j, w[j] * dpre); }
  }
  if (W1) {
    const float* w = W1 + (int64_t)r * cols1; float* dw = dW1 + (int64_t)r * cols1;
    for (int j = lane; j < cols1; j += 32) { dw[j] += dpre * b[j]; if (db) atomicAdd(db + j, w[j] * dpre); }
  }
}
}  // namespace ltb
extern "C" {
}  // extern "C"
namespace ltb {
__global__ void lstm_cell_kernel(const float* __restrict__ i, const float* __restrict__ u, const float* __restrict__ fl, const float* __restrict__ cl,
                                 const float* __restrict__ fr, const float* __restrict__ cr, const float* __restrict__ o, float* c, float* tc, float* h, int n) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  float v = i[k] * u[k];
  if (fl) { v = v + fl[k] * cl[k]; v = v + fr[k] * cr[k]; }
  const float t = tanhf(v);
  c[k] = v; tc[k] = t; h[k] = o[k] * t;
}
__global__ void lstm_cell_grad_kernel(const float* __restrict__ i, float* di, const float* __restrict__ u, float* du, const float* __restrict__ fl, float* dfl,
                                      const float* __restrict__ cl, float* dcl, const float* __restrict__ fr, float* dfr, const float* __restrict__ cr, float* dcr,
                                      const float* __restrict__ o, float* d_o, const float* __restrict__ tc, const float* __restrict__ dc,
                                      const float* __restrict__ dh, int n) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const float t = tc[k], g = dh[k];
  d_o[k] += g * t;
  const float dct = dc[k] + (g * o[k]) * (1.0f - t * t);
  di[k] += dct * u[k]; du[k] += dct * i[k];
  if (fl) { dfl[k] += dct * cl[k]; dcl[k] += dct * fl[k]; dfr[k] += dct * cr[k]; dcr[k] += dct * fr[k]; }
}
}  // namespace ltb
extern "C" {
int ltb_lstm_cell(const float* i, const float* u, const float* fl, const float* cl, const float* fr, const float* cr,
                  const float* o, float* c, float* tc, float* h, int n) {
  LTB_INITED();
  LTB_REQUIRE(i && u && o && c && tc && h && n > 0, "ltb_lstm_cell: bad argument");
  LTB_REQUIRE((fl && cl && fr && cr) || (!fl && !cl && !fr && !cr), "ltb_lstm_cell: the four child operands go together");
  LTB_LAUNCH(lstm_cell_kernel, (unsigned)ceil_div(n, 128), 128, 0, i, u, fl, cl, fr, cr, o, c, tc, h, n);
  return LTB_OK;
}
int ltb_lstm_cell_grad(const float* i, float* di, const float* u, float* du, const float* fl, float* dfl, const float* cl, float* dcl,
                       const float* fr, float* dfr, const float* cr, float* dcr, const float* o, float* d_o,
                       const float* tc, const float* dc, const float* dh, int n) {
  LTB_INITED(); LTB_SETTLE(di); LTB_SETTLE(du); LTB_SETTLE(dfl); LTB_SETTLE(dcl); LTB_SETTLE(dfr); LTB_SETTLE(dcr); LTB_SETTLE(d_o); LTB_SETTLE(dc); LTB_SETTLE(dh);
  LTB_REQUIRE(i && di && u && du && o && d_o && tc && dc && dh && n > 0, "ltb_lstm_cell_grad: bad argument");
  LTB_REQUIRE((fl && dfl && cl && dcl && fr && dfr && cr && dcr) || (!fl && !dfl && !cl && !dcl && !fr && !dfr && !cr && !dcr),
              "ltb_lstm_cell_grad: the child operands and their gradients go together");
  LTB_LAUNCH(lstm_cell_grad_kernel, (unsigned)ceil_div(n, 128), 128, 0, i, di, u, du, fl, dfl, cl, dcl, fr, dfr, cr, dcr, o, d_o, tc, dc, dh, n);
  return LTB_OK;
}
}  // extern "C"
namespace ltb {
__device__ __forceinline__ float act_fwd(int act, float v) { return act == LTB_TANH ? tanhf(v) : act == LTB_SIGMOID ? 1.0f / (expf(-v) + 1.0f) : v; }
__device__ __forceinline__ float act_slope(int act, float y) { return act == LTB_TANH ? 1.0f - y * y : act == LTB_SIGMOID ? (1.0f - y) * y : 1.0f; }
// A thread per output (b, j): the lanes of a warp share b (x is a broadcast) and read consecutive j of a weight row.
__global__ void affine_act_rows_kernel(const float* __restrict__ x0, const float* __restrict__ W0, int cols0, const float* __restrict__ x1,
                                       const float* __restrict__ W1, int cols1, const float* __restrict__ bias, int act, float* out, int batch, int width) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (j >= width) return;
  float s0 = 0.0f, s1 = 0.0f;
  const float* xr = x0 + (int64_t)b * cols0;
#pragma unroll 4
  for (int c = 0; c < cols0; ++c) s0 += xr[c] * W0[(int64_t)c * width + j];
  if (W1) {
    xr = x1 + (int64_t)b * cols1;
#pragma unroll 4
    for (int c = 0; c < cols1; ++c) s1 += xr[c] * W1[(int64_t)c * width + j];
  }
  out[(int64_t)b * width + j] = act_fwd(act, (s0 + s1) + bias[j]);
}
// The whole gradient in one launch, two kinds of blocks.  blockIdx.y < cols0 + cols1 + 1: row c of [dW0; dW1; dbias], a
// thread per column j walks the batch (dpre is recomputed from out and dout: two coalesced loads, nothing stored).
// The blocks after those: input gradients, a thread per (b, c) walks j.
__global__ void affine_act_rows_grad_kernel(const float* __restrict__ x0, float* dx0, const float* __restrict__ W0, float* dW0, int cols0,
                                            const float* __restrict__ x1, float* dx1, const float* __restrict__ W1, float* dW1, int cols1,
                                            float* dbias, int act, const float* __restrict__ out, const float* __restrict__ dout, int batch, int width) {
  const int wrows = cols0 + cols1 + 1;
  if ((int)blockIdx.y < wrows) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
    if (j >= width) return;
    const float* xs; int ld, cc; float* dst;
    if (c < cols0) { xs = x0; ld = cols0; cc = c; dst = dW0 + (int64_t)c * width + j; }
    else if (c < cols0 + cols1) { xs = x1; ld = cols1; cc = c - cols0; dst = dW1 + (int64_t)(c - cols0) * width + j; }
    else { xs = nullptr; ld = 0; cc = 0; dst = dbias + j; }
    float s = 0.0f;
#pragma unroll 4
    for (int b = 0; b < batch; ++b) {
      const float dpre = dout[(int64_t)b * width + j] * act_slope(act, out[(int64_t)b * width + j]);
      s += xs ? xs[(int64_t)b * ld + cc] * dpre : dpre;
    }
    *dst += s;
  } else {
    // input gradients: flat index over dx0 (batch x cols0, when wanted) then dx1 (batch x cols1, when wanted)
    const int64_t n0 = dx0 ? (int64_t)batch * cols0 : 0, n1 = dx1 ? (int64_t)batch * cols1 : 0;
    const int64_t t = ((int64_t)(blockIdx.y - wrows) * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= n0 + n1) return;
    const bool first = t < n0;
    const int64_t u = first ? t : t - n0;
    const int ld = first ? cols0 : cols1;
    const int b = (int)(u / ld), c = (int)(u - (int64_t)b * ld);
    const float* w = (first ? W0 : W1) + (int64_t)c * width;
    const float* o = out + (int64_t)b * width; const float* d = dout + (int64_t)b * width;
    float s = 0.0f;
#pragma unroll 4
    for (int j = 0; j < width; ++j) s += d[j] * act_slope(act, o[j]) * w[j];
    (first ? dx0 : dx1)[u] += s;
  }
}
}  // namespace ltb
extern "C" {
int ltb_affine_act_rows(const float* x0, const float* W0, int cols0, const float* x1, const float* W1, int cols1, const float* bias,
                        int act, float* out, int batch, int width) {
  LTB_INITED();
  LTB_REQUIRE(x0 && W0 && bias && out && cols0 > 0 && batch > 0 && batch <= 65535 && width > 0 && (x1 == nullptr) == (W1 == nullptr) && (!W1 || cols1 > 0),
              "ltb_affine_act_rows: bad argument");
  LTB_REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "ltb_affine_act_rows: activation must be tanh, sigmoid or -1");
  LTB_LAUNCH(affine_act_rows_kernel, dim3((unsigned)ceil_div(width, 128), batch), 128, 0, x0, W0, cols0, x1, W1, W1 ? cols1 : 0, bias, act, out, batch, width);
  return LTB_OK;
}
int ltb_affine_act_rows_grad(const float* x0, float* dx0, const float* W0, float* dW0, int cols0, const float* x1, float* dx1,
                             const float* W1, float* dW1, int cols1, float* dbias, int act, const float* out, const float* dout,
                             int batch, int width) {
  LTB_INITED(); LTB_SETTLE(dx0); LTB_SETTLE(dW0); LTB_SETTLE(dx1); LTB_SETTLE(dW1); LTB_SETTLE(dbias); LTB_SETTLE(dout);
  LTB_REQUIRE(x0 && W0 && dW0 && dbias && out && dout && cols0 > 0 && batch > 0 && width > 0, "ltb_affine_act_rows_grad: bad argument");
  LTB_REQUIRE((x1 == nullptr) == (W1 == nullptr) && (W1 == nullptr) == (dW1 == nullptr) && (!W1 || cols1 > 0) && (W1 || !dx1),
              "ltb_affine_act_rows_grad: x1, W1 and dW1 go together");
  LTB_REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "ltb_affine_act_rows_grad: activation must be tanh, sigmoid or -1");
  const int c1 = W1 ? cols1 : 0;
  const unsigned gx = (unsigned)ceil_div(width, 128);
  const int64_t inputs = (dx0 ? (int64_t)batch * cols0 : 0) + (dx1 ? (int64_t)batch * c1 : 0);
  const int64_t extra = ceil_div(inputs, (int64_t)gx * 128);
  LTB_REQUIRE(cols0 + c1 + 1 + extra <= 65535, "ltb_affine_act_rows_grad: too large for one launch");
  LTB_LAUNCH(affine_act_rows_grad_kernel, dim3(gx, (unsigned)(cols0 + c1 + 1 + extra)), 128, 0, x0, dx0, W0, dW0, cols0, x1, dx1, W1, dW1, c1,
             dbias, act, out, dout, batch, width);
  return LTB_OK;
}
int ltb_affine_act(const float* W0, const float* a, int cols0, const float* W1, const float* b, int cols1, const float* bias,
                   int act, float* out, int rows) {
  LTB_INITED();
  LTB_REQUIRE(W0 && a && bias && out && rows > 0 && cols0 > 0 && (W1 == nullptr) == (b == nullptr) && (!W1 || cols1 > 0), "ltb_affine_act: bad argument");
  LTB_REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "ltb_affine_act: activation must be tanh, sigmoid or -1");
  LTB_LAUNCH(affine_act_kernel, (unsigned)ceil_div(rows, 4), 128, 0, W0, a, cols0, W1, b, cols1, bias, act, out, rows);
  return LTB_OK;
}
int ltb_affine_act_grad(const float* W0, float* dW0, const float* a, float* da, int cols0, const float* W1, float* dW1,
                        const float* b, float* db, int cols1, float* dbias, int act, const float* out, const float* dout, int rows) {
  LTB_INITED(); LTB_SETTLE(dW0); LTB_SETTLE(da); LTB_SETTLE(dW1); LTB_SETTLE(db); LTB_SETTLE(dbias); LTB_SETTLE(dout);
  LTB_REQUIRE(W0 && dW0 && a && dbias && out && dout && rows > 0 && cols0 > 0, "ltb_affine_act_grad: bad argument");
  LTB_REQUIRE((W1 == nullptr) == (b == nullptr) && (W1 == nullptr) == (dW1 == nullptr) && (!W1 || cols1 > 0), "ltb_affine_act_grad: W1, dW1 and b go together");
  LTB_REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "ltb_affine_act_grad: activation must be tanh, sigmoid or -1");
  LTB_LAUNCH(affine_act_grad_kernel, (unsigned)ceil_div(rows, 4), 128, 0, W0, dW0, a, da, cols0, W1, dW1, b, db, cols1, dbias, act, out, dout, rows);
  return LTB_OK;
}
int ltb_mv_dot(const float* a, const float* x, float* out, int m, int k) {
  LTB_INITED(); LTB_REQUIRE(a && x && out && m > 0 && k > 0, "ltb_mv_dot: bad argument");
  LTB_LAUNCH(gemv_rows_kernel<false>, (unsigned)ceil_div((int64_t)m * 32, 256), 256, 0, a, x, out, m, k); return LTB_OK;
}
int ltb_add_cartesian(float* da, const float* y, const float* dout, int m, int k) {
  LTB_INITED(); LTB_SETTLE(da); LTB_SETTLE(dout); LTB_REQUIRE(da && y && dout && m > 0 && k > 0, "ltb_add_cartesian: bad argument");
  LTB_LAUNCH(outer_acc_kernel, grid_for((int64_t)m * k, 256), 256, 0, da, y, dout, m, k); return LTB_OK;
}
int ltb_add_composition(float* dx, const float* a, const float* dout, int m, int k) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dout); LTB_REQUIRE(dx && a && dout && m > 0 && k > 0, "ltb_add_composition: bad argument");
  LTB_LAUNCH(gemv_cols_kernel, (k + 127) / 128, 128, 0, a, dout, dx, m, k); return LTB_OK;
}

}  // extern "C"
