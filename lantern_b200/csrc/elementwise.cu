// Elementwise, broadcasting, activation, dropout and optimizer kernels: HBM-streaming work.
//
// These replace the reference's fixed <<<28,512>>> grid-stride kernels (src/main/scala/lantern/DslAPI.scala:475-842),
// its staging-time generated broadcast kernels (TensorDslCudnn.scala:153-282), cublasSgeam (TensorDslCublas.scala:318-373)
// and cudnnActivation*/cudnnAddTensor (TensorDslCudnn.scala:476-512, 1349-1429).  Semantics follow the CPU backend
// (TensorDslCPU.scala), cited per entry point.  Design: 128-bit loads/stores whenever every pointer is 16-byte
// aligned, grid sized to the SM count, one pass over memory per op.
#include <vector>

#include "common.cuh"

namespace ltb {

// ---- op functors ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bin_op(int op, float a, float b) {
  switch (op) { case LTB_ADD: return a + b; case LTB_SUB: return a - b; case LTB_MUL: return a * b; default: return a / b; }
}
__device__ __forceinline__ float un_op(int op, float v) {
  switch (op) {
    case LTB_RELU: return v < 0.0f ? 0.0f : v;                    // TensorDslCPU.scala:711-720
    case LTB_TANH: return tanhf(v);
    case LTB_SIGMOID: return 1.0f / (expf(-v) + 1.0f);            // TensorDslCPU.scala:760
    case LTB_EXP: return expf(v);
    case LTB_LOG: return logf(v);
    case LTB_SQRT: return sqrtf(v);
    default: return v * v;
  }
}
// dx += g(x, y, dy): TensorDslCPU.scala:722-781 with the fused helpers of TD.scala:789-809.
__device__ __forceinline__ float un_grad(int op, float x, float y, float dy) {
  switch (op) {
    case LTB_RELU: return x < 0.0f ? 0.0f : dy;
    case LTB_TANH: return (1.0f - y * y) * dy;
    case LTB_SIGMOID: return (1.0f - y) * y * dy;
    case LTB_EXP: return dy * y;
    case LTB_LOG: return dy / x;
    case LTB_SQRT: return dy / y / 2.0f;
    default: return dy * x * 2.0f;
  }
}

// ---- generic vectorised map over up to three inputs -------------------------------------------------------------
// F: float f(float a, float b, float c); a/b/c may be null (then 0 is passed). out may alias any input.
template <int NIN, class F>
__global__ void map_vec4(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c,
                         float* out, int64_t n4, F f) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 va = reinterpret_cast<const float4*>(a)[i];
    float4 vb = NIN > 1 ? reinterpret_cast<const float4*>(b)[i] : make_float4(0, 0, 0, 0);
    float4 vc = NIN > 2 ? reinterpret_cast<const float4*>(c)[i] : make_float4(0, 0, 0, 0);
    float4 r;
    r.x = f(va.x, vb.x, vc.x); r.y = f(va.y, vb.y, vc.y); r.z = f(va.z, vb.z, vc.z); r.w = f(va.w, vb.w, vc.w);
    reinterpret_cast<float4*>(out)[i] = r;
  }
}
template <int NIN, class F>
__global__ void map_scalar(const float* a, const float* b, const float* c, float* out, int64_t begin, int64_t n, F f) {
  int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = f(a[i], NIN > 1 ? b[i] : 0.0f, NIN > 2 ? c[i] : 0.0f);
}
template <int NIN, class F>
int launch_map(const float* a, const float* b, const float* c, float* out, int64_t n, F f) {
  if (n <= 0) return LTB_OK;
  bool vec = aligned16(a) && aligned16(out) && (NIN < 2 || aligned16(b)) && (NIN < 3 || aligned16(c));
  int64_t n4 = vec ? n / 4 : 0;
  if (n4 > 0) LTB_LAUNCH((map_vec4<NIN, F>), grid_for(n4, 256), 256, 0, a, b, c, out, n4, f);
  if (n4 * 4 < n) LTB_LAUNCH((map_scalar<NIN, F>), grid_for(n - n4 * 4, 256), 256, 0, a, b, c, out, n4 * 4, n, f);
  return LTB_OK;
}

// ---- fill -----------------------------------------------------------------------------------------------------
__global__ void fill_kernel(float* x, float v, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = v;
}
__global__ void fill_bias_kernel(float* out, const float* __restrict__ bias, int c, int64_t inner, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = bias[(i / inner) % c];
}

// ---- general broadcasting (rank <= 4) --------------------------------------------------------------------------
struct Bcast { int shape[4]; int64_t sa[4]; int64_t sb[4]; };

__device__ __forceinline__ void bcast_index(const Bcast& p, int64_t r, int64_t& ia, int64_t& ib) {
  int64_t i3 = r % p.shape[3]; r /= p.shape[3];
  int64_t i2 = r % p.shape[2]; r /= p.shape[2];
  int64_t i1 = r % p.shape[1]; int64_t i0 = r / p.shape[1];
  ia = i0 * p.sa[0] + i1 * p.sa[1] + i2 * p.sa[2] + i3 * p.sa[3];
  ib = i0 * p.sb[0] + i1 * p.sb[1] + i2 * p.sb[2] + i3 * p.sb[3];
}
__global__ void bcast_binary_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, Bcast p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) { int64_t ia, ib; bcast_index(p, i, ia, ib); out[i] = bin_op(op, a[ia], b[ib]); }
}
// Gradient of a broadcasting binary op: the operand that was broadcast receives a reduction, done with float atomics;
// the other one is a plain read-modify-write (TensorDslCPU.scala:246-263 and 300-337 for op1/op2).
__global__ void bcast_binary_grad_kernel(int op, const float* __restrict__ a, float* da, bool a_red, const float* __restrict__ b, float* db,
                                         bool b_red, const float* __restrict__ dout, Bcast p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int64_t ia, ib; bcast_index(p, i, ia, ib);
    float x = a[ia], y = b[ib], c = dout[i], g1, g2;
    switch (op) {
      case LTB_ADD: g1 = c; g2 = c; break;
      case LTB_SUB: g1 = c; g2 = 0.0f - c; break;
      case LTB_MUL: g1 = c * y; g2 = c * x; break;
      default: g1 = c / y; g2 = -1.0f * x * c / (y * y); break;
    }
    if (da) { if (a_red) atomicAdd(da + ia, g1); else da[ia] += g1; }
    if (db) { if (b_red) atomicAdd(db + ib, g2); else db[ib] += g2; }
  }
}
// x = x (op) y where y is broadcast over x (no element of x is written twice).
__global__ void bcast_inplace_kernel(int op, float* x, const float* __restrict__ y, Bcast p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) { int64_t ix, iy; bcast_index(p, i, ix, iy); x[ix] = bin_op(op, x[ix], y[iy]); }
}
// x = x (op) y where y is REDUCED into x: one warp per element of x walks, in row-major order of the broadcast
// shape, the y elements that map onto it (TensorDslCPU.scala:265-279).  ADD/SUB use a shuffle tree; MUL/DIV fold
// sequentially in lane 0 to keep the reference's order.
struct Reduce { int xshape[4]; int rshape[4]; int64_t sy[4]; };
__global__ void reduce_inplace_kernel(int op, float* x, const float* __restrict__ y, Reduce p, int64_t nx, int64_t per) {
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (warp >= nx) return;
  int xi[4]; int64_t r = warp;
  for (int d = 3; d >= 0; --d) { xi[d] = (int)(r % p.xshape[d]); r /= p.xshape[d]; }
  int red[4]; for (int d = 0; d < 4; ++d) red[d] = p.xshape[d] == 1 ? p.rshape[d] : 1;
  auto y_at = [&](int64_t j) {
    int64_t off = 0;
    for (int d = 3; d >= 0; --d) { int k = (int)(j % red[d]); j /= red[d]; off += (int64_t)(p.xshape[d] == 1 ? k : xi[d]) * p.sy[d]; }
    return y[off];
  };
  if (op == LTB_ADD || op == LTB_SUB) {
    float s = 0.0f;
    for (int64_t j = lane; j < per; j += 32) s += y_at(j);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) x[warp] = op == LTB_ADD ? x[warp] + s : x[warp] - s;
  } else if (lane == 0) {
    float v = x[warp];
    for (int64_t j = 0; j < per; ++j) v = bin_op(op, v, y_at(j));
    x[warp] = v;
  }
}

// ---- transpose-aware geam --------------------------------------------------------------------------------------
__global__ void geam_kernel(const float* __restrict__ x, int tx, float alpha, const float* __restrict__ y, int ty, float beta,
                            float* out, int rows, int cols) {
  int64_t n = (int64_t)rows * cols;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int r = (int)(i / cols), c = (int)(i % cols);
    float xv = tx ? x[(int64_t)c * rows + r] : x[i];
    float yv = ty ? y[(int64_t)c * rows + r] : y[i];
    out[i] = xv * alpha + yv * beta;
  }
}
// 32x32 shared-memory tile transpose; ACC adds into the destination (trans_grad).
template <bool ACC>
__global__ void transpose_kernel(const float* __restrict__ in, float* out, int rows, int cols) {
  __shared__ float tile[32][33];
  int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[(int64_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    int r = bx + j, c = by + threadIdx.x;   // out is [cols, rows]
    if (r < cols && c < rows) { if (ACC) out[(int64_t)r * rows + c] += tile[threadIdx.x][j]; else out[(int64_t)r * rows + c] = tile[threadIdx.x][j]; }
  }
}

// ---- multi-tensor SGD -------------------------------------------------------------------------------------------
struct SgdChunk { float* x; float* d; int64_t n; };
__global__ void sgd_multi_kernel(const SgdChunk* __restrict__ chunks, float lr) {
  SgdChunk c = chunks[blockIdx.y];
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < c.n; i += stride) { c.x[i] = c.x[i] * 1.0f + c.d[i] * (-1.0f * lr); c.d[i] = 0.0f; }
}
// x -= lr*d ; d = 0 in one pass (NNModule.scala:279-285: geam(x,1,d,-lr) then clear_grad): 16 B per parameter.
__global__ void sgd_vec4_kernel(float* x, float* d, float neg_lr, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  const float4 z = make_float4(0, 0, 0, 0);
  for (; i < n4; i += stride) {
    float4 xv = reinterpret_cast<float4*>(x)[i], dv = reinterpret_cast<float4*>(d)[i];
    xv.x = xv.x * 1.0f + dv.x * neg_lr; xv.y = xv.y * 1.0f + dv.y * neg_lr; xv.z = xv.z * 1.0f + dv.z * neg_lr; xv.w = xv.w * 1.0f + dv.w * neg_lr;
    reinterpret_cast<float4*>(x)[i] = xv; reinterpret_cast<float4*>(d)[i] = z;
  }
}
__global__ void sgd_scalar_kernel(float* x, float* d, float neg_lr, int64_t begin, int64_t n) {
  int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) { x[i] = x[i] * 1.0f + d[i] * neg_lr; d[i] = 0.0f; }
}
__global__ void adagrad_kernel(float* x, float* d, float* h, float lr, float clip, int descent, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {      // TensorDslCPU.scala:1217-1230
    float t = d[i]; if (t > clip) t = clip; if (t < -clip) t = -clip;
    float hv = h[i] + t * t; h[i] = hv;
    float upd = lr * t / sqrtf(hv + 1e-8f);
    x[i] = descent ? x[i] - upd : x[i] + upd;
    d[i] = 0.0f;
  }
}
__global__ void momentum_kernel(float* x, float* d, float* m, float lr, float mu, float clip, int nesterov, int descent, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {      // TensorDslCPU.scala:1232-1246
    float t = d[i]; if (t > clip) t = clip; if (t < -clip) t = -clip;
    float mv = m[i] * mu + t; m[i] = mv;
    t = nesterov ? t + mu * mv : mv;
    x[i] = descent ? x[i] - lr * t : x[i] + lr * t;
    d[i] = 0.0f;
  }
}

// Strided row copy used by concat: dst[r*dst_stride + j] (op)= src[r*src_stride + j], j < row_len.
template <bool ACC, int VEC>
__global__ void copy_rows_kernel(float* dst, int64_t dst_stride, const float* __restrict__ src, int64_t src_stride, int64_t row_len, int64_t n) {
  // all quantities are in units of VEC floats
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / row_len, j = i % row_len;
    if (VEC == 4) {
      float4 v = reinterpret_cast<const float4*>(src)[r * src_stride + j];
      float4* q = reinterpret_cast<float4*>(dst) + r * dst_stride + j;
      if (ACC) { float4 o = *q; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
      *q = v;
    } else {
      float v = src[r * src_stride + j];
      float* q = dst + r * dst_stride + j;
      *q = ACC ? *q + v : v;
    }
  }
}
template <bool ACC>
static int copy_rows(float* dst, int64_t dst_stride, const float* src, int64_t src_stride, int64_t row_len, int64_t rows) {
  if (rows * row_len == 0) return LTB_OK;
  if (aligned16(dst) && aligned16(src) && ((dst_stride | src_stride | row_len) & 3) == 0) {
    int64_t n = rows * (row_len / 4);
    LTB_LAUNCH((copy_rows_kernel<ACC, 4>), grid_for(n, 256), 256, 0, dst, dst_stride / 4, src, src_stride / 4, row_len / 4, n);
  } else {
    int64_t n = rows * row_len;
    LTB_LAUNCH((copy_rows_kernel<ACC, 1>), grid_for(n, 256), 256, 0, dst, dst_stride, src, src_stride, row_len, n);
  }
  return LTB_OK;
}

static bool make_bcast(const int* as, const int* bs, int rank, Bcast& p, int64_t& n, bool& a_b, bool& b_b) {
  if (rank < 1 || rank > 4 || !as || !bs) return false;
  int A[4] = {1, 1, 1, 1}, B[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { A[4 - rank + i] = as[i]; B[4 - rank + i] = bs[i]; }
  n = 1; a_b = b_b = false;
  int64_t sa = 1, sb = 1;
  for (int i = 3; i >= 0; --i) {
    if (A[i] < 1 || B[i] < 1) return false;
    if (A[i] != B[i] && A[i] != 1 && B[i] != 1) return false;
    p.shape[i] = A[i] > B[i] ? A[i] : B[i];
    p.sa[i] = A[i] == 1 ? 0 : sa; p.sb[i] = B[i] == 1 ? 0 : sb;
    if (A[i] == 1 && p.shape[i] != 1) a_b = true;
    if (B[i] == 1 && p.shape[i] != 1) b_b = true;
    sa *= A[i]; sb *= B[i]; n *= p.shape[i];
  }
  return true;
}

// ---- look-ahead fusion: issue functions and the flush ------------------------------------------------------------
int add_issue(const float* a, const float* b, float* out, int64_t n, bool relu) {
  if (relu) return launch_map<2>(a, b, nullptr, out, n, [] __device__(float x, float y, float) { float v = x + y; return v < 0.0f ? 0.0f : v; });
  return launch_map<2>(a, b, nullptr, out, n, [] __device__(float x, float y, float) { return x + y; });
}
int relu_grad_issue(const float* y, float* d, int64_t n) {
  return launch_map<2>(y, d, nullptr, d, n, [] __device__(float yv, float g0, float) { return yv > 0.0f ? g0 : 0.0f; });
}
int flush_pending() {
  const Pending p = g.pending;
  g.pending.kind = PEND_NONE;
  switch (p.kind) {
    case PEND_BN_FWD: return bn_fwd_issue(p, false);
    case PEND_ADD: return add_issue(p.a, p.b, p.out, p.n, false);
    case PEND_RELU_GRAD: return relu_grad_issue(p.relu_y, p.d, p.n);
    case PEND_RELU_ADD_GRAD: return relu_add_grad_issue(p);
    case PEND_BN_ADD: {                                         // no ReLU came: the two operations on their own, y written
      Pending q = p; q.kind = PEND_BN_FWD;
      int rc = bn_fwd_issue(q, false);
      return rc ? rc : add_issue(p.y, p.a, p.out, p.n, false);
    }
    default: return LTB_OK;
  }
}
// The held in-place ReLU gradient and the gradient of a same-shape add in one pass:
// m = y > 0 ? d : 0;  d = m;  da += m;  db += m   (da, db nullable; fa / fb: that destination holds nothing yet and is written; wb == 0: d itself is not
// rewritten, its owner has declared it dead).
// n4 float4 items, then a scalar tail from `tail`.
__global__ void relu_add_grad_kernel(const float* __restrict__ y, float* d, float* da, float* db, int64_t n4, int64_t tail, int64_t n, int fa, int fb, int wb) {
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = i0; i < n4; i += stride) {
    const float4 yv = reinterpret_cast<const float4*>(y)[i];
    float4 m = reinterpret_cast<const float4*>(d)[i];
    m.x = yv.x > 0.0f ? m.x : 0.0f; m.y = yv.y > 0.0f ? m.y : 0.0f; m.z = yv.z > 0.0f ? m.z : 0.0f; m.w = yv.w > 0.0f ? m.w : 0.0f;
    if (wb) reinterpret_cast<float4*>(d)[i] = m;
    if (da) { float4 v = fa ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(da)[i]; v.x += m.x; v.y += m.y; v.z += m.z; v.w += m.w; reinterpret_cast<float4*>(da)[i] = v; }
    if (db) { float4 v = fb ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(db)[i]; v.x += m.x; v.y += m.y; v.z += m.z; v.w += m.w; reinterpret_cast<float4*>(db)[i] = v; }
  }
  for (int64_t i = tail + i0; i < n; i += stride) {
    const float m = y[i] > 0.0f ? d[i] : 0.0f;
    if (wb) d[i] = m;
    if (da) da[i] = fa ? m : da[i] + m;
    if (db) db[i] = fb ? m : db[i] + m;
  }
}

int relu_add_grad_issue(const Pending& p) {
  const bool vec = aligned16(p.relu_y) && aligned16(p.d) && (!p.da || aligned16(p.da)) && (!p.db || aligned16(p.db));
  const int64_t n4 = vec ? p.n / 4 : 0;
  LTB_LAUNCH(relu_add_grad_kernel, grid_for(n4 ? n4 : p.n, 256), 256, 0, p.relu_y, p.d, p.da, p.db, n4, n4 * 4, p.n, p.fa, p.fb, g.fusion_no_writeback ? 0 : 1);
  return LTB_OK;
}

}  // namespace ltb

using namespace ltb;

extern "C" {

// fill / fillInPlace: TensorDslCPU.scala:30-35, 65-67.
int ltb_fill(float* x, float v, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && n >= 0, "ltb_fill: bad argument");
  if (n) LTB_LAUNCH(fill_kernel, grid_for(n, 256), 256, 0, x, v, n);
  return LTB_OK;
}
// fillWithBias: TensorDslCPU.scala:41-61.
int ltb_fill_with_bias(float* out, const float* bias, int outer, int c, int inner) {
  LTB_INITED(); filter_cache_note_write(out, (size_t)outer * c * inner * 4); LTB_REQUIRE(out && bias && outer >= 0 && c > 0 && inner > 0, "ltb_fill_with_bias: bad argument");
  int64_t n = (int64_t)outer * c * inner;
  if (n) LTB_LAUNCH(fill_bias_kernel, grid_for(n, 256), 256, 0, out, bias, c, (int64_t)inner, n);
  return LTB_OK;
}
// clipAt: TensorDslCPU.scala:113-119.
int ltb_clip(float* x, float bound, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && n >= 0, "ltb_clip: bad argument");
  return launch_map<1>(x, nullptr, nullptr, x, n, [bound] __device__(float v, float, float) { return v > bound ? bound : (v < -bound ? -bound : v); });
}

// elementWiseOpWithBroadCast: TensorDslCPU.scala:227-244.
int ltb_ew_binary(int op, const float* a, const int* as, const float* b, const int* bs, float* out, int rank) {
  LTB_INITED_NOFLUSH(); LTB_REQUIRE(a && b && out && op >= LTB_ADD && op <= LTB_DIV, "ltb_ew_binary: bad argument");
  Bcast p; int64_t n; bool ab, bb;
  LTB_REQUIRE(make_bcast(as, bs, rank, p, n, ab, bb), "ltb_ew_binary: shapes do not broadcast");
  if (g.pending.kind == PEND_BN_FWD && g.fusion_single_use && !ab && !bb && op == LTB_ADD && g.pending.n == n && a != b &&
      (a == g.pending.y || b == g.pending.y)) {                 // the held batch norm's result plus a shortcut: held once more, for the ReLU
    const float* other = a == g.pending.y ? b : a;
    if (out != g.pending.y && out != g.pending.x && out != other && aligned16(other) && aligned16(out)) {
      g.pending.kind = PEND_BN_ADD; g.pending.a = other; g.pending.out = out;
      return LTB_OK;
    }
  }
  if (g.pending.kind) { int rc = flush_pending(); if (rc) return rc; }
  if (!ab && !bb && op == LTB_ADD) {
    if (g.fusion && n > 0) { Pending h; h.kind = PEND_ADD; h.n = n; h.a = a; h.b = b; h.out = out; g.pending = h; return LTB_OK; }   // an in-place ReLU of out may join it
    return add_issue(a, b, out, n, false);
  }
  if (!ab && !bb) return launch_map<2>(a, b, nullptr, out, n, [op] __device__(float x, float y, float) { return bin_op(op, x, y); });
  LTB_LAUNCH(bcast_binary_kernel, grid_for(n, 256), 256, 0, op, a, b, out, p, n);
  return LTB_OK;
}
// backpropElementWiseOpWithBroadCast: TensorDslCPU.scala:246-263.
int ltb_ew_binary_grad(int op, const float* a, float* da, const int* as, const float* b, float* db, const int* bs, const float* dout, int rank) {
  LTB_INITED_NOFLUSH(); LTB_REQUIRE(a && b && dout && op >= LTB_ADD && op <= LTB_DIV, "ltb_ew_binary_grad: bad argument");
  Bcast p; int64_t n; bool ab, bb;
  LTB_REQUIRE(make_bcast(as, bs, rank, p, n, ab, bb), "ltb_ew_binary_grad: shapes do not broadcast");
  if (g.pending.kind == PEND_RELU_GRAD && !ab && !bb && op == LTB_ADD && g.pending.d == dout && g.pending.n == n && n > 0) {
    // the held ReLU gradient of dout and this add's gradient in one pass (dout is rewritten with the masked values)
    const float* y = g.pending.relu_y; float* d = g.pending.d;
    g.pending.kind = PEND_NONE;
    // a destination declared unset (ltb_grad_unset) is written instead of added into; da == db stays an accumulation
    const int fa = da && da != db && grad_take_unset(da, (size_t)n * 4) ? 1 : 0, fb = db && da != db && grad_take_unset(db, (size_t)n * 4) ? 1 : 0;
    LTB_SETTLE(d); if (!fa) LTB_SETTLE(da); if (!fb) LTB_SETTLE(db);
    Pending h; h.kind = PEND_RELU_ADD_GRAD; h.n = n; h.relu_y = y; h.d = d; h.da = da; h.db = db; h.fa = fa; h.fb = fb;
    // level 2: held once more -- a batch-norm backward whose dy is one of the two destinations, written by nobody else before
    // (fresh), reads the masked gradient straight from d and writes the other destination itself (ltb_bn_bwd)
    if (g.fusion_no_writeback && da && db && da != db && (fa || fb)) { g.pending = h; return LTB_OK; }
    return relu_add_grad_issue(h);
  }
  if (g.pending.kind) { int rc = flush_pending(); if (rc) return rc; }
  LTB_SETTLE(dout);
  if (!ab && !bb && op == LTB_ADD) {   // the residual add of ResNet: da += dout, db += dout (a destination declared unset: da = dout)
    const bool fa = da && da != db && grad_take_unset(da, (size_t)n * 4), fb = db && da != db && grad_take_unset(db, (size_t)n * 4);
    if (!fa) LTB_SETTLE(da);
    if (!fb) LTB_SETTLE(db);
    int rc = !da ? 0 : fa ? launch_map<1>(dout, nullptr, nullptr, da, n, [] __device__(float c, float, float) { return c; })
                          : launch_map<2>(da, dout, nullptr, da, n, [] __device__(float g0, float c, float) { return g0 + c; });
    if (rc) return rc;
    return !db ? LTB_OK : fb ? launch_map<1>(dout, nullptr, nullptr, db, n, [] __device__(float c, float, float) { return c; })
                             : launch_map<2>(db, dout, nullptr, db, n, [] __device__(float g0, float c, float) { return g0 + c; });
  }
  LTB_SETTLE(da); LTB_SETTLE(db);
  if (!da && !db) return LTB_OK;
  LTB_LAUNCH(bcast_binary_grad_kernel, grid_for(n, 256), 256, 0, op, a, da, ab, b, db, bb, dout, p, n);
  return LTB_OK;
}
// map(x, s => s op y): TensorDslCPU.scala:298-331.
int ltb_ew_scalar(int op, const float* a, float s, float* out, int64_t n) {
  LTB_INITED(); filter_cache_note_write(out, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(a && out && n >= 0 && op >= LTB_ADD && op <= LTB_DIV, "ltb_ew_scalar: bad argument");
  return launch_map<1>(a, nullptr, nullptr, out, n, [op, s] __device__(float x, float, float) { return bin_op(op, x, s); });
}
int ltb_ew_inplace_scalar(int op, float* x, float s, int64_t n) { return ltb_ew_scalar(op, x, s, x, n); }

// inplaceElementWiseOpWithBroadCastOrReduce: TensorDslCPU.scala:265-279.
int ltb_ew_inplace(int op, float* x, const int* xs, const float* y, const int* ys, int rank) {
  LTB_INITED(); LTB_SETTLE(x); LTB_SETTLE(y); { size_t cnt_ = 1; for (int i_ = 0; i_ < rank && i_ < 8 && xs; ++i_) cnt_ *= (size_t)(xs[i_] > 0 ? xs[i_] : 1); filter_cache_note_write(x, cnt_ * 4); } LTB_REQUIRE(x && y && op >= LTB_ADD && op <= LTB_DIV, "ltb_ew_inplace: bad argument");
  Bcast p; int64_t n; bool xb, yb;
  LTB_REQUIRE(make_bcast(xs, ys, rank, p, n, xb, yb), "ltb_ew_inplace: shapes do not broadcast");
  if (!xb && !yb) return launch_map<2>(x, y, nullptr, x, n, [op] __device__(float u, float v, float) { return bin_op(op, u, v); });
  if (!xb) { LTB_LAUNCH(bcast_inplace_kernel, grid_for(n, 256), 256, 0, op, x, y, p, n); return LTB_OK; }
  // y (possibly itself broadcast on other dims) is reduced into x
  Reduce r; int64_t nx = 1;
  for (int i = 0; i < 4; ++i) { r.xshape[i] = p.sa[i] == 0 && p.shape[i] != 1 ? 1 : p.shape[i]; r.rshape[i] = p.shape[i]; r.sy[i] = p.sb[i]; nx *= r.xshape[i]; }
  int64_t per = n / nx;
  LTB_LAUNCH(reduce_inplace_kernel, (unsigned)ceil_div(nx * 32, 256), 256, 0, op, x, y, r, nx, per);
  return LTB_OK;
}
// plusBias / plusBias_grad: TensorDslCPU.scala:281-288.
int ltb_plus_bias(float* main, const int* ms, const float* bias, const int* bs, int rank) { return ltb_ew_inplace(LTB_ADD, main, ms, bias, bs, rank); }
int ltb_plus_bias_grad(float* dbias, const int* bs, const float* dmain, const int* ms, int rank) { return ltb_ew_inplace(LTB_ADD, dbias, bs, dmain, ms, rank); }

// geam: TensorDslCPU.scala:342-347 / cublasSgeam at TensorDslCublas.scala:318-373.
int ltb_geam(const float* x, int tx, float alpha, const float* y, int ty, float beta, float* out, int rows, int cols) {
  LTB_INITED(); filter_cache_note_write(out, (size_t)rows * cols * 4); LTB_REQUIRE(x && y && out && rows > 0 && cols > 0, "ltb_geam: bad argument");
  LTB_REQUIRE(!((tx || ty) && (out == x || out == y)), "ltb_geam: in-place with transpose");
  int64_t n = (int64_t)rows * cols;
  if (!tx && !ty) return launch_map<2>(x, y, nullptr, out, n, [alpha, beta] __device__(float u, float v, float) { return u * alpha + v * beta; });
  LTB_LAUNCH(geam_kernel, grid_for(n, 256), 256, 0, x, tx, alpha, y, ty, beta, out, rows, cols);
  return LTB_OK;
}
// trans / trans_grad: TensorDslCPU.scala:349-374.
int ltb_trans(const float* x, float* out, int rows, int cols) {
  LTB_INITED(); LTB_REQUIRE(x && out && rows > 0 && cols > 0, "ltb_trans: bad argument");
  LTB_LAUNCH(transpose_kernel<false>, dim3((cols + 31) / 32, (rows + 31) / 32), dim3(32, 8), 0, x, out, rows, cols);
  return LTB_OK;
}
int ltb_trans_grad(float* dx, const float* dy, int rows, int cols) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_REQUIRE(dx && dy && rows > 0 && cols > 0, "ltb_trans_grad: bad argument");
  // dy is [cols, rows]; dx[rows, cols] += dy^T
  LTB_LAUNCH(transpose_kernel<true>, dim3((rows + 31) / 32, (cols + 31) / 32), dim3(32, 8), 0, dy, dx, cols, rows);
  return LTB_OK;
}

// relu/tanh/sigmoid/exp/log/sqrt/square: TensorDslCPU.scala:710-781.
int ltb_unary(int op, const float* x, float* out, int64_t n) {
  LTB_INITED_NOFLUSH(); LTB_REQUIRE(x && out && n >= 0 && op >= LTB_RELU && op <= LTB_SQUARE, "ltb_unary: bad argument");
  if (g.pending.kind && op == LTB_RELU && x == out && g.pending.n == n) {      // in-place ReLU of the result that was just held back
    const Pending h = g.pending;
    if (h.kind == PEND_BN_FWD && h.y == out) { g.pending.kind = PEND_NONE; return bn_fwd_issue(h, true); }
    if (h.kind == PEND_ADD && h.out == out) { g.pending.kind = PEND_NONE; return add_issue(h.a, h.b, h.out, h.n, true); }
    if (h.kind == PEND_BN_ADD && h.out == out) { g.pending.kind = PEND_NONE; return bn_fwd_issue(h, true); }
  }
  if (g.pending.kind) { int rc = flush_pending(); if (rc) return rc; }
  return launch_map<1>(x, nullptr, nullptr, out, n, [op] __device__(float v, float, float) { return un_op(op, v); });
}
// *_grad.  ReLU in place: the reference's CPU backend tests the clamped value with `< 0` and so never masks
// (TensorDslCPU.scala:726) while its GPU backend masks where y <= 0 (cudnnActivationBackward with beta 0,
// TensorDslCudnn.scala:1392-1429); this library masks where y <= 0, which is the derivative of what was computed.
int ltb_unary_grad(int op, const float* x, float* dx, const float* y, const float* dy, int64_t n, int in_place) {
  LTB_INITED(); LTB_REQUIRE(dx && dy && n >= 0 && op >= LTB_RELU && op <= LTB_SQUARE, "ltb_unary_grad: bad argument");
  LTB_SETTLE(dx); LTB_SETTLE(dy);
  if (op == LTB_RELU && in_place) {
    LTB_REQUIRE(y, "ltb_unary_grad: relu in place needs the result");
    if (g.fusion && n > 0) { Pending h; h.kind = PEND_RELU_GRAD; h.n = n; h.relu_y = y; h.d = dx; g.pending = h; return LTB_OK; }   // BN backward or an add's gradient may absorb it
    return relu_grad_issue(y, dx, n);
  }
  const float* xin = x ? x : y; const float* yin = y ? y : x;
  LTB_REQUIRE(xin, "ltb_unary_grad: needs x or y");
  // dx += g(x, y, dy): four streams; fold x/y into the two the op actually needs
  bool needs_x = op == LTB_RELU || op == LTB_LOG || op == LTB_SQUARE;
  const float* s = needs_x ? xin : yin;
  return launch_map<3>(dx, s, dy, dx, n, [op] __device__(float g0, float v, float d) { return g0 + un_grad(op, v, v, d); });
}

// dropout: TensorDslCPU.scala:1066-1088.  The keep mask is drawn on the host from glibc rand() in element order,
// the stream the reference's CPU backend consumes, and uploaded; cudnnDropout in the reference's GPU backend is seeded
// with time(NULL) (TensorDslCudnn.scala:1301) and cannot be reproduced.
int ltb_dropout_masked(const float* x, float* y, const float* mask, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(x && y && mask && n >= 0, "ltb_dropout_masked: bad argument");
  return launch_map<2>(x, mask, nullptr, y, n, [] __device__(float v, float m, float) { return v * m; });
}
int ltb_dropout(const float* x, float* y, float* mask, float p, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(x && y && mask && n >= 0 && p >= 0.0f && p < 1.0f, "ltb_dropout: rate must be in [0,1)");
  LTB_REQUIRE(!g.capturing, "ltb_dropout: host RNG while recording a step");
  std::vector<float> h((size_t)n);
  float scale = 1.0f / (1.0f - p);
  for (int64_t i = 0; i < n; ++i) h[i] = ((float)rand() / RAND_MAX > p) ? scale : 0.0f;
  if (n) LTB_CUDA(cudaMemcpyAsync(mask, h.data(), (size_t)n * 4, cudaMemcpyHostToDevice, g.stream));
  LTB_CUDA(cudaStreamSynchronize(g.stream));
  return ltb_dropout_masked(x, y, mask, n);
}
int ltb_dropout_grad(float* dx, const float* mask, const float* dy, int64_t n) {
  LTB_INITED(); LTB_SETTLE(dx); LTB_SETTLE(dy); LTB_REQUIRE(dx && mask && dy && n >= 0, "ltb_dropout_grad: bad argument");
  return launch_map<3>(dx, mask, dy, dx, n, [] __device__(float g0, float m, float d) { return g0 + m * d; });
}

// concat / concat_grad: TensorDslCPU.scala:1166-1212. Input k is [outer, dims[k], inner]; one strided copy per input
// (the reference's GPU kernel handles exactly two 4-D inputs on dim 1, DslAPI.scala:561-623).
int ltb_concat(float* out, const float* const* inputs, const int* dims, int n_inputs, int outer, int inner) {
  LTB_INITED(); LTB_REQUIRE(out && inputs && dims && n_inputs > 0 && outer > 0 && inner > 0, "ltb_concat: bad argument");
  int64_t total = 0;
  for (int k = 0; k < n_inputs; ++k) { LTB_REQUIRE(inputs[k] && dims[k] > 0, "ltb_concat: bad input %d", k); total += dims[k]; }
  int64_t off = 0;
  for (int k = 0; k < n_inputs; ++k) {
    int64_t len = (int64_t)dims[k] * inner;
    int rc = copy_rows<false>(out + off, total * inner, inputs[k], len, len, outer);
    if (rc) return rc;
    off += len;
  }
  return LTB_OK;
}
int ltb_concat_grad(float* const* dinputs, const float* dout, const int* dims, int n_inputs, int outer, int inner) {
  LTB_INITED(); LTB_SETTLE(dout); LTB_REQUIRE(dinputs && dout && dims && n_inputs > 0 && outer > 0 && inner > 0, "ltb_concat_grad: bad argument");
  int64_t total = 0;
  for (int k = 0; k < n_inputs; ++k) { LTB_REQUIRE(dims[k] > 0, "ltb_concat_grad: bad input %d", k); total += dims[k]; }
  int64_t off = 0;
  for (int k = 0; k < n_inputs; ++k) {
    int64_t len = (int64_t)dims[k] * inner;
    if (dinputs[k]) {
      // an input's gradient buffer declared unset (ltb_grad_unset) is written, any other is added into
      const bool fresh = grad_take_unset(dinputs[k], (size_t)len * outer * 4);
      if (!fresh) LTB_SETTLE(dinputs[k]);
      int rc = fresh ? copy_rows<false>(dinputs[k], len, dout + off, total * inner, len, outer) : copy_rows<true>(dinputs[k], len, dout + off, total * inner, len, outer);
      if (rc) return rc;
    }
    off += len;
  }
  return LTB_OK;
}

// SGD.step: NNModule.scala:265-287.
int ltb_sgd_step(float* x, float* d, float lr, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && d && n >= 0, "ltb_sgd_step: bad argument");
  if (!n) return LTB_OK;
  float neg_lr = -1.0f * lr;
  int64_t n4 = (aligned16(x) && aligned16(d)) ? n / 4 : 0;
  if (n4) LTB_LAUNCH(sgd_vec4_kernel, grid_for(n4, 256), 256, 0, x, d, neg_lr, n4);
  if (n4 * 4 < n) LTB_LAUNCH(sgd_scalar_kernel, grid_for(n - n4 * 4, 256), 256, 0, x, d, neg_lr, n4 * 4, n);
  return LTB_OK;
}
// One launch for a whole list of parameter tensors (the reference issues 2 launches per tensor, 267 tensors for ResNet-50).
int ltb_sgd_step_multi(float* const* xs, float* const* ds, const int64_t* sizes, int nt, float lr) {
  LTB_INITED(); filter_cache_note_write(nullptr, 0); LTB_REQUIRE(xs && ds && sizes && nt >= 0, "ltb_sgd_step_multi: bad argument");
  if (!nt) return LTB_OK;
  LTB_REQUIRE((size_t)nt * sizeof(SgdChunk) <= g.cur_scratch_bytes(), "ltb_sgd_step_multi: too many tensors");
  LTB_REQUIRE(!g.capturing, "ltb_sgd_step_multi: uploads its tensor list; use ltb_sgd_step on a slab while recording");
  std::vector<SgdChunk> h(nt);
  int64_t mx = 0;
  for (int i = 0; i < nt; ++i) { h[i] = {xs[i], ds[i], sizes[i]}; if (sizes[i] > mx) mx = sizes[i]; }
  LTB_CUDA(cudaMemcpyAsync(g.cur_scratch(), h.data(), nt * sizeof(SgdChunk), cudaMemcpyHostToDevice, g.stream));
  LTB_CUDA(cudaStreamSynchronize(g.stream));
  int gx = (int)(ceil_div(mx, 256) < 64 ? ceil_div(mx, 256) : 64);
  LTB_LAUNCH(sgd_multi_kernel, dim3(gx < 1 ? 1 : gx, nt), 256, 0, (const SgdChunk*)g.cur_scratch(), lr);
  return LTB_OK;
}
int ltb_adagrad_update(float* x, float* d, float* h, float lr, float clip, int descent, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && d && h && n >= 0, "ltb_adagrad_update: bad argument");
  if (n) LTB_LAUNCH(adagrad_kernel, grid_for(n, 256), 256, 0, x, d, h, lr, clip, descent, n);
  return LTB_OK;
}
int ltb_momentum_update(float* x, float* d, float* m, float lr, float mu, float clip, int nesterov, int descent, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && d && m && n >= 0, "ltb_momentum_update: bad argument");
  if (n) LTB_LAUNCH(momentum_kernel, grid_for(n, 256), 256, 0, x, d, m, lr, mu, clip, nesterov, descent, n);
  return LTB_OK;
}

}  // extern "C"
