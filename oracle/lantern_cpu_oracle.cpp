// TEST INFRASTRUCTURE -- not part of the product.
//
// CPU restatement of Lantern's CPU backend (class BackendCPU,
// src/main/scala/lantern/TensorDslCPU.scala) behind the same C ABI as the CUDA library, with the
// prefix ora_ instead of ltb_ and host pointers instead of device pointers.  Only tests/, the smoke
// check and bench.py's cpu_baseline / reference arm may load this library; the product never does.
//
// Each function cites the reference lines it follows.  Loop orders and float/double usage follow the
// reference so that sequential-summation effects are the reference's own.  Deviations, all deliberate:
//   * cblas_sgemm / cblas_sgemv come from OpenBLAS in the reference (version unpinned, -lopenblas at
//     src/main/scala/lantern/DslAPI.scala:962); here they are a plain float triple loop.
//   * relu_grad in place: the reference tests the already-clamped value with `< 0` and therefore never
//     masks anything (TensorDslCPU.scala:726); the GPU backend of the reference masks by y > 0
//     (cudnnActivationBackward, TensorDslCudnn.scala:1392-1429).  The oracle masks by y > 0.
//   * batchNorm_grad and softmax_grad are `???` on the reference CPU backend (TensorDslCPU.scala:1058-1060,
//     835); they are restated from the cuDNN semantics the reference's GPU backend relies on
//     (TensorDslCudnn.scala:1025-1109, 1431-1504) and pinned by the known-answer vectors of
//     src/test/scala/lantern/TestCudnn.scala:1051-1118 and 751-795.
//   * maxpool with padding: the reference forgets the batch base in the saved index (TensorDslCPU.scala:939);
//     the oracle adds it (the padded path is never used with pads on the training path).
//
// Parity status: pinned -- see tests/test_oracle_golden.py (known-answer vectors copied from the
// reference's ScalaTest files) and tests/test_oracle_vs_generated.py (loss trajectory of the
// reference's shipped generated MNIST program compiled from its own source).
#define LTB_FN(name) ora_##name
#include "../include/lantern_b200.h"
#include "../lantern_b200/csrc/comm_wait.h"   // the product's bounded host wait (policy shared with the CPU communicator below)
#include "../lantern_b200/csrc/tc_plan.h"   // eligibility rule of the product's tensor-core engine (shape arithmetic only)
#include "../lantern_b200/csrc/buckets.h"   // all-reduce bucket spans (host arithmetic only)

#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>
#ifdef _OPENMP
#include <immintrin.h>
#include <omp.h>
#endif

namespace {

struct Ctx {
  bool inited = false;
  char* heap = nullptr;
  size_t heap_bytes = 0;
  size_t used = 0;
  int fatal = 1;
  int last = 0;
  std::string msg;
  int threads = 1;
  int64_t calls = 0;
  int math = LTB_MATH_FP32;   // LTB_MATH_TF32: emulate the operand truncation of the product's tensor-core path
} g;

// TF32 emulation.  In LTB_MATH_TF32 mode the oracle reproduces what the product's tensor-core path computes for the
// shapes that path accepts: both operands of the contraction reduced to TF32 (10-bit mantissa, low 13 bits dropped, as the
// tensor core reads FP32 words), products and sums in FP32.  Shapes the engine declines are computed in plain FP32 on both
// sides.  This turns the 2e-3 "TF32 tolerance" into a check at FP32 rounding level.  Default is plain FP32: the reference's
// CPU backend.
inline float tf32_trunc(float v) { uint32_t u; memcpy(&u, &v, 4); u &= 0xFFFFE000u; memcpy(&v, &u, 4); return v; }
std::vector<float> truncated(const float* p, size_t n) { std::vector<float> v(n); for (size_t i = 0; i < n; ++i) v[i] = tf32_trunc(p[i]); return v; }
alignas(16) float tc_dummy[4];
bool tc_gemm_taken(bool a_kmajor, bool b_kmajor, int M, int N, int K) {
  if (g.math != LTB_MATH_TF32) return false;
  ltb::TcPlan p; return ltb::tc_plan_gemm(p, tc_dummy, a_kmajor, tc_dummy, b_kmajor, tc_dummy, M, N, K, 1.0f, false, 148);
}
// kind 0 forward, 1 data-grad, 2 weight-grad.  full_image: the filter covers the whole unpadded image (one output pixel),
// which the product computes as a matrix product over (channel, row, column).
bool tc_conv_taken(int kind, int n_img, int ck, int co, int pix, bool full_image) {
  if (g.math != LTB_MATH_TF32) return false;
  if (full_image) {
    if (kind == 0) return tc_gemm_taken(true, true, n_img, co, ck);       // y[N][K] = x[N][CHW] w[K][CHW]^T
    if (kind == 1) return tc_gemm_taken(true, false, n_img, ck, co);      // dx[N][CHW] += dy[N][K] w[K][CHW]
    return tc_gemm_taken(false, false, co, ck, n_img);                    // dw[K][CHW] += dy^T[K][N] x[N][CHW]
  }
  ltb::TcPlan p; const bool rows = ltb::tc_conv_needs_rows(pix);
  // the product pads filter rows to 4 floats (forward) or 32 (data-grad) in a staging copy when they are not
  if (kind == 0) return ltb::tc_plan_conv_fwd(p, tc_dummy, rows, tc_dummy, (ck + 3) / 4 * 4, nullptr, tc_dummy, n_img, ck, co, pix, 148);
  if (kind == 1) return ltb::tc_plan_conv_dgrad(p, tc_dummy, rows, tc_dummy, (ck + 31) / 32 * 32, tc_dummy, n_img, ck, co, pix, true, 148);
  return ltb::tc_plan_conv_wgrad(p, tc_dummy, tc_dummy, tc_dummy, n_img, ck, co, pix, 148);
}

int fail(int code, const char* what) {
  g.last = code;
  g.msg = what;
  if (g.fatal) {
    fprintf(stderr, "lantern oracle error %d: %s\n", code, what);
    exit(code < 0 ? -code : code);
  }
  return code;
}
// Wall-clock time per entry point (ora_profile / ora_profile_report): where a CPU step spends its time.
struct ProfEntry { const char* name; double seconds; long long calls; };
static ProfEntry g_prof[160]; static int g_prof_n = 0; static bool g_prof_on = false;
struct ProfScope {
  const char* name; double t0; bool on;
  explicit ProfScope(const char* n) : name(n), t0(0), on(g_prof_on) { if (on) t0 = omp_get_wtime(); }
  ~ProfScope() {
    if (!on) return;
    const double dt = omp_get_wtime() - t0;
    for (int i = 0; i < g_prof_n; ++i) if (g_prof[i].name == name) { g_prof[i].seconds += dt; ++g_prof[i].calls; return; }
    if (g_prof_n < 160) g_prof[g_prof_n++] = ProfEntry{name, dt, 1};
  }
};
#define REQUIRE(cond, what) do { if (!(cond)) return fail(LTB_E_ARG, what); } while (0)

const size_t kGranule = 256;
size_t round_up(size_t b) { return (b + kGranule - 1) / kGranule * kGranule; }

// S[i][j] = sum over k = 0 .. K-1, in that order, of A(i,k) * B[k][j], every element a float sum of its own (fused multiply-add,
// which is what the compiler makes of `acc += a * b` in the plain loops as well).  A(i,k) = A[i*ais + k*aks]; B is row-major
// with ldb floats per row; S is row-major with lds floats per row and is overwritten.  A register tile of 4 rows x 16 columns
// keeps the partial sums out of memory; the order of the additions per element is that of the plain loop, so results are
// the same bit for bit.  `threads` > 1 spreads the row blocks over that many threads.
void gemm_seq(int M, int N, int K, const float* A, size_t ais, size_t aks, const float* B, size_t ldb, float* S, size_t lds, int threads) {
  const int row_blocks = (M + 3) / 4;
#pragma omp parallel for if (threads > 1 && row_blocks > 1) num_threads(threads) schedule(static)
  for (int ib = 0; ib < row_blocks; ++ib) {
    const int i0 = ib * 4, rows = std::min(4, M - i0);
    int j0 = 0;
    for (; j0 + 16 <= N; j0 += 16) {
      __m256 acc[4][2];
      for (int r = 0; r < 4; ++r) { acc[r][0] = _mm256_setzero_ps(); acc[r][1] = _mm256_setzero_ps(); }
      const float* a0 = A + (size_t)i0 * ais;
      for (int k = 0; k < K; ++k) {
        const float* b = B + (size_t)k * ldb + j0;
        const __m256 b0 = _mm256_loadu_ps(b), b1 = _mm256_loadu_ps(b + 8);
        for (int r = 0; r < rows; ++r) {
          const __m256 a = _mm256_set1_ps(a0[(size_t)r * ais + (size_t)k * aks]);
          acc[r][0] = _mm256_fmadd_ps(a, b0, acc[r][0]); acc[r][1] = _mm256_fmadd_ps(a, b1, acc[r][1]);
        }
      }
      for (int r = 0; r < rows; ++r) { _mm256_storeu_ps(S + (size_t)(i0 + r) * lds + j0, acc[r][0]); _mm256_storeu_ps(S + (size_t)(i0 + r) * lds + j0 + 8, acc[r][1]); }
    }
    for (; j0 < N; ++j0)                                   // the ragged columns, one at a time
      for (int r = 0; r < rows; ++r) {
        float acc = 0.0f;
        const float* a = A + (size_t)(i0 + r) * ais;
        for (int k = 0; k < K; ++k) acc = __builtin_fmaf(a[(size_t)k * aks], B[(size_t)k * ldb + j0], acc);
        S[(size_t)(i0 + r) * lds + j0] = acc;
      }
  }
}

// Plain row-major sgemm with the cblas contract: C = alpha*op(A)*op(B) + beta*C.
// Summation over k is sequential in float for every output element.
void sgemm(bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda, const float* B, int ldb,
           float beta, float* C, int ldc) {
  const bool par = (double)M * N * K > 2e6 && g.threads > 1;
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static)
  for (int i = 0; i < M; ++i) {
    float* c = C + (size_t)i * ldc;
    std::vector<float> acc(N, 0.0f);
    if (!tb) {
      for (int k = 0; k < K; ++k) {
        const float a = ta ? A[(size_t)k * lda + i] : A[(size_t)i * lda + k];
        const float* b = B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) acc[j] += a * b[j];
      }
    } else {
      for (int j = 0; j < N; ++j) {
        const float* b = B + (size_t)j * ldb;
        float s = 0.0f;
        if (!ta) {
          const float* a = A + (size_t)i * lda;
          for (int k = 0; k < K; ++k) s += a[k] * b[k];
        } else {
          for (int k = 0; k < K; ++k) s += A[(size_t)k * lda + i] * b[k];
        }
        acc[j] = s;
      }
    }
    if (beta == 0.0f) for (int j = 0; j < N; ++j) c[j] = alpha * acc[j];
    else for (int j = 0; j < N; ++j) c[j] = alpha * acc[j] + beta * c[j];
  }
}

// sgemm with the TF32 emulation applied when the product would run this problem on its tensor-core engine.
// a_kmajor / b_kmajor describe op(A) / op(B) the way the product's planner sees them: A stored [M,K], B stored [N,K].
void sgemm_m(bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc) {
  if (!tc_gemm_taken(!ta, tb, M, N, K)) { sgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc); return; }
  std::vector<float> a = truncated(A, (size_t)(ta ? K : M) * lda), b = truncated(B, (size_t)(tb ? N : K) * ldb);
  sgemm(ta, tb, M, N, K, alpha, a.data(), lda, b.data(), ldb, beta, C, ldc);
}

inline float apply_op(int op, float a, float b) {
  switch (op) {
    case LTB_ADD: return a + b;
    case LTB_SUB: return a - b;
    case LTB_MUL: return a * b;
    default: return a / b;
  }
}

// Strides with 0 on broadcast (size-1) dims: "xStridesShadow", TensorDslCPU.scala:233-234.
void shadow_strides(const int* shape, int rank, int64_t* st) {
  int64_t s = 1;
  for (int i = rank - 1; i >= 0; --i) { st[i] = shape[i] == 1 ? 0 : s; s *= shape[i]; }
}
int64_t prod(const int* s, int rank) { int64_t p = 1; for (int i = 0; i < rank; ++i) p *= s[i]; return p; }

bool same_shape(const int* a, const int* b, int rank) { for (int i = 0; i < rank; ++i) if (a[i] != b[i]) return false; return true; }
bool bcast_shape(const int* a, const int* b, int rank, int* r) {
  if (rank < 1 || rank > 8) return false;
  for (int i = 0; i < rank; ++i) {
    if (a[i] < 1 || b[i] < 1) return false;
    if (a[i] != b[i] && a[i] != 1 && b[i] != 1) return false;
    r[i] = a[i] > b[i] ? a[i] : b[i];
  }
  return true;
}

// Row-major traversal of the broadcast shape calling f(idxA, idxB, idxR).
template <class F>
void traverse(const int* rshape, const int64_t* sa, const int64_t* sb, int rank, F f) {
  int idx[8] = {0};
  int64_t total = prod(rshape, rank);
  int64_t ia = 0, ib = 0;
  for (int64_t r = 0; r < total; ++r) {
    f(ia, ib, r);
    for (int d = rank - 1; d >= 0; --d) {
      ++idx[d]; ia += sa[d]; ib += sb[d];
      if (idx[d] < rshape[d]) break;
      ia -= sa[d] * rshape[d]; ib -= sb[d] * rshape[d]; idx[d] = 0;
    }
  }
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ lifetime / arena
// CPU arena: calloc(HEAP_SIZE_CPU) + bump pointer + memset-on-reset, DslAPI.scala:372-383, TD.scala:1782-1789.
int ora_init(int /*device*/, size_t heap_bytes) {
  if (g.inited) return fail(LTB_E_STATE, "ora_init: already initialised");
  if (heap_bytes == 0) heap_bytes = (size_t)1 << 30;
  g.heap = (char*)calloc(heap_bytes, 1);
  if (!g.heap) return fail(LTB_E_OOM, "ora_init: calloc failed");
  g.heap_bytes = heap_bytes; g.used = 0; g.inited = true; g.last = 0;
  return LTB_OK;
}
int ora_shutdown(void) { free(g.heap); g.heap = nullptr; g.inited = false; g.used = 0; return LTB_OK; }
int ora_set_fatal(int on) { g.fatal = on; return LTB_OK; }
int ora_last_error(char* buf, int len) {
  if (buf && len > 0) { strncpy(buf, g.msg.c_str(), len - 1); buf[len - 1] = 0; }
  return g.last;
}
int ora_set_stream(void*) { ProfScope prof_scope_("ora_set_stream"); return LTB_OK; }
void* ora_get_stream(void) { return nullptr; }
int ora_sync(void) { ProfScope prof_scope_("ora_sync"); return LTB_OK; }
int ora_set_deterministic(int) { return LTB_OK; }   // the CPU build always sums in program order
int ora_set_filter_cache(int) { return LTB_OK; }    // the CPU build reads OIHW filters as they are
int ora_params_changed(void) { return LTB_OK; }
// Deferred zero fill: the CPU restatement keeps the reference's plain rule (zeroed memory, every gradient added), so a block
// declared unset is simply filled with zeros at once and nothing else changes.
int ora_grad_unset(float* d, int64_t n) { ProfScope prof_scope_("ora_grad_unset"); REQUIRE(d && n > 0, "grad_unset: bad argument"); memset(d, 0, (size_t)n * 4); return LTB_OK; }
int ora_grad_materialize(float*, int64_t) { return LTB_OK; }
int ora_set_fusion(int) { ProfScope prof_scope_("ora_set_fusion"); return LTB_OK; }   // the CPU build executes every call at once
int ora_set_math(int mode) { ProfScope prof_scope_("ora_set_math"); g.math = mode; return LTB_OK; }
int ora_device_status(void) { return LTB_OK; }
// The device-side bounded waits have no CPU counterpart: there is nothing to wait for.
int ora_set_wait_limit(int64_t) { ProfScope prof_scope_("ora_set_wait_limit"); return LTB_OK; }
int ora_clear_device_status(void) { ProfScope prof_scope_("ora_clear_device_status"); return LTB_OK; }
int ora_selftest_bounded_wait(int64_t) { ProfScope prof_scope_("ora_selftest_bounded_wait"); return LTB_OK; }
int64_t ora_kernel_launches(void) { return 0; }
// Not in the shared header: number of host threads the oracle may use (1 = the reference's protocol,
// OPENBLAS_NUM_THREADS=1 in src/out/NIPS18evaluation/run_exp.sh:12).
int ora_set_threads(int n) { ProfScope prof_scope_("ora_set_threads"); g.threads = n < 1 ? 1 : n; return LTB_OK; }

void* ora_malloc(size_t bytes) {
  if (!g.inited) { fail(LTB_E_STATE, "ora_malloc: not initialised"); return nullptr; }
  size_t b = round_up(bytes);
  if (g.used + b > g.heap_bytes) { fail(LTB_E_OOM, "ora_malloc: arena exhausted"); return nullptr; }
  void* p = g.heap + g.used; g.used += b;
  return p;  // zero: calloc at start, memset on reset/free
}
void* ora_malloc_uninit(size_t bytes) { return ora_malloc(bytes); }
int ora_free(void* p, size_t bytes) { ProfScope prof_scope_("ora_free");
  size_t b = round_up(bytes);
  if (!p || b > g.used || (char*)p != g.heap + g.used - b) return fail(LTB_E_ARG, "ora_free: not the newest block");
  memset(p, 0, b); g.used -= b; return LTB_OK;
}
void* ora_mark(void) { return g.heap + g.used; }
int ora_reset(void* mark) { ProfScope prof_scope_("ora_reset");
  char* m = (char*)mark;
  if (m < g.heap || m > g.heap + g.used) return fail(LTB_E_ARG, "ora_reset: mark outside the used span");
  memset(m, 0, g.heap + g.used - m); g.used = m - g.heap; return LTB_OK;
}
size_t ora_arena_used(void) { return g.used; }
int ora_h2d(void* d, const void* s, size_t n) { ProfScope prof_scope_("ora_h2d"); memcpy(d, s, n); return LTB_OK; }
int ora_d2h(void* d, const void* s, size_t n) { ProfScope prof_scope_("ora_d2h"); memcpy(d, s, n); return LTB_OK; }
int ora_d2d(void* d, const void* s, size_t n) { ProfScope prof_scope_("ora_d2d"); memmove(d, s, n); return LTB_OK; }

// ------------------------------------------------------------------ fill / init
// fill, fillInPlace: TensorDslCPU.scala:30-35, 65-67.
int ora_fill(float* x, float v, int64_t n) { ProfScope prof_scope_("ora_fill"); for (int64_t i = 0; i < n; ++i) x[i] = v; return LTB_OK; }
// fillWithBias: TensorDslCPU.scala:41-61.
int ora_fill_with_bias(float* out, const float* bias, int outer, int c, int inner) { ProfScope prof_scope_("ora_fill_with_bias");
  REQUIRE(out && bias && outer >= 0 && c >= 0 && inner >= 0, "fill_with_bias: bad argument");
  size_t off = 0;
  for (int h = 0; h < outer; ++h) for (int cd = 0; cd < c; ++cd) for (int l = 0; l < inner; ++l) out[off++] = bias[cd];
  return LTB_OK;
}
// randinit: TensorDslCPU.scala:101-110 with Random.rand() = (float)rand()/RAND_MAX (TD.scala:1018-1026).
int ora_randinit(float* x, int64_t n, float scale, int seed) { ProfScope prof_scope_("ora_randinit");
  if (seed >= 0) srand((unsigned)seed);
  for (int64_t i = 0; i < n; ++i) x[i] = ((float)rand() / RAND_MAX - 0.5f) * scale;
  return LTB_OK;
}
// clipAt: TensorDslCPU.scala:113-119.
int ora_clip(float* x, float bound, int64_t n) { ProfScope prof_scope_("ora_clip");
  for (int64_t i = 0; i < n; ++i) { float t = x[i]; if (t > bound) x[i] = bound; if (t < -1.0f * bound) x[i] = -1.0f * bound; }
  return LTB_OK;
}

// ------------------------------------------------------------------ dot family
// vectorVectorDot: TensorDslCPU.scala:135-144.
int ora_vv_dot(const float* x, const float* y, float* out, int n) { ProfScope prof_scope_("ora_vv_dot");
  float v = 0.0f; for (int i = 0; i < n; ++i) v += x[i] * y[i]; out[0] = v; return LTB_OK;
}
// dot_grad case (1,1): addMul(output.d.data(0), other), TensorDslCPU.scala:173-175, TD.scala:766-773.
int ora_vv_dot_grad(float* dx, float* dy, const float* x, const float* y, const float* dout, int n) { ProfScope prof_scope_("ora_vv_dot_grad");
  float a = dout[0];
  if (dx) for (int i = 0; i < n; ++i) dx[i] = dx[i] + a * y[i];
  if (dy) for (int i = 0; i < n; ++i) dy[i] = dy[i] + a * x[i];
  return LTB_OK;
}
// matrixVectorDot: cblas_sgemv NoTrans beta 0, TensorDslCPU.scala:146-156.
int ora_mv_dot(const float* a, const float* x, float* out, int m, int k) { ProfScope prof_scope_("ora_mv_dot");
  for (int i = 0; i < m; ++i) { float s = 0.0f; for (int j = 0; j < k; ++j) s += a[(size_t)i * k + j] * x[j]; out[i] = s; }
  return LTB_OK;
}
// Fused affine map with activation: the composition of matrixVectorDot (TensorDslCPU.scala:148-156), the broadcasting
// adds and tanh / sigmoid (748-766) that the unfused programs issue, sums in the same sequential float order per product.
int ora_affine_act(const float* W0, const float* a, int cols0, const float* W1, const float* b, int cols1, const float* bias,
                   int act, float* out, int rows) { ProfScope prof_scope_("ora_affine_act");
  REQUIRE(W0 && a && bias && out && rows > 0 && cols0 > 0 && (W1 == nullptr) == (b == nullptr), "affine_act: bad argument");
  REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "affine_act: activation must be tanh, sigmoid or -1");
  for (int r = 0; r < rows; ++r) {
    float s0 = 0.0f, s1 = 0.0f;
    for (int j = 0; j < cols0; ++j) s0 += W0[(size_t)r * cols0 + j] * a[j];
    if (W1) for (int j = 0; j < cols1; ++j) s1 += W1[(size_t)r * cols1 + j] * b[j];
    float v = (s0 + s1) + bias[r];
    if (act == LTB_TANH) v = (float)tanh((double)v); else if (act == LTB_SIGMOID) v = 1.0f / ((float)exp((double)(-1.0f * v)) + 1.0f);
    out[r] = v;
  }
  return LTB_OK;
}
int ora_affine_act_grad(const float* W0, float* dW0, const float* a, float* da, int cols0, const float* W1, float* dW1,
                        const float* b, float* db, int cols1, float* dbias, int act, const float* out, const float* dout, int rows) { ProfScope prof_scope_("ora_affine_act_grad");
  REQUIRE(W0 && dW0 && a && dbias && out && dout && rows > 0 && cols0 > 0, "affine_act_grad: bad argument");
  REQUIRE((W1 == nullptr) == (b == nullptr) && (W1 == nullptr) == (dW1 == nullptr), "affine_act_grad: W1, dW1 and b go together");
  for (int r = 0; r < rows; ++r) {
    const float y = out[r];
    float dpre = dout[r];
    if (act == LTB_TANH) dpre *= 1.0f - y * y; else if (act == LTB_SIGMOID) dpre *= (1.0f - y) * y;
    dbias[r] += dpre;
    for (int j = 0; j < cols0; ++j) { dW0[(size_t)r * cols0 + j] += dpre * a[j]; if (da) da[j] += W0[(size_t)r * cols0 + j] * dpre; }
    if (W1) for (int j = 0; j < cols1; ++j) { dW1[(size_t)r * cols1 + j] += dpre * b[j]; if (db) db[j] += W1[(size_t)r * cols1 + j] * dpre; }
  }
  return LTB_OK;
}
// Batched form: matrixMatrixDot (TensorDslCPU.scala:158-169) with the broadcasting adds and the activation; every sum runs
// sequentially over its index in float, as the cblas restatement above does.
int ora_affine_act_rows(const float* x0, const float* W0, int cols0, const float* x1, const float* W1, int cols1, const float* bias,
                        int act, float* out, int batch, int width) { ProfScope prof_scope_("ora_affine_act_rows");
  REQUIRE(x0 && W0 && bias && out && cols0 > 0 && batch > 0 && width > 0 && (x1 == nullptr) == (W1 == nullptr), "affine_act_rows: bad argument");
  REQUIRE(act == -1 || act == LTB_TANH || act == LTB_SIGMOID, "affine_act_rows: activation must be tanh, sigmoid or -1");
  for (int b = 0; b < batch; ++b) for (int j = 0; j < width; ++j) {
    float s0 = 0.0f, s1 = 0.0f;
    for (int c = 0; c < cols0; ++c) s0 += x0[(size_t)b * cols0 + c] * W0[(size_t)c * width + j];
    if (W1) for (int c = 0; c < cols1; ++c) s1 += x1[(size_t)b * cols1 + c] * W1[(size_t)c * width + j];
    float v = (s0 + s1) + bias[j];
    if (act == LTB_TANH) v = (float)tanh((double)v); else if (act == LTB_SIGMOID) v = 1.0f / ((float)exp((double)(-1.0f * v)) + 1.0f);
    out[(size_t)b * width + j] = v;
  }
  return LTB_OK;
}
int ora_affine_act_rows_grad(const float* x0, float* dx0, const float* W0, float* dW0, int cols0, const float* x1, float* dx1,
                             const float* W1, float* dW1, int cols1, float* dbias, int act, const float* out, const float* dout,
                             int batch, int width) { ProfScope prof_scope_("ora_affine_act_rows_grad");
  REQUIRE(x0 && W0 && dW0 && dbias && out && dout && cols0 > 0 && batch > 0 && width > 0, "affine_act_rows_grad: bad argument");
  REQUIRE((x1 == nullptr) == (W1 == nullptr) && (W1 == nullptr) == (dW1 == nullptr) && (W1 || !dx1), "affine_act_rows_grad: x1, W1 and dW1 go together");
  std::vector<float> dpre((size_t)batch * width);
  for (size_t k = 0; k < dpre.size(); ++k) {
    const float y = out[k];
    dpre[k] = dout[k] * (act == LTB_TANH ? 1.0f - y * y : act == LTB_SIGMOID ? (1.0f - y) * y : 1.0f);
  }
  for (int j = 0; j < width; ++j) { float s = 0.0f; for (int b = 0; b < batch; ++b) s += dpre[(size_t)b * width + j]; dbias[j] += s; }
  for (int pass = 0; pass < 2; ++pass) {
    const float* x = pass ? x1 : x0; const float* W = pass ? W1 : W0; float* dW = pass ? dW1 : dW0; float* dx = pass ? dx1 : dx0;
    const int cols = pass ? cols1 : cols0;
    if (!W) continue;
    for (int c = 0; c < cols; ++c) for (int j = 0; j < width; ++j) {
      float s = 0.0f; for (int b = 0; b < batch; ++b) s += x[(size_t)b * cols + c] * dpre[(size_t)b * width + j];
      dW[(size_t)c * width + j] += s;
    }
    if (dx) for (int b = 0; b < batch; ++b) for (int c = 0; c < cols; ++c) {
      float s = 0.0f; for (int j = 0; j < width; ++j) s += dpre[(size_t)b * width + j] * W[(size_t)c * width + j];
      dx[(size_t)b * cols + c] += s;
    }
  }
  return LTB_OK;
}
// The elementwise part of an LSTM cell: the products, in-place sums and tanh the unfused programs issue
// (TensorDslCPU.scala:227-374 elementwise, 748-758 tanh), in the same order of float operations.
int ora_lstm_cell(const float* i, const float* u, const float* fl, const float* cl, const float* fr, const float* cr,
                  const float* o, float* c, float* tc, float* h, int n) { ProfScope prof_scope_("ora_lstm_cell");
  REQUIRE(i && u && o && c && tc && h && n > 0, "lstm_cell: bad argument");
  REQUIRE((fl && cl && fr && cr) || (!fl && !cl && !fr && !cr), "lstm_cell: the four child operands go together");
  for (int k = 0; k < n; ++k) {
    float v = i[k] * u[k];
    if (fl) { v = v + fl[k] * cl[k]; v = v + fr[k] * cr[k]; }
    const float t = (float)tanh((double)v);
    c[k] = v; tc[k] = t; h[k] = o[k] * t;
  }
  return LTB_OK;
}
int ora_lstm_cell_grad(const float* i, float* di, const float* u, float* du, const float* fl, float* dfl, const float* cl, float* dcl,
                       const float* fr, float* dfr, const float* cr, float* dcr, const float* o, float* d_o,
                       const float* tc, const float* dc, const float* dh, int n) { ProfScope prof_scope_("ora_lstm_cell_grad");
  REQUIRE(i && di && u && du && o && d_o && tc && dc && dh && n > 0, "lstm_cell_grad: bad argument");
  REQUIRE((fl && dfl && cl && dcl && fr && dfr && cr && dcr) || (!fl && !dfl && !cl && !dcl && !fr && !dfr && !cr && !dcr),
          "lstm_cell_grad: the child operands and their gradients go together");
  for (int k = 0; k < n; ++k) {
    const float t = tc[k], g = dh[k];
    d_o[k] += g * t;
    const float dct = dc[k] + (g * o[k]) * (1.0f - t * t);
    di[k] += dct * u[k]; du[k] += dct * i[k];
    if (fl) { dfl[k] += dct * cl[k]; dcl[k] += dct * fl[k]; dfr[k] += dct * cr[k]; dcr[k] += dct * fr[k]; }
  }
  return LTB_OK;
}
// matrixMatrixDot: TensorDslCPU.scala:158-169.
int ora_mm_dot(const float* a, const float* b, float* out, int m, int k, int n) { ProfScope prof_scope_("ora_mm_dot");
  sgemm_m(false, false, m, n, k, 1.0f, a, k, b, n, 0.0f, out, n); return LTB_OK;
}
// add_cartesian: TensorDslCPU.scala:186-196.
int ora_add_cartesian(float* da, const float* y, const float* dout, int m, int k) { ProfScope prof_scope_("ora_add_cartesian");
  for (int i = 0; i < m; ++i) for (int j = 0; j < k; ++j) da[(size_t)i * k + j] = da[(size_t)i * k + j] + y[j] * dout[i];
  return LTB_OK;
}
// add_composition: cblas_sgemv Trans beta 1, TensorDslCPU.scala:198-206.
int ora_add_composition(float* dx, const float* a, const float* dout, int m, int k) { ProfScope prof_scope_("ora_add_composition");
  for (int j = 0; j < k; ++j) { float s = 0.0f; for (int i = 0; i < m; ++i) s += a[(size_t)i * k + j] * dout[i]; dx[j] += s; }
  return LTB_OK;
}
// add_dotTrans1: x += y^T . output, TensorDslCPU.scala:208-215.
int ora_add_dot_trans1(float* db, const float* a, const float* dc, int m, int k, int n) { ProfScope prof_scope_("ora_add_dot_trans1");
  sgemm_m(true, false, k, n, m, 1.0f, a, k, dc, n, 1.0f, db, n); return LTB_OK;
}
// add_dotTrans2: x += y . output^T, TensorDslCPU.scala:217-225.
int ora_add_dot_trans2(float* da, const float* dc, const float* b, int m, int k, int n) { ProfScope prof_scope_("ora_add_dot_trans2");
  sgemm_m(false, true, m, k, n, 1.0f, dc, n, b, n, 1.0f, da, k); return LTB_OK;
}

// gemm: TensorDslCPU.scala:379-426 (four cblas_sgemm cases, beta 0).
int ora_gemm(const float* a, int ta, const float* b, int tb, float alpha, float* c, int M, int N, int K) { ProfScope prof_scope_("ora_gemm");
  REQUIRE(a && b && c && M > 0 && N > 0 && K > 0, "gemm: bad argument");
  sgemm_m(ta, tb, M, N, K, alpha, a, ta ? M : K, b, tb ? K : N, 0.0f, c, N);
  return LTB_OK;
}
// gemm_grad: TensorDslCPU.scala:428-472 (beta 1 in all eight calls).
int ora_gemm_grad(const float* a, float* da, int ta, const float* b, float* db, int tb, float alpha, const float* dc,
                  int M, int N, int K) { ProfScope prof_scope_("ora_gemm_grad");
  REQUIRE(a && b && dc && M > 0 && N > 0 && K > 0, "gemm_grad: bad argument");
  if (!ta && !tb) {
    if (da) sgemm_m(false, true, M, K, N, alpha, dc, N, b, N, 1.0f, da, K);
    if (db) sgemm_m(true, false, K, N, M, alpha, a, K, dc, N, 1.0f, db, N);
  } else if (!ta && tb) {
    if (da) sgemm_m(false, false, M, K, N, alpha, dc, N, b, K, 1.0f, da, K);
    if (db) sgemm_m(true, false, N, K, M, alpha, dc, N, a, K, 1.0f, db, K);
  } else if (ta && !tb) {
    if (da) sgemm_m(false, true, K, M, N, alpha, b, N, dc, N, 1.0f, da, M);
    if (db) sgemm_m(false, false, K, N, M, alpha, a, M, dc, N, 1.0f, db, N);
  } else {
    if (da) sgemm_m(true, true, K, M, N, alpha, b, K, dc, N, 1.0f, da, M);
    if (db) sgemm_m(true, true, N, K, M, alpha, dc, N, a, M, 1.0f, db, K);
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ convolution
namespace {
// unfoldedCopy: TensorDslCPU.scala:484-530. The reference offsets the kw slot by outputWidth*outputWidth (line 491),
// which equals outputHeight*outputWidth only for square outputs; the oracle uses the rectangular form.
void unfolded_copy(float* finput, const float* input, int kW, int kH, int dW, int dH, int padW, int padH, int nIn,
                   int iW, int iH, int oW, int oH) {
  for (int k = 0; k < nIn * kH * kW; ++k) {
    int nip = k / (kH * kW), rest = k % (kH * kW), kh = rest / kW, kw = rest % kW;
    float* dst = finput + (size_t)k * oH * oW;
    const float* src = input + (size_t)nip * iH * iW;
    for (int y = 0; y < oH; ++y) {
      int iy = y * dH - padH + kh;
      for (int x = 0; x < oW; ++x) {
        int ix = x * dW - padW + kw;
        dst[y * oW + x] = (iy < 0 || iy >= iH || ix < 0 || ix >= iW) ? 0.0f : src[iy * iW + ix];
      }
    }
  }
}
// unfoldedAcc: TensorDslCPU.scala:647-692 (same traversal order: plane, kh, kw, y, x).
void unfolded_acc(const float* finput, float* input, int kW, int kH, int dW, int dH, int padW, int padH, int nIn,
                  int iW, int iH, int oW, int oH) {
  for (int nip = 0; nip < nIn; ++nip)
    for (int kh = 0; kh < kH; ++kh)
      for (int kw = 0; kw < kW; ++kw) {
        const float* src = finput + ((size_t)(nip * kH + kh) * kW + kw) * oH * oW;
        float* dst = input + (size_t)nip * iH * iW;
        for (int y = 0; y < oH; ++y) {
          int iy = y * dH - padH + kh;
          if (iy < 0 || iy >= iH) continue;
          for (int x = 0; x < oW; ++x) {
            int ix = x * dW - padW + kw;
            if (ix < 0 || ix >= iW) continue;
            dst[iy * iW + ix] += src[y * oW + x];
          }
        }
      }
}
}  // namespace

// conv2D_batch: TensorDslCPU.scala:532-571. Output pre-filled with the bias (or zero), then per image
// im2col + sgemm(Cout x HoWo x CinKhKw, beta 1).
int ora_conv2d_fwd(const float* x, const float* w, const float* bias, float* y, int N, int C, int H, int W, int K, int R,
                   int S, int sh, int sw, int ph, int pw) { ProfScope prof_scope_("ora_conv2d_fwd");
  REQUIRE(x && w && y && N > 0 && C > 0 && K > 0 && R > 0 && S > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0, "conv2d_fwd: bad argument");
  int oH = (H + 2 * ph - R) / sh + 1, oW = (W + 2 * pw - S) / sw + 1;
  REQUIRE(oH > 0 && oW > 0, "conv2d_fwd: empty output");
  size_t ohw = (size_t)oH * oW;
  if (bias) ora_fill_with_bias(y, bias, N, K, (int)ohw); else memset(y, 0, sizeof(float) * N * K * ohw);
  const bool full_image = R == H && S == W && ph == 0 && pw == 0 && R * S > 1;
  const bool tf = tc_conv_taken(0, N, C * R * S, K, (int)ohw, full_image);
  std::vector<float> wt; if (tf) { wt = truncated(w, (size_t)K * C * R * S); w = wt.data(); }
  // Images are independent, so they run in parallel; images whose output map is small (fewer than 64 pixels) are taken
  // several at a time with their unfolded columns side by side, so that the innermost loop stays long.  Every output
  // element is still its own float sum over k = 0 .. C*R*S - 1 in order, added to the bias: the grouping changes no value.
  const int G = ohw >= 64 ? 1 : (int)std::min<size_t>((size_t)N, (64 + ohw - 1) / ohw);
  const int groups = (N + G - 1) / G;
  const bool par = g.threads > 1 && groups > 1;
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static)
  for (int gi = 0; gi < groups; ++gi) {
    const int t0 = gi * G, gn = std::min(G, N - t0);
    const int dim1 = K, dim2 = C * R * S, dim3 = (int)ohw, cols = gn * dim3;
    std::vector<float> fin((size_t)dim2 * cols), one(gn > 1 ? (size_t)dim2 * dim3 : 0), acc(cols);
    for (int u = 0; u < gn; ++u) {
      const float* img = x + (size_t)(t0 + u) * C * H * W;
      if (gn == 1) unfolded_copy(fin.data(), img, S, R, sw, sh, pw, ph, C, W, H, oW, oH);
      else {
        unfolded_copy(one.data(), img, S, R, sw, sh, pw, ph, C, W, H, oW, oH);
        for (int k = 0; k < dim2; ++k) memcpy(fin.data() + (size_t)k * cols + (size_t)u * dim3, one.data() + (size_t)k * dim3, sizeof(float) * dim3);
      }
    }
    if (tf) for (auto& v : fin) v = tf32_trunc(v);
    acc.resize((size_t)dim1 * cols);
    gemm_seq(dim1, cols, dim2, w, (size_t)dim2, 1, fin.data(), (size_t)cols, acc.data(), (size_t)cols, 1);
    for (int i = 0; i < dim1; ++i)
      for (int u = 0; u < gn; ++u) {
        float* out = y + ((size_t)(t0 + u) * K + i) * ohw;
        const float* a = acc.data() + (size_t)i * cols + (size_t)u * dim3;
        for (int j = 0; j < dim3; ++j) out[j] = a[j] + out[j];
      }
  }
  return LTB_OK;
}

// conv2D_batch_grad: TensorDslCPU.scala:575-645. ConvGradInput (per image W^T.dY into the unfolded buffer, then
// unfoldedAcc into dX) and ConvGradParam (per image dY.finput^T accumulated into dW, row sums into dbias).
int ora_conv2d_bwd(const float* x, float* dx, const float* w, float* dw, float* dbias, const float* dy, int N, int C, int H,
                   int W, int K, int R, int S, int sh, int sw, int ph, int pw) { ProfScope prof_scope_("ora_conv2d_bwd");
  REQUIRE(x && w && dy && N > 0 && C > 0 && K > 0 && R > 0 && S > 0 && sh > 0 && sw > 0, "conv2d_bwd: bad argument");
  int oH = (H + 2 * ph - R) / sh + 1, oW = (W + 2 * pw - S) / sw + 1;
  size_t ohw = (size_t)oH * oW;
  const int ckk = C * R * S;
  const bool full_image = R == H && S == W && ph == 0 && pw == 0 && R * S > 1;
  const float* w_full = w;
  if (dx) {
    const bool tf = tc_conv_taken(1, N, ckk, K, (int)ohw, full_image);
    std::vector<float> wt, dyt;
    const float* dy_d = dy;
    if (tf) { wt = truncated(w, (size_t)K * ckk); w = wt.data(); dyt = truncated(dy, (size_t)N * K * ohw); dy_d = dyt.data(); }
    // as in forward: images in parallel, small maps several at a time; each element of the unfolded gradient is its own
    // sequential sum over the K output channels
    const int G = ohw >= 64 ? 1 : (int)std::min<size_t>((size_t)N, (64 + ohw - 1) / ohw);
    const int groups = (N + G - 1) / G;
    const bool par = g.threads > 1 && groups > 1;
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static)
    for (int gi = 0; gi < groups; ++gi) {
      const int t0 = gi * G, gn = std::min(G, N - t0);
      const size_t cols = (size_t)gn * ohw;
      std::vector<float> fg((size_t)ckk * cols), gog(gn > 1 ? (size_t)K * cols : 0), one(gn > 1 ? (size_t)ckk * ohw : 0);
      const float* go = dy_d + (size_t)t0 * K * ohw;                  // [K][ohw] of the one image, or the group side by side
      if (gn > 1) {
        for (int u = 0; u < gn; ++u) for (int k = 0; k < K; ++k)
          memcpy(gog.data() + (size_t)k * cols + (size_t)u * ohw, dy_d + ((size_t)(t0 + u) * K + k) * ohw, sizeof(float) * ohw);
        go = gog.data();
      }
      // sgemm(Trans, NoTrans, ckk, ohw, K, 1, w, ckk, go, ohw, 0, fg, ohw)
      gemm_seq(ckk, (int)cols, K, w, 1, (size_t)ckk, go, cols, fg.data(), cols, 1);
      for (int u = 0; u < gn; ++u) {
        const float* src = fg.data();
        if (gn > 1) {
          for (int i = 0; i < ckk; ++i) memcpy(one.data() + (size_t)i * ohw, fg.data() + (size_t)i * cols + (size_t)u * ohw, sizeof(float) * ohw);
          src = one.data();
        }
        unfolded_acc(src, dx + (size_t)(t0 + u) * C * H * W, S, R, sw, sh, pw, ph, C, W, H, oW, oH);
      }
    }
  }
  w = w_full;
  if (dw) {
    // ConvGradParam, TensorDslCPU.scala:589-620: per image, sgemm(NoTrans, Trans, K, ckk, ohw, 1, dY_t, ohw, finput_t, ohw, 1, dW, ckk),
    // i.e. every dW element gets, image after image in order, a float sum over the pixels p = 0 .. ohw - 1 added to it.
    // The elements are independent of one another, so the work is spread over tiles of dW (4 rows x 16 columns kept in
    // registers across the whole image loop) instead of over images; per element the order of the additions is the reference's.
    // The unfolded inputs of all images are made first, in parallel, transposed to [pixel][filter row].
    const bool tf = tc_conv_taken(2, N, ckk, K, (int)ohw, full_image);
    std::vector<float> finT((size_t)N * ohw * ckk), dyt;
    const bool par = g.threads > 1;
#pragma omp parallel for if (par && N > 1) num_threads(g.threads) schedule(static)
    for (int t = 0; t < N; ++t) {
      std::vector<float> fin((size_t)ckk * ohw);
      unfolded_copy(fin.data(), x + (size_t)t * C * H * W, S, R, sw, sh, pw, ph, C, W, H, oW, oH);
      float* ft = finT.data() + (size_t)t * ohw * ckk;
      for (int c = 0; c < ckk; ++c) for (size_t q = 0; q < ohw; ++q) ft[q * ckk + c] = tf ? tf32_trunc(fin[(size_t)c * ohw + q]) : fin[(size_t)c * ohw + q];
    }
    const float* gt = dy;
    if (tf) { dyt = truncated(dy, (size_t)N * K * ohw); gt = dyt.data(); }
    const int row_blocks = (K + 3) / 4, col_blocks = (ckk + 15) / 16;
    // images in runs whose 16-column slice of the unfolded inputs fits a core's cache (dW goes back to memory between runs;
    // the order of the additions per element stays image by image)
    const int run = (int)std::max<size_t>(1, std::min<size_t>((size_t)N, 4096 / ohw));
    for (int tb0 = 0; tb0 < N; tb0 += run) {
    const int tb1 = std::min(N, tb0 + run);
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static) collapse(2)
    for (int jb = 0; jb < col_blocks; ++jb)           // column block outermost: its slice of the unfolded inputs stays in cache across the row blocks
      for (int ib = 0; ib < row_blocks; ++ib) {
        const int i0 = ib * 4, rows = std::min(4, K - i0), j0 = jb * 16, cols = std::min(16, ckk - j0);
        if (cols == 16) {
          __m256 d[4][2];
          for (int r = 0; r < rows; ++r) { d[r][0] = _mm256_loadu_ps(dw + (size_t)(i0 + r) * ckk + j0); d[r][1] = _mm256_loadu_ps(dw + (size_t)(i0 + r) * ckk + j0 + 8); }
          for (int t = tb0; t < tb1; ++t) {
            const float* a0 = gt + ((size_t)t * K + i0) * ohw;
            const float* bt = finT.data() + (size_t)t * ohw * ckk + j0;
            __m256 acc[4][2];
            for (int r = 0; r < 4; ++r) { acc[r][0] = _mm256_setzero_ps(); acc[r][1] = _mm256_setzero_ps(); }
            for (size_t q = 0; q < ohw; ++q) {
              const __m256 b0 = _mm256_loadu_ps(bt + q * ckk), b1 = _mm256_loadu_ps(bt + q * ckk + 8);
              for (int r = 0; r < rows; ++r) {
                const __m256 a = _mm256_set1_ps(a0[(size_t)r * ohw + q]);
                acc[r][0] = _mm256_fmadd_ps(a, b0, acc[r][0]); acc[r][1] = _mm256_fmadd_ps(a, b1, acc[r][1]);
              }
            }
            for (int r = 0; r < rows; ++r) { d[r][0] = _mm256_add_ps(acc[r][0], d[r][0]); d[r][1] = _mm256_add_ps(acc[r][1], d[r][1]); }
          }
          for (int r = 0; r < rows; ++r) { _mm256_storeu_ps(dw + (size_t)(i0 + r) * ckk + j0, d[r][0]); _mm256_storeu_ps(dw + (size_t)(i0 + r) * ckk + j0 + 8, d[r][1]); }
        } else {
          for (int r = 0; r < rows; ++r) for (int c = 0; c < cols; ++c) {
            float dv = dw[(size_t)(i0 + r) * ckk + j0 + c];
            for (int t = tb0; t < tb1; ++t) {
              const float* a = gt + ((size_t)t * K + i0 + r) * ohw;
              const float* bt = finT.data() + (size_t)t * ohw * ckk + j0 + c;
              float acc = 0.0f;
              for (size_t q = 0; q < ohw; ++q) acc = __builtin_fmaf(a[q], bt[q * ckk], acc);
              dv = acc + dv;
            }
            dw[(size_t)(i0 + r) * ckk + j0 + c] = dv;
          }
        }
      }
    }
    if (dbias)
      for (int t = 0; t < N; ++t) for (int i = 0; i < K; ++i) {
        float s = 0.0f; const float* d = dy + ((size_t)t * K + i) * ohw;
        for (size_t k = 0; k < ohw; ++k) s += d[k];
        dbias[i] += 1.0f * s;
      }
  } else if (dbias) {
    for (int t = 0; t < N; ++t) for (int i = 0; i < K; ++i) {
      float s = 0.0f; const float* d = dy + ((size_t)t * K + i) * ohw;
      for (size_t k = 0; k < ohw; ++k) s += d[k];
      dbias[i] += s;
    }
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ pooling
// maxPool2D_batch / maxPool_k_inplace: TensorDslCPU.scala:848-948.
int ora_maxpool_fwd(const float* x, float* y, int32_t* idx, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int pad) { ProfScope prof_scope_("ora_maxpool_fwd");
  REQUIRE(x && y && idx && N > 0 && C > 0 && kh >= 1 && kw >= 1 && sh >= 1 && sw >= 1 && pad >= 0, "maxpool_fwd: bad argument");
  REQUIRE(H + 2 * pad >= kh && W + 2 * pad >= kw, "maxpool_fwd: image too small");
  int oH = (H + 2 * pad - kh) / sh + 1, oW = (W + 2 * pad - kw) / sw + 1;
  for (int n = 0; n < N; ++n) for (int c = 0; c < C; ++c) {
    const size_t ibase = ((size_t)n * C + c) * H * W, obase = ((size_t)n * C + c) * oH * oW;
    for (int r = 0; r < oH; ++r) for (int q = 0; q < oW; ++q) {
      float best = -FLT_MAX; int32_t bi = 0;  // Float.MinValue; zero-initialised savedIdx if nothing beats it
      for (int a = 0; a < kh; ++a) for (int b = 0; b < kw; ++b) {
        int ir = r * sh - pad + a, ic = q * sw - pad + b;
        if (ir < 0 || ir >= H || ic < 0 || ic >= W) continue;
        size_t ii = ibase + (size_t)ir * W + ic;
        if (x[ii] > best) { best = x[ii]; bi = (int32_t)ii; }
      }
      y[obase + (size_t)r * oW + q] = best; idx[obase + (size_t)r * oW + q] = bi;
    }
  }
  return LTB_OK;
}
// maxPool2D_batch_grad: TensorDslCPU.scala:950-959.
int ora_maxpool_bwd(float* dx, const float* dy, const int32_t* idx, int64_t n_out) { ProfScope prof_scope_("ora_maxpool_bwd");
  for (int64_t i = 0; i < n_out; ++i) dx[idx[i]] += dy[i];
  return LTB_OK;
}
// averagePool2D_batch / averagePool_inplace: TensorDslCPU.scala:961-1006.
int ora_avgpool_fwd(const float* x, float* y, int N, int C, int H, int W, int kh, int kw, int sh, int sw) { ProfScope prof_scope_("ora_avgpool_fwd");
  REQUIRE(x && y && N > 0 && C > 0 && kh >= 1 && kw >= 1 && sh >= 1 && sw >= 1 && H >= kh && W >= kw, "avgpool_fwd: bad argument");
  int oH = (H - kh) / sh + 1, oW = (W - kw) / sw + 1;
  float ksz = kh * kw * 1.0f;
  for (size_t p = 0; p < (size_t)N * C; ++p) for (int r = 0; r < oH; ++r) for (int q = 0; q < oW; ++q) {
    float s = 0.0f;
    for (int a = 0; a < kh; ++a) for (int b = 0; b < kw; ++b) s += x[p * H * W + (size_t)(r * sh + a) * W + q * sw + b];
    y[p * oH * oW + (size_t)r * oW + q] = s / ksz;
  }
  return LTB_OK;
}
// averagePool2D_batch_grad: TensorDslCPU.scala:1008-1038.
int ora_avgpool_bwd(float* dx, const float* dy, int N, int C, int H, int W, int kh, int kw, int sh, int sw) { ProfScope prof_scope_("ora_avgpool_bwd");
  int oH = (H - kh) / sh + 1, oW = (W - kw) / sw + 1;
  int ksz = kh * kw;
  for (size_t p = 0; p < (size_t)N * C; ++p) for (int r = 0; r < oH; ++r) for (int q = 0; q < oW; ++q) {
    float d = dy[p * oH * oW + (size_t)r * oW + q] / ksz;
    for (int a = 0; a < kh; ++a) for (int b = 0; b < kw; ++b) dx[p * H * W + (size_t)(r * sh + a) * W + q * sw + b] += d;
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ batch norm
namespace {
// batchNormAv: TD.scala:521-538 -- per channel, summed image by image in float, divided by N*H*W.
void bn_average(const float* x, int N, int C, int HW, std::vector<float>& out, bool squared_diff, const float* mean) {
  out.assign(C, 0.0f);
  for (int n = 0; n < N; ++n) for (int c = 0; c < C; ++c) {
    const float* p = x + ((size_t)n * C + c) * HW;
    float r = out[c];
    if (!squared_diff) for (int l = 0; l < HW; ++l) r = r + p[l];
    else for (int l = 0; l < HW; ++l) { float d = p[l] - mean[c]; r = r + d * d; }
    out[c] = r;
  }
  float base = (float)N * HW * 1.0f;
  for (int c = 0; c < C; ++c) out[c] = out[c] / base;
}
}  // namespace

// batchNormTraining: TensorDslCPU.scala:1047-1056 for y; saved stats / running stats as cuDNN gives them to the
// reference's GPU backend (TensorDslCudnn.scala:1025-1056): exponentialAverageFactor = momentum, unbiased running var.
int ora_bn_train_fwd(const float* x, float* y, const float* gamma, const float* beta, float* run_mean, float* run_var,
                     float* save_mean, float* save_istd, int N, int C, int HW, float eps, float momentum) { ProfScope prof_scope_("ora_bn_train_fwd");
  REQUIRE(x && y && gamma && beta && save_mean && save_istd && N > 0 && C > 0 && HW > 0, "bn_train_fwd: bad argument");
  std::vector<float> mean, var;
  bn_average(x, N, C, HW, mean, false, nullptr);
  bn_average(x, N, C, HW, var, true, mean.data());
  const bool par = g.threads > 1;
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static)
  for (int n = 0; n < N; ++n) for (int c = 0; c < C; ++c) {
    float sd = (float)sqrt((double)(var[c] + eps));
    const float* p = x + ((size_t)n * C + c) * HW; float* q = y + ((size_t)n * C + c) * HW;
    for (int l = 0; l < HW; ++l) q[l] = (p[l] - mean[c]) / sd * gamma[c] + beta[c];
  }
  double m = (double)N * HW;
  for (int c = 0; c < C; ++c) {
    save_mean[c] = mean[c];
    save_istd[c] = 1.0f / (float)sqrt((double)(var[c] + eps));
    if (run_mean) run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mean[c];
    if (run_var) run_var[c] = (1.0f - momentum) * run_var[c] + momentum * (float)(var[c] * (m > 1 ? m / (m - 1) : 1.0));
  }
  return LTB_OK;
}
// batchNorm_grad: `???` on the reference CPU backend; restated from cudnnBatchNormalizationBackward as the reference
// calls it (alpha/beta = 1 for data and params, TensorDslCudnn.scala:1086-1109):
//   dbeta += sum dy; dgamma += sum dy*xhat; dx += gamma*istd/m * (m*dy - sum dy - xhat * sum dy*xhat).
int ora_bn_bwd(const float* x, float* dx, const float* dy, const float* gamma, float* dgamma, float* dbeta,
               const float* save_mean, const float* save_istd, int N, int C, int HW) { ProfScope prof_scope_("ora_bn_bwd");
  REQUIRE(x && dy && gamma && save_mean && save_istd && N > 0 && C > 0 && HW > 0, "bn_bwd: bad argument");
  double m = (double)N * HW;
  const bool par = g.threads > 1;
  // Channels are independent; a thread takes a run of 16 neighbouring channels and walks the images once for all of them
  // (for small maps a cache line holds several channels of one image).  Per channel the sums run over n, then over the
  // pixels, in order, in double, exactly as a loop over that channel alone would.
  const int chunk = 16, chunks = (C + chunk - 1) / chunk;
#pragma omp parallel for if (par) num_threads(g.threads) schedule(static)
  for (int cb = 0; cb < chunks; ++cb) {
    const int c0 = cb * chunk, cn = std::min(chunk, C - c0);
    double s1[16] = {0}, s2[16] = {0};
    for (int n = 0; n < N; ++n) for (int cc = 0; cc < cn; ++cc) {
      const int c = c0 + cc; const float mu = save_mean[c], is = save_istd[c];
      const float* p = x + ((size_t)n * C + c) * HW; const float* d = dy + ((size_t)n * C + c) * HW;
      double a1 = s1[cc], a2 = s2[cc];
      for (int l = 0; l < HW; ++l) { a1 += d[l]; a2 += (double)d[l] * ((p[l] - mu) * is); }
      s1[cc] = a1; s2[cc] = a2;
    }
    for (int cc = 0; cc < cn; ++cc) {
      if (dbeta) dbeta[c0 + cc] += (float)s1[cc];
      if (dgamma) dgamma[c0 + cc] += (float)s2[cc];
    }
    if (dx)
      for (int n = 0; n < N; ++n) for (int cc = 0; cc < cn; ++cc) {
        const int c = c0 + cc; const float mu = save_mean[c], is = save_istd[c];
        const float k = (float)(gamma[c] * is / m);
        const double t1 = s1[cc], t2 = s2[cc];
        const float* p = x + ((size_t)n * C + c) * HW; const float* d = dy + ((size_t)n * C + c) * HW;
        float* o = dx + ((size_t)n * C + c) * HW;
        for (int l = 0; l < HW; ++l) { float xh = (p[l] - mu) * is; o[l] += k * (float)(m * d[l] - t1 - xh * t2); }
      }
  }
  return LTB_OK;
}
// batchNormInference: TensorDslCPU.scala:1040-1045.
int ora_bn_inference(const float* x, float* y, const float* gamma, const float* beta, const float* rm, const float* rv,
                     int N, int C, int HW, float eps) { ProfScope prof_scope_("ora_bn_inference");
  REQUIRE(x && y && gamma && beta && rm && rv, "bn_inference: bad argument");
  for (int n = 0; n < N; ++n) for (int c = 0; c < C; ++c) {
    float sd = (float)sqrt((double)(rv[c] + eps));
    const float* p = x + ((size_t)n * C + c) * HW; float* q = y + ((size_t)n * C + c) * HW;
    for (int l = 0; l < HW; ++l) q[l] = (p[l] - rm[c]) / sd * gamma[c] + beta[c];
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ broadcasting elementwise
// elementWiseOpWithBroadCast: TensorDslCPU.scala:227-244.
int ora_ew_binary(int op, const float* a, const int* as, const float* b, const int* bs, float* out, int rank) { ProfScope prof_scope_("ora_ew_binary");
  int rs[8]; REQUIRE(a && b && out && as && bs && bcast_shape(as, bs, rank, rs), "ew_binary: shapes do not broadcast");
  if (same_shape(as, bs, rank)) {                     // no broadcast: the traversal is the identity on all three tensors
    const int64_t n = prod(rs, rank);
#pragma omp parallel for if (g.threads > 1 && n > (1 << 16)) num_threads(g.threads) schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = apply_op(op, a[i], b[i]);
    return LTB_OK;
  }
  int64_t sa[8], sb[8]; shadow_strides(as, rank, sa); shadow_strides(bs, rank, sb);
  traverse(rs, sa, sb, rank, [&](int64_t ia, int64_t ib, int64_t ir) { out[ir] = apply_op(op, a[ia], b[ib]); });
  return LTB_OK;
}
// backpropElementWiseOpWithBroadCast with the op1/op2 of add_grad, minus_grad, mul_grad, div_grad:
// TensorDslCPU.scala:246-263, 300-337.
int ora_ew_binary_grad(int op, const float* a, float* da, const int* as, const float* b, float* db, const int* bs,
                       const float* dout, int rank) { ProfScope prof_scope_("ora_ew_binary_grad");
  int rs[8]; REQUIRE(a && b && dout && bcast_shape(as, bs, rank, rs), "ew_binary_grad: shapes do not broadcast");
  if (same_shape(as, bs, rank) && da != db) {         // no broadcast and distinct destinations: every element is touched once
    const int64_t n = prod(rs, rank);
#pragma omp parallel for if (g.threads > 1 && n > (1 << 16)) num_threads(g.threads) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      const float x = a[i], y = b[i], c = dout[i];
      float g1, g2;
      switch (op) {
        case LTB_ADD: g1 = c; g2 = c; break;
        case LTB_SUB: g1 = c; g2 = 0.0f - c; break;
        case LTB_MUL: g1 = c * y; g2 = c * x; break;
        default: g1 = c / y; g2 = -1.0f * x * c / (y * y); break;
      }
      if (da) da[i] += g1;
      if (db) db[i] += g2;
    }
    return LTB_OK;
  }
  int64_t sa[8], sb[8]; shadow_strides(as, rank, sa); shadow_strides(bs, rank, sb);
  traverse(rs, sa, sb, rank, [&](int64_t ia, int64_t ib, int64_t ir) {
    float x = a[ia], y = b[ib], c = dout[ir];
    float g1, g2;
    switch (op) {
      case LTB_ADD: g1 = c; g2 = c; break;
      case LTB_SUB: g1 = c; g2 = 0.0f - c; break;
      case LTB_MUL: g1 = c * y; g2 = c * x; break;
      default: g1 = c / y; g2 = -1.0f * x * c / (y * y); break;
    }
    if (da) da[ia] += g1;
    if (db) db[ib] += g2;
  });
  return LTB_OK;
}
// map(x, s => s op y): TensorDslCPU.scala:298, 309, 320, 331.
int ora_ew_scalar(int op, const float* a, float s, float* out, int64_t n) { ProfScope prof_scope_("ora_ew_scalar");
  for (int64_t i = 0; i < n; ++i) out[i] = apply_op(op, a[i], s);
  return LTB_OK;
}
// inplaceElementWiseOpWithBroadCastOrReduce: TensorDslCPU.scala:265-279.
int ora_ew_inplace(int op, float* x, const int* xs, const float* y, const int* ys, int rank) { ProfScope prof_scope_("ora_ew_inplace");
  int rs[8]; REQUIRE(x && y && bcast_shape(xs, ys, rank, rs), "ew_inplace: shapes do not broadcast");
  int64_t sx[8], sy[8]; shadow_strides(xs, rank, sx); shadow_strides(ys, rank, sy);
  traverse(rs, sx, sy, rank, [&](int64_t ix, int64_t iy, int64_t) { x[ix] = apply_op(op, x[ix], y[iy]); });
  return LTB_OK;
}
int ora_ew_inplace_scalar(int op, float* x, float s, int64_t n) { ProfScope prof_scope_("ora_ew_inplace_scalar");
  for (int64_t i = 0; i < n; ++i) x[i] = apply_op(op, x[i], s);
  return LTB_OK;
}
// plusBias / plusBias_grad: TensorDslCPU.scala:281-288.
int ora_plus_bias(float* main, const int* ms, const float* bias, const int* bs, int rank) { ProfScope prof_scope_("ora_plus_bias"); return ora_ew_inplace(LTB_ADD, main, ms, bias, bs, rank); }
int ora_plus_bias_grad(float* dbias, const int* bs, const float* dmain, const int* ms, int rank) { ProfScope prof_scope_("ora_plus_bias_grad"); return ora_ew_inplace(LTB_ADD, dbias, bs, dmain, ms, rank); }
// geam: TensorDslCPU.scala:342-347 (no-transpose case only on the CPU; the transposed cases follow cublasSgeam's
// definition as used at TensorDslCublas.scala:318-373).
int ora_geam(const float* x, int tx, float alpha, const float* y, int ty, float beta, float* out, int rows, int cols) { ProfScope prof_scope_("ora_geam");
  REQUIRE(x && y && out && rows > 0 && cols > 0, "geam: bad argument");
  REQUIRE(!((tx || ty) && (out == x || out == y)), "geam: in-place with transpose");
  for (int i = 0; i < rows; ++i) for (int j = 0; j < cols; ++j) {
    float xv = tx ? x[(size_t)j * rows + i] : x[(size_t)i * cols + j];
    float yv = ty ? y[(size_t)j * rows + i] : y[(size_t)i * cols + j];
    out[(size_t)i * cols + j] = xv * alpha + yv * beta;
  }
  return LTB_OK;
}
// trans / trans_grad: TensorDslCPU.scala:349-374.
int ora_trans(const float* x, float* out, int rows, int cols) { ProfScope prof_scope_("ora_trans");
  for (int i = 0; i < cols; ++i) for (int j = 0; j < rows; ++j) out[(size_t)i * rows + j] = x[(size_t)j * cols + i];
  return LTB_OK;
}
int ora_trans_grad(float* dx, const float* dy, int rows, int cols) { ProfScope prof_scope_("ora_trans_grad");
  for (int i = 0; i < cols; ++i) for (int j = 0; j < rows; ++j) dx[(size_t)j * cols + i] += dy[(size_t)i * rows + j];
  return LTB_OK;
}

// ------------------------------------------------------------------ activations
// relu, tanh, sigmoid, exp, log, sqrt, square: TensorDslCPU.scala:710-781 (double libm, cast to float).
int ora_unary(int op, const float* x, float* out, int64_t n) { ProfScope prof_scope_("ora_unary");
  REQUIRE(x && out && n >= 0, "unary: bad argument");
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i], r;
    switch (op) {
      case LTB_RELU: r = v < 0.0f ? 0.0f : v; break;
      case LTB_TANH: r = (float)tanh((double)v); break;
      case LTB_SIGMOID: r = 1.0f / ((float)exp((double)(-1.0f * v)) + 1.0f); break;
      case LTB_EXP: r = (float)exp((double)v); break;
      case LTB_LOG: r = (float)log((double)v); break;
      case LTB_SQRT: r = (float)sqrt((double)v); break;
      case LTB_SQUARE: r = v * v; break;
      default: return fail(LTB_E_ARG, "unary: unknown op");
    }
    out[i] = r;
  }
  return LTB_OK;
}
// *_grad: TensorDslCPU.scala:722-781, TD.scala:789-809.
int ora_unary_grad(int op, const float* x, float* dx, const float* y, const float* dy, int64_t n, int in_place) { ProfScope prof_scope_("ora_unary_grad");
  REQUIRE(dx && dy && n >= 0, "unary_grad: bad argument");
  for (int64_t i = 0; i < n; ++i) {
    switch (op) {
      case LTB_RELU:
        if (in_place) { if (!(y[i] > 0.0f)) dx[i] = 0.0f; }   // deviation from TensorDslCPU.scala:726, see header
        else dx[i] += (x[i] < 0.0f ? 0.0f : dy[i]);
        break;
      case LTB_TANH: dx[i] = dx[i] + (1.0f - y[i] * y[i]) * dy[i]; break;
      case LTB_SIGMOID: dx[i] = dx[i] + ((1.0f - y[i]) * y[i]) * dy[i]; break;
      case LTB_EXP: dx[i] += dy[i] * y[i]; break;
      case LTB_LOG: dx[i] += dy[i] / x[i]; break;
      case LTB_SQRT: dx[i] += dy[i] / y[i] / 2.0f; break;
      case LTB_SQUARE: dx[i] += dy[i] * x[i] * 2.0f; break;
      default: return fail(LTB_E_ARG, "unary_grad: unknown op");
    }
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ softmax / loss
// softmax: TensorDslCPU.scala:783-805; max2D TD.scala:552-571; sum(dim=1) accumulates left to right.
int ora_softmax(const float* x, float* y, int rows, int cols) { ProfScope prof_scope_("ora_softmax");
  REQUIRE(x && y && rows > 0 && cols > 0, "softmax: bad argument");
  for (int b = 0; b < rows; ++b) {
    const float* p = x + (size_t)b * cols; float* q = y + (size_t)b * cols;
    float mx = -FLT_MAX; for (int i = 0; i < cols; ++i) if (p[i] > mx) mx = p[i];
    float s = 0.0f;
    for (int i = 0; i < cols; ++i) { q[i] = (float)exp((double)(p[i] - mx)); s += q[i]; }
    for (int i = 0; i < cols; ++i) q[i] = q[i] / s;
  }
  return LTB_OK;
}
// logSoftmax: TensorDslCPU.scala:807-832.
int ora_log_softmax(const float* x, float* y, int rows, int cols) { ProfScope prof_scope_("ora_log_softmax");
  REQUIRE(x && y && rows > 0 && cols > 0, "log_softmax: bad argument");
  for (int b = 0; b < rows; ++b) {
    const float* p = x + (size_t)b * cols; float* q = y + (size_t)b * cols;
    float mx = -FLT_MAX; for (int i = 0; i < cols; ++i) if (p[i] > mx) mx = p[i];
    float s = 0.0f;
    for (int i = 0; i < cols; ++i) s += (float)exp((double)(p[i] - mx));
    float logsum = mx + (float)log((double)s);
    for (int i = 0; i < cols; ++i) q[i] = p[i] - logsum;
  }
  return LTB_OK;
}
// softmax_grad: `???` on the CPU backend; cudnnSoftmaxBackward ACCURATE as called at TensorDslCudnn.scala:1465-1504:
// dx += y * (dy - sum_j dy_j*y_j).
int ora_softmax_grad(float* dx, const float* y, const float* dy, int rows, int cols) { ProfScope prof_scope_("ora_softmax_grad");
  for (int b = 0; b < rows; ++b) {
    const float* yy = y + (size_t)b * cols; const float* d = dy + (size_t)b * cols; float* o = dx + (size_t)b * cols;
    float s = 0.0f; for (int i = 0; i < cols; ++i) s += d[i] * yy[i];
    for (int i = 0; i < cols; ++i) o[i] += yy[i] * (d[i] - s);
  }
  return LTB_OK;
}
// logSoftmax_grad: TensorDslCPU.scala:837-846.
int ora_log_softmax_grad(float* dx, const float* y, const float* dy, int rows, int cols) { ProfScope prof_scope_("ora_log_softmax_grad");
  for (int b = 0; b < rows; ++b) {
    const float* yy = y + (size_t)b * cols; const float* d = dy + (size_t)b * cols; float* o = dx + (size_t)b * cols;
    float s = 0.0f; for (int i = 0; i < cols; ++i) s += d[i];
    for (int i = 0; i < cols; ++i) o[i] += d[i] - (float)exp((double)yy[i]) * s;
  }
  return LTB_OK;
}
// nllLoss / nllLoss_grad: TensorDslCPU.scala:1090-1110.
int ora_nll(const float* x, const int32_t* t, float* out, int rows, int cols) { ProfScope prof_scope_("ora_nll");
  REQUIRE(x && t && out, "nll: bad argument");
  for (int b = 0; b < rows; ++b) {
    REQUIRE(t[b] >= 0 && t[b] < cols, "nll: target out of range");
    out[b] = -1.0f * x[(size_t)b * cols + t[b]];
  }
  return LTB_OK;
}
int ora_nll_grad(float* dx, const float* dout, const int32_t* t, int rows, int cols) { ProfScope prof_scope_("ora_nll_grad");
  for (int b = 0; b < rows; ++b) dx[(size_t)b * cols + t[b]] += -1.0f * dout[b];
  return LTB_OK;
}

// ------------------------------------------------------------------ reductions
// sum / mean and grads: TensorDslCPU.scala:1115-1124 (sequential float fold).
int ora_sum(const float* x, float* out, int64_t n) { ProfScope prof_scope_("ora_sum"); float s = 0.0f; for (int64_t i = 0; i < n; ++i) s = s + x[i]; out[0] = s; return LTB_OK; }
// The CPU build has no workspace to avoid: the static-scratch variant is the same sequential sum.
int ora_sum_static_scratch(const float* x, float* out, int64_t n) { ProfScope prof_scope_("ora_sum_static_scratch"); return ora_sum(x, out, n); }
int ora_sum_grad(float* dx, const float* dout, int64_t n) { ProfScope prof_scope_("ora_sum_grad"); for (int64_t i = 0; i < n; ++i) dx[i] = dx[i] + dout[0]; return LTB_OK; }
int ora_mean(const float* x, float* out, int64_t n) { ProfScope prof_scope_("ora_mean"); float s = 0.0f; for (int64_t i = 0; i < n; ++i) s = s + x[i]; out[0] = s / (float)n; return LTB_OK; }
int ora_mean_grad(float* dx, const float* dout, int64_t n) { ProfScope prof_scope_("ora_mean_grad"); float g1 = dout[0] / (float)n; for (int64_t i = 0; i < n; ++i) dx[i] = dx[i] + g1; return LTB_OK; }
// sum(dim) / sum_grad(dim): TensorDslCPU.scala:1125-1164.
int ora_sum_dim(const float* x, float* out, int outer, int d, int inner) { ProfScope prof_scope_("ora_sum_dim");
  for (int h = 0; h < outer; ++h) {
    float* o = out + (size_t)h * inner;
    for (int l = 0; l < inner; ++l) o[l] = 0.0f;
    for (int s = 0; s < d; ++s) { const float* p = x + ((size_t)h * d + s) * inner; for (int l = 0; l < inner; ++l) o[l] += p[l]; }
  }
  return LTB_OK;
}
int ora_sum_dim_grad(float* dx, const float* dout, int outer, int d, int inner) { ProfScope prof_scope_("ora_sum_dim_grad");
  for (int h = 0; h < outer; ++h) for (int s = 0; s < d; ++s) {
    float* p = dx + ((size_t)h * d + s) * inner; const float* o = dout + (size_t)h * inner;
    for (int l = 0; l < inner; ++l) p[l] += o[l];
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ concat
// concat / concat_grad: TensorDslCPU.scala:1166-1212.
int ora_concat(float* out, const float* const* inputs, const int* dims, int n_inputs, int outer, int inner) { ProfScope prof_scope_("ora_concat");
  REQUIRE(out && inputs && dims && n_inputs > 0, "concat: bad argument");
  size_t t = 0;
  for (int h = 0; h < outer; ++h) for (int k = 0; k < n_inputs; ++k) {
    size_t stride = (size_t)dims[k] * inner; const float* p = inputs[k] + h * stride;
    for (size_t l = 0; l < stride; ++l) out[t++] = p[l];
  }
  return LTB_OK;
}
int ora_concat_grad(float* const* dinputs, const float* dout, const int* dims, int n_inputs, int outer, int inner) { ProfScope prof_scope_("ora_concat_grad");
  size_t t = 0;
  for (int h = 0; h < outer; ++h) for (int k = 0; k < n_inputs; ++k) {
    size_t stride = (size_t)dims[k] * inner;
    if (dinputs[k]) { float* p = dinputs[k] + h * stride; for (size_t l = 0; l < stride; ++l) p[l] += dout[t + l]; }
    t += stride;
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ dropout
// dropout / dropout_grad: TensorDslCPU.scala:1066-1088.
int ora_dropout(const float* x, float* y, float* mask, float p, int64_t n) { ProfScope prof_scope_("ora_dropout");
  REQUIRE(x && y && mask && p >= 0.0f && p < 1.0f, "dropout: rate must be in [0,1)");
  float scale = 1.0f / (1.0f - p);
  for (int64_t i = 0; i < n; ++i) {
    if ((float)rand() / RAND_MAX > p) { y[i] = x[i] * scale; mask[i] = scale; } else { y[i] = 0.0f; mask[i] = 0.0f; }
  }
  return LTB_OK;
}
int ora_dropout_masked(const float* x, float* y, const float* mask, int64_t n) { ProfScope prof_scope_("ora_dropout_masked"); for (int64_t i = 0; i < n; ++i) y[i] = x[i] * mask[i]; return LTB_OK; }
int ora_dropout_grad(float* dx, const float* mask, const float* dy, int64_t n) { ProfScope prof_scope_("ora_dropout_grad"); for (int64_t i = 0; i < n; ++i) dx[i] += mask[i] * dy[i]; return LTB_OK; }

// ------------------------------------------------------------------ optimizers
// SGD.step: geam(x, 1, d, -lr) then clear_grad, NNModule.scala:265-287 with geam of TensorDslCPU.scala:342-347.
int ora_sgd_step(float* x, float* d, float lr, int64_t n) { ProfScope prof_scope_("ora_sgd_step");
  float beta = -1.0f * lr;
  for (int64_t i = 0; i < n; ++i) { x[i] = x[i] * 1.0f + d[i] * beta; d[i] = 0.0f; }
  return LTB_OK;
}
int ora_sgd_step_multi(float* const* xs, float* const* ds, const int64_t* sizes, int nt, float lr) { ProfScope prof_scope_("ora_sgd_step_multi");
  for (int t = 0; t < nt; ++t) ora_sgd_step(xs[t], ds[t], lr, sizes[t]);
  return LTB_OK;
}
// adagrad_update: TensorDslCPU.scala:1217-1230.
int ora_adagrad_update(float* x, float* d, float* h, float lr, float clip, int descent, int64_t n) { ProfScope prof_scope_("ora_adagrad_update");
  for (int64_t i = 0; i < n; ++i) {
    float t = d[i]; if (t > clip) t = clip; if (t < -clip) t = -clip;
    h[i] += t * t;
    float upd = lr * t / (float)sqrt((double)(h[i] + 1e-8f));
    if (descent) x[i] -= upd; else x[i] += upd;
    d[i] = 0.0f;
  }
  return LTB_OK;
}
// momentum_update: TensorDslCPU.scala:1232-1246.
int ora_momentum_update(float* x, float* d, float* m, float lr, float mu, float clip, int nesterov, int descent, int64_t n) { ProfScope prof_scope_("ora_momentum_update");
  for (int64_t i = 0; i < n; ++i) {
    float t = d[i]; if (t > clip) t = clip; if (t < -clip) t = -clip;
    m[i] *= mu; m[i] += t;
    if (nesterov) t += mu * m[i]; else t = m[i];
    if (descent) x[i] -= lr * t; else x[i] += lr * t;
    d[i] = 0.0f;
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ data parallelism.
// The communicator has no transport of its own: a test installs one (a callback that sums a host buffer over the
// ranks in place, e.g. torch.distributed's gloo all_reduce) with ora_comm_set_transport, which is not part of the
// shared header. The update then follows the CUDA library's: the same bucket spans, sum over ranks, x -= lr/world * d,
// d = 0 (each rank's loss is the mean over its own shard).
typedef int (*ora_allreduce_fn)(float* buf, int64_t n);
static ora_allreduce_fn g_transport = nullptr;
static int g_world = 1;
// Failure detection, as in the CUDA library (csrc/comm.cu): a sum is waited for through the same bounded_wait
// (csrc/comm_wait.h) with the communicator's timeout; a transport error or a timeout marks the communicator broken, the call
// returns LTB_E_COMM and later collectives are refused until comm_destroy.  The transport runs on a helper thread so that
// the wait can give up on it (a rank that has left makes a blocking transport wait for as long as its own timeout).
static int64_t g_timeout_ms = 60000;
static bool g_broken = false;
struct TransportCall { std::atomic<int> state{0}; int rc = 0; };      // 0 running, 1 finished
static int transport_sum(float* buf, int64_t n, const char* who) {
  if (g_broken) return fail(LTB_E_COMM, (std::string(who) + ": the communicator was aborted").c_str());
  auto call = std::make_shared<TransportCall>();
  const ora_allreduce_fn fn = g_transport;
  std::thread([call, fn, buf, n] { call->rc = fn(buf, n); call->state.store(1); }).detach();
  const int r = ltb::bounded_wait([&] { return call->state.load() == 1 && call->rc == 0; },
                                  [&] { return call->state.load() == 1 && call->rc != 0; }, g_timeout_ms);
  if (r == ltb::WAIT_DONE) return LTB_OK;
  g_broken = true;
  return fail(LTB_E_COMM, (std::string(who) + (r == ltb::WAIT_TIMEOUT ? ": a collective did not finish within the communicator's timeout (a rank has left?)"
                                                                      : ": the transport reported an error") + "; the communicator was aborted").c_str());
}
int ora_comm_set_transport(ora_allreduce_fn fn) { ProfScope prof_scope_("ora_comm_set_transport"); g_transport = fn; return LTB_OK; }
int ora_comm_exposed_ms(float* out_ms) { if (out_ms) *out_ms = 0.0f; return LTB_OK; }   // the CPU transport is synchronous: nothing overlaps
int ora_comm_set_timeout_ms(int64_t ms) { ProfScope prof_scope_("ora_comm_set_timeout_ms"); g_timeout_ms = ms; return LTB_OK; }
int ora_comm_unique_id(void* out128) { ProfScope prof_scope_("ora_comm_unique_id"); memset(out128, 0, 128); return LTB_OK; }
int ora_comm_init(int rank, int world, const void*) { ProfScope prof_scope_("ora_comm_init");
  if (world < 1 || rank < 0 || rank >= world) return fail(LTB_E_ARG, "ora_comm_init: bad rank/world");
  if (world > 1 && !g_transport) return fail(LTB_E_COMM, "ora_comm_init: no transport installed for a multi-rank communicator");
  g_world = world; g_broken = false;
  return LTB_OK;
}
int ora_comm_destroy(void) { ProfScope prof_scope_("ora_comm_destroy"); g_world = 1; g_broken = false; return LTB_OK; }
int ora_comm_world(void) { ProfScope prof_scope_("ora_comm_world"); return g_world; }
int ora_allreduce_sum(float* x, int64_t n) { ProfScope prof_scope_("ora_allreduce_sum");
  if (g_world == 1 || n == 0) return LTB_OK;
  return transport_sum(x, n, "ora_allreduce_sum");
}
// Early ranges: summed at once (the transport is synchronous) and remembered, so that the step does not sum them twice.
static struct { float* ptr; int64_t n; } g_early[16];
static int g_n_early = 0;
int ora_allreduce_begin(float* d, int64_t n) { ProfScope prof_scope_("ora_allreduce_begin");
  if (g_world == 1 || n == 0 || g_n_early == 16) return LTB_OK;
  { const int rc = transport_sum(d, n, "ora_allreduce_begin"); if (rc) return rc; }
  g_early[g_n_early].ptr = d; g_early[g_n_early].n = n; ++g_n_early;
  return LTB_OK;
}
int ora_allreduce_sgd_step(float* x, float* d, float lr, int64_t n) { ProfScope prof_scope_("ora_allreduce_sgd_step");
  if (g_world == 1) return ora_sgd_step(x, d, lr, n);
  const float s = -1.0f * lr / (float)g_world;
  std::vector<char> done((size_t)n, 0);
  for (int e = 0; e < g_n_early; ++e) {
    if (g_early[e].ptr < d || g_early[e].ptr + g_early[e].n > d + n) return fail(LTB_E_ARG, "ora_allreduce_sgd_step: early range outside the span");
    for (int64_t i = g_early[e].ptr - d; i < (g_early[e].ptr - d) + g_early[e].n; ++i) done[(size_t)i] = 1;
  }
  g_n_early = 0;
  int64_t i = 0;
  while (i < n) {                                   // maximal runs that still need the sum, cut into the library's bucket spans
    if (done[(size_t)i]) { ++i; continue; }
    int64_t j = i; while (j < n && !done[(size_t)j]) ++j;
    int64_t off[ltb::kMaxBuckets], cnt[ltb::kMaxBuckets];
    const int used = ltb::bucket_spans(j - i, off, cnt);
    for (int b = 0; b < used; ++b) { const int rc = transport_sum(d + i + off[b], cnt[b], "ora_allreduce_sgd_step"); if (rc) return rc; }
    i = j;
  }
  for (int64_t k = 0; k < n; ++k) { x[k] += d[k] * s; d[k] = 0.0f; }
  return LTB_OK;
}
}  // extern "C"

// ------------------------------------------------------------------ a whole unrolled sequence of the vanilla RNN
// The operator sequence the reference stages for T steps (NNModule.scala:189-200, 240-253), issued through this file's own
// entry points: two matrix products, two broadcasting adds and tanh for the cell; product and plusBias for the output layer;
// logSoftmax, nllLoss and sum for the step's loss, added to the running total.  Backward replays the gradient calls of
// those operators in reverse order.  What the CUDA library's single-launch sequence kernels are checked against.  Those kernels
// are FP32 CUDA-core code in every math mode (a 100-wide product per row is no tensor-core work), so the operand truncation
// of the TF32 mode is switched off for the duration of the call.
namespace { struct Fp32Scope { int saved; Fp32Scope() : saved(g.math) { g.math = LTB_MATH_FP32; } ~Fp32Scope() { g.math = saved; } }; }
extern "C" {
int ora_rnn_seq_fwd(const float* x, const int32_t* y, const float* h0, const float* Wxh, const float* Whh, const float* bh, const float* Who,
                    const float* bo, float* h, float* logp, float* loss, int T, int B, int V, int H) { ProfScope prof_scope_("ora_rnn_seq_fwd");
  REQUIRE(x && y && Wxh && Whh && bh && Who && bo && h && logp && loss && T > 0 && B > 0 && V > 0 && H > 0, "rnn_seq_fwd: bad argument");
  Fp32Scope fp32_only;
  std::vector<float> zero((size_t)B * H, 0.0f), p1((size_t)B * H), p2((size_t)B * H), pre((size_t)B * H), pre2((size_t)B * H), o((size_t)B * V), nl(B);
  const int sbh[2] = {B, H}, sh1[2] = {1, H}, sbv[2] = {B, V}, sv1[2] = {1, V};
  float total = 0.0f, st = 0.0f;
  for (int t = 0; t < T; ++t) {
    const float* hp = t ? h + (size_t)(t - 1) * B * H : (h0 ? h0 : zero.data());
    float* ht = h + (size_t)t * B * H;
    ora_mm_dot(x + (size_t)t * B * V, Wxh, p1.data(), B, V, H);
    ora_mm_dot(hp, Whh, p2.data(), B, H, H);
    ora_ew_binary(LTB_ADD, p1.data(), sbh, p2.data(), sbh, pre.data(), 2);
    ora_ew_binary(LTB_ADD, pre.data(), sbh, bh, sh1, pre2.data(), 2);
    ora_unary(LTB_TANH, pre2.data(), ht, (int64_t)B * H);
    ora_mm_dot(ht, Who, o.data(), B, H, V);
    ora_plus_bias(o.data(), sbv, bo, sv1, 2);
    ora_log_softmax(o.data(), logp + (size_t)t * B * V, B, V);
    ora_nll(logp + (size_t)t * B * V, y + (size_t)t * B, nl.data(), B, V);
    ora_sum(nl.data(), &st, B);
    total = total + st;
  }
  loss[0] = total;
  return LTB_OK;
}
int ora_rnn_seq_bwd(const float* x, const int32_t* y, const float* h0, const float* Whh, const float* Who, const float* h, const float* logp,
                    const float* dloss, float* dWxh, float* dWhh, float* dbh, float* dWho, float* dbo, int T, int B, int V, int H) { ProfScope prof_scope_("ora_rnn_seq_bwd");
  REQUIRE(x && y && Whh && Who && h && logp && dloss && dWxh && dWhh && dbh && dWho && dbo && T > 0 && B > 0 && V > 0 && H > 0, "rnn_seq_bwd: bad argument");
  Fp32Scope fp32_only;
  std::vector<float> zero((size_t)B * H, 0.0f), dh((size_t)B * H, 0.0f), dhp((size_t)B * H), dpre((size_t)B * H), dlogp((size_t)B * V), dob((size_t)B * V), dnl(B);
  const int sbh[2] = {B, H}, sh1[2] = {1, H}, sbv[2] = {B, V}, sv1[2] = {1, V};
  for (int t = T - 1; t >= 0; --t) {
    const float* hp = t ? h + (size_t)(t - 1) * B * H : (h0 ? h0 : zero.data());
    const float* ht = h + (size_t)t * B * H;
    std::fill(dnl.begin(), dnl.end(), 0.0f); std::fill(dlogp.begin(), dlogp.end(), 0.0f); std::fill(dob.begin(), dob.end(), 0.0f);
    std::fill(dpre.begin(), dpre.end(), 0.0f); std::fill(dhp.begin(), dhp.end(), 0.0f);
    ora_sum_grad(dnl.data(), dloss, B);                                            // loss = loss + sum(nll): both operands get dloss
    ora_nll_grad(dlogp.data(), dnl.data(), y + (size_t)t * B, B, V);
    ora_log_softmax_grad(dob.data(), logp + (size_t)t * B * V, dlogp.data(), B, V);
    ora_plus_bias_grad(dbo, sv1, dob.data(), sbv, 2);
    ora_add_dot_trans2(dh.data(), dob.data(), Who, B, H, V);                          // dh += do Who^T (on top of what step t + 1 sent)
    ora_add_dot_trans1(dWho, ht, dob.data(), B, H, V);                                // dWho += h^T do
    ora_unary_grad(LTB_TANH, ht, dpre.data(), ht, dh.data(), (int64_t)B * H, 0);      // dpre += dh (1 - h^2)
    ora_ew_inplace(LTB_ADD, dbh, sh1, dpre.data(), sbh, 2);                           // the bias's share of the broadcasting add
    ora_add_dot_trans1(dWxh, x + (size_t)t * B * V, dpre.data(), B, V, H);
    ora_add_dot_trans1(dWhh, hp, dpre.data(), B, H, H);
    ora_add_dot_trans2(dhp.data(), dpre.data(), Whh, B, H, H);                        // for step t - 1
    dh = dhp;
  }
  return LTB_OK;
}
}  // extern "C"

// One node of the binary tree LSTM (PLDI19APP/SentimentTreeLSTM.scala:67-146, NIPS18App/SentimentTreeLSTM.scala:118-170) as
// the sequence of this file's entry points that the gate-by-gate host program issues: one affine_act per gate, lstm_cell, the
// classifier, logSoftmax, nllLoss, the two additions of the children's losses; backward replays their gradient calls in
// reverse order with the gates' gradient vectors as locals.  What the CUDA library's one-launch node kernels are checked against.
extern "C" {
static const int kSlotAct[5] = {LTB_SIGMOID, LTB_SIGMOID, LTB_SIGMOID, LTB_SIGMOID, LTB_TANH};
static bool tree_node_ok(const ltb_tree_node* n) {
  if (!n || n->hidden <= 0 || n->hidden > 512 || n->in_len <= 0 || n->classes <= 0 || n->classes > 32) return false;
  if (!n->in[0] || (n->inner && (!n->in[1] || !n->cl || !n->cr)) || !n->Why || !n->by || !n->score || !n->gates || !n->c || !n->tc || !n->h || !n->logp || !n->loss) return false;
  for (int slot = 0; slot < 5; ++slot) {
    if (!n->inner && (slot == 1 || slot == 2)) continue;
    if (!n->W[slot][0] || !n->bias[slot] || (n->inner && !n->W[slot][1])) return false;
  }
  return true;
}
int ora_tree_node_fwd(const ltb_tree_node* n) { ProfScope prof_scope_("ora_tree_node_fwd");
  REQUIRE(tree_node_ok(n), "tree_node_fwd: bad argument");
  const int Hd = n->hidden, L = n->in_len, K = n->classes;
  for (int slot = 0; slot < 5; ++slot) {
    if (!n->inner && (slot == 1 || slot == 2)) continue;
    ora_affine_act(n->W[slot][0], n->in[0], L, n->inner ? n->W[slot][1] : nullptr, n->inner ? n->in[1] : nullptr, n->inner ? L : 0, n->bias[slot], kSlotAct[slot],
                   n->gates + (size_t)slot * Hd, Hd);
  }
  float* g = n->gates;
  if (n->inner) ora_lstm_cell(g, g + 4 * Hd, g + Hd, n->cl, g + 2 * Hd, n->cr, g + 3 * Hd, n->c, n->tc, n->h, Hd);
  else ora_lstm_cell(g, g + 4 * Hd, nullptr, nullptr, nullptr, nullptr, g + 3 * Hd, n->c, n->tc, n->h, Hd);
  std::vector<float> pred(K); float nl = 0.0f;
  ora_affine_act(n->Why, n->classify_cell ? n->c : n->h, Hd, nullptr, nullptr, 0, n->by, -1, pred.data(), K);
  ora_log_softmax(pred.data(), n->logp, 1, K);
  ora_nll(n->logp, n->score, &nl, 1, K);
  if (n->loss_l) nl = nl + n->loss_l[0];
  if (n->loss_r) nl = nl + n->loss_r[0];
  n->loss[0] = nl;
  return LTB_OK;
}
int ora_tree_node_bwd(const ltb_tree_node* n) { ProfScope prof_scope_("ora_tree_node_bwd");
  REQUIRE(tree_node_ok(n) && n->dc && n->dh && n->dloss && n->dWhy && n->dby, "tree_node_bwd: bad argument");
  const int Hd = n->hidden, L = n->in_len, K = n->classes;
  const float dl = n->dloss[0];
  if (n->dloss_l) n->dloss_l[0] += dl;
  if (n->dloss_r) n->dloss_r[0] += dl;
  std::vector<float> dlogp(K, 0.0f), dpred(K, 0.0f), pred(K, 0.0f), dc(n->dc, n->dc + Hd), dh(n->dh, n->dh + Hd), dg((size_t)5 * Hd, 0.0f), dchild((size_t)2 * Hd, 0.0f);
  ora_nll_grad(dlogp.data(), &dl, n->score, 1, K);
  ora_log_softmax_grad(dpred.data(), n->logp, dlogp.data(), 1, K);
  ora_affine_act_grad(n->Why, n->dWhy, n->classify_cell ? n->c : n->h, n->classify_cell ? dc.data() : dh.data(), Hd, nullptr, nullptr, nullptr, nullptr, 0,
                      n->dby, -1, pred.data(), dpred.data(), K);
  float* g = n->gates;
  if (n->inner) {
    float* dcl = n->dcl ? n->dcl : dchild.data(); float* dcr = n->dcr ? n->dcr : dchild.data() + Hd;
    ora_lstm_cell_grad(g, dg.data(), g + 4 * Hd, dg.data() + 4 * Hd, g + Hd, dg.data() + Hd, n->cl, dcl, g + 2 * Hd, dg.data() + 2 * Hd, n->cr, dcr,
                       g + 3 * Hd, dg.data() + 3 * Hd, n->tc, dc.data(), dh.data(), Hd);
  } else {
    ora_lstm_cell_grad(g, dg.data(), g + 4 * Hd, dg.data() + 4 * Hd, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                       g + 3 * Hd, dg.data() + 3 * Hd, n->tc, dc.data(), dh.data(), Hd);
  }
  for (int slot = 4; slot >= 0; --slot) {
    if (!n->inner && (slot == 1 || slot == 2)) continue;
    REQUIRE(n->dW[slot][0] && n->dbias[slot] && (!n->inner || n->dW[slot][1]), "tree_node_bwd: missing gate gradient");
    ora_affine_act_grad(n->W[slot][0], n->dW[slot][0], n->in[0], n->din[0], L, n->inner ? n->W[slot][1] : nullptr, n->inner ? n->dW[slot][1] : nullptr,
                        n->inner ? n->in[1] : nullptr, n->inner ? n->din[1] : nullptr, n->inner ? L : 0, n->dbias[slot], kSlotAct[slot],
                        g + (size_t)slot * Hd, dg.data() + (size_t)slot * Hd, Hd);
  }
  return LTB_OK;
}
// One level of a tree: the nodes of the call one after the other (the CPU restatement has one memory: both arrays are the same).
int ora_tree_nodes_fwd(const ltb_tree_node* nodes_host, const ltb_tree_node*, int first, int count) {
  REQUIRE(nodes_host && first >= 0 && count > 0, "tree_nodes_fwd: bad argument");
  for (int i = first; i < first + count; ++i) { int rc = ora_tree_node_fwd(nodes_host + i); if (rc) return rc; }
  return LTB_OK;
}
int ora_tree_nodes_bwd(const ltb_tree_node* nodes_host, const ltb_tree_node*, int first, int count) {
  REQUIRE(nodes_host && first >= 0 && count > 0, "tree_nodes_bwd: bad argument");
  for (int i = first; i < first + count; ++i) { int rc = ora_tree_node_bwd(nodes_host + i); if (rc) return rc; }
  return LTB_OK;
}
}  // extern "C"

// ------------------------------------------------------------------ staging / replay: plain host equivalents.
extern "C" {
void* ora_host_alloc(size_t bytes) { return malloc(bytes); }
int ora_host_free(void* p) { ProfScope prof_scope_("ora_host_free"); free(p); return LTB_OK; }
int ora_d2h_async(void* d, const void* s, size_t n) { ProfScope prof_scope_("ora_d2h_async"); memcpy(d, s, n); return LTB_OK; }
int ora_branch_mark(void) { ProfScope prof_scope_("ora_branch_mark"); return LTB_OK; }        // one thread of control: a branch simply runs where it is issued
int ora_branch_begin(void) { ProfScope prof_scope_("ora_branch_begin"); return LTB_OK; }
int ora_branch_end(void) { ProfScope prof_scope_("ora_branch_end"); return LTB_OK; }
int ora_branch_join(void) { ProfScope prof_scope_("ora_branch_join"); return LTB_OK; }
int ora_marker_record(int) { ProfScope prof_scope_("ora_marker_record"); return LTB_OK; }      // the CPU oracle runs every call to completion
int ora_upload(void* d, const void* s, size_t n, int) { ProfScope prof_scope_("ora_upload"); memcpy(d, s, n); return LTB_OK; }      // one thread of control: copied at once
int ora_upload_marker(int) { return LTB_OK; }
int ora_stream_wait_marker(int) { return LTB_OK; }
int ora_marker_wait(int) { ProfScope prof_scope_("ora_marker_wait"); return LTB_OK; }
int ora_graph_begin(void) { ProfScope prof_scope_("ora_graph_begin"); return fail(LTB_E_ARG, "the CPU oracle does not record steps"); }
void* ora_graph_end(void) { return nullptr; }
int ora_graph_launch(void*) { ProfScope prof_scope_("ora_graph_launch"); return fail(LTB_E_ARG, "the CPU oracle does not record steps"); }
int ora_graph_destroy(void*) { ProfScope prof_scope_("ora_graph_destroy"); return LTB_OK; }
int ora_profile(int on) { if (on) g_prof_n = 0; g_prof_on = on != 0; return LTB_OK; }
// One line per entry point: name<TAB>calls<TAB>total milliseconds (the format of the CUDA library's report).
int ora_profile_report(char* buf, int len) {
  if (!buf || len <= 0) return LTB_E_ARG;
  std::string out;
  for (int i = 0; i < g_prof_n; ++i) { char line[256]; snprintf(line, sizeof line, "%s\t%lld\t%.6f\n", g_prof[i].name, g_prof[i].calls, g_prof[i].seconds * 1e3); out += line; }
  strncpy(buf, out.c_str(), len - 1); buf[len - 1] = 0;
  return (int)out.size() < len ? LTB_OK : LTB_E_LIMIT;
}
}
