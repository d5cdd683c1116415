// Shared state and helpers of liblantern_b200 (internal; the public contract is include/lantern_b200.h).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../include/lantern_b200.h"

namespace ltb {

constexpr int kSMs = 148;             // B200: 2 dies x 74 SMs; grids are sized in multiples of this
constexpr size_t kGranule = 256;      // arena granule (TMA wants 16 B bases/strides; 256 keeps every tensor sector-aligned)

// Look-ahead fusion (ltb_set_fusion): an operation whose result the very next call may finish in the same kernel is held back
// for one call.  BN forward or a same-shape add followed by an in-place ReLU of their result become one kernel; an in-place
// ReLU gradient followed by BN backward or by the add's gradient reading that buffer become one kernel.  Any other call
// first issues the held operation on its own, so results never change; only the moment of the launch does.
enum { PEND_NONE = 0, PEND_BN_FWD = 1, PEND_ADD = 2, PEND_RELU_GRAD = 3, PEND_RELU_ADD_GRAD = 4, PEND_BN_ADD = 5 };
struct Pending {
  int kind = PEND_NONE;
  int64_t n = 0;
  // PEND_BN_FWD
  const float *x = nullptr, *gamma = nullptr, *beta = nullptr;
  float *y = nullptr, *run_mean = nullptr, *run_var = nullptr, *save_mean = nullptr, *save_istd = nullptr;
  int N = 0, C = 0, HW = 0; float eps = 0, momentum = 0;
  // PEND_ADD: out = a + b
  const float *a = nullptr, *b = nullptr; float* out = nullptr;
  // PEND_RELU_GRAD: d = relu_y > 0 ? d : 0
  const float* relu_y = nullptr; float* d = nullptr;
  // PEND_RELU_ADD_GRAD (fusion level 2): m = relu_y > 0 ? d : 0; da += m; db += m, held so that the batch-norm backward whose dy is
  // da (or db) reads m straight from d and writes the other destination itself; fa / fb: that destination holds nothing yet
  float *da = nullptr, *db = nullptr; int fa = 0, fb = 0;
  // PEND_BN_ADD (fusion level 3): the PEND_BN_FWD fields, then out = y + a with y the held batch norm's result; an in-place ReLU of
  // out makes the three one kernel that never writes y
};

struct Context {
  bool inited = false;
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  char* heap = nullptr;
  size_t heap_bytes = 0;
  size_t used = 0;
  size_t top_used = 0;                // bytes taken from the far end of the arena for blocks that live until ltb_reset (step_alloc)
  bool keep_off = false;              // the two ends met once: nothing is kept at the far end any more
  int fatal = 1;
  int last = 0;
  std::string msg;
  int math = LTB_MATH_TF32;
  int64_t launches = 0;
  bool capturing = false;
  int64_t capture_launch_base = 0;
  int* dev_status = nullptr;          // device word set by kernels whose bounded waits run out
  int* host_status = nullptr;         // pinned mirror
  int64_t wait_limit_cycles = 2000000000ll;   // bound of every device-side spin wait (about a second; ltb_set_wait_limit)
  float* scratch = nullptr;           // private workspace for multi-stage reductions
  size_t scratch_bytes = 0;
  int sm_count = kSMs;
  bool profiling = false;             // per-launch CUDA-event timing (ltb_profile)
  const char* label = nullptr;        // optional name override for the next launches
  cudaStream_t side = nullptr;        // second stream: the weight-gradient half of conv backward runs beside the data-gradient half
  cudaStream_t copy = nullptr;        // uploads beside the compute work (ltb_upload)
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  unsigned tune = 0;                  // LTB_TUNE (environment, read by ltb_init): switches single optimisations off for A/B measurements:
                                      // 1 no in-kernel gather, 2 no tap-loop weight-grad from kept copies, 4 no kept copies, 8 no early first loads, 32 deferred zero fill off (ltb_grad_unset fills at once)
  bool deterministic = false;         // split-K sums in a fixed order (clusters, slabs) instead of atomics (ltb_set_deterministic)
  bool filter_cache = false;          // per-tap filter forms kept across calls (ltb_set_filter_cache)
  bool fusion = false;                // look-ahead fusion of BN/add with ReLU (off unless the host opts in)
  bool fusion_single_use = false;     // level 3: a batch-norm result consumed by add + in-place ReLU has no other reader and is not written
  bool fusion_no_writeback = false;   // level 2: an absorbed in-place ReLU gradient is applied on load only (its buffer is dead afterwards)
  Pending pending;
  bool hold_workspace = false;        // while two halves are in flight their staging blocks are released together at the end
  // Branch region (ltb_branch_mark .. ltb_branch_join): a run of calls issued on a third stream beside the caller's.
  cudaStream_t branch = nullptr, trunk = nullptr;
  cudaEvent_t mark_ev = nullptr, branch_done_ev = nullptr;
  bool branch_marked = false, in_branch = false, branch_ended = false;
  // Private workspace of the calling side: while a branch region is open the two streams each get one half.
  float* cur_scratch() const { return in_branch ? scratch + (scratch_bytes / 2) / sizeof(float) : scratch; }
  size_t cur_scratch_bytes() const { return branch_marked ? scratch_bytes / 2 : scratch_bytes; }
};
extern Context g;

int fail(int code, const char* fmt, ...);
int flush_pending();
int relu_add_grad_issue(const Pending& p);                 // issues the held operation on its own (elementwise.cu)
// issue functions shared by the entry points and the flush (pool_bn.cu / elementwise.cu)
int bn_fwd_issue(const Pending& p, bool relu);
int add_issue(const float* a, const float* b, float* out, int64_t n, bool relu);
int relu_grad_issue(const float* y, float* d, int64_t n);
// Host waits while a communicator exists: bounded, with NCCL's asynchronous error state polled (comm.cu).
void filter_cache_clear();           // gemm_tc.cu
void cl_cache_clear();               // gemm_tc.cu: kept channels-last copies (they live in step_alloc blocks)
void cl_cache_drop_from(const void* p);
// A block from the far end of the arena that stays until ltb_reset; nullptr when the two ends would meet (context.cu).
void* step_alloc(size_t bytes);
// A call is about to write [p, p + bytes): cached filter forms whose source overlaps it are stale (p == nullptr: all of them).
void filter_cache_note_write(const void* p, size_t bytes);
// Gradient buffers declared unset (ltb_grad_unset): logically zero, physically not yet written.
//   grad_take_unset(p, bytes)  true when [p, p + bytes) is exactly one declared block: the caller WRITES its result instead
//                              of adding (the declaration is consumed);
//   grad_settle(p, bytes)      any other use of a block that starts at p: fill it with zeros now (on the current stream).
// Both cost a look-up in a small host table, and nothing at all while no block is declared.
bool grad_take_unset(const void* p, size_t bytes);
int grad_settle(const void* p, size_t bytes);
void grad_unset_drop_from(const void* p);
void grad_unset_clear();
bool comm_active();
int comm_wait_stream(cudaStream_t s, const char* what);
int comm_wait_event(cudaEvent_t ev, const char* what);
void profile_before(const char* name);
void profile_after();

#define LTB_REQUIRE(cond, ...) do { if (!(cond)) return ::ltb::fail(LTB_E_ARG, __VA_ARGS__); } while (0)
// A gradient buffer that was declared unset and is about to be used in any way but as a whole, writable destination: zeros first.
#define LTB_SETTLE(ptr) do { int rc_s_ = ::ltb::grad_settle((ptr), 0); if (rc_s_) return rc_s_; } while (0)
#define LTB_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return ::ltb::fail(LTB_E_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); } while (0)
#define LTB_INITED_NOFLUSH() do { if (!::ltb::g.inited) return ::ltb::fail(LTB_E_STATE, "%s: library not initialised (call ltb_init)", __func__); } while (0)
// Every entry point first issues an operation held back by the look-ahead fusion; the few that may complete it use _NOFLUSH.
#define LTB_INITED() do { LTB_INITED_NOFLUSH(); if (::ltb::g.pending.kind) { int rc_ = ::ltb::flush_pending(); if (rc_) return rc_; } } while (0)

// Every kernel launch of the library goes through this macro so that ltb_kernel_launches() is exact.
#define LTB_LAUNCH(kernel, grid, block, smem, ...)                                           \
  do {                                                                                       \
    if (::ltb::g.profiling) ::ltb::profile_before(::ltb::g.label ? ::ltb::g.label : #kernel); \
    kernel<<<(grid), (block), (smem), ::ltb::g.stream>>>(__VA_ARGS__);                       \
    if (::ltb::g.profiling) ::ltb::profile_after();                                          \
    ++::ltb::g.launches;                                                                     \
    cudaError_t e_ = cudaGetLastError();                                                     \
    if (e_ != cudaSuccess) return ::ltb::fail(LTB_E_CUDA, "launch of %s failed: %s", #kernel, cudaGetErrorString(e_)); \
  } while (0)

// The same for a launch with a thread-block cluster of `cluster` CTAs along x (grid.x must be a multiple of it).
#define LTB_LAUNCH_CLUSTER(kernel, grid, block, cluster, ...)                                \
  do {                                                                                       \
    cudaLaunchConfig_t cfg_ = {};                                                            \
    cfg_.gridDim = (grid); cfg_.blockDim = (block); cfg_.dynamicSmemBytes = 0; cfg_.stream = ::ltb::g.stream; \
    cudaLaunchAttribute attr_[1];                                                            \
    attr_[0].id = cudaLaunchAttributeClusterDimension;                                       \
    attr_[0].val.clusterDim.x = (unsigned)(cluster); attr_[0].val.clusterDim.y = 1; attr_[0].val.clusterDim.z = 1; \
    cfg_.attrs = attr_; cfg_.numAttrs = 1;                                                   \
    if (::ltb::g.profiling) ::ltb::profile_before(::ltb::g.label ? ::ltb::g.label : #kernel); \
    cudaError_t e_ = cudaLaunchKernelEx(&cfg_, kernel, __VA_ARGS__);                         \
    if (::ltb::g.profiling) ::ltb::profile_after();                                          \
    ++::ltb::g.launches;                                                                     \
    if (e_ != cudaSuccess) return ::ltb::fail(LTB_E_CUDA, "cluster launch of %s failed: %s", #kernel, cudaGetErrorString(e_)); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
// Grid for a grid-stride kernel over `work` thread-items: enough CTAs to cover it, capped at `per_sm` CTAs per SM.
inline int grid_for(int64_t work, int block, int per_sm = 8) {
  int64_t need = ceil_div(work, block);
  int64_t cap = (int64_t)g.sm_count * per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

}  // namespace ltb
