// Data parallelism: NCCL communicator and the gradient all-reduce fused with the SGD update.
//
// The reference is single-GPU (src/out/PLDI19evaluation/run_exp.sh:7 pins one device); this is the one part
// of the library with no counterpart there.  One process per GPU.  NCCL is loaded with dlopen at comm_init so that
// single-GPU users need no NCCL at all and multi-GPU users share whatever libnccl the launcher already loaded.
#include <dlfcn.h>

#include <cstring>

#include "buckets.h"
#include "comm_wait.h"
#include "common.cuh"

namespace ltb {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat = 7 };
enum { ncclSum = 0 };

struct Nccl {
  void* handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;     // failure detection: polled while the host waits for a step
  int (*CommAbort)(ncclComm_t) = nullptr;
  ncclComm_t comm = nullptr;
  bool broken = false;               // the communicator was aborted after a failure or a timeout: collectives are refused from then on
  int64_t timeout_ms = 60000;        // how long the host waits for a stream that carries collectives (ltb_comm_set_timeout_ms)
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr;
  cudaEvent_t done[kMaxBuckets] = {};
  // gradient ranges whose all-reduce was started early (ltb_allreduce_begin), in the order they were started
  static const int kMaxEarly = 16;
  struct Early { float* ptr; int64_t n; cudaEvent_t done; } early[kMaxEarly] = {};
  int n_early = 0;
  // measurement: the end of backward on the compute stream and the start of the update kernel, as timed events
  cudaEvent_t t_backward_end = nullptr, t_update_start = nullptr;
  bool timed = false;
} nccl;

static int load_nccl() {
  if (nccl.handle) return LTB_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) { nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (nccl.handle) break; }
  if (!nccl.handle) return fail(LTB_E_COMM, "cannot load libnccl.so.2: %s", dlerror());
#define LTB_SYM(field, name) do { *(void**)(&nccl.field) = dlsym(nccl.handle, name); if (!nccl.field) return fail(LTB_E_COMM, "libnccl lacks %s", name); } while (0)
  LTB_SYM(GetUniqueId, "ncclGetUniqueId"); LTB_SYM(CommInitRank, "ncclCommInitRank"); LTB_SYM(CommDestroy, "ncclCommDestroy");
  LTB_SYM(AllReduce, "ncclAllReduce"); LTB_SYM(GetErrorString, "ncclGetErrorString");
  LTB_SYM(CommGetAsyncError, "ncclCommGetAsyncError"); LTB_SYM(CommAbort, "ncclCommAbort");
#undef LTB_SYM
  return LTB_OK;
}
#define LTB_NCCL(call) do { int r_ = (call); if (r_ != ncclSuccess) return fail(LTB_E_COMM, "%s failed: %s", #call, nccl.GetErrorString(r_)); } while (0)

// x -= (lr/world) * d ; d = 0 over one bucket (the averaged-gradient SGD update).
__global__ void sgd_scaled_kernel(float* x, float* d, float neg_lr_over_world, int64_t n4, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  const float4 z = make_float4(0, 0, 0, 0);
  for (int64_t j = i; j < n4; j += stride) {
    float4 xv = reinterpret_cast<float4*>(x)[j], dv = reinterpret_cast<float4*>(d)[j];
    xv.x += dv.x * neg_lr_over_world; xv.y += dv.y * neg_lr_over_world; xv.z += dv.z * neg_lr_over_world; xv.w += dv.w * neg_lr_over_world;
    reinterpret_cast<float4*>(x)[j] = xv; reinterpret_cast<float4*>(d)[j] = z;
  }
  for (int64_t j = n4 * 4 + i; j < n; j += stride) { x[j] += d[j] * neg_lr_over_world; d[j] = 0.0f; }
}

// ---- failure detection ---------------------------------------------------------------------------------------------------
// A rank that leaves (a crash, an exception in its host program) makes its peers' next collective wait for ever, and a plain
// cudaStreamSynchronize behind it never returns.  Whenever the host blocks on the library's stream while a communicator
// exists (ltb_sync, ltb_d2h, ltb_marker_wait) it therefore polls instead: the stream or event, NCCL's asynchronous error
// state, and a deadline.  On an error or when the deadline passes the communicator is aborted (which ends its kernels on
// the device, so the stream drains), further collectives are refused, and the call returns LTB_E_COMM.
static int comm_failed(const char* what, int why) {
  if (nccl.comm && nccl.CommAbort) nccl.CommAbort(nccl.comm);
  nccl.comm = nullptr; nccl.broken = true;
  // the aborted kernels end promptly; give the streams a moment to drain so that the context stays usable
  bounded_wait([] { return cudaStreamQuery(g.stream) != cudaErrorNotReady; }, [] { return false; }, 5000);
  if (nccl.comm_stream) bounded_wait([] { return cudaStreamQuery(nccl.comm_stream) != cudaErrorNotReady; }, [] { return false; }, 5000);
  return fail(LTB_E_COMM, "%s: %s; the communicator was aborted", what,
              why == WAIT_TIMEOUT ? "a collective did not finish within the communicator's timeout (a rank has left?)" : "NCCL reported an asynchronous error");
}
static bool comm_async_error() {
  int e = ncclSuccess;
  return nccl.comm && nccl.CommGetAsyncError && (nccl.CommGetAsyncError(nccl.comm, &e) != ncclSuccess || e != ncclSuccess);
}
bool comm_active() { return nccl.comm != nullptr; }
int comm_wait_stream(cudaStream_t s, const char* what) {
  cudaError_t last = cudaSuccess;
  const int r = bounded_wait([&] { last = cudaStreamQuery(s); return last != cudaErrorNotReady; }, comm_async_error, nccl.timeout_ms);
  if (r != WAIT_DONE) return comm_failed(what, r);
  if (last != cudaSuccess) return fail(LTB_E_CUDA, "%s: %s", what, cudaGetErrorString(last));
  return LTB_OK;
}
int comm_wait_event(cudaEvent_t ev, const char* what) {
  cudaError_t last = cudaSuccess;
  const int r = bounded_wait([&] { last = cudaEventQuery(ev); return last != cudaErrorNotReady; }, comm_async_error, nccl.timeout_ms);
  if (r != WAIT_DONE) return comm_failed(what, r);
  if (last != cudaSuccess) return fail(LTB_E_CUDA, "%s: %s", what, cudaGetErrorString(last));
  return LTB_OK;
}

}  // namespace ltb

using namespace ltb;

extern "C" {

int ltb_sgd_step(float* x, float* d, float lr, int64_t n);

int ltb_comm_unique_id(void* out128) {
  LTB_REQUIRE(out128, "ltb_comm_unique_id: null pointer");
  int rc = load_nccl(); if (rc) return rc;
  ncclUniqueId id; LTB_NCCL(nccl.GetUniqueId(&id));
  memcpy(out128, &id, 128);
  return LTB_OK;
}
int ltb_comm_init(int rank, int world, const void* id128) {
  LTB_INITED(); LTB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "ltb_comm_init: bad rank/world");
  if (nccl.comm) return fail(LTB_E_STATE, "ltb_comm_init: communicator already exists");
  nccl.rank = rank; nccl.world = world;
  if (world == 1) return LTB_OK;
  LTB_REQUIRE(id128, "ltb_comm_init: null id");
  int rc = load_nccl(); if (rc) return rc;
  ncclUniqueId id; memcpy(&id, id128, 128);
  LTB_NCCL(nccl.CommInitRank(&nccl.comm, world, id, rank));
  LTB_CUDA(cudaStreamCreateWithFlags(&nccl.comm_stream, cudaStreamNonBlocking));
  LTB_CUDA(cudaEventCreateWithFlags(&nccl.ready, cudaEventDisableTiming));
  for (auto& e : nccl.done) LTB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  for (auto& e : nccl.early) LTB_CUDA(cudaEventCreateWithFlags(&e.done, cudaEventDisableTiming));
  nccl.n_early = 0;
  LTB_CUDA(cudaEventCreate(&nccl.t_backward_end)); LTB_CUDA(cudaEventCreate(&nccl.t_update_start)); nccl.timed = false;
  return LTB_OK;
}
int ltb_comm_destroy(void) {
  if (nccl.comm) {
    nccl.CommDestroy(nccl.comm); nccl.comm = nullptr;
    cudaStreamDestroy(nccl.comm_stream); cudaEventDestroy(nccl.ready);
    for (auto& e : nccl.done) cudaEventDestroy(e);
    for (auto& e : nccl.early) cudaEventDestroy(e.done);
  }
  else if (nccl.broken && nccl.comm_stream) {        // aborted earlier: the communicator is gone, its stream and events are not
    cudaStreamDestroy(nccl.comm_stream); cudaEventDestroy(nccl.ready);
    for (auto& e : nccl.done) cudaEventDestroy(e);
    for (auto& e : nccl.early) cudaEventDestroy(e.done);
  }
  if (nccl.t_backward_end) { cudaEventDestroy(nccl.t_backward_end); cudaEventDestroy(nccl.t_update_start); nccl.t_backward_end = nccl.t_update_start = nullptr; }
  nccl.comm_stream = nullptr; nccl.broken = false; nccl.timed = false;
  nccl.n_early = 0;
  nccl.world = 1; nccl.rank = 0;
  return LTB_OK;
}
int ltb_comm_world(void) { return nccl.world; }
int ltb_comm_set_timeout_ms(int64_t ms) { nccl.timeout_ms = ms; return LTB_OK; }
// The part of the gradient exchange that the last data-parallel step could not hide: the time from the end of backward on
// the compute stream to the start of the update kernel, which waits for every sum.  Blocks until that step has finished.
int ltb_comm_exposed_ms(float* out_ms) {
  LTB_INITED(); LTB_REQUIRE(out_ms, "ltb_comm_exposed_ms: null pointer");
  *out_ms = 0.0f;
  if (nccl.world == 1 || !nccl.timed) return LTB_OK;
  int rc = comm_wait_stream(g.stream, "ltb_comm_exposed_ms"); if (rc) return rc;
  LTB_CUDA(cudaEventElapsedTime(out_ms, nccl.t_backward_end, nccl.t_update_start));
  return LTB_OK;
}

int ltb_allreduce_sum(float* x, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && n >= 0, "ltb_allreduce_sum: bad argument");
  if (nccl.world == 1 || n == 0) return LTB_OK;
  if (nccl.broken) return fail(LTB_E_COMM, "ltb_allreduce_sum: the communicator was aborted");
  LTB_NCCL(nccl.AllReduce(x, x, (size_t)n, ncclFloat, ncclSum, nccl.comm, g.stream));
  return LTB_OK;
}
// Starts the sum of a gradient range whose values are final while the rest of the backward pass is still running: the
// range is reduced in place on the communication stream, after everything issued so far on the compute stream.  The
// following ltb_allreduce_sgd_step over a span that contains the range does not reduce it again.  With one rank: no-op.
int ltb_allreduce_begin(float* d, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(d && n >= 0, "ltb_allreduce_begin: bad argument");
  if (nccl.world == 1 || n == 0) return LTB_OK;
  if (nccl.broken) return fail(LTB_E_COMM, "ltb_allreduce_begin: the communicator was aborted");
  if (nccl.n_early == Nccl::kMaxEarly) return LTB_OK;              // no slot left: the range is simply reduced at the step
  Nccl::Early& e = nccl.early[nccl.n_early];
  LTB_CUDA(cudaEventRecord(nccl.ready, g.stream));
  LTB_CUDA(cudaStreamWaitEvent(nccl.comm_stream, nccl.ready, 0));
  LTB_NCCL(nccl.AllReduce(d, d, (size_t)n, ncclFloat, ncclSum, nccl.comm, nccl.comm_stream));
  LTB_CUDA(cudaEventRecord(e.done, nccl.comm_stream));
  e.ptr = d; e.n = n; ++nccl.n_early;
  return LTB_OK;
}
// Gradient all-reduce fused with the update.  Ranges started early are only waited for; what is left of the span is cut
// into buckets, bucket i being reduced on the communication stream while the update kernel of bucket i-1 runs on the
// compute stream, so only the first reduction and the last update are exposed.  Each rank's loss is the mean over its own
// shard, hence the 1/world factor.
static int update_range(float* x, float* d, int64_t off, int64_t cnt, float s) {
  float* xb = x + off; float* db = d + off;
  const int64_t n4 = (aligned16(xb) && aligned16(db)) ? cnt / 4 : 0;
  LTB_LAUNCH(sgd_scaled_kernel, grid_for(cnt / 4 + 1, 256), 256, 0, xb, db, s, n4, cnt);
  return LTB_OK;
}
int ltb_allreduce_sgd_step(float* x, float* d, float lr, int64_t n) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && d && n >= 0, "ltb_allreduce_sgd_step: bad argument");
  if (nccl.world == 1) return ltb_sgd_step(x, d, lr, n);
  if (n == 0) return LTB_OK;
  if (nccl.broken) return fail(LTB_E_COMM, "ltb_allreduce_sgd_step: the communicator was aborted");
  const float s = -1.0f * lr / (float)nccl.world;
  // early ranges inside [d, d + n), sorted by address; the gaps between them are what is still to be reduced
  int order[Nccl::kMaxEarly], ne = 0;
  for (int i = 0; i < nccl.n_early; ++i) {
    const Nccl::Early& e = nccl.early[i];
    if (e.ptr >= d && e.ptr + e.n <= d + n) order[ne++] = i;
    else return fail(LTB_E_ARG, "ltb_allreduce_sgd_step: a range given to ltb_allreduce_begin lies outside this span");
  }
  for (int i = 1; i < ne; ++i) for (int j = i; j > 0 && nccl.early[order[j]].ptr < nccl.early[order[j - 1]].ptr; --j) { int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
  // Inside a recorded step an ordinary event record is only a dependency; the external form makes a node that really
  // records the event at every replay, so that ltb_comm_exposed_ms can read the last step's span.
  const unsigned rec = g.capturing ? cudaEventRecordExternal : cudaEventRecordDefault;
  LTB_CUDA(cudaEventRecordWithFlags(nccl.t_backward_end, g.stream, rec));
  LTB_CUDA(cudaEventRecord(nccl.ready, g.stream));
  LTB_CUDA(cudaStreamWaitEvent(nccl.comm_stream, nccl.ready, 0));
  int64_t cursor = 0; int rc = LTB_OK;
  // With early ranges most of the slab is already reduced or on its way: the gaps are summed now and ONE update kernel
  // follows the last sum (eleven small update kernels with their event waits cost 0.2 ms per step more, measured).
  // Without early ranges the span is one gap and the bucket pipeline below overlaps sums and updates.
  const bool single_update = ne > 0;
  for (int k = 0; k <= ne && rc == LTB_OK; ++k) {
    const int64_t gap_end = k < ne ? (int64_t)(nccl.early[order[k]].ptr - d) : n;
    if (gap_end < cursor) return fail(LTB_E_ARG, "ltb_allreduce_sgd_step: overlapping early ranges");
    if (gap_end > cursor) {                                        // a gap: reduce it now, bucket by bucket
      int64_t off[kMaxBuckets], cnt[kMaxBuckets];
      const int used = single_update ? 1 : bucket_spans(gap_end - cursor, off, cnt);
      if (single_update) { off[0] = 0; cnt[0] = gap_end - cursor; }
      for (int b = 0; b < used; ++b) {
        LTB_NCCL(nccl.AllReduce(d + cursor + off[b], d + cursor + off[b], (size_t)cnt[b], ncclFloat, ncclSum, nccl.comm, nccl.comm_stream));
        if (!single_update) LTB_CUDA(cudaEventRecord(nccl.done[b], nccl.comm_stream));
      }
      for (int b = 0; b < used && rc == LTB_OK && !single_update; ++b) {
        LTB_CUDA(cudaStreamWaitEvent(g.stream, nccl.done[b], 0));
        rc = update_range(x, d, cursor + off[b], cnt[b], s);
      }
    }
    if (k < ne) cursor = (int64_t)(nccl.early[order[k]].ptr - d) + nccl.early[order[k]].n;
  }
  if (single_update && rc == LTB_OK) {
    // everything on the communication stream so far (early ranges and gaps, in issue order) precedes this event
    LTB_CUDA(cudaEventRecord(nccl.done[0], nccl.comm_stream));
    LTB_CUDA(cudaStreamWaitEvent(g.stream, nccl.done[0], 0));
    LTB_CUDA(cudaEventRecordWithFlags(nccl.t_update_start, g.stream, rec)); nccl.timed = true;
    rc = update_range(x, d, 0, n, s);
  }
  nccl.n_early = 0;
  return rc;
}

}  // extern "C"
