// Context, arena, transfers and step replay of liblantern_b200.
//
// Replaces the runtime preamble the reference prints into every generated .cu file
// (src/main/scala/lantern/DslAPI.scala:433-473: CUDA_CALL macro, gpuMallocBase/gpuMallocAddr bump arena,
// myGpuMalloc/myGpuFree) and backend.setup()/cleanup() (TensorDslCublas.scala:113-124).
#include <cstdarg>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace ltb {

Context g;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  g.last = code; g.msg = buf;
  if (g.fatal) {   // reference convention: print and exit (DslAPI.scala:435-451)
    fprintf(stderr, "lantern_b200 error %d: %s\n", code, buf);
    exit(code < 0 ? -code : code);
  }
  return code;
}

// ---- per-launch timing with CUDA events on the launching stream (enabled by ltb_profile) ----------------------------
struct ProfRec { const char* name; cudaEvent_t a, b; };
static std::vector<ProfRec> prof_recs;
void profile_before(const char* name) {
  if (prof_recs.size() >= ((size_t)1 << 20)) { g.profiling = false; return; }     // a forgotten ltb_profile(1): stop recording, keep what is there
  ProfRec r; r.name = name;
  cudaEventCreate(&r.a); cudaEventCreate(&r.b);
  cudaEventRecord(r.a, g.stream);
  prof_recs.push_back(r);
}
void profile_after() { cudaEventRecord(prof_recs.back().b, g.stream); }
static void profile_clear() { for (auto& r : prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); } prof_recs.clear(); }

struct Graph { cudaGraphExec_t exec; cudaGraph_t graph; int64_t launches; };

static size_t round_up(size_t b) { return (b + kGranule - 1) / kGranule * kGranule; }

}  // namespace ltb

using namespace ltb;

extern "C" {

int ltb_set_fatal(int on) { g.fatal = on; return LTB_OK; }
int ltb_last_error(char* buf, int len) {
  if (buf && len > 0) { strncpy(buf, g.msg.c_str(), len - 1); buf[len - 1] = 0; }
  return g.last;
}

// Everything ltb_init obtained, in any state of completion (also the way out of a failed ltb_init).
static void release_all() {
  if (g.stream) cudaStreamSynchronize(g.stream);
  if (g.side) cudaStreamSynchronize(g.side);
  if (g.branch) cudaStreamSynchronize(g.branch);
  if (g.branch) cudaStreamDestroy(g.branch);
  if (g.mark_ev) cudaEventDestroy(g.mark_ev);
  if (g.branch_done_ev) cudaEventDestroy(g.branch_done_ev);
  if (g.heap) cudaFree(g.heap);
  if (g.dev_status) cudaFree(g.dev_status);
  if (g.scratch) cudaFree(g.scratch);
  if (g.host_status) cudaFreeHost(g.host_status);
  if (g.side) cudaStreamDestroy(g.side);
  if (g.copy) { cudaStreamSynchronize(g.copy); cudaStreamDestroy(g.copy); }
  if (g.fork_ev) cudaEventDestroy(g.fork_ev);
  if (g.join_ev) cudaEventDestroy(g.join_ev);
  if (g.own_stream && g.stream) cudaStreamDestroy(g.stream);
  const int fatal = g.fatal, last = g.last; const std::string msg = g.msg;
  g = Context();
  g.fatal = fatal; g.last = last; g.msg = msg;          // the error mode and the last message outlive the context
}

static int init_steps(int device, size_t heap_bytes) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(LTB_E_CUDA, "ltb_init: no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e));
  LTB_REQUIRE(device >= 0 && device < count, "ltb_init: device %d out of range (%d devices)", device, count);
  LTB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  LTB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(LTB_E_CUDA, "ltb_init: device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);
  g.device = device; g.sm_count = prop.multiProcessorCount;
  if (heap_bytes == 0) heap_bytes = (size_t)8 * 1024 * 1024 * 1024 + 16;   // HEAP_SIZE, DslAPI.scala:453
  heap_bytes = round_up(heap_bytes);
  LTB_CUDA(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
  g.own_stream = true;
  LTB_CUDA(cudaMalloc((void**)&g.heap, heap_bytes));
  g.heap_bytes = heap_bytes; g.used = 0;
  LTB_CUDA(cudaMalloc((void**)&g.dev_status, 256));
  LTB_CUDA(cudaMemset(g.dev_status, 0, 256));
  LTB_CUDA(cudaMallocHost((void**)&g.host_status, 256));
  g.host_status[0] = 0;
  g.scratch_bytes = (size_t)8 << 20;
  LTB_CUDA(cudaMalloc((void**)&g.scratch, g.scratch_bytes));
  LTB_CUDA(cudaStreamCreateWithFlags(&g.side, cudaStreamNonBlocking));
  LTB_CUDA(cudaStreamCreateWithFlags(&g.copy, cudaStreamNonBlocking));
  LTB_CUDA(cudaEventCreateWithFlags(&g.fork_ev, cudaEventDisableTiming));
  LTB_CUDA(cudaEventCreateWithFlags(&g.join_ev, cudaEventDisableTiming));
  LTB_CUDA(cudaStreamCreateWithFlags(&g.branch, cudaStreamNonBlocking));
  LTB_CUDA(cudaEventCreateWithFlags(&g.mark_ev, cudaEventDisableTiming));
  LTB_CUDA(cudaEventCreateWithFlags(&g.branch_done_ev, cudaEventDisableTiming));
  g.launches = 0; g.last = 0; g.msg.clear(); g.capturing = false; g.math = LTB_MATH_TF32;
  if (const char* t = getenv("LTB_TUNE")) g.tune = (unsigned)strtoul(t, nullptr, 0);
  return LTB_OK;
}

int ltb_init(int device, size_t heap_bytes) {
  if (g.inited) return fail(LTB_E_STATE, "ltb_init: already initialised");
  const int rc = init_steps(device, heap_bytes);
  if (rc) { release_all(); return rc; }        // non-fatal mode: a step that failed leaves nothing behind
  g.inited = true;
  return LTB_OK;
}

int ltb_comm_destroy(void);
}
namespace ltb { void static_sum_forget(); }
extern "C" {

// Stream markers (ltb_marker_record / ltb_marker_wait): one event per slot, created on first use.
static cudaEvent_t marker_ev[16];
static bool marker_set[16];

int ltb_shutdown(void) {
  if (!g.inited) return LTB_OK;
  if (g.pending.kind) flush_pending();
  ltb_comm_destroy();
  static_sum_forget();
  profile_clear();
  cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g.side); cudaStreamSynchronize(g.branch);
  filter_cache_clear(); cl_cache_clear();
  for (int i = 0; i < 16; ++i) { if (marker_ev[i]) cudaEventDestroy(marker_ev[i]); marker_ev[i] = nullptr; marker_set[i] = false; }
  grad_unset_clear();
  release_all();
  return LTB_OK;
}

int ltb_set_stream(void* s) {
  LTB_INITED();
  if (g.own_stream) { cudaStreamSynchronize(g.stream); cudaStreamDestroy(g.stream); g.own_stream = false; }
  g.stream = (cudaStream_t)s;
  return LTB_OK;
}
void* ltb_get_stream(void) { if (g.inited && g.pending.kind) flush_pending(); return (void*)g.stream; }   // the caller may enqueue its own work next
// With a communicator the wait is bounded and watches for a failed collective (comm.cu: comm_wait_stream).
static int stream_wait(const char* what) {
  if (comm_active()) return comm_wait_stream(g.stream, what);
  LTB_CUDA(cudaStreamSynchronize(g.stream));
  return LTB_OK;
}
int ltb_sync(void) { LTB_INITED(); return stream_wait("ltb_sync"); }
int ltb_set_fusion(int on) { LTB_INITED(); g.fusion = on != 0; g.fusion_no_writeback = on >= 2; g.fusion_single_use = on >= 3; return LTB_OK; }
int ltb_set_filter_cache(int on) {
  LTB_INITED(); LTB_REQUIRE(!g.capturing, "ltb_set_filter_cache: not while recording a step");
  if (!on && g.filter_cache) { cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g.side); cudaStreamSynchronize(g.branch); filter_cache_clear(); }
  g.filter_cache = on != 0; return LTB_OK;
}
int ltb_set_deterministic(int on) { LTB_INITED(); LTB_REQUIRE(!g.capturing, "ltb_set_deterministic: not while recording a step"); g.deterministic = on != 0; return LTB_OK; }
int ltb_params_changed(void) { LTB_INITED(); filter_cache_note_write(nullptr, 0); return LTB_OK; }
int ltb_set_math(int mode) {
  LTB_REQUIRE(mode == LTB_MATH_FP32 || mode == LTB_MATH_TF32, "ltb_set_math: unknown mode %d", mode);
  g.math = mode; return LTB_OK;
}
int ltb_device_status(void) {
  if (!g.inited) return LTB_OK;
  if (g.pending.kind) flush_pending();
  if (cudaMemcpyAsync(g.host_status, g.dev_status, 4, cudaMemcpyDeviceToHost, g.stream) != cudaSuccess) return LTB_E_CUDA;
  if (cudaStreamSynchronize(g.stream) != cudaSuccess) return LTB_E_CUDA;
  return g.host_status[0] ? LTB_E_DEVICE : LTB_OK;
}
int ltb_clear_device_status(void) {
  LTB_INITED();
  LTB_CUDA(cudaMemsetAsync(g.dev_status, 0, 4, g.stream));
  return LTB_OK;
}
int64_t ltb_kernel_launches(void) { return g.launches; }

// ------------------------------------------------------------------ arena (DslAPI.scala:453-473)
static void* arena_alloc(size_t bytes, bool zero) {
  if (!g.inited) { fail(LTB_E_STATE, "ltb_malloc: library not initialised"); return nullptr; }
  size_t b = round_up(bytes ? bytes : 1);
  if (g.used + b + g.top_used > g.heap_bytes && g.top_used && !g.capturing) {
    // The far end's kept copies are a convenience and yield to a real allocation: wait for their readers, drop them, and keep
    // nothing from now on (this arena is too tight for them).  Not possible while a step is being recorded: that is an overflow.
    cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g.side); cudaStreamSynchronize(g.branch);
    cl_cache_clear(); g.top_used = 0; g.keep_off = true;
  }
  if (g.used + b + g.top_used > g.heap_bytes) {
    fail(LTB_E_OOM, "ltb_malloc: arena exhausted (%zu used + %zu requested > %zu)", g.used, b, g.heap_bytes);
    return nullptr;
  }
  char* p = g.heap + g.used;
  g.used += b;
  if (zero && cudaMemsetAsync(p, 0, b, g.stream) != cudaSuccess) { fail(LTB_E_CUDA, "ltb_malloc: memset failed"); return nullptr; }
  return p;
}
}  // extern "C"
namespace ltb {
// ---- deferred zero fill of gradient buffers ------------------------------------------------------------------------------------
// The reference hands out zeroed memory and every gradient entry point adds into its destination.  For the activation
// gradients of a convolutional network that is a zero fill of every buffer plus a read of those zeros by the first (usually
// only) operation that adds into it.  A caller may instead declare a fresh gradient buffer unset: the first accumulating entry
// point that meets it as its whole destination and is able to (convolution data-grad, batch-norm backward, same-shape add
// gradient) writes its result; every other entry point fills the block with zeros before it touches it.
static std::vector<std::pair<const char*, size_t>> unset_blocks;
static int unset_find(const void* p) {
  for (size_t i = 0; i < unset_blocks.size(); ++i) if (unset_blocks[i].first == (const char*)p) return (int)i;
  return -1;
}
bool grad_take_unset(const void* p, size_t bytes) {
  if (unset_blocks.empty() || !p) return false;
  const int i = unset_find(p);
  if (i < 0) return false;
  if (unset_blocks[i].second != bytes) return false;               // a part or more than the block: the caller settles it instead
  unset_blocks[i] = unset_blocks.back(); unset_blocks.pop_back();
  return true;
}
int grad_settle(const void* p, size_t) {
  if (unset_blocks.empty() || !p) return LTB_OK;
  const int i = unset_find(p);
  if (i < 0) return LTB_OK;
  const size_t bytes = unset_blocks[i].second;
  unset_blocks[i] = unset_blocks.back(); unset_blocks.pop_back();
  if (cudaMemsetAsync(const_cast<void*>(p), 0, bytes, g.stream) != cudaSuccess) return fail(LTB_E_CUDA, "zero fill of a deferred gradient buffer failed");
  return LTB_OK;
}
void grad_unset_drop_from(const void* p) {
  for (size_t i = 0; i < unset_blocks.size();) { if ((const void*)unset_blocks[i].first >= p) { unset_blocks[i] = unset_blocks.back(); unset_blocks.pop_back(); } else ++i; }
}
void grad_unset_clear() { unset_blocks.clear(); }
void* step_alloc(size_t bytes) {
  if (!g.inited || g.keep_off) return nullptr;
  const size_t b = round_up(bytes ? bytes : 1);
  if (g.used + g.top_used + b + ((size_t)256 << 20) > g.heap_bytes) return nullptr;     // leave the near end room to grow
  g.top_used += b;
  return g.heap + g.heap_bytes - g.top_used;
}
}  // namespace ltb
extern "C" {
// Deferred zero fill (see grad_take_unset): d must be a block of n floats that nothing has written since it was handed out.
int ltb_grad_unset(float* d, int64_t n) {
  LTB_INITED_NOFLUSH(); LTB_REQUIRE(d && n > 0, "ltb_grad_unset: bad argument");       // bookkeeping on a buffer no held operation can name yet: nothing is issued
  if (g.tune & 32) { LTB_CUDA(cudaMemsetAsync(d, 0, (size_t)n * 4, g.stream)); return LTB_OK; }     // switch: plain zero fill at once
  grad_settle(d, 0);                                                   // declared before and never used: start over
  unset_blocks.emplace_back((const char*)d, (size_t)n * 4);
  return LTB_OK;
}
int ltb_grad_materialize(float* d, int64_t n) { LTB_INITED(); LTB_REQUIRE(d && n >= 0, "ltb_grad_materialize: bad argument"); return grad_settle(d, (size_t)n * 4); }
void* ltb_malloc(size_t bytes) { return arena_alloc(bytes, true); }
void* ltb_malloc_uninit(size_t bytes) { return arena_alloc(bytes, false); }
int ltb_free(void* p, size_t bytes) {
  LTB_INITED();
  size_t b = round_up(bytes ? bytes : 1);
  LTB_REQUIRE(p && b <= g.used && (char*)p == g.heap + g.used - b, "ltb_free: not the newest block (LIFO arena)");
  g.used -= b;
  cl_cache_drop_from(p); grad_unset_drop_from(p);
  return LTB_OK;
}
void* ltb_mark(void) { return g.heap + g.used; }
int ltb_reset(void* mark) {
  LTB_INITED();
  char* m = (char*)mark;
  LTB_REQUIRE(m >= g.heap && m <= g.heap + g.used, "ltb_reset: mark outside the used span");
  LTB_REQUIRE(!g.branch_marked, "ltb_reset: a branch region is open (ltb_branch_join missing)");
  g.used = (size_t)(m - g.heap);   // zeroing happens when a block is handed out again by ltb_malloc
  g.top_used = 0; cl_cache_clear();  // the step's kept copies go with it
  grad_unset_drop_from(m);           // and the declarations of blocks that no longer exist
  return LTB_OK;
}
size_t ltb_arena_used(void) { return g.used; }

// ------------------------------------------------------------------ transfers (GPUOps.scala:51-95)
int ltb_h2d(void* dst, const void* src, size_t bytes) {
  LTB_INITED(); filter_cache_note_write(dst, bytes); LTB_REQUIRE(dst && src, "ltb_h2d: null pointer");
  { int rc_ = grad_settle(dst, bytes); if (rc_) return rc_; }
  if (bytes) LTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g.stream));
  return LTB_OK;
}
int ltb_d2h(void* dst, const void* src, size_t bytes) {
  LTB_INITED(); LTB_REQUIRE(dst && src, "ltb_d2h: null pointer");
  { int rc_ = grad_settle(src, bytes); if (rc_) return rc_; }
  LTB_REQUIRE(!g.capturing, "ltb_d2h: blocking read-back while recording a step");
  if (bytes) LTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g.stream));
  return stream_wait("ltb_d2h");
}
int ltb_d2d(void* dst, const void* src, size_t bytes) {
  LTB_INITED(); filter_cache_note_write(dst, bytes); LTB_REQUIRE(dst && src, "ltb_d2d: null pointer");
  { int rc_ = grad_settle(dst, bytes); if (!rc_) rc_ = grad_settle(src, bytes); if (rc_) return rc_; }
  if (bytes) LTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, g.stream));
  return LTB_OK;
}
void* ltb_host_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) { fail(LTB_E_CUDA, "ltb_host_alloc: cudaMallocHost failed"); return nullptr; }
  return p;
}
int ltb_host_free(void* p) { if (p) LTB_CUDA(cudaFreeHost(p)); return LTB_OK; }
int ltb_d2h_async(void* dst, const void* src, size_t bytes) {
  LTB_INITED(); LTB_REQUIRE(dst && src, "ltb_d2h_async: null pointer");
  { int rc_ = grad_settle(src, bytes); if (rc_) return rc_; }
  if (bytes) LTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g.stream));
  return LTB_OK;
}
int ltb_marker_record(int slot) {
  LTB_INITED(); LTB_REQUIRE(slot >= 0 && slot < 16, "ltb_marker_record: slot %d out of range", slot);
  LTB_REQUIRE(!g.capturing, "ltb_marker_record: not allowed while recording a step");
  if (!marker_ev[slot]) LTB_CUDA(cudaEventCreateWithFlags(&marker_ev[slot], cudaEventDisableTiming));
  LTB_CUDA(cudaEventRecord(marker_ev[slot], g.stream));
  marker_set[slot] = true;
  return LTB_OK;
}
// Uploads beside the compute work.  ltb_upload copies from (pinned) host memory on the library's copy stream, after marker
// `after` if one is named (the point of the compute stream up to which the destination was still being read); ltb_upload_marker
// records a marker on the copy stream (the uploads so far are done when it is reached); ltb_stream_wait_marker makes the
// COMPUTE stream wait for a marker on the device, without blocking the host.
int ltb_upload(void* dst, const void* src, size_t bytes, int after) {
  LTB_INITED(); LTB_REQUIRE(dst && src && after >= -1 && after < 16, "ltb_upload: bad argument");
  LTB_REQUIRE(!g.capturing, "ltb_upload: not allowed while recording a step");
  filter_cache_note_write(dst, bytes);
  { int rc_ = grad_settle(dst, bytes); if (rc_) return rc_; }
  if (after >= 0 && marker_set[after]) LTB_CUDA(cudaStreamWaitEvent(g.copy, marker_ev[after], 0));
  if (bytes) LTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g.copy));
  return LTB_OK;
}
int ltb_upload_marker(int slot) {
  LTB_INITED(); LTB_REQUIRE(slot >= 0 && slot < 16, "ltb_upload_marker: slot %d out of range", slot);
  if (!marker_ev[slot]) LTB_CUDA(cudaEventCreateWithFlags(&marker_ev[slot], cudaEventDisableTiming));
  LTB_CUDA(cudaEventRecord(marker_ev[slot], g.copy));
  marker_set[slot] = true;
  return LTB_OK;
}
int ltb_stream_wait_marker(int slot) {
  LTB_INITED(); LTB_REQUIRE(slot >= 0 && slot < 16, "ltb_stream_wait_marker: slot %d out of range", slot);
  LTB_REQUIRE(!g.capturing, "ltb_stream_wait_marker: not allowed while recording a step");
  if (marker_set[slot]) LTB_CUDA(cudaStreamWaitEvent(g.stream, marker_ev[slot], 0));
  return LTB_OK;
}
int ltb_marker_wait(int slot) {
  LTB_INITED_NOFLUSH(); LTB_REQUIRE(slot >= 0 && slot < 16, "ltb_marker_wait: slot %d out of range", slot);
  if (marker_set[slot]) {
    if (comm_active()) return comm_wait_event(marker_ev[slot], "ltb_marker_wait");
    LTB_CUDA(cudaEventSynchronize(marker_ev[slot]));
  }
  return LTB_OK;
}

// ------------------------------------------------------------------ branch regions
// mark: remember this point of the caller's stream.  begin: the calls that follow run on the branch stream, which starts
// from the marked point.  end: back to the caller's stream.  join: the caller's stream waits for the branch.  Between mark
// and join staging blocks are not handed back (a block released by one side could be overwritten by the other side's next
// call while a kernel still reads it); they return with the next ltb_reset.  While the launch profiler is on the four
// calls do nothing, so that every kernel is timed alone.
int ltb_branch_mark(void) {
  LTB_INITED();
  if (g.profiling) return LTB_OK;
  LTB_REQUIRE(!g.branch_marked, "ltb_branch_mark: a branch region is already open");
  LTB_CUDA(cudaEventRecord(g.mark_ev, g.stream));
  g.branch_marked = true; g.branch_ended = false;
  return LTB_OK;
}
int ltb_branch_begin(void) {
  LTB_INITED();
  if (g.profiling && !g.branch_marked) return LTB_OK;
  LTB_REQUIRE(g.branch_marked && !g.in_branch && !g.branch_ended, "ltb_branch_begin: needs ltb_branch_mark first, once per region");
  LTB_CUDA(cudaStreamWaitEvent(g.branch, g.mark_ev, 0));
  g.trunk = g.stream; g.stream = g.branch; g.in_branch = true;
  return LTB_OK;
}
int ltb_branch_end(void) {
  LTB_INITED();
  if (!g.in_branch) { LTB_REQUIRE(g.profiling, "ltb_branch_end: no branch is running"); return LTB_OK; }
  LTB_CUDA(cudaEventRecord(g.branch_done_ev, g.branch));
  g.stream = g.trunk; g.in_branch = false; g.branch_ended = true;
  return LTB_OK;
}
int ltb_branch_join(void) {
  LTB_INITED();
  if (!g.branch_marked) { LTB_REQUIRE(g.profiling, "ltb_branch_join: no branch region is open"); return LTB_OK; }
  LTB_REQUIRE(!g.in_branch, "ltb_branch_join: the branch has not ended");
  if (g.branch_ended) LTB_CUDA(cudaStreamWaitEvent(g.stream, g.branch_done_ev, 0));
  g.branch_marked = g.branch_ended = false;
  return LTB_OK;
}

// ------------------------------------------------------------------ whole-step replay
int ltb_graph_begin(void) {
  LTB_INITED(); LTB_REQUIRE(!g.capturing, "ltb_graph_begin: already recording");
  LTB_REQUIRE(!g.profiling, "ltb_graph_begin: the launch profiler is on (its event pairs cannot be recorded into a step)");
  LTB_REQUIRE(!g.branch_marked && !g.in_branch, "ltb_graph_begin: a branch region is open (ltb_branch_join missing)");
  LTB_CUDA(cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeThreadLocal));
  g.capturing = true; g.capture_launch_base = g.launches;
  return LTB_OK;
}
void* ltb_graph_end(void) {
  if (!g.capturing) { fail(LTB_E_STATE, "ltb_graph_end: not recording"); return nullptr; }
  if (g.pending.kind) flush_pending();             // a held operation belongs to the recorded step
  g.capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(g.stream, &graph);
  if (e != cudaSuccess || !graph) { fail(LTB_E_CUDA, "ltb_graph_end: capture failed: %s", cudaGetErrorString(e)); return nullptr; }
  Graph* G = new Graph();
  G->graph = graph; G->launches = g.launches - g.capture_launch_base;
  g.launches = g.capture_launch_base;      // recording launched nothing
  e = cudaGraphInstantiate(&G->exec, graph, 0);
  if (e != cudaSuccess) { cudaGraphDestroy(graph); delete G; fail(LTB_E_CUDA, "ltb_graph_end: instantiate failed: %s", cudaGetErrorString(e)); return nullptr; }
  return G;
}
int ltb_graph_launch(void* graph) {
  LTB_INITED(); filter_cache_note_write(nullptr, 0); LTB_REQUIRE(graph, "ltb_graph_launch: null graph");
  Graph* G = (Graph*)graph;
  LTB_CUDA(cudaGraphLaunch(G->exec, g.stream));
  g.launches += G->launches;
  return LTB_OK;
}
int ltb_graph_destroy(void* graph) {
  if (!graph) return LTB_OK;
  Graph* G = (Graph*)graph;
  cudaGraphExecDestroy(G->exec); cudaGraphDestroy(G->graph); delete G;
  return LTB_OK;
}

// ------------------------------------------------------------------ built-in launch profiler
// ltb_profile(1) starts timing every kernel launch of the library with a CUDA event pair on the launching stream;
// ltb_profile(0) stops.  ltb_profile_report writes one line per kernel name: "name<TAB>launches<TAB>total_ms".
int ltb_profile(int on) {
  LTB_INITED(); LTB_REQUIRE(!g.capturing, "ltb_profile: not while recording a step");
  if (on) profile_clear();          // a new measurement starts; the records of the last one stay readable until then
  g.profiling = on != 0;
  return LTB_OK;
}
int ltb_profile_report(char* buf, int len) {
  LTB_INITED(); LTB_REQUIRE(buf && len > 0, "ltb_profile_report: bad buffer");
  LTB_CUDA(cudaStreamSynchronize(g.stream));
  std::vector<std::string> names; std::vector<double> ms; std::vector<int64_t> cnt;
  for (auto& r : prof_recs) {
    float t = 0; cudaEventElapsedTime(&t, r.a, r.b);
    size_t i = 0; for (; i < names.size(); ++i) if (names[i] == r.name) break;
    if (i == names.size()) { names.push_back(r.name); ms.push_back(0); cnt.push_back(0); }
    ms[i] += t; cnt[i] += 1;
  }
  std::string out;
  for (size_t i = 0; i < names.size(); ++i) { char line[512]; snprintf(line, sizeof line, "%s\t%lld\t%.6f\n", names[i].c_str(), (long long)cnt[i], ms[i]); out += line; }
  strncpy(buf, out.c_str(), len - 1); buf[len - 1] = 0;
  return (int)out.size() < len ? LTB_OK : LTB_E_LIMIT;
}

// ------------------------------------------------------------------ host-RNG initialisation
// randinit on the reference's GPU backends draws on the CPU and uploads (TensorDslCublas.scala:154-155);
// the stream is glibc rand(), consumed in element order (TensorDslCPU.scala:101-110).
int ltb_randinit(float* x, int64_t n, float scale, int seed) {
  LTB_INITED(); filter_cache_note_write(x, (size_t)(n > 0 ? n : 0) * 4); LTB_REQUIRE(x && n >= 0, "ltb_randinit: bad argument");
  LTB_REQUIRE(!g.capturing, "ltb_randinit: host RNG while recording a step");
  if (seed >= 0) srand((unsigned)seed);
  std::vector<float> h((size_t)n);
  for (int64_t i = 0; i < n; ++i) h[i] = ((float)rand() / RAND_MAX - 0.5f) * scale;
  if (n) LTB_CUDA(cudaMemcpyAsync(x, h.data(), (size_t)n * 4, cudaMemcpyHostToDevice, g.stream));
  LTB_CUDA(cudaStreamSynchronize(g.stream));
  return LTB_OK;
}

}  // extern "C"
