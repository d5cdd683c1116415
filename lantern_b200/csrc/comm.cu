// Data parallelism: NCCL communicator and the gradient all-reduce fused with the SGD update.
//
// The reference is single-GPU (src/out/PLDI19evaluation/run_exp.sh:7 pins one device); this is the one part
// of the library with no counterpart there.  One process per GPU.  NCCL is loaded with dlopen at comm_init so that
// single-GPU users need no NCCL at all and multi-GPU users share whatever libnccl the launcher already loaded.
#include <dlfcn.h>

#include <cstring>

#include "buckets.h"
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
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr;
  cudaEvent_t done[kMaxBuckets] = {};
} nccl;

static int load_nccl() {
  if (nccl.handle) return LTB_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) { nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (nccl.handle) break; }
  if (!nccl.handle) return fail(LTB_E_COMM, "cannot load libnccl.so.2: %s", dlerror());
#define LTB_SYM(field, name) do { *(void**)(&nccl.field) = dlsym(nccl.handle, name); if (!nccl.field) return fail(LTB_E_COMM, "libnccl lacks %s", name); } while (0)
  LTB_SYM(GetUniqueId, "ncclGetUniqueId"); LTB_SYM(CommInitRank, "ncclCommInitRank"); LTB_SYM(CommDestroy, "ncclCommDestroy");
  LTB_SYM(AllReduce, "ncclAllReduce"); LTB_SYM(GetErrorString, "ncclGetErrorString");
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
  return LTB_OK;
}
int ltb_comm_destroy(void) {
  if (nccl.comm) {
    nccl.CommDestroy(nccl.comm); nccl.comm = nullptr;
    cudaStreamDestroy(nccl.comm_stream); cudaEventDestroy(nccl.ready);
    for (auto& e : nccl.done) cudaEventDestroy(e);
  }
  nccl.world = 1; nccl.rank = 0;
  return LTB_OK;
}
int ltb_comm_world(void) { return nccl.world; }

int ltb_allreduce_sum(float* x, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(x && n >= 0, "ltb_allreduce_sum: bad argument");
  if (nccl.world == 1 || n == 0) return LTB_OK;
  LTB_NCCL(nccl.AllReduce(x, x, (size_t)n, ncclFloat, ncclSum, nccl.comm, g.stream));
  return LTB_OK;
}
// Gradient all-reduce fused with the update: the slab is cut into buckets; bucket i is reduced on the communication
// stream while the update kernel of bucket i-1 runs on the compute stream, so only the first reduction and the last
// update are exposed.  Each rank's loss is the mean over its own shard, hence the 1/world factor.
int ltb_allreduce_sgd_step(float* x, float* d, float lr, int64_t n) {
  LTB_INITED(); LTB_REQUIRE(x && d && n >= 0, "ltb_allreduce_sgd_step: bad argument");
  if (nccl.world == 1) return ltb_sgd_step(x, d, lr, n);
  if (n == 0) return LTB_OK;
  int64_t off[kMaxBuckets], cnt[kMaxBuckets];
  const int used = bucket_spans(n, off, cnt);
  LTB_CUDA(cudaEventRecord(nccl.ready, g.stream));
  LTB_CUDA(cudaStreamWaitEvent(nccl.comm_stream, nccl.ready, 0));
  for (int b = 0; b < used; ++b) {
    LTB_NCCL(nccl.AllReduce(d + off[b], d + off[b], (size_t)cnt[b], ncclFloat, ncclSum, nccl.comm, nccl.comm_stream));
    LTB_CUDA(cudaEventRecord(nccl.done[b], nccl.comm_stream));
  }
  float s = -1.0f * lr / (float)nccl.world;
  for (int b = 0; b < used; ++b) {
    LTB_CUDA(cudaStreamWaitEvent(g.stream, nccl.done[b], 0));
    float* xb = x + off[b]; float* db = d + off[b];
    const int64_t n4 = (aligned16(xb) && aligned16(db)) ? cnt[b] / 4 : 0;
    LTB_LAUNCH(sgd_scaled_kernel, grid_for(cnt[b] / 4 + 1, 256), 256, 0, xb, db, s, n4, cnt[b]);
  }
  return LTB_OK;
}

}  // extern "C"
