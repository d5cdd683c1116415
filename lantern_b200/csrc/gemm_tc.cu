// TF32 tensor-core engine for sm_100a: one warp-specialised kernel for every dense contraction of the training step
// (convolution forward / data-grad / weight-grad and gemm), driven by the plans of tc_plan.cpp.
//
//   warp 0      : TMA producer.  One lane issues cp.async.bulk.tensor loads of the A and B boxes of each k-iteration into a
//                 4-stage shared-memory ring; completion is signalled on the stage's "full" mbarrier by byte count.
//   warp 1      : owns the tensor memory (tcgen05.alloc / dealloc) and issues tcgen05.mma.kind::tf32 (M = 128, N = tile
//                 width, K = 8) from one lane, four per stage, accumulating in TMEM; tcgen05.commit releases the stage
//                 ("empty" mbarrier) and finally signals the epilogue.
//   warps 2..9  : epilogue.  Each warp reads its 32-lane quarter of the accumulator with tcgen05.ld (32 columns at a time)
//                 and writes the result: pixel-major for convolutions (a warp store covers 32 consecutive pixels of one
//                 channel: 128 contiguous bytes), row-major for gemm / weight-grad; optional bias, alpha, accumulation,
//                 and atomic accumulation under split-K.
// Activations are NCHW at the boundary.  For 1x1 convolutions on images of 32 pixels or more the pixel index is the
// contiguous one and the activation operand is fed M/N-major (tcgen05 allows it for tf32) straight from the tensor with a
// 4-D tiled tensor map.  R x S convolutions with stride 1 run in tap-loop form from a channels-last copy (one transposing
// pass, see to_rows_tiled_kernel): a TMA box is then a window of whole image rows whose coordinates the tap shifts, and
// zero fill outside the image is the padding.  Smaller images, strided forward convolutions and weight-grads of R x S
// filters are staged as row matrices or unfolded matrices by the helper kernels at the end of this file.
// Every mbarrier wait is bounded: after about a second it records a code in the library's device status word and the CTA
// runs to its normal teardown (TMEM is released on every path).  The single issuing lanes of warps 0 and 1 are rejoined by
// their warps (__syncwarp) before the block-wide barrier, which needs converged warps.
#include <cooperative_groups.h>
#include <cuda.h>

#include <vector>

#include "gemm.cuh"
#include "tc_plan.h"

extern "C" void* ltb_malloc_uninit(size_t bytes);
namespace ltb { void* step_alloc(size_t bytes); }
extern "C" int ltb_free(void* p, size_t bytes);

namespace cg = cooperative_groups;

namespace ltb {

constexpr int kMaxStages = 4;
constexpr int kPartPitch = 129;                    // floats per column of a CTA's partial tile in shared memory (odd: reads along either axis are conflict-free)
constexpr int kTcThreads = 320;                    // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue

struct TcOperandDev {
  int t_div[5], t_mod[5], t_mul[5], k_div[5], k_mod[5], k_mul[5], c_off[5];
  TcWalk walk;                                // the k part as a mixed-radix counter (tc_plan.h)
  int rank, nk;
  uint32_t stage_bytes, desc_lo, desc_hi;     // descriptor without the start address
  uint32_t kstep_off[8];
};
struct TcParams {
  TcOperandDev a, b;
  int M, N, bn, k_iters, k_per_split, epilogue, accumulate, atomic, stages;
  uint32_t idesc;
  float* out; const float* bias; float alpha;
  long long split_stride;      // floats between the result slabs of consecutive clusters of splits (see launch_plan)
  int early_loads;             // the producer fills the ring before the set-up barrier (0: after it)
  int cluster_z;               // splits whose partial results are summed inside the kernel: a thread-block cluster of this many CTAs along z
  long long pix_per_img, img_stride, chan_stride, ld;
  int col_mod, col_mul;        // row-major epilogue: D column n goes to column (n % col_mod) * col_mul + n / col_mod when col_mul != 0
  // Gather mode (gather_src != null): the A operand is not loaded by TMA but collected by the epilogue warps, which are idle
  // during the main loop, straight from an activation tensor src[img][chan][pix] with pix = 4 or 16 (images too small for a
  // 128-byte run of pixels), transposing it on the way into the K-major rows the tensor core reads.
  const float* gather_src; int g_pix, g_chan, g_imgs;
  int* status;
  long long wait_cycles;       // bound of every spin wait, in clock64 ticks (the context's limit, ~1 s by default)
};

// ---- PTX wrappers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when it gave up (the code is recorded, the shared abort flag raised).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code, long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) { *abort_flag = 1; atomicExch(status, code); return false; }
  }
  return true;
}
__device__ __forceinline__ void tma_load(const CUtensorMap* map, uint64_t* bar, void* dst, int rank, const int* c) {
  const uint32_t d = smem_u32(dst), b = smem_u32(bar);
  const uint64_t m = reinterpret_cast<uint64_t>(map);
  if (rank == 2)
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]) : "memory");
  else if (rank == 3)
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]) : "memory");
  else if (rank == 4)
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]) : "memory");
  else
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4]) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Box coordinates of an operand: c[d] = c_off[d] + tile part (fixed for the CTA) + ((kiter / k_div[d]) % k_mod[d]) * k_mul[d].
// The k part is advanced incrementally with additions only: the producer is a single thread, and integer divisions or
// branches per dimension cost it more cycles than the loads it issues.  The plan's TcWalk says what each level of the
// counter adds; the common case (level 0) uses increments kept in registers.
struct BoxWalker {
  int c[5], inc0[5], i0, i1;
  // Start coordinates of both operands, computed by the lanes of one warp in parallel (lane d: coordinate d of A, lane
  // 8 + d: coordinate d of B, lanes 5/6 and 13/14: the counter positions) and handed to lane 0.  Done by a single thread
  // the ten pairs of integer division and remainder cost about 3000 cycles per CTA (measured), as long as a short main loop.
  __device__ static __forceinline__ void init_pair(BoxWalker& wa, BoxWalker& wb, const TcOperandDev& a, const TcOperandDev& b,
                                                   int m_tile, int n_tile, int k0, int lane) {
    const bool second = (lane & 8) != 0;
    const TcOperandDev& o = second ? b : a;
    const int tile = second ? n_tile : m_tile, d = lane & 7;
    int v = 0;
    if (lane < 16 && d < 5) {
      v = o.c_off[d];
      if (o.t_mul[d] != 0) v += ((o.t_div[d] > 1 ? tile / o.t_div[d] : tile) % o.t_mod[d]) * o.t_mul[d];
      if (o.k_mul[d] != 0 && k0 != 0) v += ((o.k_div[d] > 1 ? k0 / o.k_div[d] : k0) % o.k_mod[d]) * o.k_mul[d];
    } else if (lane < 16 && d == 5) v = k0 ? k0 % o.walk.n0 : 0;
    else if (lane < 16 && d == 6) v = k0 ? (k0 / o.walk.n0) % o.walk.n1 : 0;
#pragma unroll
    for (int j = 0; j < 5; ++j) { wa.c[j] = __shfl_sync(0xffffffffu, v, j); wb.c[j] = __shfl_sync(0xffffffffu, v, 8 + j); }
    wa.i0 = __shfl_sync(0xffffffffu, v, 5); wa.i1 = __shfl_sync(0xffffffffu, v, 6);
    wb.i0 = __shfl_sync(0xffffffffu, v, 13); wb.i1 = __shfl_sync(0xffffffffu, v, 14);
#pragma unroll
    for (int j = 0; j < 5; ++j) { wa.inc0[j] = a.walk.inc[0][j]; wb.inc0[j] = b.walk.inc[0][j]; }
  }
  __device__ __forceinline__ void next(const TcOperandDev& o) {
    if (++i0 != o.walk.n0) {
#pragma unroll
      for (int d = 0; d < 5; ++d) c[d] += inc0[d];
    } else {
      i0 = 0;
      int lvl = 1;
      if (++i1 == o.walk.n1) { i1 = 0; lvl = 2; }
#pragma unroll
      for (int d = 0; d < 5; ++d) c[d] += o.walk.inc[lvl][d];
    }
  }
};

// ---- the engine -------------------------------------------------------------------------------------------------------
// Epilogue store helpers: pointers advance by the column stride instead of being recomputed, and the mode (plain, bias,
// accumulate, atomic) is decided outside the 32-element loops, so that a column costs two or three instructions.  With one
// epilogue warp per scheduler every extra dependent instruction is exposed latency.
template <bool FULL>
__device__ __forceinline__ void store_columns(float* p, long long stride, const uint32_t* r, float alpha, const float* bias, int lim, int mode) {
  if (mode == 2) {                               // split-K, default mode: atomic accumulation (the bias pointer is set for split 0 only)
#pragma unroll
    for (int j = 0; j < 32; ++j) { if (FULL || j < lim) atomicAdd(p, alpha * __uint_as_float(r[j]) + (bias ? bias[j] : 0.0f)); p += stride; }
  } else if (mode == 1) {                        // accumulate: all loads first, a load-add-store chain per element would serialise on latency
    // sixteen at a time: thirty-two loads in flight next to the thirty-two accumulator registers spill
#pragma unroll
    for (int h = 0; h < 32; h += 16) {
      float old[16]; const float* q = p;
#pragma unroll
      for (int j = 0; j < 16; ++j) { old[j] = (FULL || h + j < lim) ? *q : 0.0f; q += stride; }
#pragma unroll
      for (int j = 0; j < 16; ++j) { if (FULL || h + j < lim) *p = old[j] + alpha * __uint_as_float(r[h + j]); p += stride; }
    }
  } else if (bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) { if (FULL || j < lim) *p = alpha * __uint_as_float(r[j]) + bias[j]; p += stride; }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) { if (FULL || j < lim) *p = alpha * __uint_as_float(r[j]); p += stride; }
  }
}

// EPI (TcEpilogue) and MODE (0 store, 1 accumulate, 2 atomic accumulate) are compile-time: each launch then carries one
// epilogue instead of six, a third of the instructions -- these CTAs live for a few microseconds and the instruction cache
// starts cold (measured hit rate 66 % with all variants in one kernel).
template <int EPI, int MODE>
__global__ void __launch_bounds__(kTcThreads, 2)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x, n_tile = blockIdx.y;
  const int k_begin = blockIdx.z * P.k_per_split;
  const int k_end = min(P.k_iters, k_begin + P.k_per_split);
  const int n_iter = k_end - k_begin;
  const int stages = P.stages;
  const bool gather = P.gather_src != nullptr;

  // stage buffers, aligned to the 1024-byte swizzle atom
  uint8_t* stage_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t stage_bytes = P.a.stage_bytes + P.b.stage_bytes;

  // Set-up.  The producer warp initialises the barriers and, without waiting for anybody, issues the loads that fill the
  // (empty) ring: the copies are in flight while warp 1 allocates tensor memory and the block meets at the barrier below.
  // Before that barrier nobody but the producer's issuing lane touches an mbarrier.
  BoxWalker wa, wb;
  int issued = 0;
  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
      // a stage is full when the TMA bytes have landed (one arrival with the byte count) and, in gather mode, the eight
      // gathering warps have stored their rows (one arrival each)
      for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], P.gather_src ? 9 : 1); mbar_init(&empty_bar[s], 1); }
      mbar_init(&accum_bar, 1);
      abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    BoxWalker::init_pair(wa, wb, P.a, P.b, m_tile, n_tile, k_begin, lane);
    if (lane == 0) {
      const int first = !P.early_loads ? 0 : n_iter < stages ? n_iter : stages;
      for (; issued < first; ++issued) {
        uint8_t* sa = stage_base + (size_t)issued * stage_bytes; uint8_t* sb = sa + P.a.stage_bytes;
        mbar_expect_tx(&full_bar[issued], gather ? P.b.stage_bytes : stage_bytes);
        if (!gather) { tma_load(&map_a, &full_bar[issued], sa, P.a.rank, wa.c); wa.next(P.a); }
        tma_load(&map_b, &full_bar[issued], sb, P.b.rank, wb.c); wb.next(P.b);
      }
    }
    __syncwarp();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)P.bn) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0 && n_iter > issued) {
      // after a ring filled before the barrier, stage 0 is reused next, in its second round; the first `stages` fills find
      // the ring empty and wait for nobody
      int s = issued == stages ? 0 : issued; uint32_t ph = issued == stages ? 1u : 0u;
      for (int it = issued; it < n_iter; ++it) {
        if (it >= stages && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag, P.status, 1, P.wait_cycles)) break;
        uint8_t* sa = stage_base + (size_t)s * stage_bytes; uint8_t* sb = sa + P.a.stage_bytes;
        mbar_expect_tx(&full_bar[s], gather ? P.b.stage_bytes : stage_bytes);
        if (!gather) { tma_load(&map_a, &full_bar[s], sa, P.a.rank, wa.c); wa.next(P.a); }
        tma_load(&map_b, &full_bar[s], sb, P.b.rank, wb.c); wb.next(P.b);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();          // the idle lanes wait here for the issuing lane: the block-wide barrier below needs converged warps
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      bool ok = true; int s = 0; uint32_t ph = 0;
      // descriptor pieces that do not change: kept in registers so that an MMA costs two additions and the instruction
      uint32_t koa[4], kob[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) { koa[k] = P.a.kstep_off[k] >> 4; kob[k] = P.b.kstep_off[k] >> 4; }
      const uint64_t a_hi = (uint64_t)P.a.desc_hi << 32, b_hi = (uint64_t)P.b.desc_hi << 32;
      const uint32_t a_lo = P.a.desc_lo, b_lo = P.b.desc_lo, idesc = P.idesc, a_bytes = P.a.stage_bytes;
      const uint32_t ring = smem_u32(stage_base);
      for (int it = 0; it < n_iter; ++it) {
        ok = mbar_wait(&full_bar[s], ph, &abort_flag, P.status, 2, P.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = (ring + (uint32_t)s * stage_bytes) >> 4, sb = sa + (a_bytes >> 4);   // in 16-byte units (ring < 256 KB: 14 bits)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t adesc = a_hi | (uint64_t)(a_lo | ((sa + koa[k]) & 0x3FFFu));
          const uint64_t bdesc = b_hi | (uint64_t)(b_lo | ((sb + kob[k]) & 0x3FFFu));
          tc_mma_tf32(tmem_base, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&empty_bar[s]);       // the stage may be refilled once these MMAs have read it
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok) tc_commit(&accum_bar);    // accumulator complete
    }
    __syncwarp();
  } else if (n_iter > 0) {
    // ---- warps 2..9.  In gather mode they first feed the A operand: warp g owns rows 16 g .. 16 g + 15 of the tile (one image
    // of 16 pixels, or four images of 4), lane = channel within the 32-channel block of the k-iteration.  A lane reads its
    // channel's 16 pixels (64 contiguous bytes, or four runs of 16) and stores them down its column of the tile: for a fixed
    // pixel the 32 lanes write one whole 128-byte row (128-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ (r & 7)),
    // so the stores are free of bank conflicts.  The loads of the next two k-iterations are issued before this one is stored.
    if (gather) {
      const int gw = warp - 2, pix = P.g_pix, chan = P.g_chan;
      const long long row0 = (long long)m_tile * 128 + gw * 16;                   // first tile row of this warp, as a pixel index
      const long long img0 = row0 / pix;                                          // its image (pix 16) or first of four (pix 4)
      const int runs = 16 / pix;                                                  // 1 run of 16 floats or 4 runs of 4
      const uint32_t col = (uint32_t)(lane >> 2), sub = (uint32_t)(lane & 3) << 2;
      float4 cur[4], nxt[4], nx2[4];                                             // the loads of two k-iterations are in flight while one is stored
      auto fetch = [&](int it, float4* v) {
        const int c = (k_begin + it) * 32 + lane;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long img = runs == 1 ? img0 : img0 + j;
          const bool ok = c < chan && img < P.g_imgs;
          const float4* src = reinterpret_cast<const float4*>(P.gather_src + (img * chan + c) * pix) + (runs == 1 ? j : 0);
          v[j] = ok ? __ldg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
      fetch(0, cur);
      if (n_iter > 1) fetch(1, nxt);
      int s = 0; uint32_t ph = 0;
      for (int it = 0; it < n_iter; ++it) {
        if (it + 2 < n_iter) fetch(it + 2, nx2);
        bool ok = true;
        if (it >= stages) { if (lane == 0) ok = mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag, P.status, 4, P.wait_cycles); ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0; }
        if (!ok) break;
        uint8_t* sa = stage_base + (size_t)s * stage_bytes + (size_t)gw * 16 * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t r = (uint32_t)(j * 4 + i);                            // row within this warp's sixteen (gw * 16 is a multiple of 8: r & 7 is the swizzle phase)
            *reinterpret_cast<float*>(sa + r * 128 + (((col ^ (r & 7u)) << 4) | sub)) = e[i];
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");             // the tensor core reads shared memory through the async proxy
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full_bar[s])) : "memory");
#pragma unroll
        for (int j = 0; j < 4; ++j) { cur[j] = nxt[j]; nxt[j] = nx2[j]; }
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
    // ---- epilogue: TMEM lane quarter = warp index mod 4; the two warps of a quarter take alternate 32-column chunks
    const int q = warp & 3, half = (warp - 2) >> 2;
    const bool ok = mbar_wait(&accum_bar, 0, &abort_flag, P.status, 3, P.wait_cycles);
    tc_fence_after();
    if (ok) {
      const int n0 = n_tile * P.bn;
      const float alpha = P.alpha;
      constexpr int mode = MODE;
      const uint32_t tmem_row = tmem_base + ((uint32_t)(q * 32) << 16);
      float* const out_base = P.out + (long long)(blockIdx.z / P.cluster_z) * P.split_stride;   // a cluster of splits writes its own slab of partial results
      if (P.cluster_z > 1) {
        // Split-K inside a cluster: the accumulator goes to this CTA's shared memory (the pipeline stages are idle by now);
        // the cluster then adds the tiles up (below, after the block has met).  The tile is laid out so that the reads of
        // that sum run along contiguous addresses (reads from another SM's shared memory are slow when scattered):
        // part[column][row] for the pixel-major epilogue, part[row][column] for the row-major one, odd pitches.
        float* part = reinterpret_cast<float*>(stage_base);
        const int row = q * 32 + lane, rp = P.bn + 1;
        for (int c0 = half * 32; c0 < P.bn; c0 += 64) {
          uint32_t r[32];
          tc_ld32(tmem_row + (uint32_t)c0, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) part[EPI == TC_EPI_PIXEL ? (c0 + j) * kPartPitch + row : row * rp + c0 + j] = __uint_as_float(r[j]);
        }
      } else if (EPI == TC_EPI_PIXEL) {
        // lane = pixel, register j = channel: for a fixed j a warp covers 32 consecutive pixels (128 contiguous bytes)
        const long long m = (long long)m_tile * 128 + q * 32 + lane;
        const long long cs = P.chan_stride;
        float* dst = m < P.M ? out_base + (m / P.pix_per_img) * P.img_stride + (m % P.pix_per_img) : nullptr;
        for (int c0 = half * 32; c0 < P.bn; c0 += 64) {
          if (n0 + c0 >= P.N) break;                         // uniform across the warp
          uint32_t r[32];
          tc_ld32(tmem_row + (uint32_t)c0, r);
          if (dst) {
            const int lim = P.N - n0 - c0;
            const float* bias = (P.bias && (!P.atomic || blockIdx.z == 0)) ? P.bias + n0 + c0 : nullptr;
            if (lim >= 32) store_columns<true>(dst + (long long)(n0 + c0) * cs, cs, r, alpha, bias, 32, mode);
            else store_columns<false>(dst + (long long)(n0 + c0) * cs, cs, r, alpha, bias, lim, mode);
          }
        }
      } else {
        // row-major output: transpose each 32x32 block through shared memory so that a warp writes 32 consecutive columns
        // of one row (128 contiguous bytes) per instruction.  The staging tile lives in the pipeline stages, which are idle
        // once the accumulator is complete (every load has landed and every MMA has read its operands).
        float (*tile)[33] = reinterpret_cast<float (*)[33]>(stage_base + (size_t)(warp - 2) * 32 * 33 * 4);
        const long long m0 = (long long)m_tile * 128 + q * 32;
        const int rows = (int)min(32ll, (long long)P.M - m0);
        const long long ld = P.ld;
        for (int c0 = half * 32; c0 < P.bn; c0 += 64) {
          if (n0 + c0 >= P.N) break;
          uint32_t r[32];
          tc_ld32(tmem_row + (uint32_t)c0, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) tile[lane][j] = __uint_as_float(r[j]);
          __syncwarp();
          const int n = n0 + c0 + lane;
          const long long col = P.col_mul ? (long long)(n % P.col_mod) * P.col_mul + n / P.col_mod : n;
          if (n < P.N && rows > 0) {
            uint32_t t[32];
#pragma unroll
            for (int rr = 0; rr < 32; ++rr) t[rr] = __float_as_uint(tile[rr][lane]);
            // after the transpose the "columns" of store_columns are the 32 rows of this block, `ld` apart
            const float* bias = nullptr;
            float* p = out_base + m0 * ld + col;
            if (P.bias && mode == 0) {
              const float bv = P.bias[n];
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) { if (rr < rows) *p = alpha * __uint_as_float(t[rr]) + bv; p += ld; }
            } else if (rows == 32) store_columns<true>(p, ld, t, alpha, bias, 32, mode);
            else store_columns<false>(p, ld, t, alpha, bias, rows, mode);
          }
          __syncwarp();
        }
      }
    }
  }
  if (P.cluster_z > 1 && n_iter <= 0 && warp >= 2) {
    // a split without k-iterations (the split count was rounded up to the cluster size) contributes zeros
    float* part = reinterpret_cast<float*>(stage_base);
    const int part_floats = EPI == TC_EPI_PIXEL ? P.bn * kPartPitch : 128 * (P.bn + 1);
    for (int i = threadIdx.x - 64; i < part_floats; i += kTcThreads - 64) part[i] = 0.0f;
  }
  tc_fence_before();
  __syncthreads();
  if (P.cluster_z > 1) {
    // ---- the cluster sums its partial tiles in a fixed order.  The hardware cluster barrier is safe to wait at: the CTAs
    // of a cluster are scheduled together.  CTA number zr of the cluster owns a slice of the tile -- columns for the
    // pixel-major epilogue, rows for the row-major one, so that its global stores coalesce -- reads that slice from the
    // shared memory of every CTA of the cluster, rank 0 first, and writes the result the way the epilogue would.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (warp >= 2 && !abort_flag) {
      const int cz = P.cluster_z, zr = (int)cluster.block_rank();
      float* part = reinterpret_cast<float*>(stage_base);
      const float* remote[8];
#pragma unroll
      for (int z = 0; z < 8; ++z) remote[z] = z < cz ? cluster.map_shared_rank(part, z) : part;
      const int t = threadIdx.x - 64;                                  // 0 .. 255
      const int n0 = n_tile * P.bn;
      float* const out_base = P.out + (long long)(blockIdx.z / cz) * P.split_stride;
      const float alpha = P.alpha;
      // Eight outputs at a time per thread: their partial tiles are read and, when the destination is accumulated into, its
      // old values loaded, all before the first store (a load-add-store chain per element would pay the memory latency
      // once per element).
      const bool acc = MODE == 1;
      if (EPI == TC_EPI_PIXEL) {
        const int cpc = (P.bn + cz - 1) / cz, c_lo = zr * cpc + (t >> 7), c_hi = min(min(P.bn, zr * cpc + cpc), P.N - n0);
        const int row = t & 127;
        const long long m = (long long)m_tile * 128 + row;
        if (m < P.M) {
          float* dst = out_base + (m / P.pix_per_img) * P.img_stride + (m % P.pix_per_img) + (long long)n0 * P.chan_stride;
          for (int cb = c_lo; cb < c_hi; cb += 16) {                   // this thread's columns cb, cb + 2, ..., cb + 14
            float v[8], old[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = cb + 2 * u; v[u] = 0.0f; old[u] = 0.0f;
              if (c < c_hi) {
#pragma unroll
                for (int z = 0; z < 8; ++z) if (z < cz) v[u] += remote[z][c * kPartPitch + row];
                if (acc) old[u] = dst[(long long)c * P.chan_stride];
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = cb + 2 * u;
              if (c < c_hi) dst[(long long)c * P.chan_stride] = old[u] + alpha * v[u] + (P.bias ? P.bias[n0 + c] : 0.0f);
            }
          }
        }
      } else {
        // rows of the slice go round the eight warps, a lane takes every 32nd column: a warp's stores cover 128 contiguous bytes
        const int rpc = (128 + cz - 1) / cz, r_lo = zr * rpc, r_hi = min(min(128, r_lo + rpc), (int)min(128ll, (long long)P.M - (long long)m_tile * 128));
        const int w = t >> 5, cchunks = P.bn >> 5, cshift = cchunks == 4 ? 2 : cchunks == 2 ? 1 : 0;
        const int n_rows = r_hi - r_lo - w > 0 ? (r_hi - r_lo - w + 7) / 8 : 0, items = n_rows << cshift;
        for (int ib = 0; ib < items; ib += 8) {
          float v[8], old[8]; float* o[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = ib + u; v[u] = 0.0f; old[u] = 0.0f; o[u] = nullptr;
            const int row = r_lo + w + 8 * (i >> cshift), c = ((i & (cchunks - 1)) << 5) + lane, n = n0 + c;
            if (i < items && n < P.N) {
#pragma unroll
              for (int z = 0; z < 8; ++z) if (z < cz) v[u] += remote[z][row * (P.bn + 1) + c];
              const long long col = P.col_mul ? (long long)(n % P.col_mod) * P.col_mul + n / P.col_mod : n;
              o[u] = out_base + ((long long)m_tile * 128 + row) * P.ld + col;
              if (acc) old[u] = *o[u];
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) if (o[u]) *o[u] = old[u] + alpha * v[u];
        }
      }
    }
    cluster.sync();                // no CTA leaves while its shared memory may still be read
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P.bn) : "memory");
  }
}

// ---- unfold / fold helpers for convolutions that are not 1x1 stride 1 ---------------------------------------------------
// col[n][(c*R+r)*S+s][p] = x[n][c][ho*sh-ph+r][wo*sw-pw+s] (0 outside): the reference's `finput` (TensorDslCPU.scala:484-530).
// A thread owns one output pixel of one input plane (n, c) and writes all R*S taps of it: the plane and pixel
// decomposition (the only integer divisions) is paid once per R*S elements, the writes of a warp stay contiguous.
__global__ void unfold_rows_kernel(const float* __restrict__ x, float* __restrict__ col, ConvDims d, int planes_per_block, int threads_per_plane) {
  const int pix = d.oH * d.oW, rs = d.R * d.S;
  const int64_t planes = (int64_t)d.N * d.C;
  const int lane_p = threadIdx.x % threads_per_plane;
  for (int64_t plane = (int64_t)blockIdx.x * planes_per_block + threadIdx.x / threads_per_plane; plane < planes;
       plane += (int64_t)gridDim.x * planes_per_block) {
  const float* src = x + plane * (int64_t)d.H * d.W;
  float* dst = col + plane * rs * pix;                         // rows (c*R + r)*S + s of image n are consecutive
  for (int p = lane_p; p < pix; p += threads_per_plane) {
    const int ho = p / d.oW, wo = p - ho * d.oW;
    const int ih0 = ho * d.sh - d.ph, iw0 = wo * d.sw - d.pw;
    float* q = dst + p;
    for (int r = 0; r < d.R; ++r) {
      const int ih = ih0 + r;
      const bool row_ok = ih >= 0 && ih < d.H;
      for (int s = 0; s < d.S; ++s) {
        const int iw = iw0 + s;
        *q = (row_ok && iw >= 0 && iw < d.W) ? src[ih * d.W + iw] : 0.0f;
        q += pix;
      }
    }
  }
  }
}
// The same values written as the K-major row matrix col[(n*pix + p)][k] (for images too small to be fed M/N-major).
__global__ void unfold_to_rows_kernel(const float* __restrict__ x, float* __restrict__ col, ConvDims d, int64_t total) {
  const int pix = d.oH * d.oW, rs = d.R * d.S, ck = d.C * rs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int k = (int)(i % ck); int64_t t = i / ck; int p = (int)(t % pix); int n = (int)(t / pix);
    int c = k / rs, r = (k % rs) / d.S, s = k % d.S;
    int ih = (p / d.oW) * d.sh - d.ph + r, iw = (p % d.oW) * d.sw - d.pw + s;
    col[i] = (ih >= 0 && ih < d.H && iw >= 0 && iw < d.W) ? x[(((int64_t)n * d.C + c) * d.H + ih) * d.W + iw] : 0.0f;
  }
}
// The same matrix made by tiles: a CTA takes 32 input channels of one image through shared memory (their planes are one
// contiguous run of x) and writes, for every output pixel, the run of 32 x R*S consecutive floats that those channels own in
// the pixel's row.  For input planes of at most 256 pixels (the strided layers of the last stages: element by element the
// copy of 19 MB took 41 us).
constexpr int kUnfoldTilePix = 256;
__global__ void __launch_bounds__(256) unfold_to_rows_tiled_kernel(const float* __restrict__ x, float* __restrict__ col, ConvDims d) {
  __shared__ float plane[32][kUnfoldTilePix + 1];
  const int n = blockIdx.y, c0 = blockIdx.x * 32, cn = min(32, d.C - c0);
  const int hw = d.H * d.W, pix = d.oH * d.oW, rs = d.R * d.S, ck = d.C * rs;
  const float* src = x + ((int64_t)n * d.C + c0) * hw;
  for (int i = threadIdx.x; i < cn * hw; i += 256) { const int cc = i / hw; plane[cc][i - cc * hw] = src[i]; }
  __syncthreads();
  // a thread owns (channel, tap) and walks the output pixels; when the 32 channels have fewer than 256 (channel, tap) pairs
  // (a 1x1 convolution) the block's threads also share the pixels
  const int per = cn * rs, lanes = per < 256 ? per : 256, ppar = 256 / lanes;
  const int pl = threadIdx.x / lanes, il = threadIdx.x - pl * lanes;
  if (pl >= ppar) return;
  for (int i2 = il; i2 < per; i2 += lanes) {
    const int cc = i2 / rs, t = i2 - cc * rs, r = t / d.S, sx = t - r * d.S;
    float* dst = col + (int64_t)n * pix * ck + (int64_t)c0 * rs + i2;
    for (int p = pl; p < pix; p += ppar) {
      const int ho = p / d.oW, wo = p - ho * d.oW;
      const int ih = ho * d.sh - d.ph + r, iw = wo * d.sw - d.pw + sx;
      dst[(int64_t)p * ck] = (ih >= 0 && ih < d.H && iw >= 0 && iw < d.W) ? plane[cc][ih * d.W + iw] : 0.0f;
    }
  }
}
// [N][chan][pix] -> row matrix [N*pix][chan] (K-major operand for images smaller than one 128-byte row of pixels).
__global__ void to_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int chan, int pix, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int c = (int)(i % chan); int64_t t = i / chan; int p = (int)(t % pix); int64_t n = t / pix;
    dst[i] = src[(n * chan + c) * pix + p];
  }
}
// The same copy through a shared-memory tile of 32 channels x PT pixels (PT = min(pix, 32), pix a multiple of PT, chan a
// multiple of 32), coalesced on both sides.  grid (pix/PT, chan/32, N), block 256.
template <int PT>      // PT == 0: run-time tile width `pt`
__global__ void to_rows_tiled_kernel(const float* __restrict__ src, float* __restrict__ dst, int chan, int pix, int pt_rt) {
  __shared__ float tile[32][33];
  const int pt = PT ? PT : pt_rt;
  const int n = blockIdx.z, p0 = blockIdx.x * pt, c0 = blockIdx.y * 32;
  const float* s = src + ((int64_t)n * chan + c0) * pix + p0;
  for (int i = threadIdx.x; i < 32 * pt; i += blockDim.x) { const int c = i / pt, p = i - c * pt; tile[c][p] = s[(int64_t)c * pix + p]; }
  __syncthreads();
  float* d = dst + ((int64_t)n * pix + p0) * chan + c0;
  for (int i = threadIdx.x; i < 32 * pt; i += blockDim.x) { const int p = i >> 5, c = i & 31; d[(int64_t)p * chan + c] = tile[c][p]; }
}
// Channels-last copy of dy with a zero between neighbouring pixels: up[n][2a][2b][k] = dy[n][k][a][b], 0 elsewhere
// (up is uH x uW pixels).  The data-gradient of a stride-2 convolution is the stride-1 data-gradient of this tensor, so the
// tap-loop plan serves it and no fold-back pass is needed.  K a multiple of 32, oW <= 32.  grid (ceil(uH/2), K/32, N), block 256.
__global__ void to_rows_up2_kernel(const float* __restrict__ dy, float* __restrict__ up, int K, int oH, int oW, int uH, int uW) {
  __shared__ float tile[32][33];
  const int a = blockIdx.x, k0 = blockIdx.y * 32, n = blockIdx.z;
  if (a < oH)
    for (int i = threadIdx.x; i < 32 * oW; i += blockDim.x) {
      const int k = i / oW, b = i - k * oW;
      tile[k][b] = dy[(((int64_t)n * K + k0 + k) * oH + a) * oW + b];
    }
  __syncthreads();
  for (int hu = 2 * a; hu < 2 * a + 2 && hu < uH; ++hu)
    for (int i = threadIdx.x; i < uW * 32; i += blockDim.x) {
      const int wu = i >> 5, k = i & 31;
      float v = 0.0f;
      if (hu == 2 * a && a < oH && !(wu & 1) && (wu >> 1) < oW) v = tile[k][wu >> 1];
      up[(((int64_t)n * uH + hu) * uW + wu) * K + k0 + k] = v;
    }
}
// Filters w[k][c][tap] (OIHW) as one matrix per tap: out[tap][k][c] (by_c == 0, forward) or out[tap][c][k] (data-grad).
__global__ void permute_taps_kernel(const float* __restrict__ w, float* __restrict__ out, int K, int C, int taps, int by_c, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int k, c; const int inner = by_c ? K : C, outer = by_c ? C : K;
    const int a = (int)(i % inner); const int64_t t2 = i / inner; const int b = (int)(t2 % outer); const int t = (int)(t2 / outer);
    if (by_c) { k = a; c = b; } else { c = a; k = b; }
    out[i] = w[((int64_t)k * C + c) * taps + t];
  }
}
// Both per-tap forms, fwd[tap][k][c] and dgrad[tap][c][k], of several filters in one launch (every filter the optimizer has
// just written: one launch per step instead of one per 3x3 layer).  A CTA takes a tile of 32 output channels x 32 input
// channels x all taps of one filter through shared memory: the 32 x (32 taps) floats of a tile are contiguous runs of w, and
// both forms leave as runs of 32 consecutive floats (read element by element, w's stride of `taps` floats between
// neighbouring channels made this copy of 45 MB take 137 us).  Jobs are laid end to end over the tile index.
struct FormJob { const float* w; float* fwd; float* dgrad; int K, C, taps; int begin; };    // begin: first tile of this job
constexpr int kFormJobs = 24;
struct FormJobs { FormJob j[kFormJobs]; int n; int total; };
constexpr int kFormTaps = 9;                                   // filters with more taps go element by element inside their tile
__global__ void __launch_bounds__(256) filter_forms_multi_kernel(const FormJobs J) {
  __shared__ float tile[32][32 * kFormTaps + 1];
  int q = 0;
  while (q + 1 < J.n && (int)blockIdx.x >= J.j[q + 1].begin) ++q;
  const FormJob& f = J.j[q];
  const int K = f.K, C = f.C, taps = f.taps;
  const int ctiles = (C + 31) / 32, id = (int)blockIdx.x - f.begin;
  const int k0 = (id / ctiles) * 32, c0 = (id % ctiles) * 32;
  const int kn = min(32, K - k0), cn = min(32, C - c0);
  if (taps > kFormTaps) {
    for (int i = threadIdx.x; i < kn * cn * taps; i += 256) {
      const int t = i % taps, cc = (i / taps) % cn, kk = i / (taps * cn);
      const float v = f.w[((long long)(k0 + kk) * C + c0 + cc) * taps + t];
      f.fwd[((long long)t * K + k0 + kk) * C + c0 + cc] = v;
      f.dgrad[((long long)t * C + c0 + cc) * K + k0 + kk] = v;
    }
    return;
  }
  const int run = cn * taps;                                   // floats of one output channel's row inside the tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int kk = warp; kk < kn; kk += 8) {                      // a warp per row of the tile: no index arithmetic per element
    const float* src = f.w + ((long long)(k0 + kk) * C + c0) * taps;
    for (int r = lane; r < run; r += 32) tile[kk][r] = src[r];
  }
  __syncthreads();
  // both forms leave as rows of up to 32 consecutive floats, a warp per row: fwd[t][k][c0 ..] and dgrad[t][c][k0 ..]
  for (int row = warp; row < taps * kn; row += 8) {
    const int t = row / kn, kk = row - t * kn;
    if (lane < cn) f.fwd[((long long)t * K + k0 + kk) * C + c0 + lane] = tile[kk][lane * taps + t];
  }
  for (int row = warp; row < taps * cn; row += 8) {
    const int t = row / cn, cc = row - t * cn;
    if (lane < kn) f.dgrad[((long long)t * C + c0 + cc) * K + k0 + lane] = tile[lane][cc * taps + t];
  }
}
// Filter matrix w[rows][cols] copied with its rows padded by zeros to ld floats (the engine's tensor maps want a row length
// of 4 floats for K-major and 32 floats for N-major operands; 3x3 filters over 3 or 16 channels have 27 or 144).
__global__ void pad_rows_kernel(const float* __restrict__ w, float* __restrict__ out, int cols, int ld, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % ld); const int64_t r = i / ld;
    out[i] = c < cols ? w[r * cols + c] : 0.0f;
  }
}
// dx[n][c][h][w] += sum over the (r,s) taps that reach (h,w): gather form of unfoldedAcc (TensorDslCPU.scala:647-692).
// One block row per (n, c) plane; the tap loops run over at most R*S entries of the unfolded gradient.
// STRIDE 1 and 2 avoid the per-tap division and remainder (0 = any stride).
template <int STRIDE>
__global__ void fold_acc_kernel(const float* __restrict__ col, float* dx, ConvDims d, int planes_per_block, int threads_per_plane) {
  const int pix = d.oH * d.oW, hw = d.H * d.W;
  const int64_t planes = (int64_t)d.N * d.C;
  const int lane_p = threadIdx.x % threads_per_plane;
  for (int64_t plane = (int64_t)blockIdx.x * planes_per_block + threadIdx.x / threads_per_plane; plane < planes;
       plane += (int64_t)gridDim.x * planes_per_block) {
  const float* src = col + plane * d.R * d.S * pix;          // rows (c*R + r)*S + s of image n start here
  float* dst = dx + plane * hw;
  for (int i = lane_p; i < hw; i += threads_per_plane) {
    const int h = i / d.W, w = i - h * d.W;
    float acc = 0.0f;
    for (int r = 0; r < d.R; ++r) {
      const int hs = h + d.ph - r;
      if (hs < 0) continue;
      int ho;
      if (STRIDE == 1) ho = hs;
      else if (STRIDE == 2) { if (hs & 1) continue; ho = hs >> 1; }
      else { if (hs % d.sh) continue; ho = hs / d.sh; }
      if (ho >= d.oH) continue;
      for (int s = 0; s < d.S; ++s) {
        const int ws = w + d.pw - s;
        if (ws < 0) continue;
        int wo;
        if (STRIDE == 1) wo = ws;
        else if (STRIDE == 2) { if (ws & 1) continue; wo = ws >> 1; }
        else { if (ws % d.sw) continue; wo = ws / d.sw; }
        if (wo >= d.oW) continue;
        acc += src[(r * d.S + s) * pix + ho * d.oW + wo];
      }
    }
    if (acc != 0.0f || STRIDE == 1) dst[i] += acc;
  }
  }
}

// ---- split-K beyond one cluster: the slabs of partial results are summed in a fixed order -----------------------------------
// out[i] (+)= alpha * sum over the slabs of ws[slab][i] (+ bias of i's channel).  A CTA owns 128 consecutive outputs (32
// float4 per warp row); its eight warps each add every eighth slab, in order, and warp 0 adds the eight partial sums, in
// order: the association is fixed, so the result has the same bits on every run (sums combined by atomics do not).  The
// slabs have the layout of the output itself.  chan_div / chan_mod locate the bias entry: channel = (i / chan_div) % chan_mod.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, int slabs, long long slab, float* out, long long n, float alpha, int accumulate,
                                                            const float* __restrict__ bias, long long chan_div, int chan_mod, int vec) {
  __shared__ float4 partial[8][32];
  const int lane = threadIdx.x & 31, zl = threadIdx.x >> 5;
  const long long base = ((long long)blockIdx.x * 32 + lane) * 4;                  // this lane's four outputs
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (base < n) {
    for (int z = zl; z < slabs; z += 8) {
      const float* p = ws + (long long)z * slab + base;
      float4 b;
      if (vec) b = *reinterpret_cast<const float4*>(p);
      else { b.x = p[0]; b.y = base + 1 < n ? p[1] : 0.f; b.z = base + 2 < n ? p[2] : 0.f; b.w = base + 3 < n ? p[3] : 0.f; }
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
  }
  partial[zl][lane] = a;
  __syncthreads();
  if (zl != 0 || base >= n) return;
#pragma unroll
  for (int z = 1; z < 8; ++z) { const float4 b = partial[z][lane]; a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
  const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const long long i = base + e;
    if (i >= n) break;
    const float bv = bias ? bias[(i / chan_div) % chan_mod] : 0.0f;
    out[i] = (accumulate ? out[i] : 0.0f) + alpha * v[e] + bv;
  }
}

// ---- host side ----------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled = nullptr;
static bool smem_opted_in = false;

static int encode_map(const TcTensorMap& m, CUtensorMap* out) {
  if (!encode_tiled) {
    void* fn = nullptr; cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return fail(LTB_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    encode_tiled = (EncodeTiledFn)fn;
  }
  cuuint64_t dims[5], strides[4]; cuuint32_t box[5], estr[5];
  for (int d = 0; d < m.rank; ++d) { dims[d] = m.dims[d]; box[d] = m.box[d]; estr[d] = 1; if (d > 0) strides[d - 1] = m.strides[d]; }
  const CUtensorMapSwizzle sw = m.swizzle == TC_SW_128_32B ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                : m.swizzle == TC_SW_128 ? CU_TENSOR_MAP_SWIZZLE_128B : m.swizzle == TC_SW_64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : m.swizzle == TC_SW_32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)m.rank, const_cast<void*>(m.base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LTB_E_CUDA, "cuTensorMapEncodeTiled failed with code %d (rank %d, inner box %u)", (int)r, m.rank, m.box[0]);
  return LTB_OK;
}

static bool to_dev(const TcOperand& o, TcOperandDev& v) {
  for (int d = 0; d < 5; ++d) {
    v.t_div[d] = o.t_div[d]; v.t_mod[d] = o.t_mod[d]; v.t_mul[d] = o.t_mul[d];
    v.k_div[d] = o.k_div[d]; v.k_mod[d] = o.k_mod[d]; v.k_mul[d] = o.k_mod[d] > 1 ? o.k_mul[d] : 0; v.c_off[d] = o.c_off[d];
  }
  if (!tc_walk_of(o, v.walk)) return false;
  v.rank = o.map.rank; v.nk = o.nk; v.stage_bytes = o.stage_bytes;
  // UMMA layout type: 0 none, 1 128-byte swizzle with 32-byte atoms (M/N-major 32-bit operands), 2 128 B, 4 64 B, 6 32 B
  const uint32_t layout = o.map.swizzle == TC_SW_128_32B ? 1u : o.map.swizzle == TC_SW_128 ? 2u : o.map.swizzle == TC_SW_64 ? 4u : o.map.swizzle == TC_SW_32 ? 6u : 0u;
  v.desc_lo = ((o.lbo >> 4) & 0x3FFFu) << 16;                                     // leading byte offset, bits [16,30)
  v.desc_hi = ((o.sbo >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);             // stride byte offset [32,46), version 1 at [46,48), layout [61,64)
  for (int i = 0; i < 8; ++i) v.kstep_off[i] = o.kstep_off[i];
  return true;
}

static void temp_free(float* p, size_t floats);
static float* temp_alloc(size_t floats);

static int launch_plan(const TcPlan& p, const char* label) {
  CUtensorMap ma, mb;
  int rc = encode_map(p.a.map, &ma); if (rc) return rc;
  rc = encode_map(p.b.map, &mb); if (rc) return rc;
  TcParams P;
  if (!to_dev(p.a, P.a) || !to_dev(p.b, P.b)) return fail(LTB_E_STATE, "tensor-core plan whose k-iteration order has no incremental walk");
  P.M = p.M; P.N = p.N; P.bn = p.bn; P.k_iters = p.k_iters;
  // Split-K: up to eight splits of a tile form a thread-block cluster and add their partial tiles up inside the kernel
  // (through distributed shared memory, in a fixed order).  More than eight splits: every cluster of eight writes a slab of
  // partial results (a staging block with the layout of the output) and one more launch adds the slabs up, again in a fixed
  // order, and applies alpha, bias and accumulation.  No atomics, no zero fill, the same bits on every run.
  // That is the deterministic mode (ltb_set_deterministic): measured, it costs the contraction kernels about a third more
  // time (cluster barriers, partial tiles through shared memory).  By default the splits add their tiles into the output
  // atomically, as cuDNN's default algorithms do: faster, and the last bits of a sum depend on the order of arrival.
  int splits = p.splits < 1 ? 1 : p.splits, cz = 1, nslabs = 1;
  const bool atomic = splits > 1 && !g.deterministic;
  if (splits > 1 && !atomic) {
    cz = splits <= 2 ? 2 : splits <= 4 ? 4 : 8;
    nslabs = (int)ceil_div(splits, cz);
  }
  const size_t out_floats = p.epilogue == TC_EPI_PIXEL ? (size_t)ceil_div(p.M, p.pix_per_img ? p.pix_per_img : 1) * (size_t)p.img_stride : (size_t)p.M * (size_t)p.ld;
  float* ws = nullptr;
  if (nslabs > 1) {
    ws = temp_alloc((size_t)nslabs * out_floats);
    if (!ws) nslabs = 1;                                                           // no room for the slabs: one cluster per tile
  }
  if (!atomic) splits = nslabs * cz;
  P.k_per_split = (int)ceil_div(p.k_iters, splits);                                // a split may end up without iterations: it contributes zeros
  if (atomic) splits = (int)ceil_div(p.k_iters, P.k_per_split);                    // atomic mode: only splits that have work
  P.cluster_z = cz; P.early_loads = (g.tune & 8) ? 0 : 1;
  P.epilogue = p.epilogue; P.accumulate = ws ? 0 : p.accumulate; P.atomic = atomic ? 1 : 0;
  if (atomic && !p.accumulate) LTB_CUDA(cudaMemsetAsync(p.out, 0, out_floats * 4, g.stream));     // overwrite semantics: start from zero, then add
  // tf32 x tf32 -> f32: D format 1 at [4,6), A/B format 2 at [7,10)/[10,13), major bits 15/16, N>>3 at [17,23), M>>4 at [24,29)
  P.idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)p.a.mn_major << 15) | ((uint32_t)p.b.mn_major << 16) | ((uint32_t)(p.bn >> 3) << 17) | ((128u >> 4) << 24);
  P.out = ws ? ws : p.out; P.bias = ws ? nullptr : p.bias; P.alpha = ws ? 1.0f : p.alpha; P.split_stride = ws ? (long long)out_floats : 0;
  P.pix_per_img = p.pix_per_img ? p.pix_per_img : 1; P.img_stride = p.img_stride; P.chan_stride = p.chan_stride; P.ld = p.ld; P.col_mod = p.col_mod ? p.col_mod : 1; P.col_mul = p.col_mul;
  P.gather_src = p.gather_src; P.g_pix = p.g_pix; P.g_chan = p.g_chan; P.g_imgs = p.g_imgs;
  P.status = g.dev_status; P.wait_cycles = g.wait_limit_cycles;
  // 4 stages, except 3 for 128-wide tiles so that two CTAs (2 x 97 KB) share an SM and one's epilogue overlaps the other's main loop
  P.stages = p.bn == 128 ? 3 : kMaxStages;
  const size_t smem = (size_t)P.stages * (p.a.stage_bytes + p.b.stage_bytes) + 1024;
  if (cz > 1 && (size_t)128 * (p.bn + 1) * 4 > smem - 1024) return fail(LTB_E_STATE, "tensor-core plan whose partial tile does not fit the pipeline stages");
  if (!smem_opted_in) {
    const int max_smem = kMaxStages * (16384 + 32768) + 1024;
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    LTB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    smem_opted_in = true;
  }
  const int mode = atomic ? 2 : (P.accumulate ? 1 : 0);
  void (*kernel)(const CUtensorMap, const CUtensorMap, const TcParams) =
      p.epilogue == TC_EPI_PIXEL ? (mode == 2 ? tc_gemm_kernel<TC_EPI_PIXEL, 2> : mode == 1 ? tc_gemm_kernel<TC_EPI_PIXEL, 1> : tc_gemm_kernel<TC_EPI_PIXEL, 0>)
                                 : (mode == 2 ? tc_gemm_kernel<TC_EPI_ROWMAJOR, 2> : mode == 1 ? tc_gemm_kernel<TC_EPI_ROWMAJOR, 1> : tc_gemm_kernel<TC_EPI_ROWMAJOR, 0>);
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.m_tiles, p.n_tiles, splits); cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = smem; cfg.stream = g.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)cz;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (g.profiling) profile_before(label);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, P);
    if (g.profiling) profile_after();
    ++g.launches;
    if (e != cudaSuccess) return fail(LTB_E_CUDA, "launch of the tensor-core engine failed: %s (grid %d x %d x %d, cluster %d)", cudaGetErrorString(e), p.m_tiles, p.n_tiles, splits, cz);
  }
  if (ws) {
    const bool pixel = p.epilogue == TC_EPI_PIXEL;
    const long long chan_div = pixel ? (long long)(p.pix_per_img ? p.pix_per_img : 1) : 1;
    const int chan_mod = pixel ? p.N : (int)(p.ld > 0 ? p.ld : 1);
    const int vec = aligned16(ws) && out_floats % 4 == 0 ? 1 : 0;
    const unsigned grid_r = (unsigned)ceil_div((int64_t)out_floats, 128);
    LTB_LAUNCH(splitk_reduce_kernel, grid_r, 256, 0, (const float*)ws, nslabs, (long long)out_floats, p.out, (long long)out_floats, p.alpha, p.accumulate, p.bias, chan_div, chan_mod, vec);
    temp_free(ws, (size_t)nslabs * out_floats);
  }
  return LTB_OK;
}

// Self-test of the bounded wait: one warp waits, through the engine's own mbar_wait, on a barrier at which nothing ever
// arrives.  No copy is in flight and no tensor memory is held, so when the limit runs out the kernel simply records code 9
// in the status word and returns; the context stays usable.
__global__ void wait_selftest_kernel(int* status, long long limit) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, status, 9, limit);
  __syncthreads();
}

}  // namespace ltb
extern "C" {
int ltb_set_wait_limit(int64_t cycles) {
  LTB_INITED(); LTB_REQUIRE(cycles > 0, "ltb_set_wait_limit: the limit must be positive");
  ltb::g.wait_limit_cycles = cycles; return LTB_OK;
}
int ltb_selftest_bounded_wait(int64_t cycles) {
  LTB_INITED(); LTB_REQUIRE(cycles > 0 && cycles <= 4000000000ll, "ltb_selftest_bounded_wait: limit out of range (1 .. 4e9 cycles)");
  LTB_LAUNCH(ltb::wait_selftest_kernel, 1, 32, 0, ltb::g.dev_status, (long long)cycles);
  return LTB_OK;
}
}
namespace ltb {

int gemm_tc(const float* a, bool a_kmajor, const float* b, bool b_kmajor, float* c, bool, int M, int N, int K, float alpha, bool accumulate) {
  TcPlan p;
  if (!tc_plan_gemm(p, a, a_kmajor, b, b_kmajor, c, M, N, K, alpha, accumulate, g.sm_count)) return 0;
  int rc = launch_plan(p, "tc_gemm_kernel[gemm]");
  return rc ? rc : 1;
}

// ---- channels-last copies of activations ---------------------------------------------------------------------------------------
// The tap-loop convolutions read act[n][h][w][c].  Without the operand cache (ltb_set_filter_cache) every call makes its own
// copy in a staging block and gives it back.  With it, a copy made by a forward convolution, or of dy at the start of a
// convolution's backward call, is kept in a block taken from the far end of the arena (those blocks live until ltb_reset)
// and found again by address and shape: the weight-gradient of that convolution reads the forward copy of x, and data-grad
// and weight-grad share one copy of dy.  A copy is dropped when one of the entry points that report their writes
// (filter_cache_note_write) touches its source, when ltb_free releases the source, and at ltb_reset.
struct ClCopy { const float* src; int n_img, chan, pix; float* cl; int geom; };   // geom 0: channels-last copy; else the key of an unfolded matrix (unfold_key)
static std::vector<ClCopy> cl_cache;
void cl_cache_clear() { cl_cache.clear(); }
void cl_cache_drop_from(const void* p) {                   // ltb_free: everything at or above p is gone
  for (size_t i = 0; i < cl_cache.size();) { if ((const void*)cl_cache[i].src >= p) { cl_cache[i] = cl_cache.back(); cl_cache.pop_back(); } else ++i; }
}
static float* cl_lookup(const float* src, int n_img, int chan, int pix) {
  for (auto& e : cl_cache) if (e.src == src && e.n_img == n_img && e.chan == chan && e.pix == pix && e.geom == 0) return e.cl;
  return nullptr;
}
// The unfolded matrix col[n][(c, r, s)][p] of a convolution input (the forward pass of a strided or 3-channel convolution
// makes it, the weight gradient of the same convolution reads it again): kept and found like the channels-last copies.
static int unfold_key(const ConvDims& d) { return 1 + ((((((d.R * 8 + d.S) * 4 + d.sh) * 4 + d.sw) * 8 + d.ph) * 8 + d.pw) * 64 + d.W % 64); }
static float* unfold_lookup(const float* src, const ConvDims& d) {
  const int ck = d.C * d.R * d.S, pix = d.oH * d.oW, key = unfold_key(d);
  for (auto& e : cl_cache) if (e.src == src && e.n_img == d.N && e.chan == ck && e.pix == pix && e.geom == key) return e.cl;
  return nullptr;
}
static int launch_unfold(const float* x, float* col, const ConvDims& d) {
  const int pix = d.oH * d.oW;
  int tpp = 4; while (tpp < pix && tpp < 256) tpp <<= 1;       // threads per input plane: a power of two in [4, 256] (4 x 4 and 2 x 2 outputs leave no lane idle)
  const int ppb = 256 / tpp;
  const int64_t planes = (int64_t)d.N * d.C;
  LTB_LAUNCH(unfold_rows_kernel, grid_for(ceil_div(planes, ppb) * 256, 256, 16), 256, 0, x, col, d, ppb, tpp);
  return LTB_OK;
}
// 1x1 convolution with stride 2 and no padding (ResNet's downsampling branch): every gradient element goes to exactly
// one input pixel, dx[n][c][2a][2b] += col[n][c][a][b]; a thread per element of col.
__global__ void fold_1x1_s2_kernel(const float* __restrict__ col, float* dx, int oH, int oW, int H, int W, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(i % oW); const int64_t t = i / oW; const int a = (int)(t % oH); const int64_t plane = t / oH;
    dx[(plane * H + 2 * a) * W + 2 * b] += col[i];
  }
}
static int launch_fold(const float* col, float* dx, const ConvDims& d) {
  const int hw = d.H * d.W;
  int tpp = 32; while (tpp < hw && tpp < 256) tpp <<= 1;
  const int ppb = 256 / tpp;
  const int64_t planes = (int64_t)d.N * d.C;
  const unsigned grid = (unsigned)grid_for(ceil_div(planes, ppb) * 256, 256, 16);
  if (d.R == 1 && d.S == 1 && d.sh == 2 && d.sw == 2 && d.ph == 0 && d.pw == 0) {
    const int64_t total = planes * d.oH * d.oW;
    LTB_LAUNCH(fold_1x1_s2_kernel, grid_for(total, 256), 256, 0, col, dx, d.oH, d.oW, d.H, d.W, total);
    return LTB_OK;
  }
  if (d.sh == 1 && d.sw == 1) LTB_LAUNCH(fold_acc_kernel<1>, grid, 256, 0, col, dx, d, ppb, tpp);
  else if (d.sh == 2 && d.sw == 2) LTB_LAUNCH(fold_acc_kernel<2>, grid, 256, 0, col, dx, d, ppb, tpp);
  else LTB_LAUNCH(fold_acc_kernel<0>, grid, 256, 0, col, dx, d, ppb, tpp);
  return LTB_OK;
}
static bool is_pointwise(const ConvDims& d) { return d.R == 1 && d.S == 1 && d.sh == 1 && d.sw == 1 && d.ph == 0 && d.pw == 0; }
// Staging blocks go back to the arena (a LIFO pop, host arithmetic only) unless the caller holds them: conv backward runs
// its two halves on two streams and pops both halves' blocks together once both are issued.
// Nor inside a branch region (ltb_branch_mark .. ltb_branch_join): the other stream's next call would reuse the block.
static void temp_free(float* p, size_t floats) { if (!g.hold_workspace && !g.branch_marked) ltb_free(p, floats * 4); }
static float* temp_alloc(size_t floats) {
  size_t bytes = (floats * 4 + kGranule - 1) / kGranule * kGranule;
  if (g.used + bytes + g.top_used > g.heap_bytes) return nullptr;   // no room for the staging buffer: let the FP32 path run
  return (float*)ltb_malloc_uninit(floats * 4);
}
// Stages the activation operand of forward / data-grad for the engine.  `src` is [N][chan][pix] when no unfolding is needed
// (unfold == false), else the convolution input to unfold.  Result: *op points at the operand, *rows tells its form,
// *temp/*temp_floats describe the arena block to release afterwards (null when the tensor is used in place).
static int stage_activation(const float* src, bool unfold, const ConvDims& d, int chan, int pix, const float** op, bool* rows, float** temp, size_t* temp_floats) {
  *rows = tc_conv_needs_rows(pix); *temp = nullptr; *temp_floats = 0; *op = src;
  if (!unfold && (!*rows || pix == 1)) return LTB_OK;         // [N][chan][1] already is the row matrix [N][chan]
  const size_t n = (size_t)d.N * chan * pix;
  if (unfold && !*rows && g.filter_cache && !(g.tune & 4)) {         // keep it for the weight gradient of the same convolution
    if (float* kept = (float*)step_alloc(n * 4)) {
      int rc = launch_unfold(src, kept, d); if (rc) return rc;
      cl_cache.push_back(ClCopy{src, d.N, chan, pix, kept, unfold_key(d)});
      *op = kept;
      return LTB_OK;
    }
  }
  float* buf = temp_alloc(n);
  if (!buf) return 1;
  *temp = buf; *temp_floats = n; *op = buf;
  if (unfold) {
    if (*rows && d.H * d.W <= kUnfoldTilePix && d.N <= 65535) LTB_LAUNCH(unfold_to_rows_tiled_kernel, dim3((unsigned)ceil_div(d.C, 32), (unsigned)d.N), 256, 0, src, buf, d);
    else if (*rows) LTB_LAUNCH(unfold_to_rows_kernel, grid_for((int64_t)n, 256), 256, 0, src, buf, d, (int64_t)n);
    else { int rc = launch_unfold(src, buf, d); if (rc) return rc; }
  } else {
    const int pt = pix < 32 ? pix : 32;
    if (chan % 32 == 0 && pix % pt == 0 && d.N <= 65535)
      { if (pt == 32) LTB_LAUNCH(to_rows_tiled_kernel<32>, dim3(pix / 32, chan / 32, d.N), 256, 0, src, buf, chan, pix, 32);
        else LTB_LAUNCH(to_rows_tiled_kernel<0>, dim3(pix / pt, chan / 32, d.N), 32 * pt < 256 ? 128 : 256, 0, src, buf, chan, pix, pt); }
    else
      LTB_LAUNCH(to_rows_kernel, grid_for((int64_t)n, 256), 256, 0, src, buf, chan, pix, (int64_t)n);
  }
  return LTB_OK;
}

// ---- tap-loop (implicit) path for R x S convolutions with stride 1 ---------------------------------------------------------
static bool taps_geometry(const ConvDims& d, TcConvGeom& gm) {
  if (d.R * d.S == 1 || d.sh != 1 || d.sw != 1) return false;
  gm.n_img = d.N; gm.C = d.C; gm.H = d.H; gm.W = d.W; gm.K = d.K; gm.R = d.R; gm.S = d.S; gm.ph = d.ph; gm.pw = d.pw; gm.oH = d.oH; gm.oW = d.oW;
  return true;
}
static int channels_last_into(const float* src, int n_img, int chan, int pix, float* out) {
  const size_t n = (size_t)n_img * chan * pix;
  const int pt = pix < 32 ? pix : 32;
  if (chan % 32 == 0 && pix % pt == 0 && n_img <= 65535)
    { if (pt == 32) LTB_LAUNCH(to_rows_tiled_kernel<32>, dim3(pix / 32, chan / 32, n_img), 256, 0, src, out, chan, pix, 32);
      else LTB_LAUNCH(to_rows_tiled_kernel<0>, dim3(pix / pt, chan / 32, n_img), 32 * pt < 256 ? 128 : 256, 0, src, out, chan, pix, pt); }
  else
    LTB_LAUNCH(to_rows_kernel, grid_for((int64_t)n, 256), 256, 0, src, out, chan, pix, (int64_t)n);
  return LTB_OK;
}
// Channels-last copy [N][pix][chan] of a tensor [N][chan][pix].  keep: put it where it outlives the call and remember it (when
// the cache is on and the arena has room); otherwise a staging block of *floats floats to give back (*floats == 0: kept).
// *out stays null when there is no room at all.
static int channels_last(const float* src, int n_img, int chan, int pix, float** out, size_t* floats, bool keep = false) {
  const size_t n = (size_t)n_img * chan * pix;
  *floats = 0; *out = nullptr;
  if (keep && g.filter_cache && !(g.tune & 4)) {
    if (float* kept = (float*)step_alloc(n * 4)) {
      int rc = channels_last_into(src, n_img, chan, pix, kept); if (rc) return rc;
      for (size_t i = 0; i < cl_cache.size(); ++i) if (cl_cache[i].src == src && cl_cache[i].geom == 0) { cl_cache[i] = cl_cache.back(); cl_cache.pop_back(); break; }
      cl_cache.push_back(ClCopy{src, n_img, chan, pix, kept, 0});
      *out = kept;
      return LTB_OK;
    }
  }
  *out = temp_alloc(n); *floats = n;
  if (!*out) return LTB_OK;
  return channels_last_into(src, n_img, chan, pix, *out);
}
// ---- filter cache (ltb_set_filter_cache) ------------------------------------------------------------------------------------
// The per-tap forms of a filter are needed twice per step (forward and data-grad) and change once per step (the optimizer).
// With the cache on they live in private device memory, keyed by the filter's address and shape, and are refreshed -- all
// stale filters together, in ONE launch -- at the first use after a write that overlaps a filter (filter_cache_note_write, called by the optimizer, transfer,
// fill and in-place entry points with their destination; a replayed step and ltb_params_changed mark every filter).  A filter first seen while a step is being recorded takes
// the uncached path (no allocation inside a capture).
struct FilterForms { const float* w; int K, C, taps; float *fwd, *dgrad; bool stale; };
static std::vector<FilterForms> filter_cache;
static size_t filter_cache_bytes = 0;
void filter_cache_clear() {
  for (auto& e : filter_cache) { cudaFree(e.fwd); cudaFree(e.dgrad); }
  filter_cache.clear(); filter_cache_bytes = 0;
}
void filter_cache_note_write(const void* p, size_t bytes) {
  for (size_t i = 0; i < cl_cache.size();) {
    const char* sl = (const char*)cl_cache[i].src; const char* sh = sl + (size_t)cl_cache[i].n_img * cl_cache[i].chan * cl_cache[i].pix * 4;
    if (!p || ((const char*)p < sh && sl < (const char*)p + bytes)) { cl_cache[i] = cl_cache.back(); cl_cache.pop_back(); } else ++i;
  }
  if (filter_cache.empty()) return;
  const char* lo = (const char*)p; const char* hi = lo + bytes;
  for (auto& e : filter_cache) {
    const char* wl = (const char*)e.w; const char* wh = wl + (size_t)e.K * e.C * e.taps * 4;
    if (!p || (lo < wh && wl < hi)) e.stale = true;
  }
}
static FilterForms* filter_cache_entry(const float* w, const ConvDims& d) {
  const int taps = d.R * d.S;
  for (auto& e : filter_cache) if (e.w == w && e.K == d.K && e.C == d.C && e.taps == taps) return &e;
  if (g.capturing) return nullptr;
  const size_t bytes = (size_t)d.K * d.C * taps * 4;
  if (filter_cache_bytes + 2 * bytes > ((size_t)2 << 30)) { cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g.side); cudaStreamSynchronize(g.branch); filter_cache_clear(); }
  FilterForms e{w, d.K, d.C, taps, nullptr, nullptr, true};
  if (cudaMalloc((void**)&e.fwd, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMalloc((void**)&e.dgrad, bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(e.fwd); return nullptr; }
  filter_cache_bytes += 2 * bytes;
  filter_cache.push_back(e);
  return &filter_cache.back();
}
// The per-tap matrices of w: out[tap][k][c] (by_c == 0, forward) or out[tap][c][k] (data-grad).  *floats is the size of the
// staging block to give back afterwards, 0 when the matrices live in the cache.
static int tap_matrices(const float* w, const ConvDims& d, int by_c, float** out, size_t* floats) {
  const size_t n = (size_t)d.K * d.C * d.R * d.S;
  if (g.filter_cache) {
    if (FilterForms* e = filter_cache_entry(w, d)) {
      if (e->stale) {
        // every stale filter at once: after an optimizer step all of them are, and their values are final until the next write
        // (which marks them again), so the forms of the layers still to come are made here too
        FormJobs jobs; jobs.n = 0; jobs.total = 0;
        auto flush = [&]() -> int {
          if (jobs.n == 0) return LTB_OK;
          LTB_LAUNCH(filter_forms_multi_kernel, (unsigned)jobs.total, 256, 0, jobs);
          jobs.n = 0; jobs.total = 0;
          return LTB_OK;
        };
        for (auto& o : filter_cache) {
          if (!o.stale) continue;
          if (jobs.n == kFormJobs) { int rc = flush(); if (rc) return rc; }
          jobs.j[jobs.n++] = FormJob{o.w, o.fwd, o.dgrad, o.K, o.C, o.taps, jobs.total};
          jobs.total += (int)(ceil_div(o.K, 32) * ceil_div(o.C, 32));
          o.stale = false;
        }
        int rc = flush(); if (rc) return rc;
      }
      *out = by_c ? e->dgrad : e->fwd; *floats = 0;
      return LTB_OK;
    }
  }
  *out = temp_alloc(n); *floats = n;
  if (!*out) return LTB_OK;
  LTB_LAUNCH(permute_taps_kernel, grid_for((int64_t)n, 256), 256, 0, w, *out, d.K, d.C, d.R * d.S, by_c, (int64_t)n);
  return LTB_OK;
}
// w[rows][cols] with rows of ld floats: the tensor itself when ld == cols, else a zero-padded copy in a staging block
// (*out stays null when the arena has no room for it).
static int padded_filter(const float* w, int rows, int cols, int ld, const float** out, float** temp, size_t* floats) {
  *temp = nullptr; *floats = 0; *out = w;
  if (ld == cols) return LTB_OK;
  const size_t n = (size_t)rows * ld;
  float* buf = temp_alloc(n);
  *out = buf;
  if (!buf) return LTB_OK;
  *temp = buf; *floats = n;
  LTB_LAUNCH(pad_rows_kernel, grid_for((int64_t)n, 256), 256, 0, w, buf, cols, ld, (int64_t)n);
  return LTB_OK;
}
// Each returns 1 when it took the problem, 0 when not eligible (the unfolding path then runs), negative on error.
static int conv_fwd_taps(const float* x, const float* w, const float* bias, float* y, const ConvDims& d) {
  TcConvGeom gm; TcPlan p;
  if (!taps_geometry(d, gm) || !tc_plan_conv_taps_fwd(p, y, y, bias, y, gm, g.sm_count)) return 0;     // eligibility with any aligned pointers
  float *xr = nullptr, *wt = nullptr; size_t nx = 0, nw = 0;
  int rc = channels_last(x, d.N, d.C, d.H * d.W, &xr, &nx, /*keep=*/true); if (rc) return rc;     // the weight-gradient of this convolution reads it again
  if (!xr) return 0;
  rc = tap_matrices(w, d, 0, &wt, &nw);
  bool ok = !rc && wt && tc_plan_conv_taps_fwd(p, xr, wt, bias, y, gm, g.sm_count);
  if (ok) rc = launch_plan(p, "tc_gemm_kernel[conv_fwd taps]");
  if (wt && nw) temp_free(wt, nw);
  if (nx) temp_free(xr, nx);
  return rc ? rc : (ok ? 1 : 0);
}
static int conv_dgrad_taps(const float* dy, const float* w, float* dx, const ConvDims& d, bool accumulate) {
  TcConvGeom gm; TcPlan p;
  if (!taps_geometry(d, gm) || !tc_plan_conv_taps_dgrad(p, dx, dx, dx, gm, true, g.sm_count)) return 0;
  float *dyr = cl_lookup(dy, d.N, d.K, d.oH * d.oW), *wd = nullptr; size_t ny = 0, nw = 0;
  int rc = dyr ? LTB_OK : channels_last(dy, d.N, d.K, d.oH * d.oW, &dyr, &ny); if (rc) return rc;
  if (!dyr) return 0;
  rc = tap_matrices(w, d, 1, &wd, &nw);
  bool ok = !rc && wd && tc_plan_conv_taps_dgrad(p, dyr, wd, dx, gm, accumulate, g.sm_count);
  if (ok) rc = launch_plan(p, "tc_gemm_kernel[conv_dgrad taps]");
  if (wd && nw) temp_free(wd, nw);
  if (ny) temp_free(dyr, ny);
  return rc ? rc : (ok ? 1 : 0);
}
// Stride 2 (both directions): dx is the stride-1 data-gradient of dy with zeros inserted (to_rows_up2_kernel).
static int conv_dgrad_taps_up2(const float* dy, const float* w, float* dx, const ConvDims& d, bool accumulate) {
  if (d.sh != 2 || d.sw != 2 || d.R * d.S == 1 || d.K % 32 || d.oW > 32 || d.N > 65535) return 0;   // 1x1: the unfolded form with its one-to-one fold is cheaper
  TcConvGeom gm; TcPlan p;
  gm.n_img = d.N; gm.C = d.C; gm.H = d.H; gm.W = d.W; gm.K = d.K; gm.R = d.R; gm.S = d.S; gm.ph = d.ph; gm.pw = d.pw;
  gm.oH = d.H + 2 * d.ph - d.R + 1; gm.oW = d.W + 2 * d.pw - d.S + 1;              // the stride-1 output grid
  if (gm.oH < 1 || gm.oW < 1 || 2 * (d.oH - 1) >= gm.oH || 2 * (d.oW - 1) >= gm.oW) return 0;
  if (!tc_plan_conv_taps_dgrad(p, dx, dx, dx, gm, true, g.sm_count)) return 0;
  const size_t nu = (size_t)d.N * gm.oH * gm.oW * d.K;
  float* up = temp_alloc(nu);
  if (!up) return 0;
  LTB_LAUNCH(to_rows_up2_kernel, dim3((gm.oH + 1) / 2, d.K / 32, d.N), 256, 0, dy, up, d.K, d.oH, d.oW, gm.oH, gm.oW);
  float* wd = nullptr; size_t nw = 0;
  int rc = tap_matrices(w, d, 1, &wd, &nw);
  bool ok = !rc && wd && tc_plan_conv_taps_dgrad(p, up, wd, dx, gm, accumulate, g.sm_count);
  if (ok) rc = launch_plan(p, "tc_gemm_kernel[conv_dgrad taps up2]");
  if (wd && nw) temp_free(wd, nw);
  temp_free(up, nu);
  return rc ? rc : (ok ? 1 : 0);
}
static int conv_wgrad_taps(const float* x, const float* dy, float* dw, const ConvDims& d) {
  TcConvGeom gm; TcPlan p;
  if (!taps_geometry(d, gm) || !tc_plan_conv_taps_wgrad(p, dw, dw, dw, gm, g.sm_count)) return 0;
  float *dyr = cl_lookup(dy, d.N, d.K, d.oH * d.oW), *xr = cl_lookup(x, d.N, d.C, d.H * d.W); size_t ny = 0, nx = 0;
  // Both operands are read channels-last.  With the copies already there (x from this convolution's forward call, dy shared
  // with the data-grad) the tap loop reads each of them once; having to make both first only pays once the unfolded
  // matrix, nine times the size of x, would be large.
  if ((!dyr || !xr || (g.tune & 2)) && (size_t)d.N * d.C * d.R * d.S * d.oH * d.oW * 4 < ((size_t)64 << 20)) return 0;
  int rc = dyr ? LTB_OK : channels_last(dy, d.N, d.K, d.oH * d.oW, &dyr, &ny); if (rc) return rc;
  if (!dyr) return 0;
  if (!xr) rc = channels_last(x, d.N, d.C, d.H * d.W, &xr, &nx);
  bool ok = !rc && xr && tc_plan_conv_taps_wgrad(p, dyr, xr, dw, gm, g.sm_count);
  if (ok) rc = launch_plan(p, "tc_gemm_kernel[conv_wgrad taps]");
  if (xr && nx) temp_free(xr, nx);
  if (ny) temp_free(dyr, ny);
  return rc ? rc : (ok ? 1 : 0);
}
// Start of a convolution's backward call, before its two halves part onto two streams: one channels-last copy of dy for both.
int conv_bwd_prestage(const float* dy, const ConvDims& d, bool both_halves) {
  TcConvGeom gm;
  if (!g.filter_cache || !both_halves || !taps_geometry(d, gm) || d.C % 64 || d.K % 32) return LTB_OK;
  if (cl_lookup(dy, d.N, d.K, d.oH * d.oW)) return LTB_OK;
  float* dyr; size_t ny;
  int rc = channels_last(dy, d.N, d.K, d.oH * d.oW, &dyr, &ny, /*keep=*/true);
  if (!rc && dyr && ny) temp_free(dyr, ny);                 // no room to keep it: each half makes its own, as before
  return rc;
}

int conv_fwd_tc(const float* x, const float* w, const float* bias, float* y, const ConvDims& d) {
  const int ck = d.C * d.R * d.S, pix = d.oH * d.oW;
  TcPlan p;
  const bool rows = tc_conv_needs_rows(pix);
  const int ldw = (ck + 3) / 4 * 4;                                        // K-major filter rows must be a multiple of 16 bytes
  if (!tc_plan_conv_fwd(p, y /* any aligned pointer: eligibility only */, rows, y, ldw, bias, y, d.N, ck, d.K, pix, g.sm_count)) return 0;
  { int t = conv_fwd_taps(x, w, bias, y, d); if (t != 0) return t; }      // the tap-loop form when the shape allows it
  // Small images (4 or 16 pixels) of a 1x1 convolution: the kernel collects the activation itself (no row copy first).
  bool gathered = rows && is_pointwise(d) && pix > 1 && !(g.tune & 1) && tc_gather_possible(x, ck, pix);
  const float* op = x; const float* gsrc = x; bool r2; float* temp = nullptr; size_t tn = 0;
  int rc = LTB_OK;
  // Small images of a strided or 3x3 convolution: unfold into col[n][(c, r, s)][p] -- the layout the weight gradient of this
  // convolution reads, so the matrix is kept for it -- and let the kernel collect its rows from there like those of a 1x1.
  if (!gathered && rows && !is_pointwise(d) && pix > 1 && !(g.tune & 1) && g.filter_cache && !(g.tune & 4) && tc_gather_possible(y, ck, pix)) {
    float* kept = unfold_lookup(x, d);
    if (!kept && (kept = (float*)step_alloc((size_t)d.N * ck * pix * 4)) != nullptr) {
      rc = launch_unfold(x, kept, d); if (rc) return rc;
      cl_cache.push_back(ClCopy{x, d.N, ck, pix, kept, unfold_key(d)});
    }
    if (kept) { gathered = true; op = gsrc = kept; }
  }
  if (!gathered) rc = stage_activation(x, !is_pointwise(d), d, ck, pix, &op, &r2, &temp, &tn);
  if (rc) return rc < 0 ? rc : 0;
  float* wtemp; size_t wn; const float* wp;
  rc = padded_filter(w, d.K, ck, ldw, &wp, &wtemp, &wn);
  const bool ok = !rc && wp && tc_plan_conv_fwd(p, op, rows, wp, ldw, bias, y, d.N, ck, d.K, pix, g.sm_count);
  if (ok && gathered) tc_plan_gather(p, gsrc, d.N, ck, pix);
  if (ok) rc = launch_plan(p, gathered ? "tc_gemm_kernel[conv_fwd gather]" : "tc_gemm_kernel[conv_fwd]");
  if (wtemp) temp_free(wtemp, wn);
  if (temp) temp_free(temp, tn);
  return rc ? rc : (ok ? 1 : 0);
}

// *fresh: dx was declared unset (ltb_grad_unset) and holds nothing: a path that can writes its result instead of adding, the
// unfold-and-fold path fills dx with zeros first; either way *fresh is false once dx holds data.
int conv_dgrad_tc(const float* dy, const float* w, float* dx, const ConvDims& d, bool* fresh) {
  const int ck = d.C * d.R * d.S, pix = d.oH * d.oW;
  TcPlan p;
  const bool rows = tc_conv_needs_rows(pix), direct = is_pointwise(d);
  const int ldw = (ck + 31) / 32 * 32;                                     // N-major filter rows must be whole 128-byte chunks
  if (!tc_plan_conv_dgrad(p, dx, rows, dx, ldw, dx, d.N, ck, d.K, pix, direct, g.sm_count)) return 0;
  { int t = conv_dgrad_taps(dy, w, dx, d, !*fresh); if (t != 0) { if (t > 0) *fresh = false; return t; } }
  { int t = conv_dgrad_taps_up2(dy, w, dx, d, !*fresh); if (t != 0) { if (t > 0) *fresh = false; return t; } }
  const bool gathered = rows && pix > 1 && !(g.tune & 1) && tc_gather_possible(dy, d.K, pix);    // dy of a small map: collected by the kernel itself
  const float* op = dy; bool r2; float* temp = nullptr; size_t tn = 0;
  ConvDims flat = d; flat.C = d.K;                               // dy is [N][K][pix]: staged like a pointwise activation with K channels
  int rc = gathered ? LTB_OK : stage_activation(dy, false, flat, d.K, pix, &op, &r2, &temp, &tn);
  if (rc) return rc < 0 ? rc : 0;
  float* col = nullptr; const size_t ncol = (size_t)d.N * ck * pix;
  if (!direct) { col = temp_alloc(ncol); if (!col) { if (temp) temp_free(temp, tn); return 0; } }
  float* wtemp; size_t wn; const float* wp;
  rc = padded_filter(w, d.K, ck, ldw, &wp, &wtemp, &wn);
  bool ok = !rc && wp && tc_plan_conv_dgrad(p, op, rows, wp, ldw, direct ? dx : col, d.N, ck, d.K, pix, direct && !*fresh, g.sm_count);
  if (ok && !direct && *fresh) {                                  // the fold-back adds into dx: start from zeros
    if (cudaMemsetAsync(dx, 0, (size_t)d.N * d.C * d.H * d.W * 4, g.stream) != cudaSuccess) { ok = false; rc = fail(LTB_E_CUDA, "conv data-grad: zero fill failed"); }
  }
  if (ok && gathered) tc_plan_gather(p, dy, d.N, d.K, pix);
  if (ok) rc = launch_plan(p, gathered ? "tc_gemm_kernel[conv_dgrad gather]" : "tc_gemm_kernel[conv_dgrad]");
  if (ok && !rc && !direct) rc = launch_fold(col, dx, d);
  if (ok && !rc) *fresh = false;
  if (wtemp) temp_free(wtemp, wn);
  if (col) temp_free(col, ncol);
  if (temp) temp_free(temp, tn);
  return rc ? rc : (ok ? 1 : 0);
}

int conv_wgrad_tc(const float* x, const float* dy, float* dw, const ConvDims& d) {
  const int ck = d.C * d.R * d.S, pix = d.oH * d.oW;
  TcPlan p;
  if (!tc_plan_conv_wgrad(p, dy, dy, dw, d.N, ck, d.K, pix, g.sm_count)) return 0;
  { int t = conv_wgrad_taps(x, dy, dw, d); if (t != 0) return t; }
  const float* xin = x; float* col = nullptr; const size_t n = (size_t)d.N * ck * pix;
  if (!is_pointwise(d)) {
    if (float* kept = unfold_lookup(x, d)) xin = kept;               // forward left its unfolded matrix behind
    else {
      col = temp_alloc(n); if (!col) return 0;
      int rc0 = launch_unfold(x, col, d); if (rc0) return rc0;
      xin = col;
    }
  }
  // the probe above used dy in place of x: the caller's x may still be declined (a view that is not 16-byte aligned)
  if (!tc_plan_conv_wgrad(p, xin, dy, dw, d.N, ck, d.K, pix, g.sm_count)) { if (col) temp_free(col, n); return 0; }
  int rc = launch_plan(p, "tc_gemm_kernel[conv_wgrad]");
  if (col) temp_free(col, n);
  return rc ? rc : 1;
}

}  // namespace ltb
