// A whole unrolled sequence of the vanilla recurrent network in one launch (two for the backward pass).
//
// The reference stages the cell h_t = tanh(x_t Wxh + h_{t-1} Whh + bh) and the output layer o_t = h_t Who + bo operator by
// operator (NNModule.scala:189-200), unrolls T steps (DynamicRNNFix, NNModule.scala:240-253) and adds
// sum(nll(logSoftmax(o_t), y_t)) over the steps: for T = 20 that is some 260 kernels of a few microseconds each, forward and
// backward, and the step runs at the launch rate of the host, not at any limit of the device.
//
// The batch rows of such a sequence never meet: row b of h_t depends on row b of h_{t-1} only.  So the rows are dealt out to
// CTAs (two rows per CTA at batch 256: one CTA per SM); a CTA copies the weight matrices and ALL T steps of its rows into
// shared memory once and never leaves the SM.  Only the recurrence itself is sequential (one matrix-vector product and one
// barrier per step); everything that does not depend on the step before -- x_t Wxh for all t, the output layer, the
// log-softmax, and in the backward pass do_t Who^T and all five gradient sums -- runs as register-tiled matrix products
// over the CTA's T x rows lines at once.  The CTAs' gradient sums are written to slabs and added into the gradient tensors
// in CTA order by a second small launch (no atomics: the same bits on every run).
#include "common.cuh"

namespace ltb {

constexpr int kSeqThreads = 512;

// CTAs of the running forward launch that have written their part of the loss; back at zero when the launch ends.
__device__ unsigned seq_done_count;

__device__ __forceinline__ float warp_max(float v) { for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }
__device__ __forceinline__ float warp_add(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }
__host__ __device__ __forceinline__ int up4(int v) { return (v + 3) & ~3; }

// C[m][n] = sum_k A[m][k] W[k][n] (+ bias[n]) on shared memory, a 4 x 4 block of C per thread: the W row is read as one float4
// (consecutive lanes, consecutive columns), the four A values are broadcasts.  Row counts and column pitches are multiples of 4
// (padding rows and columns hold zeros).
__device__ __forceinline__ void mm_tiles(const float* A, int lda, const float* W, int ldw, float* C, int ldc, const float* bias, int M4, int N4, int K) {
  const int nt = N4 >> 2, tiles = (M4 >> 2) * nt;
  for (int tile = threadIdx.x; tile < tiles; tile += kSeqThreads) {
    const int m0 = (tile / nt) << 2, n0 = (tile % nt) << 2;
    float acc[4][4] = {};
    const float* a = A + (size_t)m0 * lda;
    for (int k = 0; k < K; ++k) {
      const float4 w = *reinterpret_cast<const float4*>(W + (size_t)k * ldw + n0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float av = a[i * lda + k];
        acc[i][0] += av * w.x; acc[i][1] += av * w.y; acc[i][2] += av * w.z; acc[i][3] += av * w.w;
      }
    }
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) bv = *reinterpret_cast<const float4*>(bias + n0);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<float4*>(C + (size_t)(m0 + i) * ldc + n0) = make_float4(acc[i][0] + bv.x, acc[i][1] + bv.y, acc[i][2] + bv.z, acc[i][3] + bv.w);
  }
}

// out[a][b] = sum_row A[row][a] B[row][b] for a < Ma, b < Nb (global memory, row pitch Nb), 4 x 4 per thread, both operands read as float4.
__device__ __forceinline__ void outer_tiles(const float* A, int lda, const float* Bm, int ldb, float* out, int Ma, int Nb, int rows) {
  const int nt = up4(Nb) >> 2, tiles = (up4(Ma) >> 2) * nt;
  for (int tile = threadIdx.x; tile < tiles; tile += kSeqThreads) {
    const int a0 = (tile / nt) << 2, b0 = (tile % nt) << 2;
    float acc[4][4] = {};
    for (int r = 0; r < rows; ++r) {
      const float4 av = *reinterpret_cast<const float4*>(A + (size_t)r * lda + a0);
      const float4 bv = *reinterpret_cast<const float4*>(Bm + (size_t)r * ldb + b0);
      const float aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[i][0] += aa[i] * bv.x; acc[i][1] += aa[i] * bv.y; acc[i][2] += aa[i] * bv.z; acc[i][3] += aa[i] * bv.w; }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (a0 + i < Ma && b0 + j < Nb) out[(size_t)(a0 + i) * Nb + b0 + j] = acc[i][j];
  }
}

// Shared memory of the forward kernel (pitches Vq = up4(V), Hq = up4(H); L = up4(T * rows) lines, line (t, r) = t * rows + r):
//   Wxh [V][Hq], Whh [H][Hq], Who [H][Vq], bh [Hq], bo [Vq], x -> o [L][Vq], hx [rows + L][Hq] (h0, then h_0 .. h_{T-1}).
// loss_part[cta] receives the CTA's sum of -logp[y]; the last CTA to finish adds the parts in CTA order into loss[0].
__global__ void __launch_bounds__(kSeqThreads) rnn_seq_fwd_kernel(const float* __restrict__ x, const int32_t* __restrict__ y, const float* __restrict__ h0,
                                                                  const float* __restrict__ Wxh, const float* __restrict__ Whh, const float* __restrict__ bh,
                                                                  const float* __restrict__ Who, const float* __restrict__ bo, float* __restrict__ h_out,
                                                                  float* __restrict__ logp_out, float* loss, float* loss_part,
                                                                  int T, int B, int V, int H, int rows) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  const int Vq = up4(V), Hq = up4(H), L = up4(T * rows);
  float* s_wxh = sm; float* s_whh = s_wxh + V * Hq; float* s_who = s_whh + H * Hq; float* s_bh = s_who + H * Vq; float* s_bo = s_bh + Hq;
  float* s_x = s_bo + Vq; float* s_hx = s_x + L * Vq;
  __shared__ float s_loss[kSeqThreads / 32];
  __shared__ bool s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b0 = blockIdx.x * rows, nr = min(rows, B - b0);
  for (int i = tid; i < V * Hq; i += kSeqThreads) { const int r = i / Hq, c = i - r * Hq; s_wxh[i] = c < H ? Wxh[r * H + c] : 0.0f; }
  for (int i = tid; i < H * Hq; i += kSeqThreads) { const int r = i / Hq, c = i - r * Hq; s_whh[i] = c < H ? Whh[r * H + c] : 0.0f; }
  for (int i = tid; i < H * Vq; i += kSeqThreads) { const int r = i / Vq, c = i - r * Vq; s_who[i] = c < V ? Who[r * V + c] : 0.0f; }
  for (int i = tid; i < Hq; i += kSeqThreads) s_bh[i] = i < H ? bh[i] : 0.0f;
  for (int i = tid; i < Vq; i += kSeqThreads) s_bo[i] = i < V ? bo[i] : 0.0f;
  for (int i = tid; i < L * Vq; i += kSeqThreads) {
    const int line = i / Vq, c = i - line * Vq, t = line / rows, r = line - t * rows;
    s_x[i] = (t < T && r < nr && c < V) ? x[((size_t)t * B + b0 + r) * V + c] : 0.0f;
  }
  for (int i = tid; i < rows * Hq; i += kSeqThreads) { const int r = i / Hq, c = i - r * Hq; s_hx[i] = (h0 && r < nr && c < H) ? h0[(size_t)(b0 + r) * H + c] : 0.0f; }
  __syncthreads();
  // every step's input part at once: hx[line] = x[line] Wxh + bh
  mm_tiles(s_x, Vq, s_wxh, Hq, s_hx + rows * Hq, Hq, s_bh, L, Hq, V);
  __syncthreads();
  // the recurrence: one thread per (row, hidden unit); a warp reads consecutive columns of Whh, h_{t-1} is a broadcast
  for (int t = 0; t < T; ++t) {
    const float* hp = s_hx + (size_t)t * rows * Hq; float* hc = s_hx + (size_t)(t + 1) * rows * Hq;
    for (int i = tid; i < rows * Hq; i += kSeqThreads) {
      const int r = i / Hq, j = i - r * Hq;
      const float* hr = hp + r * Hq;
      float c0 = 0.0f, c1 = 0.0f;
      int k = 0;
      for (; k + 1 < H; k += 2) { c0 += hr[k] * s_whh[k * Hq + j]; c1 += hr[k + 1] * s_whh[(k + 1) * Hq + j]; }
      if (k < H) c0 += hr[k] * s_whh[k * Hq + j];
      hc[i] = j < H ? tanhf(hc[i] + (c0 + c1)) : 0.0f;
    }
    __syncthreads();
  }
  // output layer of every step at once: o[line] = h[line] Who + bo (over the x lines, no longer needed)
  mm_tiles(s_hx + rows * Hq, Hq, s_who, Vq, s_x, Vq, s_bo, L, Vq, H);
  __syncthreads();
  for (int i = tid; i < T * nr * H; i += kSeqThreads) {
    const int c = i % H, rest = i / H, r = rest % nr, t = rest / nr;
    h_out[((size_t)t * B + b0 + r) * H + c] = s_hx[(size_t)((t + 1) * rows + r) * Hq + c];
  }
  // logSoftmax and the loss: one warp per line (max, sum of exponentials, x - (max + log sum): TensorDslCPU.scala:805-835)
  float my_loss = 0.0f;
  for (int line = warp; line < T * rows; line += kSeqThreads / 32) {
    const int t = line / rows, r = line - t * rows;
    if (r >= nr) continue;
    const float* o = s_x + (size_t)line * Vq;
    float m = -3.4028235e38f;
    for (int v = lane; v < V; v += 32) m = fmaxf(m, o[v]);
    m = warp_max(m);
    float s = 0.0f;
    for (int v = lane; v < V; v += 32) s += expf(o[v] - m);
    s = warp_add(s);
    const float lse = m + logf(s);
    float* lp = logp_out + ((size_t)t * B + b0 + r) * V;
    for (int v = lane; v < V; v += 32) lp[v] = o[v] - lse;
    if (lane == 0) { const int target = y[(size_t)t * B + b0 + r]; my_loss += -(o[target] - lse); }
  }
  if (lane == 0) s_loss[warp] = my_loss;
  __syncthreads();
  if (tid == 0) {
    float s = 0.0f;
    for (int w = 0; w < kSeqThreads / 32; ++w) s += s_loss[w];
    loss_part[blockIdx.x] = s;
    __threadfence();
    s_last = atomicAdd(&seq_done_count, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last && tid == 0) {                         // the last CTA to finish: the parts are all there; added in CTA order
    __threadfence();
    float s = 0.0f;
    for (unsigned c = 0; c < gridDim.x; ++c) s += ((volatile float*)loss_part)[c];
    loss[0] = s;
    seq_done_count = 0;                             // ready for the next launch
  }
}

// Backward.  Shared memory: Whh^T [H][Hq] and Who^T [V][Hq] (transposed while loading, so that both products below read
// consecutive columns), x [L][Vq], hx [rows + L][Hq] (h0, h_0 .. h_{T-1}), do [L][Vq], dp [L][Hq] (first do Who^T, then the
// gradient at the cell's pre-activation).  The CTA's sums go to slab[cta][...] in the order dWxh, dWhh, dbh, dWho, dbo.
__global__ void __launch_bounds__(kSeqThreads) rnn_seq_bwd_kernel(const float* __restrict__ x, const int32_t* __restrict__ y, const float* __restrict__ h0,
                                                                  const float* __restrict__ Whh, const float* __restrict__ Who, const float* __restrict__ h_all,
                                                                  const float* __restrict__ logp, const float* __restrict__ dloss, float* __restrict__ slab,
                                                                  int T, int B, int V, int H, int rows) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  const int Vq = up4(V), Hq = up4(H), L = up4(T * rows);
  float* s_whhT = sm; float* s_whoT = s_whhT + H * Hq; float* s_x = s_whoT + V * Hq; float* s_hx = s_x + L * Vq;
  float* s_do = s_hx + (rows + L) * Hq; float* s_dp = s_do + L * Vq;
  const int tid = threadIdx.x;
  const int b0 = blockIdx.x * rows, nr = min(rows, B - b0);
  const int n_sums = 2 * V * H + H * H + H + V;
  const float dl = dloss[0];
  for (int i = tid; i < H * Hq; i += kSeqThreads) { const int jp = i / Hq, j = i - jp * Hq; s_whhT[i] = j < H ? Whh[j * H + jp] : 0.0f; }     // [j'][j] = Whh[j][j']
  for (int i = tid; i < V * Hq; i += kSeqThreads) { const int v = i / Hq, j = i - v * Hq; s_whoT[i] = j < H ? Who[j * V + v] : 0.0f; }        // [v][j] = Who[j][v]
  for (int i = tid; i < L * Vq; i += kSeqThreads) {
    const int line = i / Vq, c = i - line * Vq, t = line / rows, r = line - t * rows;
    const bool live = t < T && r < nr && c < V;
    const size_t g = ((size_t)t * B + b0 + r) * V + c;
    s_x[i] = live ? x[g] : 0.0f;
    // nllLoss_grad then logSoftmax_grad (TensorDslCPU.scala:1100-1110, 837-846): do = dl * (exp(logp) - onehot(y))
    s_do[i] = live ? dl * (expf(logp[g]) - (y[(size_t)t * B + b0 + r] == c ? 1.0f : 0.0f)) : 0.0f;
  }
  for (int i = tid; i < (rows + L) * Hq; i += kSeqThreads) {
    const int line = i / Hq, c = i - line * Hq, t = line / rows - 1, r = line % rows;               // line 0 .. rows-1: h0
    float v = 0.0f;
    if (r < nr && c < H && t < T) v = t < 0 ? (h0 ? h0[(size_t)(b0 + r) * H + c] : 0.0f) : h_all[((size_t)t * B + b0 + r) * H + c];
    s_hx[i] = v;
  }
  __syncthreads();
  // what reaches h_t from the output layer, every step at once: dp[line] = do[line] Who^T
  mm_tiles(s_do, Vq, s_whoT, Hq, s_dp, Hq, nullptr, L, Hq, V);
  __syncthreads();
  // the recurrence, backwards in time: dpre_t = (dp_t + dpre_{t+1} Whh^T) (1 - h_t^2)
  for (int t = T - 1; t >= 0; --t) {
    const float* nx = s_dp + (size_t)(t + 1) * rows * Hq; float* cu = s_dp + (size_t)t * rows * Hq;
    const float* hc = s_hx + (size_t)(t + 1) * rows * Hq;
    for (int i = tid; i < rows * Hq; i += kSeqThreads) {
      const int r = i / Hq, j = i - r * Hq;
      float c0 = 0.0f, c1 = 0.0f;
      if (t + 1 < T) {
        const float* dr = nx + r * Hq;
        int k = 0;
        for (; k + 1 < H; k += 2) { c0 += dr[k] * s_whhT[k * Hq + j]; c1 += dr[k + 1] * s_whhT[(k + 1) * Hq + j]; }
        if (k < H) c0 += dr[k] * s_whhT[k * Hq + j];
      }
      const float hv = hc[i];
      cu[i] = j < H ? (cu[i] + (c0 + c1)) * (1.0f - hv * hv) : 0.0f;
    }
    __syncthreads();
  }
  // the five sums over the CTA's lines: dWxh = x^T dpre, dWhh = h_prev^T dpre, dbh, dWho = h^T do, dbo
  float* out = slab + (size_t)blockIdx.x * n_sums;
  const int lines = T * rows;
  outer_tiles(s_x, Vq, s_dp, Hq, out, V, H, lines);
  outer_tiles(s_hx, Hq, s_dp, Hq, out + V * H, H, H, lines);                                       // line (t, r) of hx is h_{t-1}
  outer_tiles(s_hx + rows * Hq, Hq, s_do, Vq, out + V * H + H * H + H, H, V, lines);
  for (int j = tid; j < H; j += kSeqThreads) { float a = 0.0f; for (int l = 0; l < lines; ++l) a += s_dp[(size_t)l * Hq + j]; out[V * H + H * H + j] = a; }
  for (int v = tid; v < V; v += kSeqThreads) { float a = 0.0f; for (int l = 0; l < lines; ++l) a += s_do[(size_t)l * Vq + v]; out[2 * V * H + H * H + H + v] = a; }
}
// d[i] += slab[0][i] + slab[1][i] + ... for the five gradient tensors (segments of the slab row in the order of the kernel above).
__global__ void rnn_seq_sum_kernel(const float* __restrict__ slab, int ctas, int n_sums, float* dWxh, float* dWhh, float* dbh, float* dWho, float* dbo, int V, int H) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_sums) return;
  float a = 0.0f;
  for (int c = 0; c < ctas; ++c) a += slab[(size_t)c * n_sums + i];
  const int o1 = V * H, o2 = o1 + H * H, o3 = o2 + H, o4 = o3 + H * V;
  if (i < o1) dWxh[i] += a; else if (i < o2) dWhh[i - o1] += a; else if (i < o3) dbh[i - o2] += a; else if (i < o4) dWho[i - o3] += a; else dbo[i - o4] += a;
}

static int seq_opted_device = -1;                   // the device whose kernels have been given the large shared-memory limit

// Rows per CTA: one CTA per SM when the batch allows it, fewer rows (more CTAs) when T steps of that many rows do not fit the
// 227 KB of an SM beside the weights.
static bool seq_plan(int T, int B, int V, int H, int* rows, size_t* smem_fwd, size_t* smem_bwd) {
  const size_t Vq = (size_t)up4(V), Hq = (size_t)up4(H);
  int r = (int)ceil_div(B, g.sm_count); if (r < 1) r = 1;
  for (; r >= 1; --r) {
    const size_t L = (size_t)up4(T * r);
    *smem_fwd = ((size_t)V * Hq + (size_t)H * Hq + (size_t)H * Vq + Hq + Vq + L * Vq + ((size_t)r + L) * Hq) * 4;
    *smem_bwd = ((size_t)H * Hq + (size_t)V * Hq + L * Vq + ((size_t)r + L) * Hq + L * Vq + (L + (size_t)r) * Hq) * 4;
    if (*smem_bwd <= (size_t)220 * 1024 && *smem_fwd <= (size_t)220 * 1024 && ceil_div(B, r) <= 65535) { *rows = r; return true; }
  }
  return false;
}

}  // namespace ltb

using namespace ltb;

extern "C" {

int ltb_rnn_seq_fwd(const float* x, const int32_t* y, const float* h0, const float* Wxh, const float* Whh, const float* bh, const float* Who,
                    const float* bo, float* h, float* logp, float* loss, int T, int B, int V, int H) {
  LTB_INITED(); LTB_REQUIRE(x && y && Wxh && Whh && bh && Who && bo && h && logp && loss && T > 0 && B > 0 && V > 0 && H > 0, "ltb_rnn_seq_fwd: bad argument");
  int rows; size_t sf, sb;
  if (!seq_plan(T, B, V, H, &rows, &sf, &sb))
    return fail(LTB_E_LIMIT, "ltb_rnn_seq_fwd: the weights (vocabulary %d, hidden %d) and %d steps of one batch row do not fit one SM's shared memory", V, H, T);
  if (seq_opted_device != g.device) {
    LTB_REQUIRE(!g.capturing, "ltb_rnn_seq_fwd: the first call sets the kernels up and must come before a step is recorded");
    LTB_CUDA(cudaFuncSetAttribute(rnn_seq_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    LTB_CUDA(cudaFuncSetAttribute(rnn_seq_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    seq_opted_device = g.device;
  }
  const int ctas = (int)ceil_div(B, rows);
  LTB_REQUIRE((size_t)ctas * 4 <= g.cur_scratch_bytes(), "ltb_rnn_seq_fwd: batch too large for the library's workspace");
  LTB_LAUNCH(rnn_seq_fwd_kernel, ctas, kSeqThreads, sf, x, y, h0, Wxh, Whh, bh, Who, bo, h, logp, loss, g.cur_scratch(), T, B, V, H, rows);
  return LTB_OK;
}

int ltb_rnn_seq_bwd(const float* x, const int32_t* y, const float* h0, const float* Whh, const float* Who, const float* h, const float* logp,
                    const float* dloss, float* dWxh, float* dWhh, float* dbh, float* dWho, float* dbo, int T, int B, int V, int H) {
  LTB_INITED(); LTB_SETTLE(dloss); LTB_SETTLE(dWxh); LTB_SETTLE(dWhh); LTB_SETTLE(dbh); LTB_SETTLE(dWho); LTB_SETTLE(dbo); LTB_REQUIRE(x && y && Whh && Who && h && logp && dloss && dWxh && dWhh && dbh && dWho && dbo && T > 0 && B > 0 && V > 0 && H > 0, "ltb_rnn_seq_bwd: bad argument");
  int rows; size_t sf, sb;
  if (!seq_plan(T, B, V, H, &rows, &sf, &sb) || seq_opted_device != g.device) return fail(LTB_E_STATE, "ltb_rnn_seq_bwd: no forward call came before");
  const int ctas = (int)ceil_div(B, rows), n_sums = 2 * V * H + H * H + H + V;
  float* slab = (float*)ltb_malloc_uninit((size_t)ctas * n_sums * 4);                 // staging block, given back below (LIFO)
  if (!slab) return g.last;
  LTB_LAUNCH(rnn_seq_bwd_kernel, ctas, kSeqThreads, sb, x, y, h0, Whh, Who, h, logp, dloss, slab, T, B, V, H, rows);
  LTB_LAUNCH(rnn_seq_sum_kernel, (unsigned)ceil_div(n_sums, 256), 256, 0, (const float*)slab, ctas, n_sums, dWxh, dWhh, dbh, dWho, dbo, V, H);
  return ltb_free(slab, (size_t)ctas * n_sums * 4);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------------------
// One node of the binary tree LSTM per launch.
//
// Operator by operator a node is some 45 kernels forward and backward, gate by gate (ltb_affine_act, ltb_lstm_cell) still 18;
// every one of them works on vectors of 150 floats, so a tree runs at the launch rate of the host.  Here the forward pass of
// a node is one launch: a warp per gate row (750 rows for an inner node: 94 CTAs that read the ten 150x150 matrices out of
// L2 once), and the last CTA to finish combines the gates into the cell, runs the classifier and the loss.  The backward
// pass is one launch too: what precedes the gate gradients in the chain rule (loss, classifier, cell: a few thousand
// operations on vectors of 150) is recomputed by EVERY CTA for itself in shared memory, so no CTA waits for another; CTA 0
// alone writes that part's results.  Then a CTA is one of two kinds: rows of the weight gradients (dW[g][j][:] += dpre in[:]),
// or partial sums of the input gradients (32 inputs x 32 gate rows per warp, added atomically).
namespace ltb {

constexpr int kNodeThreads = 256, kNodeWarps = kNodeThreads / 32;
constexpr int kNodeMaxHidden = 512;                   // the backward prologue keeps 7 vectors of this length in shared memory

__device__ unsigned node_done_count;                  // CTAs of the running forward launch that have stored their gates
constexpr int kNodesPerLaunch = 128;
__device__ unsigned nodes_done_count[kNodesPerLaunch]; // the same, one per node of a batched launch

__device__ __forceinline__ float act_apply(int slot, float v) { return slot == 4 ? tanhf(v) : 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ int node_slot(bool inner, int g) { return inner ? g : (g == 0 ? 0 : g + 2); }   // leaf rows: slots 0, 3, 4

// bx: this CTA's index among the n_ctas CTAs that work on node P; done: their completion counter (zero between launches)
__device__ __forceinline__ void node_fwd_body(const ltb_tree_node& P, unsigned* done, unsigned n_ctas, int bx) {
  __shared__ float s_in[kNodeMaxHidden];
  __shared__ float s_pred[32];
  __shared__ bool s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hd = P.hidden, L = P.in_len, G = P.inner ? 5 : 3;
  const int row = bx * kNodeWarps + warp;
  if (row < G * Hd) {
    const int slot = node_slot(P.inner, row / Hd), j = row % Hd;
    float a = 0.0f;
    const float* w0 = P.W[slot][0] + (size_t)j * L; const float* x0 = P.in[0];
    for (int k = lane; k < L; k += 32) a += w0[k] * x0[k];
    if (P.inner) {
      float b = 0.0f;
      const float* w1 = P.W[slot][1] + (size_t)j * L; const float* x1 = P.in[1];
      for (int k = lane; k < L; k += 32) b += w1[k] * x1[k];
      a = warp_add(a) + warp_add(b);
    } else {
      a = warp_add(a);
    }
    if (lane == 0) { P.gates[slot * Hd + j] = act_apply(slot, a + P.bias[slot][j]); __threadfence(); }
  }
  __syncthreads();
  if (tid == 0) { __threadfence(); s_last = atomicAdd(done, 1u) == n_ctas - 1; }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last CTA: all gates are in memory (read past L1: other SMs wrote them)
  for (int j = tid; j < Hd; j += kNodeThreads) {
    const float ig = __ldcg(P.gates + j), og = __ldcg(P.gates + 3 * Hd + j), uv = __ldcg(P.gates + 4 * Hd + j);
    float c = ig * uv;
    if (P.inner) c = (c + __ldcg(P.gates + Hd + j) * P.cl[j]) + __ldcg(P.gates + 2 * Hd + j) * P.cr[j];
    const float tc = tanhf(c), h = og * tc;
    P.c[j] = c; P.tc[j] = tc; P.h[j] = h;
    s_in[j] = P.classify_cell ? c : h;
  }
  __syncthreads();
  for (int k = warp; k < P.classes; k += kNodeWarps) {
    float a = 0.0f;
    for (int j = lane; j < Hd; j += 32) a += P.Why[(size_t)k * Hd + j] * s_in[j];
    a = warp_add(a);
    if (lane == 0) s_pred[k] = a + P.by[k];
  }
  __syncthreads();
  if (warp == 0) {
    const float o = lane < P.classes ? s_pred[lane] : -3.4028235e38f;
    const float m = warp_max(o);
    const float s = warp_add(lane < P.classes ? expf(o - m) : 0.0f);
    const float lse = m + logf(s);
    if (lane < P.classes) P.logp[lane] = o - lse;
    if (lane == 0) {
      float loss = -(s_pred[P.score[0]] - lse);
      if (P.loss_l) loss += P.loss_l[0];
      if (P.loss_r) loss += P.loss_r[0];
      P.loss[0] = loss;
      *done = 0;                                      // ready for the next launch
    }
  }
}
__global__ void __launch_bounds__(kNodeThreads) tree_node_fwd_kernel(const ltb_tree_node P) { node_fwd_body(P, &node_done_count, gridDim.x, (int)blockIdx.x); }
// Several independent nodes (one level of a tree) in one launch: blockIdx.y picks the node out of an array in device memory,
// the CTA copies its node's description into shared memory first.  done[] has one counter per node of the launch.
__device__ __forceinline__ const ltb_tree_node& node_to_shared(const ltb_tree_node* nodes, int i) {
  __shared__ ltb_tree_node sp;
  const int* src = reinterpret_cast<const int*>(nodes + i); int* dst = reinterpret_cast<int*>(&sp);
  for (int k = threadIdx.x; k < (int)(sizeof(ltb_tree_node) / 4); k += blockDim.x) dst[k] = src[k];
  __syncthreads();
  return sp;
}
__global__ void __launch_bounds__(kNodeThreads) tree_nodes_fwd_kernel(const ltb_tree_node* nodes) {
  unsigned* done = nodes_done_count;
  const ltb_tree_node& P = node_to_shared(nodes, (int)blockIdx.y);
  const unsigned n_ctas = (unsigned)(((P.inner ? 5 : 3) * P.hidden + kNodeWarps - 1) / kNodeWarps);
  if (blockIdx.x >= n_ctas) return;                                    // the grid is sized for an inner node; a leaf needs fewer CTAs
  node_fwd_body(P, done + blockIdx.y, n_ctas, (int)blockIdx.x);
}

// Backward.  Grid: n_w CTAs of weight-gradient rows, then n_x CTAs of input-gradient partial sums (none for a leaf).
// SHARED: several nodes of one launch add into the same parameter gradients (a level of a tree): those additions are atomic.
template <bool SHARED>
__device__ __forceinline__ void node_bwd_body(const ltb_tree_node& P, int n_w, int bx) {
  __shared__ float s_dpre[5 * kNodeMaxHidden];        // gradient at each gate's pre-activation
  __shared__ float s_dpred[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hd = P.hidden, L = P.in_len, G = P.inner ? 5 : 3;
  const float dl = P.dloss[0];
  const int score = P.score[0];
  if (tid < 32) s_dpred[tid] = tid < P.classes ? dl * (expf(P.logp[tid]) - (tid == score ? 1.0f : 0.0f)) : 0.0f;   // nllLoss_grad, logSoftmax_grad
  __syncthreads();
  for (int j = tid; j < Hd; j += kNodeThreads) {
    float dcls = 0.0f;                                // classifier's gradient at its input
    for (int k = 0; k < P.classes; ++k) dcls += P.Why[(size_t)k * Hd + j] * s_dpred[k];
    const float dh = P.dh[j] + (P.classify_cell ? 0.0f : dcls), dc = P.dc[j] + (P.classify_cell ? dcls : 0.0f);
    const float ig = P.gates[j], og = P.gates[3 * Hd + j], uv = P.gates[4 * Hd + j], tc = P.tc[j];
    const float dct = dc + dh * og * (1.0f - tc * tc);
    s_dpre[0 * Hd + j] = (dct * uv) * ig * (1.0f - ig);
    s_dpre[3 * Hd + j] = (dh * tc) * og * (1.0f - og);
    s_dpre[4 * Hd + j] = (dct * ig) * (1.0f - uv * uv);
    if (P.inner) {
      const float fl = P.gates[Hd + j], fr = P.gates[2 * Hd + j];
      s_dpre[1 * Hd + j] = (dct * P.cl[j]) * fl * (1.0f - fl);
      s_dpre[2 * Hd + j] = (dct * P.cr[j]) * fr * (1.0f - fr);
      if (bx == 0) {
        if (P.dcl) P.dcl[j] += dct * fl;
        if (P.dcr) P.dcr[j] += dct * fr;
      }
    }
    if (bx == 0) {
      const float v = P.classify_cell ? P.c[j] : P.h[j];
      for (int k = 0; k < P.classes; ++k) { if (SHARED) atomicAdd(P.dWhy + (size_t)k * Hd + j, s_dpred[k] * v); else P.dWhy[(size_t)k * Hd + j] += s_dpred[k] * v; }
    }
  }
  if (bx == 0) {
    if (tid < P.classes) { if (SHARED) atomicAdd(P.dby + tid, s_dpred[tid]); else P.dby[tid] += s_dpred[tid]; }
    if (tid == 0) { if (P.dloss_l) P.dloss_l[0] += dl; if (P.dloss_r) P.dloss_r[0] += dl; }
  }
  __syncthreads();
  if (bx < n_w) {
    const int row = bx * kNodeWarps + warp;
    if (row >= G * Hd) return;
    const int slot = node_slot(P.inner, row / Hd), j = row % Hd;
    const float dp = s_dpre[slot * Hd + j];
    float* d0 = P.dW[slot][0] + (size_t)j * L; const float* x0 = P.in[0];
    for (int k = lane; k < L; k += 32) { if (SHARED) atomicAdd(d0 + k, dp * x0[k]); else d0[k] += dp * x0[k]; }
    if (P.inner) {
      float* d1 = P.dW[slot][1] + (size_t)j * L; const float* x1 = P.in[1];
      for (int k = lane; k < L; k += 32) { if (SHARED) atomicAdd(d1 + k, dp * x1[k]); else d1[k] += dp * x1[k]; }
    }
    if (lane == 0) atomicAdd(P.dbias[slot] + j, dp);   // two slots may share a bias vector
    return;
  }
  // input gradients: warp = (input, block of 32 inputs, gate, block of 32 gate rows); din[k] += sum_j dpre[j] W[j][k]
  const int kb = (L + 31) / 32, jb = (Hd + 31) / 32;
  int w = (bx - n_w) * kNodeWarps + warp;
  const int n_in = P.inner ? 2 : 1;
  if (w >= n_in * kb * G * jb) return;
  const int j0 = (w % jb) * 32; w /= jb;
  const int slot = node_slot(P.inner, w % G); w /= G;
  const int k = (w % kb) * 32 + lane; const int input = w / kb;
  float* din = P.din[input];
  if (!din || k >= L) return;
  const float* wm = P.W[slot][input];
  const int j1 = min(j0 + 32, Hd);
  float a = 0.0f;
  for (int j = j0; j < j1; ++j) a += s_dpre[slot * Hd + j] * wm[(size_t)j * L + k];
  atomicAdd(din + k, a);
}

__global__ void __launch_bounds__(kNodeThreads) tree_node_bwd_kernel(const ltb_tree_node P, int n_w) { node_bwd_body<false>(P, n_w, (int)blockIdx.x); }
__global__ void __launch_bounds__(kNodeThreads) tree_nodes_bwd_kernel(const ltb_tree_node* nodes) {
  const ltb_tree_node& P = node_to_shared(nodes, (int)blockIdx.y);
  const int G = P.inner ? 5 : 3, n_w = (G * P.hidden + kNodeWarps - 1) / kNodeWarps;
  const bool any_din = P.din[0] || (P.inner && P.din[1]);
  const int x_warps = any_din ? (P.inner ? 2 : 1) * ((P.in_len + 31) / 32) * G * ((P.hidden + 31) / 32) : 0;
  if ((int)blockIdx.x >= n_w + (x_warps + kNodeWarps - 1) / kNodeWarps) return;
  node_bwd_body<true>(P, n_w, (int)blockIdx.x);
}

}  // namespace ltb

extern "C" {

static int tree_node_check(const ltb_tree_node* n, const char* who) {
  LTB_REQUIRE(n, "tree_node: null node");
  const int G = n->inner ? 5 : 3;
  LTB_REQUIRE(n->hidden > 0 && n->hidden <= kNodeMaxHidden && n->in_len > 0 && n->classes > 0 && n->classes <= 32, "tree_node: hidden must be 1..512, classes 1..32");
  LTB_REQUIRE(n->in[0] && (!n->inner || (n->in[1] && n->cl && n->cr)) && n->Why && n->by && n->score && n->gates && n->c && n->tc && n->h && n->logp && n->loss,
              "tree_node: missing operand");
  for (int g = 0; g < G; ++g) {
    const int slot = n->inner ? g : (g == 0 ? 0 : g + 2);
    LTB_REQUIRE(n->W[slot][0] && n->bias[slot] && (!n->inner || n->W[slot][1]), "tree_node: missing gate matrix or bias");
  }
  (void)who;
  return LTB_OK;
}

int ltb_tree_node_fwd(const ltb_tree_node* n) {
  LTB_INITED();
  if (int rc = tree_node_check(n, "ltb_tree_node_fwd")) return rc;
  const int G = n->inner ? 5 : 3;
  LTB_LAUNCH(tree_node_fwd_kernel, (unsigned)ceil_div(G * n->hidden, kNodeWarps), kNodeThreads, 0, *n);
  return LTB_OK;
}

int ltb_tree_node_bwd(const ltb_tree_node* n) {
  LTB_INITED();
  if (int rc = tree_node_check(n, "ltb_tree_node_bwd")) return rc;
  const int G = n->inner ? 5 : 3;
  LTB_REQUIRE(n->dc && n->dh && n->dloss && n->dWhy && n->dby, "ltb_tree_node_bwd: missing gradient operand");
  for (int g = 0; g < G; ++g) {
    const int slot = n->inner ? g : (g == 0 ? 0 : g + 2);
    LTB_REQUIRE(n->dW[slot][0] && n->dbias[slot] && (!n->inner || n->dW[slot][1]), "ltb_tree_node_bwd: missing gate gradient");
  }
  const int n_w = (int)ceil_div(G * n->hidden, kNodeWarps);
  const bool any_din = n->din[0] || (n->inner && n->din[1]);
  const int x_warps = any_din ? (n->inner ? 2 : 1) * (int)ceil_div(n->in_len, 32) * G * (int)ceil_div(n->hidden, 32) : 0;
  LTB_LAUNCH(tree_node_bwd_kernel, (unsigned)(n_w + ceil_div(x_warps, kNodeWarps)), kNodeThreads, 0, *n, n_w);
  return LTB_OK;
}

// One level of a tree -- `count` nodes that do not depend on one another -- in one launch each way.  nodes_host and nodes_dev
// are the same array on the host (read here: checks, grid size) and in device memory (read by the kernels); the nodes of the
// call are [first, first + count).
int ltb_tree_nodes_fwd(const ltb_tree_node* nodes_host, const ltb_tree_node* nodes_dev, int first, int count) {
  LTB_INITED(); LTB_REQUIRE(nodes_host && nodes_dev && first >= 0 && count > 0, "ltb_tree_nodes_fwd: bad argument");
  for (int at = first; at < first + count; at += kNodesPerLaunch) {
    const int n = first + count - at < kNodesPerLaunch ? first + count - at : kNodesPerLaunch;
    int ctas = 1;
    for (int i = at; i < at + n; ++i) {
      if (int rc = tree_node_check(nodes_host + i, "ltb_tree_nodes_fwd")) return rc;
      const int c = (int)ceil_div((nodes_host[i].inner ? 5 : 3) * nodes_host[i].hidden, kNodeWarps);
      if (c > ctas) ctas = c;
    }
    LTB_LAUNCH(tree_nodes_fwd_kernel, dim3((unsigned)ctas, (unsigned)n), kNodeThreads, 0, nodes_dev + at);
  }
  return LTB_OK;
}
int ltb_tree_nodes_bwd(const ltb_tree_node* nodes_host, const ltb_tree_node* nodes_dev, int first, int count) {
  LTB_INITED(); LTB_REQUIRE(nodes_host && nodes_dev && first >= 0 && count > 0, "ltb_tree_nodes_bwd: bad argument");
  for (int at = first; at < first + count; at += kNodesPerLaunch) {
    const int n = first + count - at < kNodesPerLaunch ? first + count - at : kNodesPerLaunch;
    int ctas = 1;
    for (int i = at; i < at + n; ++i) {
      const ltb_tree_node* q = nodes_host + i;
      if (int rc = tree_node_check(q, "ltb_tree_nodes_bwd")) return rc;
      const int G = q->inner ? 5 : 3;
      LTB_REQUIRE(q->dc && q->dh && q->dloss && q->dWhy && q->dby, "ltb_tree_nodes_bwd: missing gradient operand");
      for (int g = 0; g < G; ++g) {
        const int slot = q->inner ? g : (g == 0 ? 0 : g + 2);
        LTB_REQUIRE(q->dW[slot][0] && q->dbias[slot] && (!q->inner || q->dW[slot][1]), "ltb_tree_nodes_bwd: missing gate gradient");
      }
      const bool any_din = q->din[0] || (q->inner && q->din[1]);
      const int x_warps = any_din ? (q->inner ? 2 : 1) * (int)ceil_div(q->in_len, 32) * G * (int)ceil_div(q->hidden, 32) : 0;
      const int c = (int)ceil_div(G * q->hidden, kNodeWarps) + (int)ceil_div(x_warps, kNodeWarps);
      if (c > ctas) ctas = c;
    }
    LTB_LAUNCH(tree_nodes_bwd_kernel, dim3((unsigned)ctas, (unsigned)n), kNodeThreads, 0, nodes_dev + at);
  }
  return LTB_OK;
}

}  // extern "C"
