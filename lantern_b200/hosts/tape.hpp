// Host-side runtime for hand-mirrored "as-if-generated" Lantern programs.
//
// Lantern's TensorR operators run the forward computation, call the continuation, and then run the
// gradient code as the continuation returns (shift/reset, src/main/scala/lantern/TensorDifferentiation.scala:
// 1146-1506).  The staged result is straight-line code: forward calls in program order followed by the
// *_grad calls in exactly the reverse order.  `Tape` reproduces that order without a staging compiler: every
// operator issues its forward backend call immediately and pushes its gradient call; backward() pops them.
//
// All tensor math goes through the C ABI of include/lantern_b200.h (LTB_FN picks the library the file is
// compiled against), so this file contains no arithmetic of its own.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <vector>

#include "../../include/lantern_b200.h"

#define BK(name) LTB_FN(name)

namespace lantern_host {

// TensorR: value + gradient (TD.scala:1146-1160). rank 1, 2 or 4.
struct TR {
  float* x = nullptr;
  float* d = nullptr;
  int shape[4] = {1, 1, 1, 1};
  int rank = 0;
  bool is_input = false;   // leaf without gradient (TensorR.isInput)
  int64_t count() const { int64_t n = 1; for (int i = 0; i < rank; ++i) n *= shape[i]; return n; }
};

inline float* alloc_value(int64_t n) { return (float*)BK(malloc_uninit)((size_t)n * 4); }
// Gradient buffers of one step are carved out of ONE zero-filled block taken at the start of the step (the reference
// zeroes its whole arena span once per step, DslAPI.scala:475-484: one bulk fill instead of one small fill per tensor, each
// of which is a node of its own in the recorded step).  The block's size is what the previous step of the same program
// asked for; a request that does not fit (first step, data-dependent programs) is served by the library's zeroing malloc.
struct ZeroPool { char* base = nullptr; size_t cap = 0, used = 0, asked = 0; };
inline ZeroPool& zero_pool() { static ZeroPool p; return p; }
inline void zero_pool_begin(size_t bytes) {
  ZeroPool& p = zero_pool();
  p.base = bytes ? (char*)BK(malloc)(bytes) : nullptr;
  p.cap = p.base ? bytes : 0; p.used = 0; p.asked = 0;
}
inline size_t zero_pool_end() { ZeroPool& p = zero_pool(); size_t a = p.asked; p.base = nullptr; p.cap = p.used = 0; return a; }
inline float* alloc_zero(int64_t n) {
  ZeroPool& p = zero_pool();
  const size_t bytes = ((size_t)n * 4 + 255) / 256 * 256;
  p.asked += bytes;
  if (p.used + bytes <= p.cap) { float* r = (float*)(p.base + p.used); p.used += bytes; return r; }
  return (float*)BK(malloc)((size_t)n * 4);
}

// The gradient buffer of an activation.  Large ones (4 MB and more: the feature maps of the convolutional programs) are not
// zero-filled but declared unset (ltb_grad_unset): the operator that would be the first to add into the buffer writes it
// instead, and any other use fills it with zeros first, so results do not depend on the choice.  Off while tracing (the trace
// reads every buffer) and by deferred_grads() = false.
inline bool& tracing();
inline bool& deferred_grads() { static bool on = true; return on; }
inline float* alloc_grad(int64_t n) {
  if (n >= (1 << 20) && deferred_grads() && !tracing()) {
    float* p = alloc_value(n);
    if (p) BK(grad_unset)(p, n);
    return p;
  }
  return alloc_zero(n);
}

// Debug trace: when on, every tensor an operator allocates is remembered so that a step can be dumped
// (per-tensor checksums of value and gradient) and two libraries compared operator by operator.
inline bool& tracing() { static bool on = false; return on; }
inline std::vector<TR>& trace_list() { static std::vector<TR> v; return v; }
inline TR traced(const TR& t) { if (tracing()) trace_list().push_back(t); return t; }

inline TR make(std::initializer_list<int> shp, bool with_grad = true) {
  TR t; t.rank = (int)shp.size(); int i = 0; for (int s : shp) t.shape[i++] = s;
  t.x = alloc_value(t.count());
  if (with_grad) t.d = alloc_grad(t.count());
  return traced(t);
}
inline TR view(const TR& t, std::initializer_list<int> shp) {   // Tensor.resize: same buffers, new shape
  TR v = t; v.rank = (int)shp.size(); int i = 0; for (int s : shp) v.shape[i++] = s; for (; i < 4; ++i) v.shape[i] = 1;
  return v;
}

struct Tape {
  std::vector<std::function<void()>> grads;
  void push(std::function<void()> f) { grads.push_back(std::move(f)); }
  void backward() { for (auto it = grads.rbegin(); it != grads.rend(); ++it) (*it)(); grads.clear(); }

  // convBBP, TD.scala:1394-1410
  TR conv(const TR& in, const TR& w, const TR* bias, int stride, int pad) {
    int N = in.shape[0], C = in.shape[1], H = in.shape[2], W = in.shape[3], K = w.shape[0], R = w.shape[2], S = w.shape[3];
    TR y = make({N, K, (H + 2 * pad - R) / stride + 1, (W + 2 * pad - S) / stride + 1});
    BK(conv2d_fwd)(in.x, w.x, bias ? bias->x : nullptr, y.x, N, C, H, W, K, R, S, stride, stride, pad, pad);
    float* dbias = bias ? bias->d : nullptr;
    push([=] { BK(conv2d_bwd)(in.x, in.is_input ? nullptr : in.d, w.x, w.d, dbias, y.d, N, C, H, W, K, R, S, stride, stride, pad, pad); });
    return y;
  }
  // batchNorm, TD.scala:1324-1329
  TR batch_norm(const TR& in, const TR& gamma, const TR& beta, float* run_mean, float* run_var) {
    int N = in.shape[0], C = in.shape[1], HW = in.shape[2] * in.shape[3];
    TR y = make({N, C, in.shape[2], in.shape[3]});
    float* sm = alloc_value(C); float* si = alloc_value(C);
    BK(bn_train_fwd)(in.x, y.x, gamma.x, beta.x, run_mean, run_var, sm, si, N, C, HW, 1e-5f, 0.1f);
    push([=] { BK(bn_bwd)(in.x, in.is_input ? nullptr : in.d, y.d, gamma.x, gamma.d, beta.d, sm, si, N, C, HW); });
    return y;
  }
  // relu, TD.scala:1276-1284
  TR relu(const TR& in, bool in_place) {
    int64_t n = in.count();
    if (in_place) {
      BK(unary)(LTB_RELU, in.x, in.x, n);
      push([=] { BK(unary_grad)(LTB_RELU, in.x, in.d, in.x, in.d, n, 1); });
      return in;
    }
    TR y = in; y.x = alloc_value(n); y.d = alloc_grad(n); y.is_input = false; traced(y);
    BK(unary)(LTB_RELU, in.x, y.x, n);
    push([=] { BK(unary_grad)(LTB_RELU, in.x, in.d, y.x, y.d, n, 0); });
    return y;
  }
  TR unary(int op, const TR& in) {     // tanh / sigmoid / exp / log, TD.scala:1252-1316
    int64_t n = in.count();
    TR y = in; y.x = alloc_value(n); y.d = alloc_grad(n); y.is_input = false; traced(y);
    BK(unary)(op, in.x, y.x, n);
    push([=] { if (!in.is_input) BK(unary_grad)(op, in.x, in.d, y.x, y.d, n, 0); });
    return y;
  }
  // maxPoolBK, TD.scala:1413-1423
  TR max_pool(const TR& in, int k, int s) {
    int N = in.shape[0], C = in.shape[1], H = in.shape[2], W = in.shape[3];
    TR y = make({N, C, (H - k) / s + 1, (W - k) / s + 1});
    int32_t* idx = (int32_t*)BK(malloc_uninit)((size_t)y.count() * 4);
    BK(maxpool_fwd)(in.x, y.x, idx, N, C, H, W, k, k, s, s, 0);
    int64_t n_out = y.count();
    push([=] { if (!in.is_input) BK(maxpool_bwd)(in.d, y.d, idx, n_out); });
    return y;
  }
  // averagePoolBK, TD.scala:1385-1391
  TR avg_pool(const TR& in, int k, int s) {
    int N = in.shape[0], C = in.shape[1], H = in.shape[2], W = in.shape[3];
    TR y = make({N, C, (H - k) / s + 1, (W - k) / s + 1});
    BK(avgpool_fwd)(in.x, y.x, N, C, H, W, k, k, s, s);
    push([=] { if (!in.is_input) BK(avgpool_bwd)(in.d, y.d, N, C, H, W, k, k, s, s); });
    return y;
  }
  // broadcasting binary operators, TD.scala:1162-1218 (shapes padded to a common rank by dimBroadcast)
  TR binary(int op, const TR& a, const TR& b) {
    int rank = a.rank > b.rank ? a.rank : b.rank;
    struct Sh { int a[4], b[4], r[4]; } s;
    for (int i = 0; i < rank; ++i) {
      int ia = i - (rank - a.rank), ib = i - (rank - b.rank);
      s.a[i] = ia >= 0 ? a.shape[ia] : 1; s.b[i] = ib >= 0 ? b.shape[ib] : 1;
      s.r[i] = s.a[i] > s.b[i] ? s.a[i] : s.b[i];
    }
    TR y; y.rank = rank; for (int i = 0; i < rank; ++i) y.shape[i] = s.r[i];
    y.x = alloc_value(y.count()); y.d = alloc_grad(y.count()); traced(y);
    BK(ew_binary)(op, a.x, s.a, b.x, s.b, y.x, rank);
    push([=] { BK(ew_binary_grad)(op, a.x, a.is_input ? nullptr : a.d, s.a, b.x, b.is_input ? nullptr : b.d, s.b, y.d, rank); });
    return y;
  }
  // plusBias, TD.scala:1220-1226 region / CPU.scala:281-288: in place on `main`
  TR plus_bias(const TR& main, const TR& bias) {
    struct Sh { int m[4], b[4]; } s;
    int rank = main.rank;
    for (int i = 0; i < rank; ++i) { int ib = i - (rank - bias.rank); s.m[i] = main.shape[i]; s.b[i] = ib >= 0 ? bias.shape[ib] : 1; }
    BK(plus_bias)(main.x, s.m, bias.x, s.b, rank);
    push([=] { if (!bias.is_input) BK(plus_bias_grad)(bias.d, s.b, main.d, s.m, rank); });
    return main;
  }
  // dot (2,2) and (2,1), TD.scala:1220-1226
  // act(W0.a (+ W1.b) + bias) in one call and one gradient call (an LSTM gate); b == nullptr: one product only.
  // Equivalent to unary(act, plus_bias(plus_bias(dot(W0, a), dot(W1, b)), bias)); act == -1: no activation.
  TR affine_act(int act, const TR& W0, const TR& a, const TR* W1, const TR* b, const TR& bias) {
    const int rows = W0.shape[0], c0 = W0.shape[1], c1 = W1 ? W1->shape[1] : 0;
    TR y = make({rows});
    const float *w1x = W1 ? W1->x : nullptr, *bx = b ? b->x : nullptr;
    float *w1d = W1 ? W1->d : nullptr, *bd = (b && !b->is_input) ? b->d : nullptr;
    BK(affine_act)(W0.x, a.x, c0, w1x, bx, c1, bias.x, act, y.x, rows);
    float* ad = a.is_input ? nullptr : a.d;
    push([=] { BK(affine_act_grad)(W0.x, W0.d, a.x, ad, c0, w1x, w1d, bx, bd, c1, bias.d, act, y.x, y.d, rows); });
    return y;
  }
  // Batched: act(x0 W0 (+ x1 W1) + bias) over the rows of x0 / x1, weights stored [in, out]; one call forward, one backward.
  TR affine_act_rows(int act, const TR& x0, const TR& W0, const TR* x1, const TR* W1, const TR& bias) {
    const int batch = x0.shape[0], c0 = x0.shape[1], width = W0.shape[1], c1 = x1 ? x1->shape[1] : 0;
    TR y = make({batch, width});
    const float *x1x = x1 ? x1->x : nullptr, *w1x = W1 ? W1->x : nullptr;
    float *x1d = (x1 && !x1->is_input) ? x1->d : nullptr, *w1d = W1 ? W1->d : nullptr;
    float* x0d = x0.is_input ? nullptr : x0.d;
    BK(affine_act_rows)(x0.x, W0.x, c0, x1x, w1x, c1, bias.x, act, y.x, batch, width);
    push([=] { BK(affine_act_rows_grad)(x0.x, x0d, W0.x, W0.d, c0, x1x, x1d, w1x, w1d, c1, bias.d, act, y.x, y.d, batch, width); });
    return y;
  }
  // cell = i*u (+ fl*cl + fr*cr), hidden = o*tanh(cell) in one call and one gradient call; the child operands are null for a leaf.
  void lstm_cell(const TR& i, const TR& u, const TR* fl, const TR* cl, const TR* fr, const TR* cr, const TR& o, TR* cell, TR* hidden) {
    const int n = (int)i.count();
    TR c = make({n}), h = make({n});
    float* tc = alloc_value(n);
    const float *flx = fl ? fl->x : nullptr, *clx = cl ? cl->x : nullptr, *frx = fr ? fr->x : nullptr, *crx = cr ? cr->x : nullptr;
    float *fld = fl ? fl->d : nullptr, *cld = cl ? cl->d : nullptr, *frd = fr ? fr->d : nullptr, *crd = cr ? cr->d : nullptr;
    BK(lstm_cell)(i.x, u.x, flx, clx, frx, crx, o.x, c.x, tc, h.x, n);
    push([=] { BK(lstm_cell_grad)(i.x, i.d, u.x, u.d, flx, fld, clx, cld, frx, frd, crx, crd, o.x, o.d, tc, c.d, h.d, n); });
    *cell = c; *hidden = h;
  }
  // The whole unrolled vanilla RNN (cell, output layer, logSoftmax + NLL summed over steps and batch) as ONE forward call and
  // one backward call: x [T][B][V], targets y [T][B], weights stored [in, out]; the initial hidden state is zero.
  TR rnn_sequence(const TR& x, const int32_t* y, const TR& Wxh, const TR& Whh, const TR& bh, const TR& Who, const TR& bo, int T, int B) {
    const int V = Wxh.shape[0], H = Wxh.shape[1];
    TR loss = make({1});
    float* h = alloc_value((int64_t)T * B * H); float* logp = alloc_value((int64_t)T * B * V);
    BK(rnn_seq_fwd)(x.x, y, nullptr, Wxh.x, Whh.x, bh.x, Who.x, bo.x, h, logp, loss.x, T, B, V, H);
    push([=] { BK(rnn_seq_bwd)(x.x, y, nullptr, Whh.x, Who.x, h, logp, loss.d, Wxh.d, Whh.d, bh.d, Who.d, bo.d, T, B, V, H); });
    return loss;
  }
  // One node of the binary tree LSTM as ONE forward call and one backward call (ltb_tree_node_fwd / _bwd).  W and bias are
  // indexed by gate slot (i, fl, fr, o, u; a leaf leaves fl and fr empty and has one input); in0 / in1 are the children's first
  // state vector (or the embedding row), cl / cr their second one; the node's loss is nll + loss_l + loss_r.
  struct NodeOut { TR loss, cell, hidden; };
  NodeOut tree_node(bool inner, bool classify_cell, const TR& in0, const TR* in1, const TR (&W)[5][2], const TR (&bias)[5], const TR* cl, const TR* cr,
                    const TR& Why, const TR& by, const int32_t* score, const TR* loss_l, const TR* loss_r) {
    const int Hd = Why.shape[1], K = Why.shape[0], L = (int)in0.count();
    const int64_t pitch = ((int64_t)Hd + 63) / 64 * 64;
    float* vals = alloc_value(8 * pitch + 64);                     // gates [5], c, tc, h, then logp and the loss
    float* grads = alloc_zero(2 * pitch + 64);                     // dc, dh, dloss
    ltb_tree_node n = {};
    n.hidden = Hd; n.in_len = L; n.classes = K; n.inner = inner ? 1 : 0; n.classify_cell = classify_cell ? 1 : 0;
    n.in[0] = in0.x; n.din[0] = in0.is_input ? nullptr : in0.d;
    if (inner) { n.in[1] = in1->x; n.din[1] = in1->is_input ? nullptr : in1->d; n.cl = cl->x; n.cr = cr->x; n.dcl = cl->d; n.dcr = cr->d; }
    for (int g = 0; g < 5; ++g) {
      if (!inner && (g == 1 || g == 2)) continue;
      for (int k = 0; k < (inner ? 2 : 1); ++k) { n.W[g][k] = W[g][k].x; n.dW[g][k] = W[g][k].d; }
      n.bias[g] = bias[g].x; n.dbias[g] = bias[g].d;
    }
    n.Why = Why.x; n.by = by.x; n.dWhy = Why.d; n.dby = by.d; n.score = score;
    if (loss_l) { n.loss_l = loss_l->x; n.dloss_l = loss_l->d; }
    if (loss_r) { n.loss_r = loss_r->x; n.dloss_r = loss_r->d; }
    n.gates = vals; n.c = vals + 5 * pitch; n.tc = vals + 6 * pitch; n.h = vals + 7 * pitch; n.logp = vals + 8 * pitch; n.loss = vals + 8 * pitch + 32;
    n.dc = grads; n.dh = grads + pitch; n.dloss = grads + 2 * pitch;
    BK(tree_node_fwd)(&n);
    push([=] { BK(tree_node_bwd)(&n); });
    NodeOut out;
    out.cell.rank = out.hidden.rank = out.loss.rank = 1;
    out.cell.shape[0] = out.hidden.shape[0] = Hd; out.loss.shape[0] = 1;
    out.cell.x = n.c; out.cell.d = grads; out.hidden.x = n.h; out.hidden.d = grads + pitch; out.loss.x = n.loss; out.loss.d = grads + 2 * pitch;
    traced(out.cell); traced(out.hidden); traced(out.loss);
    return out;
  }
  TR dot(const TR& a, const TR& b) {
    if (b.rank == 2) {
      int m = a.shape[0], k = a.shape[1], n = b.shape[1];
      TR y = make({m, n});
      BK(mm_dot)(a.x, b.x, y.x, m, k, n);
      push([=] {
        if (!a.is_input) BK(add_dot_trans2)(a.d, y.d, b.x, m, k, n);
        if (!b.is_input) BK(add_dot_trans1)(b.d, a.x, y.d, m, k, n);
      });
      return y;
    }
    int m = a.shape[0], k = a.shape[1];
    TR y = make({m});
    BK(mv_dot)(a.x, b.x, y.x, m, k);
    push([=] {
      if (!a.is_input) BK(add_cartesian)(a.d, b.x, y.d, m, k);
      if (!b.is_input) BK(add_composition)(b.d, a.x, y.d, m, k);
    });
    return y;
  }
  // gemm, TD.scala:1228-1233
  TR gemm(const TR& a, bool ta, const TR& b, bool tb, float alpha) {
    int M = ta ? a.shape[1] : a.shape[0], K = ta ? a.shape[0] : a.shape[1], N = tb ? b.shape[0] : b.shape[1];
    TR y = make({M, N});
    BK(gemm)(a.x, ta, b.x, tb, alpha, y.x, M, N, K);
    push([=] { BK(gemm_grad)(a.x, a.is_input ? nullptr : a.d, ta, b.x, b.is_input ? nullptr : b.d, tb, alpha, y.d, M, N, K); });
    return y;
  }
  // dropout, TD.scala:1437-1445
  TR dropout(const TR& in, float p) {
    int64_t n = in.count();
    TR y = in; y.x = alloc_value(n); y.d = alloc_zero(n);
    float* mask = alloc_value(n);
    BK(dropout)(in.x, y.x, mask, p, n);
    push([=] { if (!in.is_input) BK(dropout_grad)(in.d, mask, y.d, n); });
    return y;
  }
  // concat along dim 1 of 4-D tensors, TD.scala:1481-1490
  TR concat1(const TR& a, const TR& b) {
    int N = a.shape[0], inner = a.shape[2] * a.shape[3];
    TR y = make({N, a.shape[1] + b.shape[1], a.shape[2], a.shape[3]});
    struct P { const float* in[2]; float* din[2]; int dims[2]; } p = {{a.x, b.x}, {a.d, b.d}, {a.shape[1], b.shape[1]}};
    BK(concat)(y.x, p.in, p.dims, 2, N, inner);
    push([=] { BK(concat_grad)(p.din, y.d, p.dims, 2, N, inner); });
    return y;
  }
  // logSoftmaxB, nllLossB, sum, mean: TD.scala:1352-1383, 1492-1506
  TR log_softmax(const TR& in) {
    int r = in.shape[0], c = in.shape[1];
    TR y = make({r, c});
    BK(log_softmax)(in.x, y.x, r, c);
    push([=] { BK(log_softmax_grad)(in.d, y.x, y.d, r, c); });
    return y;
  }
  TR nll(const TR& in, const int32_t* target) {
    int r = in.shape[0], c = in.shape[1];
    TR y = make({r});
    BK(nll)(in.x, target, y.x, r, c);
    push([=] { BK(nll_grad)(in.d, y.d, target, r, c); });
    return y;
  }
  TR sum(const TR& in) {
    int64_t n = in.count();
    TR y = make({1});
    BK(sum)(in.x, y.x, n);
    push([=] { BK(sum_grad)(in.d, y.d, n); });
    return y;
  }
  TR mean(const TR& in) {
    int64_t n = in.count();
    TR y = make({1});
    BK(mean)(in.x, y.x, n);
    push([=] { BK(mean_grad)(in.d, y.d, n); });
    return y;
  }
};

}  // namespace lantern_host
