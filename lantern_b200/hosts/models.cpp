// Hand-mirrored host programs for the reference's training apps.
//
// The Scala generator cannot run without a JVM, so each program below is written the way the staged output
// of the corresponding app is structured: parameters allocated first (before the arena mark), then per batch
// upload -> forward -> seed gradient -> backward (reverse order) -> loss read-back -> SGD over every parameter
// tensor -> arena reset.  References:
//   MNIST CNN   src/main/scala/lantern/NIPS18App/MnistCNN.scala:36-60, 168-194 and its shipped output
//               src/out/NIPS18evaluation/evaluationCNN/Lantern/Lantern.cpp
//   ResNet-50   src/main/scala/lantern/PLDI19APP/resnet50FromOnnx.scala:135-214 with the architecture of
//               src/out/PLDI19evaluation/resnet50/pytorch/resnet50.py:55-160 (op mapping ONNXLib.scala:833-1071)
//   SqueezeNet  src/main/scala/lantern/PLDI19APP/squeezenetFromOnnx.scala:111-226 with the architecture of
//               src/out/PLDI19evaluation/squeezenet/pytorch/pytorch_squeeze_cifar10.py:21-92
// The exported C functions carry the prefix given by HOST_FN (ltbh_ for the CUDA library).
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "loader.hpp"
#include "tape.hpp"

#ifndef HOST_FN
#define HOST_FN(name) ltbh_##name
#endif

using namespace lantern_host;

namespace {

struct ParamDecl { std::vector<int> shape; int init; float scale; int64_t count; int64_t offset; bool state = false; };   // state: a running statistic, not trained (no gradient, not all-reduced)
enum { INIT_ZERO = 0, INIT_RAND = 1, INIT_ONE = 2 };

struct Model {
  virtual ~Model() {}
  std::string name;
  int batch = 0;
  int in_c = 0, in_h = 0, in_w = 0;
  int64_t label_count = 0;     // int32 targets per step (0: one per sample)
  std::vector<ParamDecl> decls;
  float* slab_x = nullptr;   // all parameter tensors, contiguous (each padded to 64 floats)
  float* slab_d = nullptr;   // their gradients, same layout
  int64_t slab_count = 0;
  void* mark = nullptr;
  float* stage_x = nullptr;  // pinned staging for the batch
  int32_t* stage_y = nullptr;
  float* loss_host = nullptr;  // pinned, 1 float
  void* graph = nullptr;
  bool use_graph = false;
  float graph_lr = 0.f;
  size_t zero_bytes = 0;       // bytes of zero-initialised gradient buffers the largest step so far asked for (0: not known yet)
  bool early_reduce = false;   // this step runs data-parallel with an update: finished gradient ranges are summed during backward
  bool branches = true;        // independent runs of calls (shortcut convolutions) are issued as branch regions
  bool fused_cells = true;     // recursive models: one call per gate (ltb_affine_act) instead of one per operator
  bool level_batches = true;   // tree-LSTM with whole nodes per call: a whole LEVEL of the tree per call (ltb_tree_nodes_fwd)
  bool whole_sequence = true;  // with fused cells: the vanilla RNN's whole unrolled sequence (ltb_rnn_seq_fwd) and a whole tree node (ltb_tree_node_fwd) in one call
  bool resident = false;       // read the batch from dev_x/dev_y instead of uploading it
  float* dev_x = nullptr; int32_t* dev_y = nullptr;
  float* dev_loss = nullptr;   // the loss of the last step, kept outside the arena span that the step resets
  // The classifier's output of the last step (CNN programs: batch x classes), copied out of the arena span that the step
  // resets so that predictions (arg-max per row) can be read afterwards.
  float* dev_logits = nullptr; int64_t logit_count = 0; TR last_logits;
  // Two steps in flight (submit / collect): staging pair p = step & 1; marker p = its upload done, marker 2 + p = its step done.
  bool feeding = false;
  int64_t submitted = 0;
  float* feed_x[2] = {nullptr, nullptr}; int32_t* feed_y[2] = {nullptr, nullptr}; float* feed_loss = nullptr;
  float* dstage_x[2] = {nullptr, nullptr}; int32_t* dstage_y[2] = {nullptr, nullptr};   // device side of the two staging pairs (uploads run beside the step before)

  int declare(std::initializer_list<int> shape, int init, float scale = 0.f) {
    ParamDecl d; d.shape.assign(shape.begin(), shape.end()); d.init = init; d.scale = scale;
    d.count = 1; for (int s : d.shape) d.count *= s;
    d.offset = slab_count;
    slab_count += (d.count + 63) / 64 * 64;
    decls.push_back(d);
    return (int)decls.size() - 1;
  }
  TR P(int i) const {
    const ParamDecl& d = decls[i];
    TR t; t.rank = (int)d.shape.size(); for (int k = 0; k < t.rank; ++k) t.shape[k] = d.shape[k];
    t.x = slab_x + d.offset; t.d = slab_d + d.offset; return t;
  }
  // Allocation and initialisation in declaration order; rand() is consumed only by INIT_RAND tensors, in order,
  // after srand(seed) -- the order MnistCNN's generated code draws its weights in.
  void finalize(int seed) {
    slab_x = alloc_zero(slab_count);
    slab_d = alloc_zero(slab_count);
    bool first = true;
    for (auto& d : decls) {
      if (d.init == INIT_RAND) { BK(randinit)(slab_x + d.offset, d.count, d.scale, first ? seed : -1); first = false; }
      else if (d.init == INIT_ONE) BK(fill)(slab_x + d.offset, 1.0f, d.count);
    }
    if (first && seed >= 0) srand((unsigned)seed);
    if (label_count == 0) label_count = batch;
    stage_x = (float*)BK(host_alloc)((size_t)batch * in_c * in_h * in_w * 4);
    stage_y = (int32_t*)BK(host_alloc)((size_t)label_count * 4);
    loss_host = (float*)BK(host_alloc)(4);
    dev_x = alloc_value((int64_t)batch * in_c * in_h * in_w);
    dev_y = (int32_t*)BK(malloc_uninit)((size_t)label_count * 4);
    dev_loss = alloc_value(1);
    for (int p = 0; p < 2; ++p) { dstage_x[p] = alloc_value((int64_t)batch * in_c * in_h * in_w); dstage_y[p] = (int32_t*)BK(malloc_uninit)((size_t)label_count * 4); }
    if (logit_count > 0) dev_logits = alloc_value(logit_count);
    mark = BK(mark)();
  }
  virtual TR forward(Tape& t, const TR& x, const int32_t* y) = 0;

  // One training step's device work, in the order of the generated programs.
  void enqueue(float lr, bool update) {
    Tape tape;
    zero_pool_begin(zero_bytes);
    int64_t nin = (int64_t)batch * in_c * in_h * in_w;
    TR x; x.rank = 4; x.shape[0] = batch; x.shape[1] = in_c; x.shape[2] = in_h; x.shape[3] = in_w; x.is_input = true;
    int32_t* y;
    if (resident) {           // batch already in device memory (measurement of the device-side step alone)
      x.x = dev_x; y = dev_y;
    } else {                  // the generated programs upload every batch: resnet50FromOnnx.scala:173-174
      x.x = alloc_value(nin);
      y = (int32_t*)BK(malloc_uninit)((size_t)label_count * 4);
      BK(h2d)(x.x, stage_x, (size_t)nin * 4);
      BK(h2d)(y, stage_y, (size_t)label_count * 4);
    }
    early_reduce = update && BK(comm_world)() > 1;
    last_logits = TR();
    TR loss = forward(tape, x, y);
    if (dev_logits && last_logits.x && last_logits.count() == logit_count) BK(d2d)(dev_logits, last_logits.x, (size_t)logit_count * 4);
    BK(fill)(loss.d, 1.0f, 1);                       // gradR_loss: y.d.setAsOne(), TD.scala:1763-1780
    BK(d2d)(dev_loss, loss.x, 4);
    tape.backward();
    BK(d2h_async)(loss_host, dev_loss, 4);
    if (update) apply_update(lr);
    if (tracing()) dump_trace();
    { const size_t asked = zero_pool_end(); if (asked > zero_bytes) zero_bytes = asked; }   // the largest step so far: a smaller tree leaves part of the block unused
    BK(reset)(mark);
  }
  // Data parallelism: pushed on the tape at a point of the forward pass, this fires in the backward pass once every layer
  // after that point is done, i.e. when the gradients of the parameters declared from `first_decl` up to offset `hi` of the
  // slab are final; their all-reduce then overlaps the rest of the backward pass (measured on 2 GPUs: 5.64 -> 5.47 ms per step).
  void reduce_when_final(Tape& t, int first_decl, int64_t hi) {
    if (!early_reduce) return;
    float* d = slab_d + decls[first_decl].offset; const int64_t n = hi - decls[first_decl].offset;
    t.push([=] { BK(allreduce_begin)(d, n); });
  }
  // SGD of the CNN apps (NNModule.scala:265-287: geam x -= lr*d, then d = 0), fused with the gradient all-reduce when the
  // communicator has more than one rank.
  virtual void apply_update(float lr) {
    if (BK(comm_world)() > 1) BK(allreduce_sgd_step)(slab_x, slab_d, lr, slab_count);
    else BK(sgd_step)(slab_x, slab_d, lr, slab_count);
  }
  std::string trace_text;
  // One line per operator output, in forward order (read back before the reset): index, element count, shape, sum|x|,
  // sum|d|, non-zero counts, smallest non-zero |x|, then sum x^2, sum d^2 and eight signed sums of x and of d.  A signed sum
  // is sum_i s_k(i) v_i with s_k(i) = +-1 from a fixed hash of (i, k): for two tensors a, b the mean over k of
  // (S_k(a) - S_k(b))^2 estimates |a - b|^2, so two libraries can be compared tensor by tensor from these few numbers.
  void dump_trace() {
    trace_text.clear();
    std::vector<float> h;
    int idx = 0;
    for (const TR& t : trace_list()) {
      int64_t n = t.count(); h.resize((size_t)n);
      double ax = 0, ad = 0, minx = 1e30, x2 = 0, d2 = 0, px[8] = {0}, pd[8] = {0}; long long nzx = 0, nzd = 0;
      auto signs = [](int64_t i) { uint64_t z = (uint64_t)i + 0x9E3779B97F4A7C15ull; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); };
      BK(d2h)(h.data(), t.x, (size_t)n * 4);
      for (int64_t i = 0; i < n; ++i) {
        const double v = h[i], a = std::fabs(v); ax += a; x2 += v * v; if (a != 0) { ++nzx; if (a < minx) minx = a; }
        const uint64_t s = signs(i); for (int k = 0; k < 8; ++k) px[k] += ((s >> k) & 1) ? v : -v;
      }
      if (t.d) {
        BK(d2h)(h.data(), t.d, (size_t)n * 4);
        for (int64_t i = 0; i < n; ++i) {
          const double v = h[i]; ad += std::fabs(v); d2 += v * v; nzd += h[i] != 0;
          const uint64_t s = signs(i); for (int k = 0; k < 8; ++k) pd[k] += ((s >> (8 + k)) & 1) ? v : -v;
        }
      }
      char line[1024];
      int w = snprintf(line, sizeof line, "%d %lld [%d,%d,%d,%d] %.9e %.9e %lld %lld %.3e %.9e %.9e", idx++, (long long)n, t.shape[0], t.shape[1], t.shape[2], t.shape[3], ax, ad, nzx, nzd, minx, x2, d2);
      for (int k = 0; k < 8; ++k) w += snprintf(line + w, sizeof line - w, " %.9e", px[k]);
      for (int k = 0; k < 8; ++k) w += snprintf(line + w, sizeof line - w, " %.9e", pd[k]);
      snprintf(line + w, sizeof line - w, "\n");
      trace_text += line;
    }
    trace_list().clear();
  }
  void load(const float* xh, const int32_t* yh) {
    memcpy(stage_x, xh, (size_t)batch * in_c * in_h * in_w * 4);
    memcpy(stage_y, yh, (size_t)label_count * 4);
  }
  int step_async(const float* xh, const int32_t* yh, float lr, bool update) {
    if (!resident && xh) load(xh, yh);
    if (use_graph && update && zero_bytes > 0) {        // the first step runs eagerly: it measures the gradient pool
      if (graph && graph_lr != lr) { BK(graph_destroy)(graph); graph = nullptr; }
      if (!graph) {
        int rc = BK(graph_begin)(); if (rc) return rc;
        enqueue(lr, true);
        graph = BK(graph_end)(); graph_lr = lr;
        if (!graph) return LTB_E_CUDA;
      }
      return BK(graph_launch)(graph);
    }
    enqueue(lr, update);
    return 0;
  }
  float step(const float* xh, const int32_t* yh, float lr, bool update) {
    step_async(xh, yh, lr, update);
    BK(sync)();
    return *loss_host;
  }
  // Training with two steps in flight.  The generated programs upload a batch, run the step and block on the loss copy
  // (resnet50FromOnnx.scala:173-186), so the device idles while the host prepares the next batch.  submit() copies the
  // batch into one of two pinned staging pairs, queues the upload, the step (reading the batch at its fixed device
  // address, so the recorded step is the same every time) and a 4-byte loss copy, and returns; collect(k) waits for
  // step k alone.  The staging pair of step k is refilled by step k + 2, after its upload marker has fired.
  void feed_mode(bool on) {
    if (feeding == on) return;
    if (graph) { BK(graph_destroy)(graph); graph = nullptr; }      // the recorded step reads the batch from another place
    if (on && !feed_loss) {
      const size_t xb = (size_t)batch * in_c * in_h * in_w * 4;
      for (int p = 0; p < 2; ++p) { feed_x[p] = (float*)BK(host_alloc)(xb); feed_y[p] = (int32_t*)BK(host_alloc)((size_t)label_count * 4); }
      feed_loss = (float*)BK(host_alloc)(8);
    }
    if (on) BK(sync)();
    feeding = resident = on;
  }
  // Staging pair for the next submit, free to be written (a loader decodes a batch straight into it).
  int feed_slot(float** x, int32_t** y) {
    feed_mode(true);
    const int p = (int)(submitted & 1);
    if (submitted >= 2) { int rc = BK(marker_wait)(p); if (rc) return rc; }
    *x = feed_x[p]; *y = feed_y[p];
    return 0;
  }
  // xh == nullptr: the caller has filled the pair returned by feed_slot.
  int64_t submit(const float* xh, const int32_t* yh, float lr) {
    float* sx; int32_t* sy;
    if (feed_slot(&sx, &sy)) return -1;
    const int p = (int)(submitted & 1);
    const size_t xb = (size_t)batch * in_c * in_h * in_w * 4;
    if (xh) { memcpy(sx, xh, xb); memcpy(sy, yh, (size_t)label_count * 4); }
    // The upload runs on the copy stream beside the step before it (marker 4 + p: the device staging pair was read for the last
    // time by step submitted - 2; marker p: the upload has left the host staging pair); the compute stream then waits for the
    // upload on the device and moves the batch to where the recorded step reads it.
    const size_t yb = (size_t)label_count * 4;
    if (BK(upload)(dstage_x[p], sx, xb, submitted >= 2 ? 4 + p : -1) || BK(upload)(dstage_y[p], sy, yb, -1) || BK(upload_marker)(p)) return -1;
    if (BK(stream_wait_marker)(p) || BK(d2d)(dev_x, dstage_x[p], xb) || BK(d2d)(dev_y, dstage_y[p], yb) || BK(marker_record)(4 + p)) return -1;
    if (step_async(nullptr, nullptr, lr, true)) return -1;
    if (BK(d2h_async)(feed_loss + p, dev_loss, 4) || BK(marker_record)(2 + p)) return -1;
    return submitted++;
  }
  int collect(int64_t k, float* loss) {
    if (k < 0 || k >= submitted || k + 2 < submitted) return LTB_E_ARG;     // only the last two steps keep their loss
    const int p = (int)(k & 1);
    int rc = BK(marker_wait)(2 + p); if (rc) return rc;
    *loss = feed_loss[p];
    return 0;
  }
};

// ------------------------------------------------------------------------------------------------ MNIST CNN
struct Mnist : Model {
  int c1w, c1b, c2w, c2b, l1w, l1b, l2w, l2b;
  Mnist(int b, int seed) {
    name = "mnist"; batch = b; in_c = 1; in_h = in_w = 28; logit_count = (int64_t)b * 10;
    // Conv2D: uniform(+-sqrt(6/fan_in)) == (rand-0.5)*2*sqrt(6/fan_in), bias 0 (NNModule.scala:128-146);
    // Linear1D: (rand-0.5)/sqrt(in), weight stored [in,out] (NNModule.scala:112-117).
    c1w = declare({10, 1, 5, 5}, INIT_RAND, 2.0f * sqrtf(6.0f / 25.0f));  c1b = declare({10}, INIT_ZERO);
    c2w = declare({20, 10, 5, 5}, INIT_RAND, 2.0f * sqrtf(6.0f / 250.0f)); c2b = declare({20}, INIT_ZERO);
    l1w = declare({320, 50}, INIT_RAND, 1.0f / sqrtf(320.0f)); l1b = declare({50}, INIT_ZERO);
    l2w = declare({50, 10}, INIT_RAND, 1.0f / sqrtf(50.0f));   l2b = declare({10}, INIT_ZERO);
    finalize(seed);
  }
  TR forward(Tape& t, const TR& x, const int32_t* y) override {   // MnistCNN.scala:43-59
    TR b1 = P(c1b), b2 = P(c2b);
    TR s0 = t.conv(x, P(c1w), &b1, 1, 0);
    TR s1 = t.max_pool(t.relu(s0, false), 2, 2);
    TR s2 = t.conv(s1, P(c2w), &b2, 1, 0);
    TR s25 = t.max_pool(t.relu(s2, false), 2, 2);
    TR flat = view(s25, {batch, 320});
    TR s3 = t.dropout(t.plus_bias(t.dot(flat, P(l1w)), P(l1b)), 0.5f);
    TR out = t.plus_bias(t.dot(s3, P(l2w)), P(l2b));
    last_logits = out;
    return t.sum(t.nll(t.log_softmax(out), y));
  }
};

// ------------------------------------------------------------------------------------------------ min-char-rnn
// Vanilla RNN of NNModule.scala:189-200 (VanillaRNNCell = Linear1D2 + tanh, Linear1D) unrolled by DynamicRNNFix
// (NNModule.scala:240-253) as the app VanillaRNN.scala:187-291 uses it: vocabulary 80 one-hot inputs x[T][B][80],
// hidden 100, T = 20 steps, per step  h = tanh(x_t.W1 + h.W2 + b);  o = h.Wo (+)= bo;  loss += sum(nll(logSoftmax(o), y_t));
// Adagrad lr-as-given, clip 5.  The targets arrive as y[t][b] (the generated code gathers them per step from a
// [b][t] host array, NNModule.scala:246-248; the order of the buffer is this host program's choice).
struct VanillaRnn : Model {
  static constexpr int T = 20;
  const int V, Hd;                  // 80 / 100 for the benchmark configuration; 26 / 50 in the reference's shipped generated program
  int w1, w2, bh, wo, bo;
  float* slab_h = nullptr;          // Adagrad accumulators, same layout as the parameter slab
  VanillaRnn(int b, int seed, int vocab, int hidden) : V(vocab), Hd(hidden) {
    name = "rnn"; batch = b; in_c = T; in_h = 1; in_w = V; label_count = (int64_t)T * b;
    w1 = declare({V, Hd}, INIT_RAND, 1.0f / sqrtf((float)V));   w2 = declare({Hd, Hd}, INIT_RAND, 1.0f / sqrtf((float)Hd));
    bh = declare({Hd}, INIT_ZERO);
    wo = declare({Hd, V}, INIT_RAND, 1.0f / sqrtf((float)Hd));  bo = declare({V}, INIT_ZERO);
    finalize(seed);
    slab_h = alloc_zero(slab_count);   // allocated after the mark was taken: move the mark above it
    mark = BK(mark)();
  }
  TR forward(Tape& t, const TR& x, const int32_t* y) override {
    if (fused_cells && whole_sequence)                 // all T steps in one call (ltb_rnn_seq_fwd / _bwd): 4 launches per sequence
      return t.rnn_sequence(x, y, P(w1), P(w2), P(bh), P(wo), P(bo), T, batch);
    TR h = make({batch, Hd});                          // cell.init: zeros
    BK(fill)(h.x, 0.0f, h.count());
    TR loss = make({1});
    BK(fill)(loss.x, 0.0f, 1);
    for (int s = 0; s < T; ++s) {
      TR xt; xt.rank = 2; xt.shape[0] = batch; xt.shape[1] = V; xt.x = x.x + (int64_t)s * batch * V; xt.is_input = true;
      TR o;
      if (fused_cells) {       // the cell and the output layer as one call each (ltb_affine_act_rows)
        TR w2t = P(w2);
        h = t.affine_act_rows(LTB_TANH, xt, P(w1), &h, &w2t, P(bh));
        o = t.affine_act_rows(-1, h, P(wo), nullptr, nullptr, P(bo));
      } else {
        TR pre = t.binary(LTB_ADD, t.binary(LTB_ADD, t.dot(xt, P(w1)), t.dot(h, P(w2))), P(bh));
        h = t.unary(LTB_TANH, pre);
        o = t.plus_bias(t.dot(h, P(wo)), P(bo));
      }
      loss = t.binary(LTB_ADD, loss, t.sum(t.nll(t.log_softmax(o), y + (int64_t)s * batch)));
    }
    return loss;
  }
  void apply_update(float lr) override {               // NNModule.scala:289-295 -> Backend.adagrad_update (TD.scala:377)
    BK(adagrad_update)(slab_x, slab_d, slab_h, lr, 5.0f, 1, slab_count);
  }
};

// ------------------------------------------------------------------------------------------------ TreeLSTM (sentiment)
// PLDI19APP/SentimentTreeLSTM.scala:67-146: Leaf (3 gates from a 300-d embedding), Node (5 gates from the two children),
// Out (5-way classifier at every node), recursion LOOPTM over the (lch, rch) arrays from node 0, losses added up the
// tree, Adagrad lr-as-given with the default clip 1.0 over the 22 tensors, one tree per step.
// One quirk of the app is kept on purpose: Leaf and Node return ArrayBuffer(hidden, cell) and the caller destructures it
// as ArrayBuffer(cell, hidden) (lines 131 and 135), so the classifier reads the cell state and the children's two states
// reach the parent with their roles exchanged.  This program does exactly the same.
// A step's "labels" carry the tree: y[0] = node count n <= 99, then four arrays with a stride of 99 ints: scores (0..4),
// words (row of the embedding table), left child, right child (-1 = none; node 0 is the root).  The embedding table
// (1000 rows x 300, N(0, 0.1), fixed seed) stands in for the GloVe file the app reads; it is data, not a parameter.
struct TreeLstm : Model {
  static constexpr int E = 300, Hd = 150, O = 5, MAXN = 99, VOCAB = 1000;
  int Wi, bi, Wo, bo, Wu, bu;
  int U0i, U1i, bbi, U00f, U01f, U10f, U11f, bbf, U0o, U1o, bbo, U0u, U1u, bbu;
  int Why, by;
  float* slab_h = nullptr;
  float* table = nullptr;
  struct State { TR loss, first, second; };   // the app's ArrayBuffer(loss, "hidden", "cell") with its exchanged roles
  // pldi19 == false: the earlier NIPS18App/SentimentTreeLSTM.scala:118-170, whose generated program ships under
  // src/out/NIPS18evaluation/evaluationTreeLSTM/Lantern/Lantern.cpp: the same cell without the exchanged roles, and a
  // hand-written Adagrad loop without gradient clipping.
  const bool pldi19;

  TreeLstm(int, int seed, bool pldi19_variant) : pldi19(pldi19_variant) {
    name = "treelstm"; batch = 1; in_c = in_h = in_w = 1; label_count = 1 + 4 * MAXN;
    auto W = [&](int r, int c) { return declare({r, c}, INIT_RAND, 0.01f); };
    auto Z = [&](int n) { return declare({n}, INIT_ZERO); };
    Wi = W(Hd, E); bi = Z(Hd); Wo = W(Hd, E); bo = Z(Hd); Wu = W(Hd, E); bu = Z(Hd);
    U0i = W(Hd, Hd); U1i = W(Hd, Hd); bbi = Z(Hd);
    U00f = W(Hd, Hd); U01f = W(Hd, Hd); U10f = W(Hd, Hd); U11f = W(Hd, Hd); bbf = Z(Hd);
    U0o = W(Hd, Hd); U1o = W(Hd, Hd); bbo = Z(Hd);
    U0u = W(Hd, Hd); U1u = W(Hd, Hd); bbu = Z(Hd);
    Why = W(O, Hd); by = Z(O);
    finalize(seed);
    slab_h = alloc_zero(slab_count);
    table = alloc_value((int64_t)VOCAB * E);
    {
      std::vector<float> h((size_t)VOCAB * E);
      uint64_t st = 0x9E3779B97F4A7C15ull;              // own generator: the weights' rand() stream stays untouched
      auto u01 = [&]() { st = st * 6364136223846793005ull + 1442695040888963407ull; return (double)((st >> 11) + 1) / 9007199254740993.0; };
      for (size_t i = 0; i + 1 < h.size() + 1; i += 2) {
        const double r = std::sqrt(-2.0 * std::log(u01())), a = 6.283185307179586 * u01();
        h[i] = (float)(0.1 * r * std::cos(a)); if (i + 1 < h.size()) h[i + 1] = (float)(0.1 * r * std::sin(a));
      }
      BK(h2d)(table, h.data(), h.size() * 4); BK(sync)();
    }
    mark = BK(mark)();
  }
  // With fused cells (the default) a gate is one call forward and one backward (ltb_affine_act) instead of the five and
  // about eight small kernels of the operator-by-operator form, which is kept for comparison (model_use_fused_cells).
  TR gate(Tape& t, int op, int W0, const TR& a, int W1, const TR& b, int bias) {      // (W0.a plusBias W1.b plusBias bias).op
    if (fused_cells) { TR w1 = P(W1); return t.affine_act(op, P(W0), a, &w1, &b, P(bias)); }
    return t.unary(op, t.plus_bias(t.plus_bias(t.dot(P(W0), a), t.dot(P(W1), b)), P(bias)));
  }
  TR leaf_gate(Tape& t, int op, int W, const TR& e, int bias) {                       // (W.e plusBias bias).op
    if (fused_cells) return t.affine_act(op, P(W), e, nullptr, nullptr, P(bias));
    return t.unary(op, t.plus_bias(t.dot(P(W), e), P(bias)));
  }
  TR out(Tape& t, const TR& in, const int32_t* score) {                              // Out.apply, lines 111-118
    TR pred = fused_cells ? t.affine_act(-1, P(Why), in, nullptr, nullptr, P(by)) : t.plus_bias(t.dot(P(Why), in), P(by));
    return t.nll(t.log_softmax(view(pred, {1, O})), score);
  }
  State visit(Tape& t, const int32_t* host, const int32_t* dev, int i) {
    const int32_t *scores = dev + 1, *words = host + 1 + MAXN, *lch = host + 1 + 2 * MAXN, *rch = host + 1 + 3 * MAXN;
    State s;
    if (fused_cells && whole_sequence) {               // the whole node in one call forward and one backward (ltb_tree_node_fwd / _bwd)
      TR none, W[5][2], bias[5];
      Tape::NodeOut o;
      if (lch[i] < 0) {
        TR e; e.rank = 1; e.shape[0] = E; e.x = table + (int64_t)words[i] * E; e.is_input = true;
        W[0][0] = P(Wi); W[3][0] = P(Wo); W[4][0] = P(Wu); bias[0] = P(bi); bias[3] = P(bo); bias[4] = P(bu);
        o = t.tree_node(false, pldi19, e, nullptr, W, bias, nullptr, nullptr, P(Why), P(by), scores + i, nullptr, nullptr);
      } else {
        State l = visit(t, host, dev, lch[i]), r = visit(t, host, dev, rch[i]);
        W[0][0] = P(U0i); W[0][1] = P(U1i); W[1][0] = P(U00f); W[1][1] = P(U01f); W[2][0] = P(U10f); W[2][1] = P(U11f);
        W[3][0] = P(U0o); W[3][1] = P(U1o); W[4][0] = P(U0u); W[4][1] = P(U1u);
        bias[0] = P(bbi); bias[1] = P(bbf); bias[2] = P(bbf); bias[3] = P(bbo); bias[4] = P(bbu);
        o = t.tree_node(true, pldi19, l.first, &r.first, W, bias, &l.second, &r.second, P(Why), P(by), scores + i, &l.loss, &r.loss);
      }
      s.loss = o.loss;
      s.first = pldi19 ? o.cell : o.hidden; s.second = pldi19 ? o.hidden : o.cell;   // the PLDI19 application's exchanged roles
      return s;
    }
    if (lch[i] < 0) {                                                                // leaf, lines 72-85 and 130-133
      TR e; e.rank = 1; e.shape[0] = E; e.x = table + (int64_t)words[i] * E; e.is_input = true;
      TR ig = leaf_gate(t, LTB_SIGMOID, Wi, e, bi);
      TR og = leaf_gate(t, LTB_SIGMOID, Wo, e, bo);
      TR uv = leaf_gate(t, LTB_TANH, Wu, e, bu);
      TR cell, hidden;
      if (fused_cells) t.lstm_cell(ig, uv, nullptr, nullptr, nullptr, nullptr, og, &cell, &hidden);
      else { cell = t.binary(LTB_MUL, ig, uv); hidden = t.binary(LTB_MUL, og, t.unary(LTB_TANH, cell)); }
      if (!pldi19) { s.loss = out(t, hidden, scores + i); s.first = hidden; s.second = cell; return s; }
      // val ArrayBuffer(cell', hidden') = leaf(...): cell' = hidden, hidden' = cell
      s.loss = out(t, /*hidden'*/ cell, scores + i);
      s.first = /*hidden'*/ cell; s.second = /*cell'*/ hidden;
      return s;
    }
    State l = visit(t, host, dev, lch[i]), r = visit(t, host, dev, rch[i]);
    const TR &hl = l.first, &cl = l.second, &hr = r.first, &cr = r.second;           // ArrayBuffer(loss, hiddenl, celll) = l
    TR ig = gate(t, LTB_SIGMOID, U0i, hl, U1i, hr, bbi);
    TR fl = gate(t, LTB_SIGMOID, U00f, hl, U01f, hr, bbf);
    TR fr = gate(t, LTB_SIGMOID, U10f, hl, U11f, hr, bbf);
    TR og = gate(t, LTB_SIGMOID, U0o, hl, U1o, hr, bbo);
    TR uv = gate(t, LTB_TANH, U0u, hl, U1u, hr, bbu);
    TR cell, hidden;
    if (fused_cells) t.lstm_cell(ig, uv, &fl, &cl, &fr, &cr, og, &cell, &hidden);
    else {
      cell = t.plus_bias(t.plus_bias(t.binary(LTB_MUL, ig, uv), t.binary(LTB_MUL, fl, cl)), t.binary(LTB_MUL, fr, cr));
      hidden = t.binary(LTB_MUL, og, t.unary(LTB_TANH, cell));
    }
    if (!pldi19) {        // loss = lossl + lossr + nll, NIPS18App/SentimentTreeLSTM.scala:158
      s.loss = t.binary(LTB_ADD, t.binary(LTB_ADD, l.loss, r.loss), out(t, hidden, scores + i));
      s.first = hidden; s.second = cell;
      return s;
    }
    s.loss = t.plus_bias(t.plus_bias(out(t, /*hidden'*/ cell, scores + i), l.loss), r.loss);
    s.first = cell; s.second = hidden;
    return s;
  }
  // The whole tree level by level (ltb_tree_nodes_fwd / _bwd): all leaves in one call, then all nodes whose children are done,
  // and so on up to the root; the descriptions of all nodes are uploaded once.  A 25-leaf tree is some ten calls each way
  // instead of 49.
  std::vector<ltb_tree_node> level_nodes;          // sorted by height; kept until the backward calls have been issued
  TR forward_levels(Tape& t, const int32_t* host, const int32_t* dev, int n) {
    const int32_t *scores = dev + 1, *words = host + 1 + MAXN, *lch = host + 1 + 2 * MAXN, *rch = host + 1 + 3 * MAXN;
    std::vector<int> height(n, -1), order(n), pos(n);
    std::function<int(int)> hgt = [&](int i) -> int {
      if (height[i] >= 0) return height[i];
      if (lch[i] < 0) return height[i] = 0;
      const int a = hgt(lch[i]), b = hgt(rch[i]);
      return height[i] = 1 + (a > b ? a : b);
    };
    int top = 0;
    for (int i = 0; i < n; ++i) { const int h = hgt(i); if (h > top) top = h; }
    std::vector<int> first(top + 2, 0);
    for (int i = 0; i < n; ++i) ++first[height[i] + 1];
    for (int h = 0; h <= top; ++h) first[h + 1] += first[h];
    { std::vector<int> fill(first.begin(), first.end() - 1); for (int i = 0; i < n; ++i) { pos[i] = fill[height[i]]++; order[pos[i]] = i; } }
    const int64_t pitch = ((int64_t)Hd + 63) / 64 * 64, vstride = 8 * pitch + 64, gstride = 2 * pitch + 64;
    float* vals = alloc_value(n * vstride);
    float* grads = alloc_zero(n * gstride);
    level_nodes.assign((size_t)n, ltb_tree_node{});
    auto V = [&](int i) { return vals + (int64_t)pos[i] * vstride; };
    auto G = [&](int i) { return grads + (int64_t)pos[i] * gstride; };
    for (int i = 0; i < n; ++i) {
      ltb_tree_node& q = level_nodes[(size_t)pos[i]];
      const bool inner = lch[i] >= 0;
      q.hidden = Hd; q.classes = O; q.inner = inner ? 1 : 0; q.classify_cell = pldi19 ? 1 : 0;
      auto setW = [&](int slot, int k, int idx) { const TR w = P(idx); q.W[slot][k] = w.x; q.dW[slot][k] = w.d; };
      auto setB = [&](int slot, int idx) { const TR b = P(idx); q.bias[slot] = b.x; q.dbias[slot] = b.d; };
      if (!inner) {
        q.in_len = E; q.in[0] = table + (int64_t)words[i] * E;
        setW(0, 0, Wi); setW(3, 0, Wo); setW(4, 0, Wu); setB(0, bi); setB(3, bo); setB(4, bu);
      } else {
        const int l = lch[i], r = rch[i];
        // the children's first state vector feeds the gates, their second one the cell (the PLDI19 application's exchanged roles:
        // first = cell, second = hidden)
        q.in_len = Hd;
        q.in[0] = pldi19 ? V(l) + 5 * pitch : V(l) + 7 * pitch; q.din[0] = pldi19 ? G(l) : G(l) + pitch;
        q.in[1] = pldi19 ? V(r) + 5 * pitch : V(r) + 7 * pitch; q.din[1] = pldi19 ? G(r) : G(r) + pitch;
        q.cl = pldi19 ? V(l) + 7 * pitch : V(l) + 5 * pitch; q.dcl = pldi19 ? G(l) + pitch : G(l);
        q.cr = pldi19 ? V(r) + 7 * pitch : V(r) + 5 * pitch; q.dcr = pldi19 ? G(r) + pitch : G(r);
        q.loss_l = V(l) + 8 * pitch + 32; q.dloss_l = G(l) + 2 * pitch; q.loss_r = V(r) + 8 * pitch + 32; q.dloss_r = G(r) + 2 * pitch;
        setW(0, 0, U0i); setW(0, 1, U1i); setW(1, 0, U00f); setW(1, 1, U01f); setW(2, 0, U10f); setW(2, 1, U11f);
        setW(3, 0, U0o); setW(3, 1, U1o); setW(4, 0, U0u); setW(4, 1, U1u);
        setB(0, bbi); setB(1, bbf); setB(2, bbf); setB(3, bbo); setB(4, bbu);
      }
      { const TR w = P(Why), b = P(by); q.Why = w.x; q.dWhy = w.d; q.by = b.x; q.dby = b.d; }
      q.score = scores + i;
      float* v = V(i); float* g = G(i);
      q.gates = v; q.c = v + 5 * pitch; q.tc = v + 6 * pitch; q.h = v + 7 * pitch; q.logp = v + 8 * pitch; q.loss = v + 8 * pitch + 32;
      q.dc = g; q.dh = g + pitch; q.dloss = g + 2 * pitch;
    }
    ltb_tree_node* dev_nodes = (ltb_tree_node*)BK(malloc_uninit)((size_t)n * sizeof(ltb_tree_node));
    BK(h2d)(dev_nodes, level_nodes.data(), (size_t)n * sizeof(ltb_tree_node));
    const ltb_tree_node* hn = level_nodes.data();
    for (int h = 0; h <= top; ++h) {
      const int f = first[h], c = first[h + 1] - first[h];
      BK(tree_nodes_fwd)(hn, dev_nodes, f, c);
      t.push([=] { BK(tree_nodes_bwd)(hn, dev_nodes, f, c); });
    }
    TR loss; loss.rank = 1; loss.shape[0] = 1; loss.x = V(0) + 8 * pitch + 32; loss.d = G(0) + 2 * pitch;
    return loss;
  }
  TR forward(Tape& t, const TR&, const int32_t* y) override {
    const int n = stage_y[0];
    if (n < 1 || n > MAXN) { TR z = make({1}); BK(fill)(z.x, 0.0f, 1); return z; }
    if (fused_cells && whole_sequence && level_batches) return forward_levels(t, stage_y, y, n);
    return visit(t, stage_y, y, 0).loss;
  }
  void apply_update(float lr) override { BK(adagrad_update)(slab_x, slab_d, slab_h, lr, pldi19 ? 1.0f : 3.0e38f, 1, slab_count); }
  // Replaces the embedding table (rows x 300 floats, rows <= VOCAB) by the caller's.
  int set_table(const float* host, int rows) {
    if (rows < 1 || rows > VOCAB) return LTB_E_ARG;
    int rc = BK(h2d)(table, host, (size_t)rows * E * 4);
    return rc ? rc : BK(sync)();
  }
};

// ------------------------------------------------------------------------------------------------ ResNet-50 (CIFAR)
struct ResNet50 : Model {
  struct ConvBN { int w, gamma, beta, rmean, rvar; };
  struct Block { ConvBN a, b, c, down; bool has_down; int stride; };
  ConvBN stem; std::vector<Block> blocks; int fcw, fcb;

  ConvBN conv_bn(int cin, int cout, int k) {
    ConvBN cb;
    cb.w = declare({cout, cin, k, k}, INIT_RAND, 2.0f * sqrtf(6.0f / (float)(cin * k * k)));
    cb.gamma = declare({cout}, INIT_ONE); cb.beta = declare({cout}, INIT_ZERO);
    cb.rmean = declare({cout}, INIT_ZERO); cb.rvar = declare({cout}, INIT_ONE);
    decls[cb.rmean].state = decls[cb.rvar].state = true;   // each replica keeps the running statistics of its own batches
    return cb;
  }
  // max_blocks < 16 gives a prefix of the network (stem, max pool, the first max_blocks bottleneck blocks) closed by an
  // average pool over the whole remaining map and the classifier: shallow enough for its TF32 gradients to be compared
  // tightly, made of exactly the layer types and the issue order of the full program.
  ResNet50(int b, int seed, int max_blocks = 16) {
    name = max_blocks < 16 ? "resnet50_prefix" : "resnet50"; batch = b; in_c = 3; in_h = in_w = 32; logit_count = (int64_t)b * 10;
    stem = conv_bn(3, 64, 3);
    int inplanes = 64; const int layers[4] = {3, 4, 6, 3}; const int planes[4] = {64, 128, 256, 512};
    for (int s = 0; s < 4; ++s)
      for (int i = 0; i < layers[s] && (int)blocks.size() < max_blocks; ++i) {
        Block bl; bl.stride = (i == 0 && s > 0) ? 2 : 1;
        bl.a = conv_bn(inplanes, planes[s], 1); bl.b = conv_bn(planes[s], planes[s], 3); bl.c = conv_bn(planes[s], planes[s] * 4, 1);
        bl.has_down = (i == 0);
        if (bl.has_down) bl.down = conv_bn(inplanes, planes[s] * 4, 1);
        inplanes = planes[s] * 4;
        blocks.push_back(bl);
      }
    fcw = declare({10, inplanes}, INIT_RAND, 1.0f / sqrtf((float)inplanes)); fcb = declare({10}, INIT_ZERO);
    finalize(seed);
  }
  TR cbn(Tape& t, const TR& x, const ConvBN& p, int stride, int pad, bool relu) {
    TR y = t.batch_norm(t.conv(x, P(p.w), nullptr, stride, pad), P(p.gamma), P(p.beta), P(p.rmean).x, P(p.rvar).x);
    return relu ? t.relu(y, true) : y;
  }
  TR forward(Tape& t, const TR& x, const int32_t* y) override {
    TR h = t.max_pool(cbn(t, x, stem, 1, 1, true), 2, 2);
    const size_t stage_start[3] = {3, 7, 13};            // first block of stages 2, 3, 4: the slab above each is final when backward gets there
    for (size_t bi = 0; bi < blocks.size(); ++bi) {       // Bottleneck.forward, resnet50.py:72-93
      const Block& bl = blocks[bi];
      for (int k = 0; k < 3 && blocks.size() == 16; ++k)
        if (bi == stage_start[k]) reduce_when_final(t, bl.a.w, k == 2 ? slab_count : decls[blocks[stage_start[k + 1]].a.w].offset);
      // A block with a shortcut convolution has two runs of calls that meet only at the sum: the shortcut (conv + BN) is
      // issued as a branch beside the three conv + BN of the main path.  Backward replays the tape in reverse, so every
      // marker pushes its counterpart: the shortcut's gradients run as a branch from the sum's gradient on, and are joined
      // before the gradient of the block's first convolution, which accumulates into the same input gradient.
      const bool fork = bl.has_down && branches;
      if (fork) BK(branch_mark)();
      TR o = t.conv(h, P(bl.a.w), nullptr, 1, 0);
      if (fork) t.push([] { BK(branch_join)(); });
      o = t.relu(t.batch_norm(o, P(bl.a.gamma), P(bl.a.beta), P(bl.a.rmean).x, P(bl.a.rvar).x), true);
      o = cbn(t, o, bl.b, bl.stride, 1, true);
      o = cbn(t, o, bl.c, 1, 0, false);
      TR res = h;
      if (bl.has_down) {
        if (fork) { BK(branch_begin)(); t.push([] { BK(branch_end)(); }); }
        res = cbn(t, h, bl.down, bl.stride, 0, false);
        if (fork) { BK(branch_end)(); t.push([] { BK(branch_begin)(); }); BK(branch_join)(); t.push([] { BK(branch_mark)(); }); }
      }
      h = t.relu(t.binary(LTB_ADD, o, res), true);
    }
    TR p = t.avg_pool(h, h.shape[2], 1);                                         // 2x2 on the full network's last map
    TR flat = view(p, {batch, h.shape[1]});
    TR logits = t.plus_bias(t.gemm(flat, false, P(fcw), true, 1.0f), P(fcb));   // ONNX Gemm, ONNXLib.scala:956-974
    last_logits = logits;
    return t.mean(t.nll(t.log_softmax(logits), y));                              // resnet50FromOnnx.scala:153-156
  }
};

// ------------------------------------------------------------------------------------------------ SqueezeNet (CIFAR)
struct SqueezeNet : Model {
  struct Conv { int w, b; };
  struct Fire { Conv s, e1, e3; };
  Conv first, last; std::vector<Fire> fires;
  Conv conv(int cin, int cout, int k) {
    Conv c; c.w = declare({cout, cin, k, k}, INIT_RAND, 2.0f * sqrtf(6.0f / (float)(cin * k * k))); c.b = declare({cout}, INIT_ZERO); return c;
  }
  SqueezeNet(int b, int seed) {
    name = "squeezenet"; batch = b; in_c = 3; in_h = in_w = 32; logit_count = (int64_t)b * 10;
    first = conv(3, 96, 3);
    const int cfg[8][4] = {{96, 16, 64, 64}, {128, 16, 64, 64}, {128, 32, 128, 128}, {256, 32, 128, 128},
                           {256, 48, 192, 192}, {384, 48, 192, 192}, {384, 64, 256, 256}, {512, 64, 256, 256}};
    for (auto& c : cfg) { Fire f; f.s = conv(c[0], c[1], 1); f.e1 = conv(c[1], c[2], 1); f.e3 = conv(c[1], c[3], 3); fires.push_back(f); }
    last = conv(512, 10, 4);
    finalize(seed);
  }
  TR cr(Tape& t, const TR& x, const Conv& c, int pad) { TR b = P(c.b); return t.relu(t.conv(x, P(c.w), &b, 1, pad), true); }
  TR fire(Tape& t, const TR& x, const Fire& f) {
    TR s = cr(t, x, f.s, 0);
    return t.concat1(cr(t, s, f.e1, 0), cr(t, s, f.e3, 1));
  }
  TR forward(Tape& t, const TR& x, const int32_t* y) override {
    TR h = t.max_pool(cr(t, x, first, 1), 2, 2);
    for (int i = 0; i < 3; ++i) h = fire(t, h, fires[i]);
    h = t.max_pool(h, 2, 2);
    for (int i = 3; i < 7; ++i) {
      if (i == 4) reduce_when_final(t, fires[4].s.w, slab_count);
      h = fire(t, h, fires[i]);
    }
    h = t.max_pool(h, 2, 2);
    h = fire(t, h, fires[7]);
    TR lb = P(last.b);
    TR logits = view(t.conv(h, P(last.w), &lb, 1, 0), {batch, 10});
    last_logits = logits;
    return t.mean(t.nll(t.log_softmax(logits), y));
  }
};

}  // namespace

extern "C" {

void* HOST_FN(model_create)(const char* name, int batch, int seed) {
  std::string n(name);
  BK(set_fusion)(3);     // generated programs issue every device operation through the library: the one-call look-ahead is safe, and a
                         // gradient buffer has no reader after the operator that absorbs its in-place ReLU gradient (level 2); in the
                         // networks of this file the last batch norm of a residual block is read by the block's sum only (level 3)
  BK(set_filter_cache)(1);   // and they write parameters only through the optimizer, transfer and fill entry points
  if (n == "mnist") return new Mnist(batch, seed);
  if (n == "resnet50") return new ResNet50(batch, seed);
  if (n == "resnet50_prefix") return new ResNet50(batch, seed, 1);        // stem + the first bottleneck block + classifier
  if (n == "squeezenet") return new SqueezeNet(batch, seed);
  if (n == "rnn") return new VanillaRnn(batch, seed, 80, 100);
  if (n == "rnn_26_50") return new VanillaRnn(batch, seed, 26, 50);     // sizes of src/out/NIPS18evaluation/evaluationRNN/Lantern.cpp
  if (n == "treelstm") return new TreeLstm(batch, seed, true);
  if (n == "treelstm_nips18") return new TreeLstm(batch, seed, false);
  return nullptr;
}
void HOST_FN(model_destroy)(void* m) {
  Model* M = (Model*)m;
  if (M->graph) BK(graph_destroy)(M->graph);
  BK(host_free)(M->stage_x); BK(host_free)(M->stage_y); BK(host_free)(M->loss_host);
  for (int p = 0; p < 2; ++p) { BK(host_free)(M->feed_x[p]); BK(host_free)(M->feed_y[p]); }
  BK(host_free)(M->feed_loss);
  delete M;
}
int HOST_FN(model_num_params)(void* m) { return (int)((Model*)m)->decls.size(); }
int64_t HOST_FN(model_param_count)(void* m, int i) { return ((Model*)m)->decls[i].count; }
int HOST_FN(model_param_is_state)(void* m, int i) { return ((Model*)m)->decls[i].state ? 1 : 0; }   // 1: a batch-norm running statistic
float* HOST_FN(model_param_ptr)(void* m, int i) { Model* M = (Model*)m; return M->slab_x + M->decls[i].offset; }
float* HOST_FN(model_grad_ptr)(void* m, int i) { Model* M = (Model*)m; return M->slab_d + M->decls[i].offset; }
int64_t HOST_FN(model_slab_count)(void* m) { return ((Model*)m)->slab_count; }
float* HOST_FN(model_slab_params)(void* m) { return ((Model*)m)->slab_x; }
float* HOST_FN(model_slab_grads)(void* m) { return ((Model*)m)->slab_d; }
int64_t HOST_FN(model_input_count)(void* m) { Model* M = (Model*)m; return (int64_t)M->batch * M->in_c * M->in_h * M->in_w; }
// TreeLSTM only: load the embedding table (rows x 300) the leaves read.
int HOST_FN(model_set_table)(void* m, const float* host, int rows) {
  TreeLstm* T = dynamic_cast<TreeLstm*>((Model*)m);
  return T ? T->set_table(host, rows) : LTB_E_ARG;
}
int64_t HOST_FN(model_label_count)(void* m) { return ((Model*)m)->label_count; }
// Recursive models: gates as single fused calls (default) or operator by operator, as the reference stages them.
// on: 0 operator by operator, 1 one call per gate / cell, 2 (default) in addition the vanilla RNN's whole sequence in one call.
int HOST_FN(model_use_fused_cells)(void* m, int on) {
  Model* M = (Model*)m;
  if (M->graph) { BK(graph_destroy)(M->graph); M->graph = nullptr; }
  M->fused_cells = on != 0; M->whole_sequence = on >= 2; M->level_batches = on >= 3; return 0;
}
// Issue independent runs of calls as branch regions (default) or everything in program order on one stream.
// Large activation gradients declared unset instead of zero-filled (ltb_grad_unset; default on).  Process-wide: it is a property
// of how the tape allocates, not of one model.
int HOST_FN(model_use_deferred_zero)(void*, int on) { deferred_grads() = on != 0; return 0; }
int HOST_FN(model_use_branches)(void* m, int on) {
  Model* M = (Model*)m;
  if (M->graph) { BK(graph_destroy)(M->graph); M->graph = nullptr; }
  M->branches = on != 0; return 0;
}
// A recorded step can only be replayed when every step issues the same operations: not so for one tree per step.
// Nor when a step touches the host: the MNIST program draws its dropout mask from rand() every step.
int HOST_FN(model_use_graph)(void* m, int on) { Model* M = (Model*)m; M->use_graph = on != 0 && M->name != "treelstm" && M->name != "mnist"; return 0; }
// Keep one batch resident in device memory; later steps read it there and upload nothing (x_host/y_host are ignored).
int HOST_FN(model_set_resident)(void* m, const float* x_host, const int32_t* y_host) {
  Model* M = (Model*)m;
  M->feed_mode(false);
  if (M->graph) { BK(graph_destroy)(M->graph); M->graph = nullptr; }
  if (!x_host) { M->resident = false; return 0; }
  M->load(x_host, y_host);
  BK(h2d)(M->dev_x, M->stage_x, (size_t)M->batch * M->in_c * M->in_h * M->in_w * 4);
  BK(h2d)(M->dev_y, M->stage_y, (size_t)M->label_count * 4);
  BK(sync)();
  M->resident = true;
  return 0;
}
// Blocking step: returns the loss of this batch. update=0 leaves the parameter gradients in place for inspection.
float HOST_FN(model_step)(void* m, const float* x_host, const int32_t* y_host, float lr, int update) {
  Model* M = (Model*)m;
  if (M->feeding) M->feed_mode(false);
  return M->step(x_host, y_host, lr, update != 0);
}
// Non-blocking step: the loss is available from model_last_loss after the library's sync.
int HOST_FN(model_step_async)(void* m, const float* x_host, const int32_t* y_host, float lr) {
  Model* M = (Model*)m;
  if (M->feeding) M->feed_mode(false);
  return M->step_async(x_host, y_host, lr, true);
}
// Two steps in flight: submit returns the step's number (or -1) without waiting; collect(k) waits for step k and gives its
// loss.  Only the last two submitted steps can be collected.
int64_t HOST_FN(model_submit)(void* m, const float* x_host, const int32_t* y_host, float lr) { return ((Model*)m)->submit(x_host, y_host, lr); }
int HOST_FN(model_collect)(void* m, int64_t step, float* loss) { return ((Model*)m)->collect(step, loss); }
float HOST_FN(model_last_loss)(void* m) { return *((Model*)m)->loss_host; }
// The classifier's output of the last step (batch x classes floats); returns the number of floats, 0 for programs without one.
int64_t HOST_FN(model_logits)(void* m, float* host_out) {
  Model* M = (Model*)m;
  if (!M->dev_logits || BK(d2h)(host_out, M->dev_logits, (size_t)M->logit_count * 4)) return 0;
  return M->logit_count;
}

// ---- data and parameter files in the reference's formats (loader.hpp)
void* HOST_FN(loader_open_floats)(const char* data_path, const char* target_path, int64_t floats_per_sample, float mean, float stdev) {
  Loader* L = new Loader;
  L->open_floats(data_path, target_path, floats_per_sample, mean, stdev);
  return L;                                      // a loader that failed to open has length 0 and a message (loader_error)
}
void* HOST_FN(loader_open_cifar)(const char* path, int64_t bytes_per_sample) {
  Loader* L = new Loader;
  L->open_cifar(path, bytes_per_sample);
  return L;
}
const char* HOST_FN(loader_error)(void* l) { return ((Loader*)l)->error.c_str(); }
int64_t HOST_FN(loader_length)(void* l) { Loader* L = (Loader*)l; return L->error.empty() ? L->length : 0; }
int HOST_FN(loader_fill)(void* l, int64_t index, int batch, float* x, int32_t* y) {
  Loader* L = (Loader*)l;
  return L->error.empty() && L->fill(index, batch, x, y) ? 0 : LTB_E_ARG;
}
void HOST_FN(loader_close)(void* l) { Loader* L = (Loader*)l; L->close(); delete L; }
// One pass over the loader's batches (at most max_batches when positive) with two steps in flight: batch i + 1 is decoded
// into pinned staging while the device runs step i.  losses (nullable) receives one value per batch.  Returns the number
// of steps, or a negative error code.
int64_t HOST_FN(model_train_epoch)(void* m, void* l, float lr, float* losses, int64_t max_batches) {
  Model* M = (Model*)m; Loader* L = (Loader*)l;
  if (!L->error.empty() || L->sample_count != (int64_t)M->in_c * M->in_h * M->in_w || M->label_count != M->batch) return LTB_E_ARG;
  int64_t n = L->batches(M->batch);
  if (max_batches > 0 && max_batches < n) n = max_batches;
  int64_t prev = -1;
  for (int64_t i = 0; i < n; ++i) {
    float* sx; int32_t* sy; float loss;
    if (M->feed_slot(&sx, &sy) || !L->fill(i, M->batch, sx, sy)) return LTB_E_STATE;
    const int64_t k = M->submit(nullptr, nullptr, lr);
    if (k < 0) return LTB_E_CUDA;
    if (prev >= 0) { if (M->collect(prev, &loss)) return LTB_E_CUDA; if (losses) losses[i - 1] = loss; }
    prev = k;
  }
  if (prev >= 0) { float loss; if (M->collect(prev, &loss)) return LTB_E_CUDA; if (losses) losses[n - 1] = loss; }
  return n;
}
// Parameter file: every tensor's floats back to back, unpadded, in declaration order (ONNXLib.scala:157-185).
int HOST_FN(model_save_params)(void* m, const char* path) {
  Model* M = (Model*)m;
  std::vector<float> slab((size_t)M->slab_count);
  if (BK(d2h)(slab.data(), M->slab_x, slab.size() * 4)) return LTB_E_CUDA;
  FILE* f = fopen(path, "wb");
  if (!f) return LTB_E_ARG;
  bool ok = true;
  for (const ParamDecl& d : M->decls) ok = ok && fwrite(slab.data() + d.offset, 4, (size_t)d.count, f) == (size_t)d.count;
  return fclose(f) == 0 && ok ? 0 : LTB_E_STATE;
}
int HOST_FN(model_load_params)(void* m, const char* path) {
  Model* M = (Model*)m;
  MappedFile f;
  if (!f.open(path)) return LTB_E_ARG;
  int64_t total = 0;
  for (const ParamDecl& d : M->decls) total += d.count;
  if ((int64_t)(f.bytes / 4) != total || f.bytes % 4) { f.close(); return LTB_E_ARG; }      // not this model's file
  std::vector<float> slab((size_t)M->slab_count, 0.0f);
  const float* src = (const float*)f.data;
  for (const ParamDecl& d : M->decls) { memcpy(slab.data() + d.offset, src, (size_t)d.count * 4); src += d.count; }
  f.close();
  if (BK(sync)() || BK(h2d)(M->slab_x, slab.data(), slab.size() * 4) || BK(sync)()) return LTB_E_CUDA;
  return 0;
}
// Debug: run one step without update and write per-operator checksums (see Model::dump_trace) into buf.
int HOST_FN(model_trace)(void* m, const float* x_host, const int32_t* y_host, char* buf, int len) {
  Model* M = (Model*)m;
  tracing() = true; trace_list().clear();
  BK(set_fusion)(1);     // the trace reads every gradient buffer after the step: masked gradients are written back as the separate calls would
  M->step(x_host, y_host, 0.0f, false);
  BK(set_fusion)(3);
  tracing() = false;
  strncpy(buf, M->trace_text.c_str(), len - 1); buf[len - 1] = 0;
  return (int)M->trace_text.size();
}

}  // extern "C"
