/*
 * lantern_b200.h -- C ABI of the B200-native tensor backend for Lantern.
 *
 * Lantern's Scala front end stages model code into one C++/CUDA host program; every
 * tensor operation in that program is whatever text the active `Backend` object spliced in
 * (trait Backend, src/main/scala/lantern/TensorDifferentiation.scala:137-379).  This header is
 * the set of C symbols a `BackendB200` emits calls to: one entry point per Backend method on
 * the CNN/RNN training path, taking the information the Scala method has in hand when it
 * prints the call (raw arena pointers + integer shapes + scalars by value).
 *
 * Conventions (identical to the reference's generated code):
 *   - all tensors are dense row-major float32; 4-D tensors are NCHW, filters OIHW;
 *     indices and class targets are int32;
 *   - "ow" = the destination is overwritten, "acc" = the result is ADDED into the destination
 *     (the reference CPU backend accumulates every gradient, TensorDslCPU.scala passim);
 *   - buffers are owned by the caller and come from the arena below; the library keeps no
 *     pointer past a call (exception: the communicator);
 *   - all work is issued on one stream in program order; only ltb_d2h / ltb_sync block.
 *
 * Every function returns 0 on success or a negative LTB_E_* code (pointer-returning functions
 * return NULL).  In fatal mode (the default, matching CUDA_CALL/CUBLAS_CALL/CUDNN_CALL in
 * src/main/scala/lantern/DslAPI.scala:435-451) an error prints to stderr and exit()s; with
 * ltb_set_fatal(0) the code is returned and ltb_last_error() holds the message.
 *
 * The same declarations, compiled with -DLTB_FN(n)=ora_##n, are the ABI of the CPU oracle used
 * by the tests (host pointers instead of device pointers).
 */
#ifndef LANTERN_B200_H
#define LANTERN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifndef LTB_FN
#define LTB_FN(name) ltb_##name
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LTB_OK = 0,
  LTB_E_CUDA = -1,      /* a CUDA runtime/driver call failed */
  LTB_E_ARG = -2,       /* bad shape / null pointer / unsupported combination */
  LTB_E_OOM = -3,       /* arena exhausted (reference: abort(), DslAPI.scala:462-464) */
  LTB_E_STATE = -4,     /* not initialised / initialised twice */
  LTB_E_COMM = -5,      /* NCCL failure or timeout */
  LTB_E_DEVICE = -6,    /* a kernel reported a bounded wait that ran out */
  LTB_E_LIMIT = -7      /* a stated size limit of the entry point was exceeded */
};

/* Binary op codes for the broadcasting family (Backend + - * /, TD.scala:222-258). */
enum { LTB_ADD = 0, LTB_SUB = 1, LTB_MUL = 2, LTB_DIV = 3 };
/* Unary op codes (Backend relu/tanh/sigmoid/exp/log/sqrt/square, TD.scala:319-335). */
enum { LTB_RELU = 0, LTB_TANH = 1, LTB_SIGMOID = 2, LTB_EXP = 3, LTB_LOG = 4, LTB_SQRT = 5, LTB_SQUARE = 6 };
/* Math mode, the counterpart of `cudnnMathType` (TensorDslCudnn.scala:133-136). */
enum { LTB_MATH_FP32 = 0, LTB_MATH_TF32 = 1 };

/* ---------------------------------------------------------------- lifetime / context
 * Replaces backend.setup()/cleanup(): TensorDslCublas.scala:113-124, TensorDslCudnn.scala:143-151
 * and the arena globals of DslAPI.scala:453-473. heap_bytes==0 selects the reference's 8 GiB + 16. */
int    LTB_FN(init)(int device, size_t heap_bytes);
int    LTB_FN(shutdown)(void);
int    LTB_FN(set_fatal)(int on);
int    LTB_FN(last_error)(char* buf, int len);          /* returns the last status code */
int    LTB_FN(set_stream)(void* cuda_stream);           /* adopt a caller stream (cudaStream_t) */
void*  LTB_FN(get_stream)(void);
int    LTB_FN(sync)(void);
int    LTB_FN(set_math)(int mode);                      /* LTB_MATH_TF32 (default) or LTB_MATH_FP32 */
/* Look-ahead fusion, off by default. When on, batch-norm forward and same-shape add are issued one call late so that an
 * in-place ReLU of their result joins the same kernel, and an in-place ReLU gradient is held so that the batch-norm
 * backward or add gradient that reads it applies it on the fly. Results are those of the separate calls; only the moment
 * of the launch moves: a held operation is issued by the next call of this library whatever it is (sync, copies,
 * get_stream and graph_end included; malloc, malloc_uninit and grad_unset only keep books on a block no held operation can
 * name yet and issue nothing). A host that enqueues its own work on the stream must call get_stream or sync first.
 * Level 2: in addition the caller declares that the gradient buffer an in-place ReLU gradient works on is not read again
 * after the batch-norm backward or add gradient that absorbed it (true of every staged program: that operator is the
 * buffer's only reader).  The absorbing kernel then applies the mask on load only and no longer writes the masked gradient
 * back into that buffer; every result (dx, dgamma, dbeta, da, db) is unchanged.
 * Level 3: in addition the caller declares that a batch-norm result whose next two calls are a same-shape add with it as one
 * operand and an in-place ReLU of the sum has no other reader (true of a residual block's last batch norm; NOT something
 * reverse-mode structure guarantees, so a generic staged program stays at level 2).  The three calls then become one kernel
 * that writes the sum and never the batch norm's own result; the sum and the saved / running statistics are unchanged. */
int    LTB_FN(set_fusion)(int on);
/* Filter cache, off by default (no counterpart in the reference, where cuDNN reads OIHW filters as they are). The tensor-core
 * engine reads the filter of an R x S convolution as one matrix per tap; forward and data-grad each need their own form, and
 * without the cache both are rebuilt at every call. With it on they are kept, keyed by the filter's address and shape, and
 * rebuilt once after the parameters changed. The library notes a change by itself in every entry point through which a
 * generated program writes parameters: the optimizer steps (sgd_step*, adagrad_update, momentum_update, allreduce_*), h2d,
 * d2d, fill*, randinit, clip, geam, the in-place elementwise forms, and a replayed step. A host that writes a filter by
 * any other route (as the output of another operator, or with its own kernel) must call params_changed afterwards. */
/* Deterministic mode, off by default (the counterpart of choosing cuDNN's deterministic algorithms, which the reference does
 * not do: it takes whatever cudnnFind*Algorithm ranks first, TensorDslCudnn.scala:515-624). A contraction whose output has few
 * tiles is split over its reduction dimension. By default the splits add their partial results into the output atomically,
 * in whatever order they finish, so the last bits of such a sum can differ from run to run. With this mode on, up to eight
 * splits form a thread-block cluster that adds its tiles up in a fixed order through shared memory, and larger splits go
 * through slabs of partial results summed in a fixed order by one more launch: a step of the tensor-core path then gives
 * the same bits on every run, at about a third more time in the contraction kernels.  The CUDA-core fallback paths (shapes the
 * engine declines, the FP32 math mode) do not split over K at all in this mode. */
int    LTB_FN(set_deterministic)(int on);
int    LTB_FN(set_filter_cache)(int on);
int    LTB_FN(params_changed)(void);
/* Deferred zero fill of gradient buffers (no counterpart in the reference, whose arena hands out zeroed memory and whose
 * gradient operators all add into their destination, TensorDslCublas.scala:18-25, TensorDslCPU.scala:575-692).  For the
 * activation gradients of a convolutional network that is a zero fill of every buffer plus a read of those zeros by the
 * first -- usually the only -- operator that adds into it.  grad_unset(d, n) declares the n floats at d, a fresh block that
 * nothing has written, to be a gradient buffer whose zero fill is deferred: it COUNTS as zero.  The first entry point that
 * meets exactly that block as an accumulation destination and is able to -- conv2d_bwd (dx, tensor-core path), bn_bwd (dx),
 * the gradient of a same-shape add (da, db) -- writes its result instead of adding; every other entry point that is handed
 * the block (any gradient operator, the transfers) fills it with zeros first, so results never depend on the declaration.
 * grad_materialize(d, n) does that filling on request (before the caller reads the block by other means).  Declarations
 * end with the arena span that holds the block (ltb_reset, ltb_free). */
int    LTB_FN(grad_unset)(float* d, int64_t n);
int    LTB_FN(grad_materialize)(float* d, int64_t n);
int    LTB_FN(device_status)(void);                     /* 0, or LTB_E_DEVICE if a kernel's bounded wait expired */
/* Failure detection on the device (no counterpart in the reference, whose kernels never wait on anything). Every spin wait
 * inside a kernel of this library (on a TMA or tensor-core completion barrier) gives up after a limit, records a code in
 * a status word that device_status reads, and lets the kernel run to its normal end, so the context stays usable.
 *   set_wait_limit:         the limit in SM clock ticks (default 2e9, about a second);
 *   clear_device_status:    back to 0 (stream-ordered);
 *   selftest_bounded_wait:  launches one warp that waits, through the same wait routine, on a barrier at which nothing
 *                           ever arrives: after `cycles` ticks device_status reports LTB_E_DEVICE. Nothing faults or hangs. */
int    LTB_FN(set_wait_limit)(int64_t cycles);
int    LTB_FN(clear_device_status)(void);
int    LTB_FN(selftest_bounded_wait)(int64_t cycles);
int64_t LTB_FN(kernel_launches)(void);                  /* kernels launched by this library so far */

/* ---------------------------------------------------------------- arena
 * myGpuMalloc / myGpuFree (DslAPI.scala:453-473), getCudaMallocAddr / resetCudaMallocAddr
 * (TensorDslCublas.scala:18-25).  Memory is ZERO when handed out by ltb_malloc, because
 * Tensor.zeros is a bare mallocArray (TD.scala:1075-1076).  ltb_malloc_uninit is for op outputs
 * that are fully overwritten by the next call; it skips the zero fill. Granule 256 B. */
void*  LTB_FN(malloc)(size_t bytes);
void*  LTB_FN(malloc_uninit)(size_t bytes);
int    LTB_FN(free)(void* p, size_t bytes);             /* LIFO pop: p must be the newest block */
void*  LTB_FN(mark)(void);
int    LTB_FN(reset)(void* mark);
size_t LTB_FN(arena_used)(void);

/* Transfers: gpu_array_copy_* of src/main/scala/common/GPUOps.scala:51-95. d2h blocks. */
int LTB_FN(h2d)(void* dst, const void* src, size_t bytes);
int LTB_FN(d2h)(void* dst, const void* src, size_t bytes);
int LTB_FN(d2d)(void* dst, const void* src, size_t bytes);   /* copyFloatArray, TD.scala:150 */
/* Pinned host staging and a non-blocking read-back, so the per-step loss copy (MnistCNN.scala:185) need not
 * stall the stream; the value is valid after the next ltb_sync(). */
void* LTB_FN(host_alloc)(size_t bytes);
int   LTB_FN(host_free)(void* p);
int   LTB_FN(d2h_async)(void* dst_pinned, const void* src, size_t bytes);
/* Stream markers (no counterpart in the reference, whose generated programs block on every transfer,
 * GPUOps.scala:63-65): marker_record notes the current end of the library's stream in one of 16 slots, marker_wait
 * blocks the calling thread until the work issued before that record has finished (returns at once for a slot
 * never recorded).  They let a host program keep two steps in flight -- refill a pinned staging buffer, or read a
 * loss written by d2h_async, as soon as the step that used it is done -- instead of draining the stream with
 * ltb_sync after every step.  Not allowed while recording a step. */
int   LTB_FN(marker_record)(int slot);
int   LTB_FN(marker_wait)(int slot);
/* Uploads beside the compute work (no counterpart in the reference, whose training loops upload on the one stream and block,
 * resnet50FromOnnx.scala:173-186).  upload copies from pinned host memory on the library's copy stream; it starts after
 * marker `after` (-1: at once) -- the point of the compute stream up to which the destination was still being read.
 * upload_marker records a marker on the copy stream (marker_wait on it tells the host that the staging buffer is free
 * again); stream_wait_marker makes the compute stream wait for a marker on the device without blocking the host. */
int   LTB_FN(upload)(void* dst, const void* src, size_t bytes, int after);
int   LTB_FN(upload_marker)(int slot);
int   LTB_FN(stream_wait_marker)(int slot);

/* Fused affine map with activation on vectors, for the recursive models (one LSTM gate per call instead of five).  The
 * Backend trait has no such method; the reference fuses the same expression for its CPU backend only (Tensor.linearTanh /
 * linear2Tanh, TensorDifferentiation.scala:947-990).
 *   affine_act:      out[r] = act(sum_j W0[r][j] a[j] (+ sum_j W1[r][j] b[j]) + bias[r])
 *                    W0 [rows x cols0], W1 [rows x cols1] row-major; W1 and b may both be NULL; act = LTB_SIGMOID, LTB_TANH or
 *                    -1 (none).
 *   affine_act_grad: dpre = dout * act'(out); dbias += dpre; dW0 += dpre a^T; da += W0^T dpre; likewise dW1, db.
 *                    da / db may be NULL (a leaf input).  Everything accumulates, as the separate gradients do
 *                    (TensorDslCPU.scala:186-225, 748-766). */
int LTB_FN(affine_act)(const float* W0, const float* a, int cols0, const float* W1, const float* b, int cols1, const float* bias,
                       int act, float* out, int rows);
int LTB_FN(affine_act_grad)(const float* W0, float* dW0, const float* a, float* da, int cols0, const float* W1, float* dW1,
                            const float* b, float* db, int cols1, float* dbias, int act, const float* out, const float* dout, int rows);

/* The batched form, for a recurrent cell over a minibatch (weights stored [in, out] as the reference's Linear1D does,
 * NNModule.scala:112-117; the cell is tanh(x W0 + h W1 + bias), NNModule.scala:189-200):
 *   affine_act_rows:      out[b][j] = act(sum_c x0[b][c] W0[c][j] (+ sum_c x1[b][c] W1[c][j]) + bias[j]),  b < batch, j < width
 *   affine_act_rows_grad: dpre = dout * act'(out); dbias += column sums of dpre; dW0 += x0^T dpre; dx0 += dpre W0^T; likewise
 *                         dW1, dx1.  dx0 / dx1 may be NULL (an input); x1, W1, dW1 go together and may be NULL. */
int LTB_FN(affine_act_rows)(const float* x0, const float* W0, int cols0, const float* x1, const float* W1, int cols1, const float* bias,
                            int act, float* out, int batch, int width);
int LTB_FN(affine_act_rows_grad)(const float* x0, float* dx0, const float* W0, float* dW0, int cols0, const float* x1, float* dx1,
                                 const float* W1, float* dW1, int cols1, float* dbias, int act, const float* out, const float* dout,
                                 int batch, int width);

/* The elementwise part of a (tree) LSTM cell in one call, and its gradient in one call (no Backend counterpart; the
 * expression is NIPS18App/SentimentTreeLSTM.scala:150-156 = PLDI19APP/SentimentTreeLSTM.scala:136-141):
 *   c = i*u (+ fl*cl + fr*cr when fl is not NULL: an inner node);  tc = tanh(c);  h = o*tc       (tc is kept for the gradient)
 *   lstm_cell_grad: dct = dc + dh*o*(1 - tc^2); do += dh*tc; di += dct*u; du += dct*i; dfl += dct*cl; dcl += dct*fl;
 *                   dfr += dct*cr; dcr += dct*fr.  fl, cl, fr, cr and their gradients are all NULL for a leaf. */
int LTB_FN(lstm_cell)(const float* i, const float* u, const float* fl, const float* cl, const float* fr, const float* cr,
                      const float* o, float* c, float* tc, float* h, int n);
int LTB_FN(lstm_cell_grad)(const float* i, float* di, const float* u, float* du, const float* fl, float* dfl, const float* cl, float* dcl,
                           const float* fr, float* dfr, const float* cr, float* dcr, const float* o, float* d_o,
                           const float* tc, const float* dc, const float* dh, int n);

/* A whole unrolled sequence of the vanilla recurrent network in one call (no Backend counterpart: the reference stages the
 * cell of NNModule.scala:189-200 operator by operator and unrolls it, DynamicRNNFix, NNModule.scala:240-253; the loss is
 * sum over the steps of sum(nllLoss(logSoftmax(o_t), y_t)), as the generated min-char-rnn programs compute it).
 *   x [T][B][V] inputs, y [T][B] classes, h0 [B][H] or NULL (zeros); Wxh [V][H], Whh [H][H], bh [H], Who [H][V], bo [V].
 *   rnn_seq_fwd: h[t] = tanh(x[t] Wxh + h[t-1] Whh + bh); logp[t] = logSoftmax(h[t] Who + bo); loss[0] = -sum logp[t][b][y[t][b]].
 *                h [T][B][H] and logp [T][B][V] are kept for the gradient.
 *   rnn_seq_bwd: ACCUMULATES the gradient of dloss[0] * loss into dWxh, dWhh, dbh, dWho, dbo (inputs and h0 get none).
 * The weights must fit one SM's shared memory (LTB_E_LIMIT otherwise: use the per-step calls); the first call must come
 * before a step is recorded. */
int LTB_FN(rnn_seq_fwd)(const float* x, const int32_t* y, const float* h0, const float* Wxh, const float* Whh, const float* bh,
                        const float* Who, const float* bo, float* h, float* logp, float* loss, int T, int B, int V, int H);
int LTB_FN(rnn_seq_bwd)(const float* x, const int32_t* y, const float* h0, const float* Whh, const float* Who, const float* h,
                        const float* logp, const float* dloss, float* dWxh, float* dWhh, float* dbh, float* dWho, float* dbo,
                        int T, int B, int V, int H);

/* One node of the binary tree LSTM in one call forward and one call backward (no Backend counterpart: the reference stages a
 * node operator by operator, PLDI19APP/SentimentTreeLSTM.scala:67-146 = NIPS18App/SentimentTreeLSTM.scala:118-170).
 * Gate slots: 0 input gate i, 1 forget gate of the left child fl, 2 forget gate of the right child fr, 3 output gate o
 * (all sigmoid), 4 update u (tanh).  A leaf uses slots 0, 3, 4 over ONE input (the embedding row); an inner node all five
 * over TWO inputs (the children's first state vector):  gate[g] = act(W[g][0] in[0] (+ W[g][1] in[1]) + bias[g]).
 *   c = i*u (+ fl*cl + fr*cr);  tc = tanh(c);  h = o*tc;
 *   logp = logSoftmax(Why (classify_cell ? c : h) + by);  loss[0] = -logp[score[0]] (+ loss_l[0] + loss_r[0]).
 * tree_node_bwd reads the gradients that arrived in dc, dh, dloss and ACCUMULATES into dW, dbias, din, dcl, dcr, dWhy, dby,
 * dloss_l, dloss_r (any of din, dcl, dcr, dloss_l, dloss_r may be NULL: an input, a leaf). */
typedef struct ltb_tree_node {
  int hidden;                 /* length of every gate, of c and of h */
  int in_len;                 /* length of the gate inputs: the embedding for a leaf, hidden for an inner node */
  int classes;                /* rows of the classifier, at most 32 */
  int inner;                  /* 0: leaf, 1: inner node */
  int classify_cell;          /* the classifier reads c (the exchanged roles of the PLDI19 application) instead of h */
  const float* in[2];         /* gate inputs (in[1] NULL for a leaf) */
  float* din[2];
  const float* W[5][2];       /* [hidden][in_len] each; unused slots NULL */
  float* dW[5][2];
  const float* bias[5];       /* [hidden]; slots 1 and 2 may name the same vector */
  float* dbias[5];
  const float* cl;            /* the children's second state vector (inner node) */
  const float* cr;
  float* dcl;
  float* dcr;
  const float* Why;           /* classifier [classes][hidden] */
  const float* by;
  float* dWhy;
  float* dby;
  const int32_t* score;       /* the node's class, in device memory */
  const float* loss_l;        /* the children's accumulated losses (inner node) */
  const float* loss_r;
  float* dloss_l;
  float* dloss_r;
  float* gates;               /* out: [5][hidden] activations, kept for the gradient */
  float* c;                   /* out: [hidden] each */
  float* tc;
  float* h;
  float* logp;                /* out: [classes] */
  float* loss;                /* out: [1] */
  const float* dc;            /* gradients arriving from the parent and from the root's loss */
  const float* dh;
  const float* dloss;
} ltb_tree_node;
int LTB_FN(tree_node_fwd)(const ltb_tree_node* node);
int LTB_FN(tree_node_bwd)(const ltb_tree_node* node);
/* One LEVEL of a tree -- `count` nodes that do not depend on one another (all leaves; then all nodes whose children are done;
 * ...) -- in one call each way.  nodes_host and nodes_dev are the same array of descriptions in host memory (read by the call:
 * checks, launch size) and in device memory (read by the kernels: the caller uploads the array once per tree); the nodes of
 * the call are [first, first + count).  Results are those of tree_node_fwd / tree_node_bwd on each node; two nodes of one
 * backward call may have a common child only if they are the same node's parents -- they are not, in a tree. */
int LTB_FN(tree_nodes_fwd)(const ltb_tree_node* nodes_host, const ltb_tree_node* nodes_dev, int first, int count);
int LTB_FN(tree_nodes_bwd)(const ltb_tree_node* nodes_host, const ltb_tree_node* nodes_dev, int first, int count);

/* Branch regions (no counterpart in the reference, whose generated programs issue everything on one stream): two runs of
 * calls that do not depend on each other -- the shortcut convolution of a residual block and its main path, the two
 * expand convolutions of a fire module -- may overlap on the device.
 *   ltb_branch_mark()   remembers the current point of the stream (both runs may read what was issued before it);
 *   ltb_branch_begin()  the calls that follow are issued on a second stream that starts from the marked point;
 *   ltb_branch_end()    back to the first stream;
 *   ltb_branch_join()   the first stream waits for the branch: from here on its results may be used.
 * Calls issued between mark and begin belong to the first run.  The caller guarantees that the branch and the calls issued
 * on the first stream between mark and join touch no common buffer other than read-only inputs (gradients ACCUMULATE into
 * their destinations, so two runs that end in the same gradient buffer must be separated by the join).  One region at a
 * time; not nested.  Staging memory taken inside a region is returned by the next ltb_reset, not at the end of its call. */
int   LTB_FN(branch_mark)(void);
int   LTB_FN(branch_begin)(void);
int   LTB_FN(branch_end)(void);
int   LTB_FN(branch_join)(void);

/* Whole-step replay. Shapes are static and the bump arena hands out the same addresses every iteration after
 * ltb_reset, so one training step can be recorded once and replayed: graph_begin starts recording the calls
 * that follow on the library's stream, graph_end returns a handle, graph_launch replays it.  Calls that
 * touch the host (randinit, dropout, d2h) are not allowed while recording. */
int   LTB_FN(graph_begin)(void);
void* LTB_FN(graph_end)(void);
int   LTB_FN(graph_launch)(void* graph);
int   LTB_FN(graph_destroy)(void* graph);

/* Built-in launch profiler: while on, every kernel launch of the library is bracketed by a CUDA event pair on the
 * launching stream. The report has one line per kernel: name<TAB>launches<TAB>total milliseconds. */
int   LTB_FN(profile)(int on);
int   LTB_FN(profile_report)(char* buf, int len);

/* ---------------------------------------------------------------- fill / init (CPU.scala:30-67, 101-119) */
int LTB_FN(fill)(float* x, float value, int64_t n);                                  /* fill, fillInPlace */
int LTB_FN(fill_with_bias)(float* out, const float* bias, int outer, int c, int inner); /* fillWithBias */
/* randinit: (rand()/RAND_MAX - 0.5)*scale drawn on the HOST with glibc rand() in element order, then
 * uploaded (TensorDslCublas.scala:154-155); seed >= 0 calls srand(seed) first. */
int LTB_FN(randinit)(float* x, int64_t n, float scale, int seed);
int LTB_FN(clip)(float* x, float bound, int64_t n);                                  /* clipAt */

/* ---------------------------------------------------------------- dot family (TD.scala:186-219, CPU.scala:135-225) */
int LTB_FN(vv_dot)(const float* x, const float* y, float* out, int n);               /* out[0] = x.y           ow */
int LTB_FN(vv_dot_grad)(float* dx, float* dy, const float* x, const float* y, const float* dout, int n); /* acc; dx/dy nullable */
int LTB_FN(mv_dot)(const float* a, const float* x, float* out, int m, int k);        /* out[m] = A[m,k] x[k]   ow */
int LTB_FN(mm_dot)(const float* a, const float* b, float* out, int m, int k, int n); /* out[m,n] = A[m,k]B[k,n] ow */
int LTB_FN(add_cartesian)(float* da, const float* y, const float* dout, int m, int k);   /* dA[i,j] += y[j]*dout[i] */
int LTB_FN(add_composition)(float* dx, const float* a, const float* dout, int m, int k); /* dx[k] += A^T dout      */
int LTB_FN(add_dot_trans1)(float* db, const float* a, const float* dc, int m, int k, int n); /* dB[k,n] += A^T dC   */
int LTB_FN(add_dot_trans2)(float* da, const float* dc, const float* b, int m, int k, int n); /* dA[m,k] += dC B^T   */

/* gemm / gemm_grad (TD.scala:279-280, CPU.scala:379-472): C[M,N] = alpha * op(A) op(B), op(A) is M x K.
 * A is stored [M,K] (transA=0) or [K,M] (transA=1); B is [K,N] or [N,K]. Gradients accumulate;
 * dA or dB may be NULL (isInput). */
int LTB_FN(gemm)(const float* a, int trans_a, const float* b, int trans_b, float alpha, float* c, int M, int N, int K);
int LTB_FN(gemm_grad)(const float* a, float* da, int trans_a, const float* b, float* db, int trans_b,
                      float alpha, const float* dc, int M, int N, int K);

/* ---------------------------------------------------------------- convolution (TD.scala:292-296, CPU.scala:484-692)
 * x[N,C,H,W], w[K,C,R,S], bias[K] or NULL, y[N,K,Ho,Wo] ow, Ho=(H+2ph-R)/sh+1. Cross-correlation,
 * dilation 1, groups 1.  Backward: dx acc (NULL when the input is a leaf), dw acc, dbias acc (nullable). */
int LTB_FN(conv2d_fwd)(const float* x, const float* w, const float* bias, float* y,
                       int N, int C, int H, int W, int K, int R, int S, int sh, int sw, int ph, int pw);
int LTB_FN(conv2d_bwd)(const float* x, float* dx, const float* w, float* dw, float* dbias, const float* dy,
                       int N, int C, int H, int W, int K, int R, int S, int sh, int sw, int ph, int pw);

/* ---------------------------------------------------------------- pooling (TD.scala:298-302, CPU.scala:848-1038)
 * Max pool: output starts at -FLT_MAX, window scanned row-major with strict '>', so the first maximum
 * wins; idx[i] is the flat int32 index of the winner in the WHOLE batch tensor (CPU.scala:906-909).
 * pad must be 0 for avg pool (CPU.scala:1003-1005). Backward passes accumulate. */
int LTB_FN(maxpool_fwd)(const float* x, float* y, int32_t* idx, int N, int C, int H, int W,
                        int kh, int kw, int sh, int sw, int pad);
int LTB_FN(maxpool_bwd)(float* dx, const float* dy, const int32_t* idx, int64_t n_out);
int LTB_FN(avgpool_fwd)(const float* x, float* y, int N, int C, int H, int W, int kh, int kw, int sh, int sw);
int LTB_FN(avgpool_bwd)(float* dx, const float* dy, int N, int C, int H, int W, int kh, int kw, int sh, int sw);

/* ---------------------------------------------------------------- batch norm (TD.scala:304-306)
 * Spatial BN over N*HW per channel.  Forward follows CPU.scala:1047-1056 (mean, biased variance,
 * eps inside the sqrt); saved statistics and running-stat update follow what the reference's GPU
 * backend gets from cuDNN (TensorDslCudnn.scala:1025-1109): save_mean, save_istd = 1/sqrt(var+eps),
 * run = (1-momentum)*run + momentum*batch (unbiased variance for run_var); run_* may be NULL.
 * Backward accumulates dx, dgamma, dbeta (alpha=beta=1 at TensorDslCudnn.scala:1106-1108). */
int LTB_FN(bn_train_fwd)(const float* x, float* y, const float* gamma, const float* beta,
                         float* run_mean, float* run_var, float* save_mean, float* save_istd,
                         int N, int C, int HW, float eps, float momentum);
int LTB_FN(bn_bwd)(const float* x, float* dx, const float* dy, const float* gamma, float* dgamma, float* dbeta,
                   const float* save_mean, const float* save_istd, int N, int C, int HW);
int LTB_FN(bn_inference)(const float* x, float* y, const float* gamma, const float* beta,
                         const float* run_mean, const float* run_var, int N, int C, int HW, float eps);

/* ---------------------------------------------------------------- broadcasting elementwise (TD.scala:222-275, CPU.scala:227-374)
 * Shapes are what Tensor.dimBroadcast (TD.scala:998-1016) returns: both right-aligned and padded
 * with leading 1s to the same rank (<= 4); every dim pair is equal or one side is 1. */
int LTB_FN(ew_binary)(int op, const float* a, const int* ashape, const float* b, const int* bshape, float* out, int rank); /* ow */
int LTB_FN(ew_binary_grad)(int op, const float* a, float* da, const int* ashape, const float* b, float* db, const int* bshape,
                           const float* dout, int rank);                              /* acc; da/db nullable */
int LTB_FN(ew_scalar)(int op, const float* a, float s, float* out, int64_t n);         /* tensor (op) scalar, ow */
int LTB_FN(ew_inplace)(int op, float* x, const int* xshape, const float* y, const int* yshape, int rank); /* x = x (op) y, y broadcast or reduced into x */
int LTB_FN(ew_inplace_scalar)(int op, float* x, float s, int64_t n);
/* plusBias / plusEqual and their grads are ew_inplace(LTB_ADD, ...) with the roles the Backend gives them
 * (CPU.scala:281-296); provided as named entry points for the emitted code. */
int LTB_FN(plus_bias)(float* main, const int* mshape, const float* bias, const int* bshape, int rank);
int LTB_FN(plus_bias_grad)(float* dbias, const int* bshape, const float* dmain, const int* mshape, int rank);
/* geam (TD.scala:273): out = alpha*op(x) + beta*op(y); out is rows x cols; may alias x or y when no transpose. */
int LTB_FN(geam)(const float* x, int trans_x, float alpha, const float* y, int trans_y, float beta, float* out, int rows, int cols);
int LTB_FN(trans)(const float* x, float* out, int rows, int cols);                    /* out[cols,rows] ow */
int LTB_FN(trans_grad)(float* dx, const float* dy, int rows, int cols);               /* dx[rows,cols] += dy^T */

/* ---------------------------------------------------------------- activations (TD.scala:319-335, CPU.scala:710-781)
 * unary: out may alias x (relu in place). unary_grad: dx acc, from x (input), y (result), dy.
 * relu in place: the caller passes dx == dy and in_place=1; the gradient is masked where the
 * (already clamped) value is not positive -- see the note at ltb_unary_grad in the sources. */
int LTB_FN(unary)(int op, const float* x, float* out, int64_t n);
int LTB_FN(unary_grad)(int op, const float* x, float* dx, const float* y, const float* dy, int64_t n, int in_place);

/* ---------------------------------------------------------------- softmax / loss (TD.scala:338-346, CPU.scala:783-846, 1090-1110) */
int LTB_FN(softmax)(const float* x, float* y, int rows, int cols);
int LTB_FN(log_softmax)(const float* x, float* y, int rows, int cols);
int LTB_FN(softmax_grad)(float* dx, const float* y, const float* dy, int rows, int cols);      /* acc */
int LTB_FN(log_softmax_grad)(float* dx, const float* y, const float* dy, int rows, int cols);  /* acc */
int LTB_FN(nll)(const float* x, const int32_t* target, float* out, int rows, int cols);        /* out[b] = -x[b,t[b]] */
int LTB_FN(nll_grad)(float* dx, const float* dout, const int32_t* target, int rows, int cols); /* dx[b,t[b]] -= dout[b] */

/* ---------------------------------------------------------------- reductions (TD.scala:352-366, CPU.scala:1115-1164) */
int LTB_FN(sum)(const float* x, float* out, int64_t n);            /* out[0] ow */
int LTB_FN(sum_grad)(float* dx, const float* dout, int64_t n);     /* dx[i] += dout[0] */
int LTB_FN(mean)(const float* x, float* out, int64_t n);
int LTB_FN(mean_grad)(float* dx, const float* dout, int64_t n);    /* dx[i] += dout[0]/n */
/* sum() for callers that may not allocate: same result as sum(), bit for bit, but the partial sums live in a fixed
 * device array inside the library instead of a workspace, and the call allocates nothing (no cudaMalloc, no arena
 * block). Has no counterpart in the reference. The first call on a device does a one-time address look-up and should
 * come before any stream capture. Limit: n <= 2^30 elements, else LTB_E_LIMIT. One array per device: calls that
 * overlap in time (two streams, two threads) race; calls on one stream do not. */
int LTB_FN(sum_static_scratch)(const float* x, float* out, int64_t n);   /* out[0] ow */
int LTB_FN(sum_dim)(const float* x, float* out, int outer, int d, int inner);         /* out[outer,inner] ow */
int LTB_FN(sum_dim_grad)(float* dx, const float* dout, int outer, int d, int inner);  /* acc */

/* ---------------------------------------------------------------- concat (TD.scala:369-370, CPU.scala:1166-1212)
 * Inputs i has shape [outer, dims[i], inner]; out is [outer, sum(dims), inner]. */
int LTB_FN(concat)(float* out, const float* const* inputs, const int* dims, int n_inputs, int outer, int inner);
int LTB_FN(concat_grad)(float* const* dinputs, const float* dout, const int* dims, int n_inputs, int outer, int inner); /* acc; entries nullable */

/* ---------------------------------------------------------------- dropout (TD.scala:312-313, CPU.scala:1066-1088)
 * ltb_dropout draws the keep mask on the host from glibc rand() in element order (rand()/RAND_MAX > p
 * keeps and scales by 1/(1-p)), exactly the stream the CPU backend consumes, and uploads it.
 * ltb_dropout_masked applies a mask the caller already has on the device. */
int LTB_FN(dropout)(const float* x, float* y, float* mask, float p, int64_t n);
int LTB_FN(dropout_masked)(const float* x, float* y, const float* mask, int64_t n);
int LTB_FN(dropout_grad)(float* dx, const float* mask, const float* dy, int64_t n);   /* acc */

/* ---------------------------------------------------------------- optimizers (NNModule.scala:265-303, CPU.scala:1217-1246)
 * sgd_step = geam(x, 1, d, -lr) followed by clear_grad, fused; the multi form walks n tensors in one launch. */
int LTB_FN(sgd_step)(float* x, float* d, float lr, int64_t n);
int LTB_FN(sgd_step_multi)(float* const* xs, float* const* ds, const int64_t* sizes, int n_tensors, float lr);
int LTB_FN(adagrad_update)(float* x, float* d, float* h, float lr, float clip, int descent, int64_t n);
int LTB_FN(momentum_update)(float* x, float* d, float* m, float lr, float mu, float clip, int nesterov, int descent, int64_t n);

/* ---------------------------------------------------------------- data parallelism (no counterpart in the reference,
 * which is single-GPU: src/out/PLDI19evaluation/run_exp.sh:7).  One process per GPU; rank 0 creates the id
 * and the launcher distributes it.  allreduce_sgd_step: d <- sum over ranks of d, then
 * x -= lr * d / world, d = 0, bucket by bucket so the update of one bucket overlaps the reduction of the next. */
int LTB_FN(comm_unique_id)(void* out128);
int LTB_FN(comm_init)(int rank, int world, const void* id128);
int LTB_FN(comm_destroy)(void);
int LTB_FN(comm_world)(void);
/* Failure detection between ranks: while a communicator exists, every host-side wait on the library's stream (sync, d2h,
 * marker_wait) polls NCCL's asynchronous error state and gives up after this many milliseconds (default 60000; 0 = wait for
 * ever). On an error or a timeout the communicator is aborted, the call returns LTB_E_COMM, and later collectives are
 * refused with LTB_E_COMM until comm_destroy / comm_init. */
int LTB_FN(comm_set_timeout_ms)(int64_t ms);
/* Measurement: milliseconds between the end of backward on the compute stream and the start of the update kernel of the
 * last allreduce_sgd_step that followed allreduce_begin calls (the part of the exchange that backward did not hide);
 * 0 with one rank. Waits for that step to finish. */
int LTB_FN(comm_exposed_ms)(float* out_ms);
int LTB_FN(allreduce_sum)(float* x, int64_t n);
/* Starts, while backward is still running, the sum of a gradient range that is already final; the allreduce_sgd_step
 * that follows over a span containing it only waits for that sum. No-op with one rank. */
int LTB_FN(allreduce_begin)(float* d, int64_t n);
int LTB_FN(allreduce_sgd_step)(float* x, float* d, float lr, int64_t n);

#ifdef __cplusplus
}
#endif
#endif /* LANTERN_B200_H */
