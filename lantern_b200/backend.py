"""Python mirror of the reference's `Backend` trait over the C ABI.

Method names, argument meaning and accumulate/overwrite behaviour follow
src/main/scala/lantern/TensorDifferentiation.scala:137-379, so tests written against this class read like
the reference's own (src/test/scala/lantern/TestCudnn.scala etc.).  A `Tensor` is a (pointer, shape) pair in
the library's arena, a `TensorR` pairs a value `x` with its gradient `d` (TD.scala:1146-1160).
"""
import ctypes

import numpy as np

ADD, SUB, MUL, DIV = 0, 1, 2, 3
RELU, TANH, SIGMOID, EXP, LOG, SQRT, SQUARE = range(7)


def _prod(shape):
    p = 1
    for s in shape:
        p *= int(s)
    return p


class Tensor:
    """Dense row-major float32 tensor living in the backend's arena (Tensor, TD.scala:386)."""

    def __init__(self, backend, ptr, shape, dtype=np.float32):
        self.backend, self.ptr, self.shape, self.dtype = backend, ptr, tuple(int(s) for s in shape), dtype

    @property
    def scalarCount(self):
        return _prod(self.shape)

    @property
    def rank(self):
        return len(self.shape)

    def resize(self, *shape):
        shape = list(shape)
        if -1 in shape:
            i = shape.index(-1)
            shape[i] = self.scalarCount // max(1, -_prod(shape))
        assert _prod(shape) == self.scalarCount
        return Tensor(self.backend, self.ptr, shape, self.dtype)

    def toCPU(self):
        out = np.empty(self.shape, dtype=self.dtype)
        self.backend.lib.d2h(out.ctypes.data, self.ptr, out.nbytes)
        return out

    def offset(self, elems, shape):
        return Tensor(self.backend, self.ptr + 4 * int(elems), shape, self.dtype)


class TensorR:
    """Value + gradient pair (TensorR, TD.scala:1146)."""

    def __init__(self, x, d=None, isInput=False):
        self.x = x
        self.d = d if d is not None else x.backend.zeros(*x.shape)
        self.isInput = isInput


def _ints(seq):
    return (ctypes.c_int * len(seq))(*[int(s) for s in seq])


def dimBroadcast(a, b):
    """Tensor.dimBroadcast, TD.scala:998-1016: right-align, pad with 1s, check compatibility."""
    a, b = list(a), list(b)
    r = max(len(a), len(b))
    a = [1] * (r - len(a)) + a
    b = [1] * (r - len(b)) + b
    res = []
    for x, y in zip(a, b):
        if not (x == 1 or y == 1 or x == y):
            raise ValueError("dimensions not compatible for broadcasting %s with %s" % (a, b))
        res.append(max(x, y))
    return a, b, res


class Backend:
    """Mirror of `trait Backend`; `lib` is a BoundLibrary (the CUDA product, or the CPU oracle in tests)."""

    def __init__(self, lib):
        self.lib = lib

    # ---- lifetime / memory (TD.scala:139-177)
    def setup(self, device=0, heap_bytes=1 << 30):
        self.lib.init(device, heap_bytes)

    def cleanup(self):
        self.lib.shutdown()

    def mallocArray(self, length, dtype=np.float32, zero=True):
        n = int(length) * np.dtype(dtype).itemsize
        return self.lib.malloc(n) if zero else self.lib.malloc_uninit(n)

    def zeros(self, *shape):
        return Tensor(self, self.mallocArray(_prod(shape)), shape)

    def empty(self, *shape):
        return Tensor(self, self.mallocArray(_prod(shape), zero=False), shape)

    def fromNumpy(self, a):
        dt = np.int32 if np.issubdtype(np.asarray(a).dtype, np.integer) else np.float32
        a = np.ascontiguousarray(a, dtype=dt)
        t = Tensor(self, self.mallocArray(max(1, a.size), dt, zero=False), a.shape, dt)
        if a.size:
            self.lib.h2d(t.ptr, a.ctypes.data, a.nbytes)
        return t

    def copyFloatArray(self, dest, src, length):
        self.lib.d2d(dest.ptr, src.ptr, 4 * int(length))

    def copyTensorData(self, dest, src):
        assert dest.scalarCount == src.scalarCount
        self.copyFloatArray(dest, src, dest.scalarCount)

    def makeTensor(self, dims, *scalars):
        return self.fromNumpy(np.array(scalars, dtype=np.float32).reshape(dims))

    def fill(self, dims, value):
        t = self.empty(*dims)
        self.lib.fill(t.ptr, float(value), t.scalarCount)
        return t

    def fillInPlace(self, x, value):
        self.lib.fill(x.ptr, float(value), x.scalarCount)

    def fillWithBias(self, dims, bias, dim):
        t = self.empty(*dims)
        self.lib.fill_with_bias(t.ptr, bias.ptr, _prod(dims[:dim]), dims[dim], _prod(dims[dim + 1:]))
        return t

    def randinit(self, dims, scale=1.0, seed=None):
        t = self.empty(*dims)
        self.lib.randinit(t.ptr, t.scalarCount, float(scale), -1 if seed is None else int(seed))
        return t

    def clipAt(self, x, bound):
        self.lib.clip(x.ptr, float(bound), x.scalarCount)

    # ---- dot family (TD.scala:186-219)
    def vectorVectorDot(self, x, y):
        out = self.empty(1)
        self.lib.vv_dot(x.ptr, y.ptr, out.ptr, x.shape[0])
        return out

    def matrixVectorDot(self, x, y):
        out = self.empty(x.shape[0])
        self.lib.mv_dot(x.ptr, y.ptr, out.ptr, x.shape[0], x.shape[1])
        return out

    def matrixMatrixDot(self, x, y):
        out = self.empty(x.shape[0], y.shape[1])
        self.lib.mm_dot(x.ptr, y.ptr, out.ptr, x.shape[0], x.shape[1], y.shape[1])
        return out

    def dot(self, x, y):
        k = (x.rank, y.rank)
        if k == (1, 1):
            return self.vectorVectorDot(x, y)
        if k == (2, 1):
            return self.matrixVectorDot(x, y)
        if k == (2, 2):
            return self.matrixMatrixDot(x, y)
        raise ValueError("Incompatible shapes: %s, %s" % (x.shape, y.shape))

    def dot_grad(self, x, y, output):
        k = (x.x.rank, y.x.rank)
        if k == (1, 1):
            self.lib.vv_dot_grad(0 if x.isInput else x.d.ptr, 0 if y.isInput else y.d.ptr, x.x.ptr, y.x.ptr,
                                 output.d.ptr, x.x.shape[0])
        elif k == (2, 1):
            if not x.isInput:
                self.add_cartesian(x.d, y.x, output.d)
            if not y.isInput:
                self.add_composition(y.d, x.x, output.d)
        else:
            if not x.isInput:
                self.add_dotTrans2(x.d, output.d, y.x)
            if not y.isInput:
                self.add_dotTrans1(y.d, x.x, output.d)

    def add_cartesian(self, x, y, output):
        self.lib.add_cartesian(x.ptr, y.ptr, output.ptr, x.shape[0], x.shape[1])

    def add_composition(self, x, y, output):
        self.lib.add_composition(x.ptr, y.ptr, output.ptr, y.shape[0], y.shape[1])

    def add_dotTrans1(self, x, y, output):     # x += y^T . output
        self.lib.add_dot_trans1(x.ptr, y.ptr, output.ptr, y.shape[0], y.shape[1], output.shape[1])

    def add_dotTrans2(self, x, y, output):     # x += y . output^T
        self.lib.add_dot_trans2(x.ptr, y.ptr, output.ptr, x.shape[0], x.shape[1], output.shape[1])

    # ---- broadcasting elementwise (TD.scala:222-258)
    def _binary(self, op, x, y):
        if not isinstance(y, Tensor):
            out = self.empty(*x.shape)
            self.lib.ew_scalar(op, x.ptr, float(y), out.ptr, x.scalarCount)
            return out
        xs, ys, rs = dimBroadcast(x.shape, y.shape)
        out = self.empty(*rs)
        self.lib.ew_binary(op, x.ptr, _ints(xs), y.ptr, _ints(ys), out.ptr, len(rs))
        return out, tuple(xs), tuple(ys)

    def _binary_grad(self, op, x, y, output):
        xs, ys, _ = dimBroadcast(x.x.shape, y.x.shape)
        self.lib.ew_binary_grad(op, x.x.ptr, 0 if x.isInput else x.d.ptr, _ints(xs), y.x.ptr, 0 if y.isInput else y.d.ptr,
                                _ints(ys), output.d.ptr, len(xs))

    def _inplace(self, op, x, y):
        if not isinstance(y, Tensor):
            self.lib.ew_inplace_scalar(op, x.ptr, float(y), x.scalarCount)
            return
        xs, ys, _ = dimBroadcast(x.shape, y.shape)
        self.lib.ew_inplace(op, x.ptr, _ints(xs), y.ptr, _ints(ys), len(xs))

    def plus(self, x, y): return self._binary(ADD, x, y)
    def minus(self, x, y): return self._binary(SUB, x, y)
    def mul(self, x, y): return self._binary(MUL, x, y)
    def div(self, x, y): return self._binary(DIV, x, y)
    def add_grad(self, x, y, output, xShape=None, yShape=None): self._binary_grad(ADD, x, y, output)
    def minus_grad(self, x, y, output, xShape=None, yShape=None): self._binary_grad(SUB, x, y, output)
    def mul_grad(self, x, y, output, xShape=None, yShape=None): self._binary_grad(MUL, x, y, output)
    def div_grad(self, x, y, output, xShape=None, yShape=None): self._binary_grad(DIV, x, y, output)
    def plus_inplace(self, x, y): self._inplace(ADD, x, y)
    def minus_inplace(self, x, y): self._inplace(SUB, x, y)
    def mul_inplace(self, x, y): self._inplace(MUL, x, y)
    def div_inplace(self, x, y): self._inplace(DIV, x, y)

    def plusBias(self, main, bias):
        ms, bs, _ = dimBroadcast(main.shape, bias.shape)
        self.lib.plus_bias(main.ptr, _ints(ms), bias.ptr, _ints(bs), len(ms))
        return main

    def plusBias_grad(self, main, bias):
        if not bias.isInput:
            ms, bs, _ = dimBroadcast(main.d.shape, bias.d.shape)
            self.lib.plus_bias_grad(bias.d.ptr, _ints(bs), main.d.ptr, _ints(ms), len(ms))

    def plusEqual(self, base, adder):
        self._inplace(ADD, base, adder)
        return base

    def plusEqual_grad(self, base, adder):
        if not adder.isInput:
            self._inplace(ADD, adder.d, base.d)

    def geam(self, x, transX, alpha, y, transY, beta, output):
        rows, cols = (output.shape if output.rank == 2 else (1, output.scalarCount))
        self.lib.geam(x.ptr, int(transX), float(alpha), y.ptr, int(transY), float(beta), output.ptr, rows, cols)

    def trans(self, x):
        out = self.empty(x.shape[1], x.shape[0])
        self.lib.trans(x.ptr, out.ptr, x.shape[0], x.shape[1])
        return out

    def trans_grad(self, x, y):
        self.lib.trans_grad(x.d.ptr, y.d.ptr, x.x.shape[0], x.x.shape[1])

    # ---- gemm (TD.scala:279-280)
    def gemm(self, x, transX, y, transY, alpha):
        M = x.shape[1] if transX else x.shape[0]
        K = x.shape[0] if transX else x.shape[1]
        N = y.shape[0] if transY else y.shape[1]
        out = self.empty(M, N)
        self.lib.gemm(x.ptr, int(transX), y.ptr, int(transY), float(alpha), out.ptr, M, N, K)
        return out

    def gemm_grad(self, x, transX, y, transY, alpha, output):
        M, N = output.x.shape
        K = x.x.shape[0] if transX else x.x.shape[1]
        self.lib.gemm_grad(x.x.ptr, 0 if x.isInput else x.d.ptr, int(transX), y.x.ptr, 0 if y.isInput else y.d.ptr,
                           int(transY), float(alpha), output.d.ptr, M, N, K)

    # ---- convolution / pooling / batch norm (TD.scala:292-306)
    @staticmethod
    def _pads(pads):
        pads = list(pads)
        if len(pads) == 1:
            return pads[0], pads[0]
        if len(pads) == 2:
            return pads[0], pads[1]
        return pads[0], pads[2]          # TensorDslCPU.scala:534

    def conv2D_batch(self, input, kernel, bias, strides, pads):
        ph, pw = self._pads(pads)
        sh, sw = strides[0], strides[1]
        N, C, H, W = input.shape
        K, _, R, S = kernel.shape
        out = self.empty(N, K, (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1)
        self.lib.conv2d_fwd(input.ptr, kernel.ptr, bias.ptr if bias is not None else 0, out.ptr, N, C, H, W, K, R, S, sh, sw, ph, pw)
        return out, None, 0

    def conv2D_batch_grad(self, input, finput, filter, res, bias, padding, strides, dilations=(1, 1), counter=0):
        assert tuple(dilations) == (1, 1)
        N, C, H, W = input.x.shape
        K, _, R, S = filter.x.shape
        self.lib.conv2d_bwd(input.x.ptr, 0 if input.isInput else input.d.ptr, filter.x.ptr, filter.d.ptr,
                            bias.d.ptr if bias is not None else 0, res.d.ptr, N, C, H, W, K, R, S, strides[0], strides[1],
                            padding[0], padding[1])

    def maxPool2D_batch(self, input, kernel, strides, pads=None):
        N, C, H, W = input.shape
        pad = 0 if pads is None else pads[0]
        oh, ow = (H + 2 * pad - kernel[0]) // strides[0] + 1, (W + 2 * pad - kernel[1]) // strides[1] + 1
        out = self.empty(N, C, oh, ow)
        idx = Tensor(self, self.mallocArray(out.scalarCount, np.int32, zero=False), out.shape, np.int32)
        self.lib.maxpool_fwd(input.ptr, out.ptr, idx.ptr, N, C, H, W, kernel[0], kernel[1], strides[0], strides[1], pad)
        return out, idx

    def maxPool2D_batch_grad(self, input, output, sidx, kernel=None, strides=None, pads=None):
        self.lib.maxpool_bwd(input.d.ptr, output.d.ptr, sidx.ptr, output.d.scalarCount)

    def averagePool2D_batch(self, input, kernel, strides, pads=(0, 0, 0, 0)):
        assert all(p == 0 for p in pads)
        N, C, H, W = input.shape
        out = self.empty(N, C, (H - kernel[0]) // strides[0] + 1, (W - kernel[1]) // strides[1] + 1)
        self.lib.avgpool_fwd(input.ptr, out.ptr, N, C, H, W, kernel[0], kernel[1], strides[0], strides[1])
        return out

    def averagePool2D_batch_grad(self, input, output, kernel, strides, pads=(0, 0, 0, 0)):
        N, C, H, W = input.x.shape
        self.lib.avgpool_bwd(input.d.ptr, output.d.ptr, N, C, H, W, kernel[0], kernel[1], strides[0], strides[1])

    def batchNormTraining(self, x, scale, bias, runningMean, runningVar, eps=1e-5, momentum=0.1):
        N, C = x.shape[0], x.shape[1]
        HW = _prod(x.shape[2:])
        y, sm, si = self.empty(*x.shape), self.empty(C), self.empty(C)
        self.lib.bn_train_fwd(x.ptr, y.ptr, scale.ptr, bias.ptr, runningMean.ptr if runningMean else 0,
                              runningVar.ptr if runningVar else 0, sm.ptr, si.ptr, N, C, HW, eps, momentum)
        return y, sm, si, 0

    def batchNorm_grad(self, input, res, scale, bias, saveMean, saveInvVariance, counterId=0):
        N, C = input.x.shape[0], input.x.shape[1]
        HW = _prod(input.x.shape[2:])
        self.lib.bn_bwd(input.x.ptr, 0 if input.isInput else input.d.ptr, res.d.ptr, scale.x.ptr, scale.d.ptr, bias.d.ptr,
                        saveMean.ptr, saveInvVariance.ptr, N, C, HW)

    def batchNormInference(self, x, scale, bias, runningMean, runningVar, eps=1e-5):
        N, C = x.shape[0], x.shape[1]
        y = self.empty(*x.shape)
        self.lib.bn_inference(x.ptr, y.ptr, scale.ptr, bias.ptr, runningMean.ptr, runningVar.ptr, N, C, _prod(x.shape[2:]), eps)
        return y

    # ---- dropout (TD.scala:312-313)
    def dropout(self, input, prob=0.5):
        y, mask = self.empty(*input.shape), self.empty(*input.shape)
        self.lib.dropout(input.ptr, y.ptr, mask.ptr, float(prob), input.scalarCount)
        return y, mask, 0

    def dropout_grad(self, input, output, prob, helper, size=0):
        self.lib.dropout_grad(input.d.ptr, helper.ptr, output.d.ptr, input.x.scalarCount)

    # ---- activations (TD.scala:319-335)
    def _unary(self, op, x, inPlace=False):
        out = x if inPlace else self.empty(*x.shape)
        self.lib.unary(op, x.ptr, out.ptr, x.scalarCount)
        return out

    def _unary_grad(self, op, input, res, inPlace=False):
        self.lib.unary_grad(op, input.x.ptr, input.d.ptr, res.x.ptr, res.d.ptr, input.x.scalarCount, int(inPlace))

    def relu(self, x, inPlace=False): return self._unary(RELU, x, inPlace)
    def tanh(self, x): return self._unary(TANH, x)
    def sigmoid(self, x): return self._unary(SIGMOID, x)
    def exp(self, x): return self._unary(EXP, x)
    def log(self, x): return self._unary(LOG, x)
    def sqrt(self, x): return self._unary(SQRT, x)
    def square(self, x): return self._unary(SQUARE, x)
    def relu_grad(self, input, res, inPlace=False): self._unary_grad(RELU, input, res, inPlace)
    def tanh_grad(self, input, res): self._unary_grad(TANH, input, res)
    def sigmoid_grad(self, input, res): self._unary_grad(SIGMOID, input, res)
    def exp_grad(self, input, res): self._unary_grad(EXP, input, res)
    def log_grad(self, input, res): self._unary_grad(LOG, input, res)
    def sqrt_grad(self, input, res): self._unary_grad(SQRT, input, res)
    def square_grad(self, input, res): self._unary_grad(SQUARE, input, res)

    # ---- softmax / loss (TD.scala:338-346)
    def softmax(self, x, dim=1):
        assert x.rank == 2 and dim == 1
        y = self.empty(*x.shape)
        self.lib.softmax(x.ptr, y.ptr, x.shape[0], x.shape[1])
        return y

    def logSoftmax(self, x, dim=1):
        assert x.rank == 2 and dim == 1
        y = self.empty(*x.shape)
        self.lib.log_softmax(x.ptr, y.ptr, x.shape[0], x.shape[1])
        return y

    def softmax_grad(self, input, res, dim=1):
        self.lib.softmax_grad(input.d.ptr, res.x.ptr, res.d.ptr, res.x.shape[0], res.x.shape[1])

    def logSoftmax_grad(self, input, res, dim=1):
        self.lib.log_softmax_grad(input.d.ptr, res.x.ptr, res.d.ptr, res.x.shape[0], res.x.shape[1])

    def nllLoss(self, x, target):
        out = self.empty(x.shape[0])
        self.lib.nll(x.ptr, target.ptr, out.ptr, x.shape[0], x.shape[1])
        return out

    def nllLoss_grad(self, input, res, target):
        self.lib.nll_grad(input.d.ptr, res.d.ptr, target.ptr, input.x.shape[0], input.x.shape[1])

    # ---- reductions (TD.scala:352-366)
    def sum(self, x, dim=None):
        if dim is None:
            out = self.empty(1)
            self.lib.sum(x.ptr, out.ptr, x.scalarCount)
            return out
        outer, d, inner = _prod(x.shape[:dim]), x.shape[dim], _prod(x.shape[dim + 1:])
        out = self.empty(*(x.shape[:dim] + x.shape[dim + 1:]))
        self.lib.sum_dim(x.ptr, out.ptr, outer, d, inner)
        return out

    def sum_grad(self, input, res, dim=None):
        if dim is None:
            self.lib.sum_grad(input.d.ptr, res.d.ptr, input.x.scalarCount)
        else:
            s = input.x.shape
            self.lib.sum_dim_grad(input.d.ptr, res.d.ptr, _prod(s[:dim]), s[dim], _prod(s[dim + 1:]))

    def mean(self, x):
        out = self.empty(1)
        self.lib.mean(x.ptr, out.ptr, x.scalarCount)
        return out

    def mean_grad(self, input, res):
        self.lib.mean_grad(input.d.ptr, res.d.ptr, input.x.scalarCount)

    # ---- concat (TD.scala:369-370)
    def concat(self, dim, tensors):
        s0 = tensors[0].shape
        outer, inner = _prod(s0[:dim]), _prod(s0[dim + 1:])
        dims = [t.shape[dim] for t in tensors]
        out = self.empty(*(s0[:dim] + (sum(dims),) + s0[dim + 1:]))
        ptrs = (ctypes.c_void_p * len(tensors))(*[t.ptr for t in tensors])
        self.lib.concat(out.ptr, ctypes.addressof(ptrs), _ints(dims), len(tensors), outer, inner)
        return out

    def concat_grad(self, dim, tensorRs, output):
        s0 = tensorRs[0].x.shape
        outer, inner = _prod(s0[:dim]), _prod(s0[dim + 1:])
        dims = [t.x.shape[dim] for t in tensorRs]
        ptrs = (ctypes.c_void_p * len(tensorRs))(*[0 if t.isInput else t.d.ptr for t in tensorRs])
        self.lib.concat_grad(ctypes.addressof(ptrs), output.d.ptr, _ints(dims), len(tensorRs), outer, inner)

    # ---- optimizers (TD.scala:377-378, NNModule.scala:265-303)
    def sgd_step(self, tr, learning_rate):
        self.lib.sgd_step(tr.x.ptr, tr.d.ptr, float(learning_rate), tr.x.scalarCount)

    def adagrad_update(self, tr, t, learning_rate, gradClip, descent=True):
        self.lib.adagrad_update(tr.x.ptr, tr.d.ptr, t.ptr, float(learning_rate), float(gradClip), int(descent), tr.x.scalarCount)

    def momentum_update(self, tr, t, learning_rate, momentum, gradClip, nesterov, descent=True):
        self.lib.momentum_update(tr.x.ptr, tr.d.ptr, t.ptr, float(learning_rate), float(momentum), float(gradClip),
                                 int(nesterov), int(descent), tr.x.scalarCount)
