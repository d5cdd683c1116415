"""Known-answer vectors transcribed from the reference's own ScalaTest files (numbers only).

Each case is a function of a `Backend` (lantern_b200.backend.Backend over either library) that performs the
calls of the cited reference test and asserts the reference's expected values with the reference's tolerance
(Tensor.assertEqual, src/main/scala/lantern/TensorDifferentiation.scala:1126-1138: absolute 1e-4).
`T` = src/test/scala/lantern/TestTensorDifferentiation.scala, `C` = TestCudnn.scala, `B` = TestBroadcast.scala,
`U` = TestCublas.scala.
"""
import ctypes

import numpy as np

from lantern_b200.backend import TensorR

TOL = 1e-4


def _eq(expect, got, tol=TOL):
    expect = np.asarray(expect, dtype=np.float32).reshape(got.shape)
    assert np.all(np.abs(expect - got) <= tol), "expected\n%s\ngot\n%s" % (expect, got)


def _glibc_rand(n, seed=None):
    """(float)rand()/RAND_MAX from glibc, as Random.rand() (TD.scala:1018-1026)."""
    libc = ctypes.CDLL(None)
    if seed is not None:
        libc.srand(seed)
    return np.array([np.float32(libc.rand()) / np.float32(2147483647) for _ in range(n)], dtype=np.float32)


def conv_forward(b):                      # T:1096-1115
    x = b.fromNumpy(np.array([1, 2, 3, 4, 5, 6, 7, 8, 1, 2, 3, 4, 5, 6, 7, 8], np.float32).reshape(1, 1, 4, 4))
    k = b.fromNumpy(np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2))
    y, _, _ = b.conv2D_batch(x, k, b.zeros(1), (2, 2), (0, 0, 0, 0))
    _eq([44, 64, 44, 64], y.toCPU())


def conv_forward_bias_one(b):             # C:641-661
    x = b.fromNumpy(np.array([1, 2, 3, 4, 5, 6, 7, 8, 1, 2, 3, 4, 5, 6, 7, 8], np.float32).reshape(1, 1, 4, 4))
    k = b.fromNumpy(np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2))
    y, _, _ = b.conv2D_batch(x, k, b.fill((1,), 1.0), (2, 2), (0, 0, 0, 0))
    _eq([45, 65, 45, 65], y.toCPU())


def conv_pad(b):                          # T:1117-1135, 1157-1174
    x, k = b.fill((1, 1, 4, 4), 1.0), b.fill((1, 1, 3, 3), 1.0)
    y, _, _ = b.conv2D_batch(x, k, b.zeros(1), (3, 3), (1, 1, 1, 1))
    _eq([4, 4, 4, 4], y.toCPU())
    y, _, _ = b.conv2D_batch(x, k, None, (3, 3), (1, 1, 1, 1))
    _eq([4, 4, 4, 4], y.toCPU())


def conv_pad2(b):                         # T:1137-1155
    x = b.fromNumpy(np.array([1, 2, 3, 4, 5, 6, 7, 8, 2, 3, 4, 5, 6, 7, 8, 9], np.float32).reshape(1, 1, 4, 4))
    y, _, _ = b.conv2D_batch(x, b.fill((1, 1, 3, 3), 1.0), b.zeros(1), (3, 3), (1, 1, 1, 1))
    _eq([14, 22, 18, 26], y.toCPU())


def _conv_grad(b, ishape, kshape, strides, pad):
    x, k, bias = TensorR(b.fill(ishape, 1.0)), TensorR(b.fill(kshape, 1.0)), TensorR(b.zeros(1))
    y, _, _ = b.conv2D_batch(x.x, k.x, bias.x, strides, (pad,) * 4)
    out = TensorR(y, b.fill(y.shape, 1.0))          # d(sum)/dy = 1
    b.conv2D_batch_grad(x, None, k, out, bias, (pad, pad), strides, (1, 1))
    return x.d.toCPU(), k.d.toCPU(), bias.d.toCPU()


def conv_backprop(b):                     # T:1178-1208
    dx, dk, db = _conv_grad(b, (1, 1, 3, 3), (1, 1, 2, 2), (1, 1), 0)
    _eq([1, 2, 1, 2, 4, 2, 1, 2, 1], dx); _eq([4] * 4, dk); _eq([4], db)


def conv_backprop_pad(b):                 # T:1210-1244
    dx, dk, db = _conv_grad(b, (1, 1, 4, 4), (1, 1, 3, 3), (3, 3), 1)
    _eq([1] * 16, dx); _eq([1, 2, 1, 2, 4, 2, 1, 2, 1], dk); _eq([4], db)


def conv_bias_grad(b):                    # C:663-694
    dx, dk, db = _conv_grad(b, (1, 1, 4, 4), (1, 1, 3, 3), (1, 1), 0)
    _eq([1, 2, 2, 1, 2, 4, 4, 2, 2, 4, 4, 2, 1, 2, 2, 1], dx); _eq([4] * 9, dk); _eq([4], db)


def maxpool(b):                           # C:797-836
    x = TensorR(b.fromNumpy(np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3)))
    y, idx = b.maxPool2D_batch(x.x, (2, 2), (1, 1), None)
    _eq([5, 6, 8, 9], y.toCPU())
    assert idx.toCPU().ravel().tolist() == [4, 5, 7, 8]
    b.maxPool2D_batch_grad(x, TensorR(y, b.fill(y.shape, 1.0)), idx)
    _eq([0, 0, 0, 0, 1, 1, 0, 1, 1], x.d.toCPU())


def avgpool(b):                           # C:838-877, T:1246-1271
    x = TensorR(b.fromNumpy(np.arange(1, 10, dtype=np.float32).reshape(1, 1, 3, 3)))
    y = b.averagePool2D_batch(x.x, (2, 2), (1, 1))
    _eq([3, 4, 6, 7], y.toCPU())
    b.averagePool2D_batch_grad(x, TensorR(y, b.fill(y.shape, 1.0)), (2, 2), (1, 1))
    _eq([.25, .5, .25, .5, 1, .5, .25, .5, .25], x.d.toCPU())
    x = TensorR(b.fill((1, 1, 4, 4), 1.0))
    y = b.averagePool2D_batch(x.x, (2, 2), (2, 2))
    b.averagePool2D_batch_grad(x, TensorR(y, b.fill(y.shape, 1.0)), (2, 2), (2, 2))
    _eq([.25] * 16, x.d.toCPU())
    x = TensorR(b.fill((1, 1, 4, 4), 1.0))
    y = b.averagePool2D_batch(x.x, (2, 2), (1, 1))
    b.averagePool2D_batch_grad(x, TensorR(y, b.fill(y.shape, 1.0)), (2, 2), (1, 1))
    _eq([.25, .5, .5, .25, .5, 1, 1, .5, .5, 1, 1, .5, .25, .5, .5, .25], x.d.toCPU())


def softmax(b):                           # C:751-772
    x = TensorR(b.fromNumpy(np.array([[1, 2, 3], [4, 5, 6]], np.float32)))
    y = b.softmax(x.x)
    _eq([0.0900305733, 0.2447284758, 0.6652409434] * 2, y.toCPU())
    b.softmax_grad(x, TensorR(y, b.fill(y.shape, 1.0)))
    _eq([0.0000000107, 0.0000000292, 0.0000000793] * 2, x.d.toCPU())


def log_softmax(b):                       # C:774-795
    x = TensorR(b.fromNumpy(np.array([[1, 2, 3], [4, 5, 6]], np.float32)))
    y = b.logSoftmax(x.x)
    _eq([-2.4076058865, -1.4076058865, -0.4076058865, -2.4076061249, -1.4076061249, -0.4076061249], y.toCPU())
    b.logSoftmax_grad(x, TensorR(y, b.fill(y.shape, 1.0)))
    _eq([0.7299082279, 0.2658145428, -0.9957230091, 0.7299083471, 0.2658147216, -0.9957225323], x.d.toCPU())


def nll_loss(b):                          # C:917-938
    x = TensorR(b.fromNumpy(np.array([[1, 2, 3], [4, 5, 6]], np.float32)))
    t = b.fromNumpy(np.array([1, 0], np.int32))
    ls = TensorR(b.logSoftmax(x.x))
    loss = b.nllLoss(ls.x, t)
    _eq([1.4076058865, 2.4076061249], loss.toCPU())
    b.nllLoss_grad(ls, TensorR(loss, b.fill(loss.shape, 1.0)), t)
    b.logSoftmax_grad(x, ls)
    _eq([0.0900305808, -0.7552714944, 0.6652410030, -0.9099694490, 0.2447284311, 0.6652408242], x.d.toCPU())


def batchnorm_inference(b):               # C:1032-1049
    x = b.fill((3, 2, 3, 3), 1.0)
    y = b.batchNormInference(x, b.fill((2,), 3.0), b.fill((2,), 2.0), b.fill((2,), 3.0), b.fill((2,), 4.0))
    _eq([-1.0] * 54, y.toCPU())


BN_RESULT = [
    -4.70055, -2.42800, 0.33646, -1.71884, -3.37612, -3.03992, -0.07803, 1.66236, -2.64498,
    -4.40594, -2.17456, 0.45260, -2.48382, -3.67889, -3.86906, 0.42170, -4.03358, -0.95436,
    -0.62918, 0.73989, 2.56785, -3.27966, -1.47426, -0.98174, -0.55874, -0.70138, 0.62703,
    -0.44310, 0.65435, -0.73941, -2.76659, 0.87396, 1.42567, 1.76504, -2.91541, -3.78245,
    -3.30510, 1.85414, 2.58171, -0.99299, 2.04517, -2.28546, -2.79128, -3.18326, -1.24514,
    -2.01499, 1.94021, -0.85590, 1.60013, -0.91634, -2.54044, 1.48045, 0.51965, 0.44109]
BN_GRAD = [
    3.09040, -0.20212, 3.45742, -1.22957, 1.17154, 0.68444, -3.60681, 1.53643, 0.11224,
    1.99813, -1.06226, 1.89603, -0.63810, 1.00096, 1.26179, 1.93841, 1.48743, -2.73582,
    -2.80830, 2.87292, 0.22452, 1.03179, -1.58392, -2.29750, -2.91035, -2.70368, 3.03643,
    -3.43702, 1.61933, -3.03063, -0.25029, 1.31812, 0.56144, 0.09597, -0.04617, 1.14300,
    1.06865, 1.25857, 0.20445, -2.28120, 0.98180, -0.40863, 0.32422, 0.89211, -1.91587,
    -1.28113, -0.14428, -2.87085, 0.32216, -2.78796, -0.56045, 0.48630, 1.80406, 1.91181]


def batchnorm_training(b):                # C:1051-1118 (srand(42); 54 x rand()-0.5; scale 2, bias -1; relu after)
    xin = (_glibc_rand(54, seed=42) - np.float32(0.5)).reshape(3, 2, 3, 3)
    x = TensorR(b.fromNumpy(xin))
    scale, bias = TensorR(b.fill((2,), 2.0)), TensorR(b.fill((2,), -1.0))
    rm, rv = b.fill((2,), 1.0), b.fill((2,), 1.0)
    y, sm, si, _ = b.batchNormTraining(x.x, scale.x, bias.x, rm, rv)
    _eq(BN_RESULT, y.toCPU())
    yr = TensorR(y)
    r = b.relu(y)
    b.relu_grad(yr, TensorR(r, b.fill(r.shape, 1.0)))
    b.batchNorm_grad(x, yr, scale, bias, sm, si)
    _eq(BN_GRAD, x.d.toCPU())
    # running statistics: exponentialAverageFactor 0.1 (TensorDslCudnn.scala:1027), unbiased variance
    m = 27.0
    mean = xin.mean(axis=(0, 2, 3)); var = xin.var(axis=(0, 2, 3))
    _eq(0.9 * 1.0 + 0.1 * mean, rm.toCPU(), 1e-5)
    _eq(0.9 * 1.0 + 0.1 * var * m / (m - 1), rv.toCPU(), 1e-5)


def gemm_all_transposes(b):               # U:84-110 (gemm == dot of explicit transposes, alpha 0.5)
    r = np.random.default_rng(0)
    m1, m2, m3, m4 = (r.random(s, dtype=np.float32) - 0.5 for s in ((2, 3), (3, 4), (4, 3), (3, 2)))
    for a, ta, bb, tb in ((m1, 0, m2, 0), (m1, 0, m3, 1), (m4, 1, m2, 0), (m4, 1, m3, 1)):
        got = b.gemm(b.fromNumpy(a), ta, b.fromNumpy(bb), tb, 0.5).toCPU()
        via_dot = b.dot(b.trans(b.fromNumpy(a)) if ta else b.fromNumpy(a), b.trans(b.fromNumpy(bb)) if tb else b.fromNumpy(bb)).toCPU() * 0.5
        _eq(via_dot, got)
        _eq(0.5 * (a.T if ta else a) @ (bb.T if tb else bb), got)


def gemm_grad_all_transposes(b):          # U:112-160 (gemm_grad == 0.5 * dot_grad through explicit transposes)
    r = np.random.default_rng(1)
    m1, m2, m3, m4 = (r.random(s, dtype=np.float32) - 0.5 for s in ((2, 3), (3, 4), (4, 3), (3, 2)))
    for a, ta, bb, tb in ((m1, 0, m2, 0), (m1, 0, m3, 1), (m4, 1, m2, 0), (m4, 1, m3, 1)):
        A, Bm = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(bb))
        out = b.gemm(A.x, ta, Bm.x, tb, 0.5)
        b.gemm_grad(A, ta, Bm, tb, 0.5, TensorR(out, b.fill(out.shape, 1.0)))
        ones = np.ones(out.shape, np.float32)
        opa, opb = (a.T if ta else a), (bb.T if tb else bb)
        da, db = 0.5 * ones @ opb.T, 0.5 * opa.T @ ones
        _eq(da.T if ta else da, A.d.toCPU()); _eq(db.T if tb else db, Bm.d.toCPU())


def broadcast_add(b):                     # B:51-130
    t1 = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    for t2, expect, gb in ((np.array([[6, 5, 4], [3, 2, 1]], np.float32), [7] * 6, [1] * 6),
                           (np.array([[1], [2]], np.float32), [2, 3, 4, 6, 7, 8], [3, 3]),
                           (np.array([[3, 4, 5]], np.float32), [4, 6, 8, 7, 9, 11], [2, 2, 2])):
        a, c = TensorR(b.fromNumpy(t1)), TensorR(b.fromNumpy(t2))
        out, xs, ys = b.plus(a.x, c.x)
        _eq(expect, out.toCPU())
        out2, _, _ = b.plus(c.x, a.x)
        _eq(expect, out2.toCPU())
        b.add_grad(a, c, TensorR(out, b.fill(out.shape, 1.0)), xs, ys)
        _eq([1] * 6, a.d.toCPU()); _eq(gb, c.d.toCPU())


def relu_tanh_sigmoid(b):                 # C:696-749 (values from the definitions; tolerance 1e-4)
    v = np.array([-1, 2, -3, 4, 0, 0.5], np.float32).reshape(2, 3)
    x = TensorR(b.fromNumpy(v))
    r = b.relu(x.x); _eq(np.maximum(v, 0), r.toCPU())
    b.relu_grad(x, TensorR(r, b.fill(r.shape, 1.0))); _eq((v >= 0).astype(np.float32), x.d.toCPU())
    x = TensorR(b.fromNumpy(v)); t = b.tanh(x.x); _eq(np.tanh(v), t.toCPU())
    b.tanh_grad(x, TensorR(t, b.fill(t.shape, 1.0))); _eq(1 - np.tanh(v) ** 2, x.d.toCPU())
    x = TensorR(b.fromNumpy(v)); s = b.sigmoid(x.x); sg = 1 / (1 + np.exp(-v)); _eq(sg, s.toCPU())
    b.sigmoid_grad(x, TensorR(s, b.fill(s.shape, 1.0))); _eq(sg * (1 - sg), x.d.toCPU())


def sum_concat(b):                        # T:1273-1305, C:963-1030
    v = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    x = b.fromNumpy(v)
    _eq([v.sum()], b.sum(x).toCPU())
    for d in range(3):
        _eq(v.sum(axis=d), b.sum(x, d).toCPU())
    a, c = np.arange(16, dtype=np.float32).reshape(1, 2, 2, 4), -np.arange(24, dtype=np.float32).reshape(1, 3, 2, 4)
    A, Cc = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(c))
    out = b.concat(1, [A.x, Cc.x])
    _eq(np.concatenate([a, c], axis=1), out.toCPU())
    b.concat_grad(1, [A, Cc], TensorR(out, b.fromNumpy(np.arange(40, dtype=np.float32).reshape(1, 5, 2, 4))))
    _eq(np.arange(16), A.d.toCPU()); _eq(np.arange(16, 40), Cc.d.toCPU())


def dropout_identity(b):                  # T:1042-1094, C:879-915 (p = 0 is the identity)
    v = np.arange(12, dtype=np.float32).reshape(3, 4)
    x = TensorR(b.fromNumpy(v))
    y, mask, _ = b.dropout(x.x, 0.0)
    _eq(v, y.toCPU())
    b.dropout_grad(x, TensorR(y, b.fill(y.shape, 1.0)), 0.0, mask)
    _eq(np.ones_like(v), x.d.toCPU())


def exp_log_sqrt_square(b):               # T:1307-1379, U:249-323
    v = np.array([0.5, 1.0, 2.0, 4.0], np.float32)
    for fwd, gradf, ref, dref in ((b.exp, b.exp_grad, np.exp(v), np.exp(v)), (b.log, b.log_grad, np.log(v), 1 / v),
                                  (b.sqrt, b.sqrt_grad, np.sqrt(v), 0.5 / np.sqrt(v)), (b.square, b.square_grad, v * v, 2 * v)):
        x = TensorR(b.fromNumpy(v)); y = fwd(x.x); _eq(ref, y.toCPU())
        gradf(x, TensorR(y, b.fill(y.shape, 1.0))); _eq(dref, x.d.toCPU())


CASES = [conv_forward, conv_forward_bias_one, conv_pad, conv_pad2, conv_backprop, conv_backprop_pad, conv_bias_grad,
         maxpool, avgpool, softmax, log_softmax, nll_loss, batchnorm_inference, batchnorm_training,
         gemm_all_transposes, gemm_grad_all_transposes, broadcast_add, relu_tanh_sigmoid, sum_concat,
         dropout_identity, exp_log_sqrt_square]
