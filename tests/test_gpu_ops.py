"""Op-by-op parity of the CUDA library against the CPU oracle on seeded inputs, through the C ABI.
FP32 paths: 1e-4 relative; TF32 tensor-core paths: 2e-3 relative; indices bit-exact."""
import numpy as np
import pytest

from lantern_b200.backend import TensorR
from tests.golden.reference_known_answers import CASES
from tests.parity import FP32_RTOL, TF32_RTOL, assert_close, check

pytestmark = pytest.mark.gpu
R = lambda seed: np.random.default_rng(seed)


@pytest.mark.parametrize("case", CASES, ids=[c.__name__ for c in CASES])
def test_reference_known_answers_on_gpu(gpu, case):
    case(gpu)


@pytest.mark.parametrize("n", [1, 3, 4, 7, 1023, 4096, 100003])
@pytest.mark.parametrize("op", range(7))
def test_unary_and_grad(ora, gpu, n, op):
    v = R(n + op).random(n, dtype=np.float32) * 3 - (1.5 if op < 3 else -0.05)
    dy = R(1).standard_normal(n).astype(np.float32)

    def f(b):
        x = TensorR(b.fromNumpy(v))
        y = b._unary(op, x.x)
        b._unary_grad(op, x, TensorR(y, b.fromNumpy(dy)))
        return {"y": y.toCPU(), "dx": x.d.toCPU()}
    check(f, ora, gpu)


def test_relu_in_place_and_unaligned_views(ora, gpu):
    v = R(5).standard_normal(1001).astype(np.float32)

    def f(b):
        t = b.fromNumpy(v)
        view = t.offset(1, (1000,))                      # 4-byte aligned only: scalar path
        b.relu(view, True)
        x = TensorR(view, b.fromNumpy(np.ones(1000, np.float32)))
        b.relu_grad(x, x, True)
        return {"y": t.toCPU(), "d": x.d.toCPU()}
    check(f, ora, gpu)


SHAPES = [((2, 3), (2, 3)), ((2, 3), (2, 1)), ((2, 3), (1, 3)), ((2, 3), (3,)), ((4, 5, 6, 7), (5, 1, 1)), ((4, 5, 6, 7), (4, 5, 6, 7)),
          ((1, 5, 1, 7), (4, 1, 6, 1)), ((128, 10), (10,)), ((3, 1), (1, 4)), ((37, 64, 4, 4), (37, 64, 4, 4))]


@pytest.mark.parametrize("sa,sb", SHAPES)
@pytest.mark.parametrize("op", range(4))
def test_broadcast_binary_and_grad(ora, gpu, sa, sb, op):
    a = R(1).random(sa, dtype=np.float32) + 0.5
    c = R(2).random(sb, dtype=np.float32) + 0.5

    def f(b):
        A, C = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(c))
        out, xs, ys = b._binary(op, A.x, C.x)
        dout = b.fromNumpy(R(3).standard_normal(out.shape).astype(np.float32))
        b._binary_grad(op, A, C, TensorR(out, dout))
        return {"out": out.toCPU(), "da": A.d.toCPU(), "db": C.d.toCPU()}
    check(f, ora, gpu, rtol=2e-4 if op == 3 else FP32_RTOL)


@pytest.mark.parametrize("xs,ys", [((4, 6), (4, 6)), ((4, 6), (6,)), ((6,), (4, 6)), ((1, 5, 1, 1), (3, 5, 2, 2)), ((3, 5, 2, 2), (1, 5, 1, 1)),
                                   ((10,), (128, 10)), ((4, 1), (4, 9))])
@pytest.mark.parametrize("op", range(4))
def test_inplace_broadcast_or_reduce(ora, gpu, xs, ys, op):
    x0 = R(1).random(xs, dtype=np.float32) + 0.5
    y0 = R(2).random(ys, dtype=np.float32) * 0.2 + 0.9

    def f(b):
        x = b.fromNumpy(x0)
        b._inplace(op, x, b.fromNumpy(y0))
        b._inplace(op, x, 1.25)
        return {"x": x.toCPU(), "s": b._binary(op, x, 0.75).toCPU()}
    check(f, ora, gpu, rtol=5e-4 if op >= 2 else FP32_RTOL)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(2, 4, 3), (100, 50, 320), (128, 10, 2048), (65, 129, 33), (256, 100, 100), (1, 80, 100)])
def test_gemm_and_grad_fp32(ora, gpu, ta, tb, M, N, K):
    a = R(1).standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    c = R(2).standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    dc = R(3).standard_normal((M, N)).astype(np.float32)

    def f(b):
        b.lib.set_math(0)
        A, C = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(c))
        out = b.gemm(A.x, ta, C.x, tb, 0.5)
        b.gemm_grad(A, ta, C, tb, 0.5, TensorR(out, b.fromNumpy(dc)))
        b.lib.set_math(1)
        return {"out": out.toCPU(), "da": A.d.toCPU(), "db": C.d.toCPU()}
    check(f, ora, gpu)


@pytest.mark.parametrize("m,k,n", [(100, 320, 50), (20, 50, 26), (7, 5, 3)])
def test_dot_family(ora, gpu, m, k, n):
    a, bm, v = (R(i).standard_normal(s).astype(np.float32) for i, s in enumerate(((m, k), (k, n), (k,))))

    def f(b):
        b.lib.set_math(0)
        A, Bm, V = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(bm)), TensorR(b.fromNumpy(v))
        mm = b.dot(A.x, Bm.x); b.dot_grad(A, Bm, TensorR(mm, b.fromNumpy(R(9).standard_normal((m, n)).astype(np.float32))))
        mv = b.dot(A.x, V.x); b.dot_grad(A, V, TensorR(mv, b.fromNumpy(R(8).standard_normal(m).astype(np.float32))))
        V2 = TensorR(b.fromNumpy(v * 2))
        vv = b.dot(V.x, V2.x); b.dot_grad(V, V2, TensorR(vv, b.fromNumpy(np.array([0.7], np.float32))))
        b.lib.set_math(1)
        return {"mm": mm.toCPU(), "mv": mv.toCPU(), "vv": vv.toCPU(), "dA": A.d.toCPU(), "dB": Bm.d.toCPU(), "dV": V.d.toCPU(), "dV2": V2.d.toCPU()}
    check(f, ora, gpu)


CONVS = [  # N, C, H, W, K, R, stride, pad, bias
    (2, 1, 28, 28, 10, 5, 1, 0, True), (2, 10, 12, 12, 20, 5, 1, 0, True), (3, 3, 32, 32, 64, 3, 1, 1, False),
    (2, 64, 16, 16, 64, 1, 1, 0, False), (2, 64, 16, 16, 64, 3, 1, 1, False), (2, 128, 16, 16, 128, 3, 2, 1, False),
    (2, 256, 16, 16, 512, 1, 2, 0, False), (4, 512, 4, 4, 10, 4, 1, 0, True), (2, 16, 9, 7, 24, 3, 2, 1, True),
    (1, 5, 6, 6, 7, 2, 3, 1, True)]


@pytest.mark.parametrize("cfg", CONVS, ids=[str(c) for c in CONVS])
def test_conv_fwd_bwd_fp32(ora, gpu, cfg):
    N, C, H, W, K, Rk, s, p, has_bias = cfg
    x0 = R(1).standard_normal((N, C, H, W)).astype(np.float32)
    w0 = (R(2).standard_normal((K, C, Rk, Rk)) / np.sqrt(C * Rk * Rk)).astype(np.float32)
    b0 = R(3).standard_normal(K).astype(np.float32)

    def f(b):
        b.lib.set_math(0)
        x, w = TensorR(b.fromNumpy(x0)), TensorR(b.fromNumpy(w0))
        bias = TensorR(b.fromNumpy(b0)) if has_bias else None
        y, _, _ = b.conv2D_batch(x.x, w.x, bias.x if bias else None, (s, s), (p, p, p, p))
        dy = b.fromNumpy(R(4).standard_normal(y.shape).astype(np.float32))
        b.conv2D_batch_grad(x, None, w, TensorR(y, dy), bias, (p, p), (s, s))
        b.lib.set_math(1)
        out = {"y": y.toCPU(), "dx": x.d.toCPU(), "dw": w.d.toCPU()}
        if bias:
            out["db"] = bias.d.toCPU()
        return out
    check(f, ora, gpu)


@pytest.mark.parametrize("cfg", [(2, 3, 8, 8, 2, 2, 0), (2, 3, 9, 7, 3, 2, 1), (4, 16, 32, 32, 2, 2, 0), (1, 1, 3, 3, 2, 1, 0), (3, 5, 6, 10, 2, 2, 0)])
def test_maxpool_indices_bit_exact(ora, gpu, cfg):
    N, C, H, W, k, s, pad = cfg
    v = np.round(R(1).standard_normal((N, C, H, W)) * 2).astype(np.float32) / 2      # many ties

    def f(b):
        x = TensorR(b.fromNumpy(v))
        y, idx = b.maxPool2D_batch(x.x, (k, k), (s, s), None if pad == 0 else (pad,) * 4)
        b.maxPool2D_batch_grad(x, TensorR(y, b.fromNumpy(R(2).standard_normal(y.shape).astype(np.float32))), idx)
        return {"y": y.toCPU(), "idx": idx.toCPU(), "dx": x.d.toCPU()}
    check(f, ora, gpu, exact=("idx", "y"))


@pytest.mark.parametrize("cfg", [(2, 3, 4, 4, 2, 2), (2, 3, 4, 4, 2, 1), (8, 2048, 2, 2, 2, 1), (1, 2, 7, 5, 3, 2)])
def test_avgpool(ora, gpu, cfg):
    N, C, H, W, k, s = cfg
    v = R(1).standard_normal((N, C, H, W)).astype(np.float32)

    def f(b):
        x = TensorR(b.fromNumpy(v))
        y = b.averagePool2D_batch(x.x, (k, k), (s, s))
        b.averagePool2D_batch_grad(x, TensorR(y, b.fromNumpy(R(2).standard_normal(y.shape).astype(np.float32))), (k, k), (s, s))
        return {"y": y.toCPU(), "dx": x.d.toCPU()}
    check(f, ora, gpu)


@pytest.mark.parametrize("cfg", [(3, 2, 3, 3), (16, 64, 16, 16), (8, 256, 4, 4), (32, 512, 2, 2), (5, 7, 3, 5), (128, 10, 1, 1),
                                 (128, 64, 32, 32), (64, 128, 8, 8), (128, 3, 16, 16), (7, 300, 2, 6),
                                 # several channels per CTA (no cluster): row widths 64 / 128 / 512, an idle last row, 12-byte rows
                                 (128, 2048, 2, 2), (128, 1024, 4, 4), (128, 512, 8, 8), (5, 301, 2, 2), (96, 330, 4, 4)])
def test_batchnorm_train_fwd_bwd(ora, gpu, cfg):
    N, C, H, W = cfg
    v = (R(1).standard_normal((N, C, H, W)) * 2 + 3).astype(np.float32)      # non-zero mean: exercises the shifted sums
    g0, b0 = (R(2).random(C, dtype=np.float32) + 0.5), R(3).standard_normal(C).astype(np.float32)

    def f(b):
        x = TensorR(b.fromNumpy(v))
        scale, bias = TensorR(b.fromNumpy(g0)), TensorR(b.fromNumpy(b0))
        rm, rv = b.fill((C,), 0.0), b.fill((C,), 1.0)
        y, sm, si, _ = b.batchNormTraining(x.x, scale.x, bias.x, rm, rv)
        b.batchNorm_grad(x, TensorR(y, b.fromNumpy(R(4).standard_normal(v.shape).astype(np.float32))), scale, bias, sm, si)
        yi = b.batchNormInference(x.x, scale.x, bias.x, rm, rv)
        return {"y": y.toCPU(), "mean": sm.toCPU(), "istd": si.toCPU(), "rm": rm.toCPU(), "rv": rv.toCPU(), "dx": x.d.toCPU(),
                "dgamma": scale.d.toCPU(), "dbeta": bias.d.toCPU(), "yi": yi.toCPU()}
    check(f, ora, gpu, rtol=2e-4)


@pytest.mark.parametrize("rows,cols", [(2, 3), (128, 10), (100, 10), (20, 80), (1, 5), (7, 1000)])
def test_softmax_family_and_nll(ora, gpu, rows, cols):
    v = (R(1).standard_normal((rows, cols)) * 3).astype(np.float32)
    t = R(2).integers(0, cols, rows).astype(np.int32)

    def f(b):
        x, x2 = TensorR(b.fromNumpy(v)), TensorR(b.fromNumpy(v))
        tgt = b.fromNumpy(t)
        ls = TensorR(b.logSoftmax(x.x))
        loss = b.nllLoss(ls.x, tgt)
        total, avg = b.sum(loss), b.mean(loss)
        L = TensorR(loss)
        b.sum_grad(L, TensorR(total, b.fill((1,), 1.0))); b.mean_grad(L, TensorR(avg, b.fill((1,), 2.0)))
        b.nllLoss_grad(ls, L, tgt); b.logSoftmax_grad(x, ls)
        sm = b.softmax(x2.x)
        b.softmax_grad(x2, TensorR(sm, b.fromNumpy(R(3).standard_normal(v.shape).astype(np.float32))))
        return {"ls": ls.x.toCPU(), "loss": loss.toCPU(), "sum": total.toCPU(), "mean": avg.toCPU(), "dx": x.d.toCPU(),
                "sm": sm.toCPU(), "dx2": x2.d.toCPU()}
    check(f, ora, gpu, rtol=2e-4)


def test_reductions_concat_trans_geam(ora, gpu):
    v = R(1).standard_normal((6, 5, 8)).astype(np.float32)
    big = R(2).standard_normal(300001).astype(np.float32)

    def f(b):
        x = TensorR(b.fromNumpy(v))
        out = {"sum_big": b.sum(b.fromNumpy(big)).toCPU()}
        for d in range(3):
            s = b.sum(x.x, d); out["sum%d" % d] = s.toCPU()
            b.sum_grad(x, TensorR(s, b.fromNumpy(R(3 + d).standard_normal(s.shape).astype(np.float32))), d)
        out["dx"] = x.d.toCPU()
        a4, c4 = R(7).standard_normal((3, 4, 5, 5)).astype(np.float32), R(8).standard_normal((3, 6, 5, 5)).astype(np.float32)
        A, C = TensorR(b.fromNumpy(a4)), TensorR(b.fromNumpy(c4))
        cat = b.concat(1, [A.x, C.x]); out["cat"] = cat.toCPU()
        b.concat_grad(1, [A, C], TensorR(cat, b.fromNumpy(R(9).standard_normal(cat.shape).astype(np.float32))))
        out["dA"], out["dC"] = A.d.toCPU(), C.d.toCPU()
        m = TensorR(b.fromNumpy(R(10).standard_normal((37, 53)).astype(np.float32)))
        t = b.trans(m.x); out["t"] = t.toCPU()
        b.trans_grad(m, TensorR(t, b.fromNumpy(R(11).standard_normal((53, 37)).astype(np.float32)))); out["dm"] = m.d.toCPU()
        o = b.empty(37, 53); b.geam(m.x, False, 0.3, m.d, False, -1.7, o); out["geam"] = o.toCPU()
        o2 = b.empty(53, 37); b.geam(t, False, 2.0, m.x, True, 0.5, o2); out["geam_t"] = o2.toCPU()
        fb = b.fillWithBias((2, 5, 3), b.fromNumpy(np.arange(5, dtype=np.float32)), 1); out["fb"] = fb.toCPU()
        c = b.fromNumpy(R(12).standard_normal(1000).astype(np.float32) * 3); b.clipAt(c, 1.5); out["clip"] = c.toCPU()
        return out
    check(f, ora, gpu, rtol=3e-4)


def test_dropout_and_randinit_follow_the_host_rand_stream(ora, gpu):
    v = R(1).standard_normal(5000).astype(np.float32)

    def f(b):
        w = b.randinit((7, 11), 0.3, seed=42)
        x = TensorR(b.fromNumpy(v))
        y, mask, _ = b.dropout(x.x, 0.5)
        b.dropout_grad(x, TensorR(y, b.fill(y.shape, 2.0)), 0.5, mask)
        return {"w": w.toCPU(), "y": y.toCPU(), "mask": mask.toCPU(), "dx": x.d.toCPU()}
    check(f, ora, gpu, exact=("w", "mask", "y"))


def test_optimizers(ora, gpu):
    n = 10007
    x0, d0 = R(1).standard_normal(n).astype(np.float32), (R(2).standard_normal(n) * 3).astype(np.float32)

    def f(b):
        out = {}
        p = TensorR(b.fromNumpy(x0), b.fromNumpy(d0)); b.sgd_step(p, 0.1); out["sgd_x"], out["sgd_d"] = p.x.toCPU(), p.d.toCPU()
        p = TensorR(b.fromNumpy(x0), b.fromNumpy(d0)); h = b.zeros(n)
        b.adagrad_update(p, h, 0.1, 1.0); p.d = b.fromNumpy(d0 * 0.5); b.adagrad_update(p, h, 0.1, 1.0)
        out["ada_x"], out["ada_h"], out["ada_d"] = p.x.toCPU(), h.toCPU(), p.d.toCPU()
        for nest in (0, 1):
            p = TensorR(b.fromNumpy(x0), b.fromNumpy(d0)); m = b.zeros(n)
            b.momentum_update(p, m, 0.05, 0.9, 5.0, nest); p.d = b.fromNumpy(d0); b.momentum_update(p, m, 0.05, 0.9, 5.0, nest)
            out["mom%d_x" % nest], out["mom%d_m" % nest] = p.x.toCPU(), m.toCPU()
        return out
    check(f, ora, gpu)


def test_arena_semantics_and_error_codes(gpu):
    import lantern_b200
    lib = gpu.lib
    used = lib.arena_used()
    p = lib.malloc(1000)
    assert p % 256 == 0 and lib.arena_used() == used + 1024
    z = np.empty(250, np.float32); lib.d2h(z.ctypes.data, p, 1000)
    assert not z.any()                                   # zero on hand-out
    lib.fill(p, 3.0, 250)
    q = lib.malloc_uninit(8)
    with pytest.raises(lantern_b200.LanternError):
        lib.free(p, 1000)                                # not the newest block
    lib.free(q, 8); lib.free(p, 1000)
    p2 = lib.malloc(1000)
    assert p2 == p
    lib.d2h(z.ctypes.data, p2, 1000)
    assert not z.any()                                   # zero again after reuse
    with pytest.raises(lantern_b200.LanternError) as e:
        lib.malloc(1 << 50)
    assert e.value.code == -3
    with pytest.raises(lantern_b200.LanternError) as e:
        lib.gemm(0, 0, 0, 0, 1.0, 0, 4, 4, 4)
    assert e.value.code == -2
    assert lib.kernel_launches() > 0


# ------------------------------------------------------------------------------------------------ TF32 tensor-core engine
def _tf32_check(f, ora, gpu):
    """Two gates: within 2e-3 of the plain FP32 oracle (the TF32 tolerance), and within 1e-4 of the oracle emulating the
    operand truncation of the tensor-core path, which shows the engine computes exactly the TF32 product it claims."""
    from tests.parity import assert_close
    got = f(gpu, 1)
    ref32 = f(ora, 0)
    ref_tf = f(ora, 1)
    for k in got:
        assert_close(ref32[k], got[k], TF32_RTOL, k + " vs FP32 oracle")
        assert_close(ref_tf[k], got[k], FP32_RTOL, k + " vs TF32-emulating oracle")

@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 64, 32), (256, 128, 64), (384, 320, 96), (128, 2048, 256), (256, 100, 100), (8, 10, 2048)])
def test_gemm_and_grad_tf32(ora, gpu, ta, tb, M, N, K):
    """Eligible shapes run on tcgen05 (2e-3), the others fall back to the FP32 path; both must hold the TF32 tolerance."""
    a = R(1).standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    c = R(2).standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    dc = R(3).standard_normal((M, N)).astype(np.float32)

    def f(b, math=1):
        b.lib.set_math(math)
        A, C = TensorR(b.fromNumpy(a)), TensorR(b.fromNumpy(c))
        out = b.gemm(A.x, ta, C.x, tb, 0.5)
        b.gemm_grad(A, ta, C, tb, 0.5, TensorR(out, b.fromNumpy(dc)))
        return {"out": out.toCPU(), "da": A.d.toCPU(), "db": C.d.toCPU()}
    _tf32_check(f, ora, gpu)


TC_CONVS = [  # N, C, H, W, K, R, stride, pad: the ResNet-50 / SqueezeNet layer shapes at small batch (partial tiles included)
    (2, 64, 16, 16, 64, 1, 1, 0), (2, 64, 16, 16, 256, 1, 1, 0), (3, 256, 16, 16, 64, 1, 1, 0), (4, 128, 8, 8, 512, 1, 1, 0),
    (5, 512, 8, 8, 128, 1, 1, 0), (9, 256, 4, 4, 1024, 1, 1, 0), (9, 1024, 4, 4, 256, 1, 1, 0), (33, 512, 2, 2, 2048, 1, 1, 0),
    (33, 2048, 2, 2, 512, 1, 1, 0), (2, 64, 16, 16, 64, 3, 1, 1), (2, 128, 16, 16, 128, 3, 2, 1), (3, 128, 8, 8, 128, 3, 1, 1),
    (9, 256, 8, 8, 256, 3, 2, 1), (9, 256, 4, 4, 256, 3, 1, 1), (17, 512, 4, 4, 512, 3, 2, 1), (17, 512, 2, 2, 512, 3, 1, 1),
    (2, 256, 16, 16, 512, 1, 2, 0), (5, 512, 8, 8, 1024, 1, 2, 0), (9, 1024, 4, 4, 2048, 1, 2, 0), (4, 16, 32, 32, 64, 1, 1, 0),
    (4, 96, 16, 16, 16, 1, 1, 0), (8, 512, 4, 4, 10, 4, 1, 0), (3, 96, 32, 32, 16, 1, 1, 0), (3, 16, 16, 16, 64, 3, 1, 1),
    # SqueezeNet fire modules: channel counts that are not multiples of 32 (K tails filled with zeros by the TMA unit)
    (8, 48, 8, 8, 192, 1, 1, 0), (8, 48, 8, 8, 192, 3, 1, 1), (8, 256, 8, 8, 48, 1, 1, 0), (8, 384, 8, 8, 48, 1, 1, 0),
    (8, 128, 16, 16, 32, 1, 1, 0), (8, 32, 16, 16, 128, 3, 1, 1), (8, 64, 4, 4, 256, 3, 1, 1), (8, 512, 4, 4, 64, 1, 1, 0),
    # more stride-1 windows for the tap-loop plans: 32x32 images, 5x5 taps, image counts that leave partial tiles
    (4, 64, 32, 32, 64, 3, 1, 1), (6, 64, 8, 8, 64, 5, 1, 2), (5, 128, 16, 16, 64, 3, 1, 1), (21, 64, 2, 2, 128, 3, 1, 1),
    # large enough (unfolded matrix >= 64 MB) for the tap-loop weight-grad
    (112, 64, 16, 16, 64, 3, 1, 1), (30, 64, 32, 32, 64, 3, 1, 1),
    # small images whose count fills whole 128-byte rows: fed M/N-major straight from NCHW (no transposing copy)
    (8, 256, 4, 4, 1024, 1, 1, 0), (16, 512, 2, 2, 2048, 1, 1, 0), (8, 1024, 4, 4, 256, 1, 1, 0), (40, 64, 2, 2, 64, 1, 1, 0),
    (8, 256, 8, 8, 256, 3, 2, 1), (16, 512, 4, 4, 512, 3, 2, 1), (8, 512, 8, 8, 1024, 1, 2, 0),
    # filter rows that the engine needs padded (3x3 over 3 / 16 / 48 channels, 1x1 over 16 / 48), the stems of ResNet-50 and
    # SqueezeNet, and a filter that covers the whole image (SqueezeNet's classifier: a matrix product)
    (4, 3, 32, 32, 64, 3, 1, 1), (3, 3, 32, 32, 96, 3, 1, 1), (4, 16, 16, 16, 64, 1, 1, 0), (5, 48, 8, 8, 192, 3, 1, 1),
    (64, 512, 4, 4, 10, 4, 1, 0), (6, 16, 16, 16, 64, 3, 1, 1), (7, 20, 8, 8, 40, 1, 1, 0)]


@pytest.mark.parametrize("cfg", TC_CONVS, ids=[str(c) for c in TC_CONVS])
def test_conv_fwd_bwd_tf32(ora, gpu, cfg):
    N, C, H, W, K, Rk, s, p = cfg
    x0 = R(1).standard_normal((N, C, H, W)).astype(np.float32)
    w0 = (R(2).standard_normal((K, C, Rk, Rk)) / np.sqrt(C * Rk * Rk)).astype(np.float32)
    b0 = R(3).standard_normal(K).astype(np.float32)

    def f(b, math=1):
        b.lib.set_math(math)
        x, w, bias = TensorR(b.fromNumpy(x0)), TensorR(b.fromNumpy(w0)), TensorR(b.fromNumpy(b0))
        y, _, _ = b.conv2D_batch(x.x, w.x, bias.x, (s, s), (p, p, p, p))
        dy = b.fromNumpy(R(4).standard_normal(y.shape).astype(np.float32))
        # gradients accumulate: start from non-zero destinations
        x.d, w.d = b.fromNumpy(x0 * 0.25), b.fromNumpy(w0 * 0.5)
        b.conv2D_batch_grad(x, None, w, TensorR(y, dy), bias, (p, p), (s, s))
        return {"y": y.toCPU(), "dx": x.d.toCPU(), "dw": w.d.toCPU(), "db": bias.d.toCPU()}
    _tf32_check(f, ora, gpu)


def test_tensor_core_engine_reports_no_timeouts(gpu):
    assert gpu.lib.device_status() == 0


def test_a_device_wait_that_runs_out_is_reported_and_the_context_stays_usable(ora, gpu):
    """Failure detection on the device without a fault: one warp waits, through the engine's own bounded wait, on a barrier
    at which nothing ever arrives (no copy in flight, no tensor memory held).  After the limit the kernel records a code and
    returns; the host reads LTB_E_DEVICE, clears it, and the next tensor-core launch works as before."""
    lib = gpu.lib
    assert lib.device_status() == 0
    lib.selftest_bounded_wait(200000)                    # about 0.1 ms of SM clock
    lib.sync()
    assert lib.device_status() == -6                     # LTB_E_DEVICE
    assert lib.device_status() == -6                     # sticky until cleared
    lib.clear_device_status()
    assert lib.device_status() == 0
    lib.set_wait_limit(3000000000)                       # the engine's own limit is a run-time value
    try:
        a = R(1).standard_normal((256, 64)).astype(np.float32); c = R(2).standard_normal((64, 128)).astype(np.float32)

        def f(b, math=1):
            b.lib.set_math(math)
            return {"out": b.gemm(b.fromNumpy(a), 0, b.fromNumpy(c), 0, 1.0).toCPU()}
        _tf32_check(f, ora, gpu)
    finally:
        lib.set_wait_limit(2000000000)
    assert lib.device_status() == 0


# ---------------------------------------------------------------------------------------------- look-ahead fusion
@pytest.mark.parametrize("cfg", [(16, 64, 16, 16), (8, 256, 4, 4), (128, 64, 32, 32), (5, 7, 3, 5), (33, 512, 2, 2)])
def test_lookahead_fusion_gives_the_results_of_separate_calls(ora, gpu, cfg):
    """conv-net block fragment: y = relu_(bn(x)); z = relu_(y + s); backward through both. With ltb_set_fusion(1) the
    BN+ReLU, add+ReLU, ReLU-grad+add-grad and ReLU-grad+BN-backward pairs run as single kernels; every tensor, including
    the in-place masked gradients, must be bit-identical to the unfused run and within tolerance of the oracle."""
    N, C, H, W = cfg
    v = (R(1).standard_normal((N, C, H, W)) * 2 + 0.5).astype(np.float32)
    sk = R(5).standard_normal((N, C, H, W)).astype(np.float32)
    g0, b0 = (R(2).random(C, dtype=np.float32) + 0.5), R(3).standard_normal(C).astype(np.float32)
    dz0 = R(4).standard_normal((N, C, H, W)).astype(np.float32)

    def f(b, fusion=0):
        b.lib.set_fusion(fusion)
        try:
            x, s = TensorR(b.fromNumpy(v)), TensorR(b.fromNumpy(sk))
            scale, bias = TensorR(b.fromNumpy(g0)), TensorR(b.fromNumpy(b0))
            rm, rv = b.fill((C,), 0.0), b.fill((C,), 1.0)
            y, sm, si, _ = b.batchNormTraining(x.x, scale.x, bias.x, rm, rv)
            yr = TensorR(b.relu(y, True))                                  # in place: joins the BN kernel
            z = TensorR(b.relu(b.plus(yr.x, s.x)[0], True))                # in place: joins the add kernel
            z.d = b.fromNumpy(dz0)
            b.relu_grad(z, z, True)                                        # held ...
            b.add_grad(yr, s, z)                                           # ... and absorbed by the add's gradient
            b.relu_grad(yr, yr, True)                                      # held ...
            b.batchNorm_grad(x, yr, scale, bias, sm, si)                   # ... and absorbed by BN backward
            out = {"y": yr.x.toCPU(), "z": z.x.toCPU(), "dz": z.d.toCPU(), "dy": yr.d.toCPU(), "ds": s.d.toCPU(), "dx": x.d.toCPU(),
                   "dgamma": scale.d.toCPU(), "dbeta": bias.d.toCPU(), "rm": rm.toCPU(), "rv": rv.toCPU()}
        finally:
            b.lib.set_fusion(0)
        return out
    ref = f(ora)
    plain = f(gpu, 0)
    fused = f(gpu, 1)
    for k in ref:
        assert np.array_equal(plain[k], fused[k]), k + ": fused and separate kernels differ"
    for k in ("y", "z", "rm", "rv"):
        assert_close(ref[k], fused[k], 2e-4, k)
    # gradients pass through two ReLU masks: an activation within rounding of zero may fall on the other side in the two
    # implementations and switch single elements on or off, so a handful of elements out of millions may differ
    for k in ("dz", "dy", "ds", "dx"):
        bad = np.abs(ref[k] - fused[k]) > 2e-4 * np.abs(ref[k]).max()
        assert bad.mean() < 2e-5, (k, int(bad.sum()), bad.size)
    for k in ("dgamma", "dbeta"):
        assert_close(ref[k], fused[k], 2e-2, k)          # a flipped element is a visible part of a per-channel sum


def test_lookahead_fusion_flushes_on_any_other_call(ora, gpu):
    """A held operation that nothing joins is issued by the next call, whatever it is."""
    v = R(1).standard_normal((4, 32, 8, 8)).astype(np.float32)
    g0, b0 = np.ones(32, np.float32), np.zeros(32, np.float32)

    def f(b, fusion=0):
        b.lib.set_fusion(fusion)
        try:
            x = TensorR(b.fromNumpy(v))
            rm, rv = b.fill((32,), 0.0), b.fill((32,), 1.0)
            y, sm, si, _ = b.batchNormTraining(x.x, b.fromNumpy(g0), b.fromNumpy(b0), rm, rv)
            y_now = y.toCPU()                                              # a copy, not a ReLU: BN must have run by now
            t = b.tanh(y)                                                  # not a ReLU either
            a = b.plus(y, t)[0]                                            # held add ...
            a_sum = b.sum(a)                                               # ... flushed by a reduction that reads it
            yd = TensorR(y, b.fromNumpy(v * 0.5))
            b.relu_grad(yd, yd, True)                                      # held ReLU gradient ...
            d_now = yd.d.toCPU()                                           # ... flushed by the read-back
            out = {"y": y_now, "t": t.toCPU(), "a": a.toCPU(), "sum": a_sum.toCPU(), "d": d_now}
        finally:
            b.lib.set_fusion(0)
        return out
    ref, got = f(ora), f(gpu, 1)
    for k in ref:
        assert_close(ref[k], got[k], 2e-4, k)


@pytest.mark.parametrize("n", [0, 1, 3, 5, 1027, 65537])
def test_empty_ragged_and_misaligned_vectors(ora, gpu, n):
    """Element counts that are zero, smaller than a float4 or not a multiple of four, on buffers that start one float past
    a 16-byte boundary (the vectorised kernels must fall back to their scalar forms), through the streaming operators."""
    v = (R(1).standard_normal(n + 1) * 2).astype(np.float32)
    d0 = R(2).standard_normal(n + 1).astype(np.float32)

    def f(b):
        full, dfull = b.fromNumpy(v), b.fromNumpy(d0)
        x, d = full.offset(1, (n,)), dfull.offset(1, (n,))               # misaligned views of n elements
        out = {}
        if n:
            out["relu"] = b.relu(x).toCPU(); out["tanh"] = b.tanh(x).toCPU()
            out["scaled"] = b.mul(x, 0.5).toCPU()
            out["sum"] = b.sum(x).toCPU()
        t = TensorR(x, d)
        b.lib.unary_grad(0, x.ptr, d.ptr, x.ptr, d.ptr, n, 1)               # in-place ReLU gradient
        b.lib.sgd_step(x.ptr, d.ptr, 0.1, n)
        b.lib.clip(x.ptr, 1.5, n)
        b.lib.fill(d.ptr, 2.0, n)
        out["x"], out["d"], out["guard_x"], out["guard_d"] = full.toCPU()[1:], dfull.toCPU()[1:], full.toCPU()[:1], dfull.toCPU()[:1]
        return out
    check(f, ora, gpu)


def test_sgd_step_over_a_list_of_tensors(ora, gpu):
    """ltb_sgd_step_multi: one launch over a list of parameter tensors of ragged sizes (an empty one and misaligned ones
    among them) gives what ltb_sgd_step gives tensor by tensor: x -= lr * d, d = 0."""
    import ctypes
    sizes = [1, 7, 0, 64, 1023, 4096, 100003, 5]
    xs0 = [R(10 + i).standard_normal(n + 1).astype(np.float32) for i, n in enumerate(sizes)]
    ds0 = [R(50 + i).standard_normal(n + 1).astype(np.float32) for i, n in enumerate(sizes)]

    def f(b):
        xf = [b.fromNumpy(a) for a in xs0]; df = [b.fromNumpy(a) for a in ds0]
        off = [i % 2 for i in range(len(sizes))]                               # every other tensor starts one float past a 16-byte boundary
        xp = (ctypes.c_void_p * len(sizes))(*[t.ptr + 4 * o for t, o in zip(xf, off)])
        dp = (ctypes.c_void_p * len(sizes))(*[t.ptr + 4 * o for t, o in zip(df, off)])
        sz = (ctypes.c_int64 * len(sizes))(*sizes)
        b.lib.sgd_step_multi(ctypes.addressof(xp), ctypes.addressof(dp), ctypes.addressof(sz), len(sizes), 0.25)
        out = {}
        for i, (t, d) in enumerate(zip(xf, df)):
            out["x%d" % i], out["d%d" % i] = t.toCPU(), d.toCPU()
        return out
    a = f(ora)
    check(f, ora, gpu)
    for i, (n, o) in enumerate(zip(sizes, [i % 2 for i in range(len(sizes))])):   # and against the formula itself; elements outside the spans untouched
        want = xs0[i].copy(); want[o:o + n] -= np.float32(0.25) * ds0[i][o:o + n]
        assert np.allclose(a["x%d" % i], want, rtol=1e-6, atol=1e-7)
        dz = ds0[i].copy(); dz[o:o + n] = 0
        assert np.array_equal(a["d%d" % i], dz)


def test_pointwise_weight_grad_with_a_misaligned_input_view(ora, gpu):
    """A 1x1 convolution whose x is a view one float past a 16-byte boundary: the tensor-core weight-gradient plan must
    decline it (TMA needs 16-byte bases) and the FP32 path take over, not a half-built plan reach the launch."""
    N, C, H, K = 4, 64, 8, 64
    xv = R(1).standard_normal(N * C * H * H + 1).astype(np.float32)
    w0 = (R(2).standard_normal((K, C, 1, 1)) / 8).astype(np.float32)
    dy0 = R(3).standard_normal((N, K, H, H)).astype(np.float32)

    def f(b, math=1):
        b.lib.set_math(math)
        x = b.fromNumpy(xv).offset(1, (N, C, H, H))
        w = TensorR(b.fromNumpy(w0)); dy = b.fromNumpy(dy0)
        dx = b.zeros(N, C, H, H)
        b.lib.conv2d_bwd(x.ptr, dx.ptr, w.x.ptr, w.d.ptr, 0, dy.ptr, N, C, H, H, K, 1, 1, 1, 1, 0, 0)
        return {"dw": w.d.toCPU(), "dx": dx.toCPU()}
    got, ref = f(gpu, 1), f(ora, 0)
    assert_close(ref["dw"], got["dw"], FP32_RTOL, "dw (declined by the engine: FP32 path)")
    assert_close(ref["dx"], got["dx"], TF32_RTOL, "dx (dy and w are aligned: tensor-core path)")


@pytest.mark.parametrize("T,B,V,H", [(20, 256, 80, 100), (20, 1, 80, 100), (7, 37, 26, 50), (3, 300, 33, 17)])
def test_rnn_whole_sequence_kernels(ora, gpu, T, B, V, H):
    """ltb_rnn_seq_fwd / ltb_rnn_seq_bwd (every step of the unrolled vanilla RNN inside one launch, the rows of the batch dealt
    out to CTAs) against the oracle issuing the reference's operator sequence: hidden states, log-probabilities, loss, and the
    five gradients accumulated onto non-zero destinations.  Twice in a row: the launch leaves its completion counter at zero."""
    rng = R(9)
    ids = rng.integers(0, V, (T + 1, B))
    x0 = (rng.standard_normal((T, B, V)) * 0.1).astype(np.float32)
    x0[np.arange(T)[:, None], np.arange(B)[None, :], ids[:T]] += 1.0                       # near one-hot, every entry live
    y0 = ids[1:].astype(np.int32)
    W = {"xh": (rng.standard_normal((V, H)) / np.sqrt(V)).astype(np.float32), "hh": (rng.standard_normal((H, H)) / np.sqrt(H)).astype(np.float32),
         "bh": (rng.standard_normal(H) * 0.1).astype(np.float32), "ho": (rng.standard_normal((H, V)) / np.sqrt(H)).astype(np.float32),
         "bo": (rng.standard_normal(V) * 0.1).astype(np.float32)}

    def f(b):
        b.lib.set_math(0)
        x, y = b.fromNumpy(x0), b.fromNumpy(y0)
        w = {k: TensorR(b.fromNumpy(v), b.fromNumpy(v * 0.5)) for k, v in W.items()}
        out = {}
        for rep in range(2):
            h, logp, loss = b.empty(T, B, H), b.empty(T, B, V), b.empty(1)
            b.lib.rnn_seq_fwd(x.ptr, y.ptr, 0, w["xh"].x.ptr, w["hh"].x.ptr, w["bh"].x.ptr, w["ho"].x.ptr, w["bo"].x.ptr, h.ptr, logp.ptr, loss.ptr, T, B, V, H)
            dloss = b.fill((1,), 0.5)
            b.lib.rnn_seq_bwd(x.ptr, y.ptr, 0, w["hh"].x.ptr, w["ho"].x.ptr, h.ptr, logp.ptr, dloss.ptr,
                              w["xh"].d.ptr, w["hh"].d.ptr, w["bh"].d.ptr, w["ho"].d.ptr, w["bo"].d.ptr, T, B, V, H)
            out["h%d" % rep], out["logp%d" % rep], out["loss%d" % rep] = h.toCPU(), logp.toCPU(), loss.toCPU()
        for k in w:
            out["d" + k] = w[k].d.toCPU()
        return out
    check(f, ora, gpu)


@pytest.mark.parametrize("inner,classify_cell,Hd,L", [(1, 1, 150, 150), (1, 0, 150, 150), (0, 1, 150, 300), (0, 0, 150, 300), (1, 0, 40, 40)])
def test_tree_node_and_gradient(ora, gpu, inner, classify_cell, Hd, L):
    """ltb_tree_node_fwd / ltb_tree_node_bwd (a whole tree-LSTM node per launch) against the oracle issuing the gate-by-gate
    operator sequence: gates, cell, hidden, log-probabilities and loss; then every gradient accumulated onto non-zero
    destinations -- an inner node (five gates over two inputs, the two forget gates sharing one bias) and a leaf (three
    gates over the embedding, no input gradient), with the classifier on the cell and on the hidden vector.  Twice in a row:
    the forward launch leaves its completion counter at zero."""
    import ctypes
    from lantern_b200 import parse_struct
    Node = parse_struct("ltb_tree_node")
    K = 5
    rng = R(21)
    v = lambda *shape, scale=1.0: (rng.standard_normal(shape) * scale).astype(np.float32)
    slots = (0, 1, 2, 3, 4) if inner else (0, 3, 4)
    data = {"in0": v(L, scale=0.5), "in1": v(L, scale=0.5), "cl": v(Hd), "cr": v(Hd), "Why": v(K, Hd, scale=0.1), "by": v(K, scale=0.1),
            "dc": v(Hd), "dh": v(Hd), "dloss": np.array([0.75], np.float32), "loss_l": np.array([1.25], np.float32), "loss_r": np.array([2.5], np.float32)}
    for g in slots:
        data["W%d0" % g] = v(Hd, L, scale=1.0 / np.sqrt(L)); data["W%d1" % g] = v(Hd, L, scale=1.0 / np.sqrt(L))
    data["b0"], data["b12"], data["b3"], data["b4"] = v(Hd, scale=0.1), v(Hd, scale=0.1), v(Hd, scale=0.1), v(Hd, scale=0.1)
    bias_of = {0: "b0", 1: "b12", 2: "b12", 3: "b3", 4: "b4"}
    grads = ["in0", "in1", "cl", "cr", "Why", "by", "loss_l", "loss_r", "b0", "b12", "b3", "b4"] + ["W%d%d" % (g, k) for g in slots for k in (0, 1)]

    def f(b):
        t = {k: b.fromNumpy(a) for k, a in data.items()}
        d = {k: b.fromNumpy(data[k] * 0.25) for k in grads}                           # accumulate onto non-zero values
        score = b.fromNumpy(np.array([3], np.int32))
        out = {}
        for rep in range(2):
            gates, c, tc, h, logp, loss = b.fill((5, Hd), 0.0), b.fill((Hd,), 0.0), b.fill((Hd,), 0.0), b.fill((Hd,), 0.0), b.fill((K,), 0.0), b.fill((1,), 0.0)
            n = Node()
            n.hidden, n.in_len, n.classes, n.inner, n.classify_cell = Hd, L, K, inner, classify_cell
            getattr(n, "in")[0] = t["in0"].ptr
            if inner:
                getattr(n, "in")[1] = t["in1"].ptr
                n.din[0], n.din[1] = d["in0"].ptr, d["in1"].ptr
                n.cl, n.cr, n.dcl, n.dcr = t["cl"].ptr, t["cr"].ptr, d["cl"].ptr, d["cr"].ptr
                n.loss_l, n.loss_r, n.dloss_l, n.dloss_r = t["loss_l"].ptr, t["loss_r"].ptr, d["loss_l"].ptr, d["loss_r"].ptr
            for g in slots:
                for k in ((0, 1) if inner else (0,)):
                    n.W[g][k], n.dW[g][k] = t["W%d%d" % (g, k)].ptr, d["W%d%d" % (g, k)].ptr
                n.bias[g], n.dbias[g] = t[bias_of[g]].ptr, d[bias_of[g]].ptr
            n.Why, n.by, n.dWhy, n.dby, n.score = t["Why"].ptr, t["by"].ptr, d["Why"].ptr, d["by"].ptr, score.ptr
            n.gates, n.c, n.tc, n.h, n.logp, n.loss = gates.ptr, c.ptr, tc.ptr, h.ptr, logp.ptr, loss.ptr
            n.dc, n.dh, n.dloss = t["dc"].ptr, t["dh"].ptr, t["dloss"].ptr
            b.lib.tree_node_fwd(ctypes.addressof(n))
            b.lib.tree_node_bwd(ctypes.addressof(n))
            g_all = gates.toCPU()
            out["gates%d" % rep] = g_all if inner else g_all[[0, 3, 4]]
            out["c%d" % rep], out["h%d" % rep], out["logp%d" % rep], out["loss%d" % rep] = c.toCPU(), h.toCPU(), logp.toCPU(), loss.toCPU()
        used = [k for k in grads if inner or k not in ("in0", "in1", "cl", "cr", "loss_l", "loss_r", "b12") and not k.endswith("1")]
        for k in used:
            out["d" + k] = d[k].toCPU()
        return out
    check(f, ora, gpu)


@pytest.mark.parametrize("classify_cell", [0, 1])
def test_tree_levels_and_gradient(ora, gpu, classify_cell):
    """ltb_tree_nodes_fwd / ltb_tree_nodes_bwd: a small tree (four leaves, two inner nodes over them, the root) level by level --
    three calls forward, three backward, node descriptions read from an array in device memory -- against the oracle running
    the nodes one after the other: every node's cell, hidden vector and loss, the root's accumulated loss, and every weight
    gradient."""
    import ctypes
    from lantern_b200 import parse_struct
    Node = parse_struct("ltb_tree_node")
    Hd, E, K, n = 150, 300, 5, 7
    rng = R(31)
    v = lambda *shape, scale=1.0: (rng.standard_normal(shape) * scale).astype(np.float32)
    W = {"leaf%d" % g: v(Hd, E, scale=1 / np.sqrt(E)) for g in (0, 3, 4)}
    W.update({"in%d%d" % (g, k): v(Hd, Hd, scale=1 / np.sqrt(Hd)) for g in range(5) for k in (0, 1)})
    W.update({"bl%d" % g: v(Hd, scale=0.1) for g in (0, 3, 4)}); W.update({"bi%d" % g: v(Hd, scale=0.1) for g in (0, 1, 3, 4)})
    W["Why"], W["by"] = v(K, Hd, scale=0.1), v(K, scale=0.1)
    emb = v(4, E, scale=0.5)
    scores0 = rng.integers(0, K, n).astype(np.int32)
    kids = {4: (0, 1), 5: (2, 3), 6: (4, 5)}            # nodes 0..3 leaves, 4 and 5 over them, 6 the root; already sorted by height

    def f(b):
        lib = b.lib
        w = {k: TensorR(b.fromNumpy(a), b.fromNumpy(a * 0.25)) for k, a in W.items()}
        e, scores = b.fromNumpy(emb), b.fromNumpy(scores0)
        pitch = 192
        vals, grads = b.fill((n, 8 * pitch + 64), 0.0), b.fill((n, 2 * pitch + 64), 0.0)
        V = lambda i: vals.ptr + 4 * i * (8 * pitch + 64)
        G = lambda i: grads.ptr + 4 * i * (2 * pitch + 64)
        first = 5 if classify_cell else 7                # which state vector the parent's gates read (cell or hidden), in pitches
        arr = (Node * n)()
        for i in range(n):
            q = arr[i]
            q.hidden, q.classes, q.classify_cell, q.inner = Hd, K, classify_cell, int(i >= 4)
            if i < 4:
                q.in_len = E
                getattr(q, "in")[0] = e.ptr + 4 * i * E
                for g in (0, 3, 4):
                    q.W[g][0], q.dW[g][0], q.bias[g], q.dbias[g] = w["leaf%d" % g].x.ptr, w["leaf%d" % g].d.ptr, w["bl%d" % g].x.ptr, w["bl%d" % g].d.ptr
            else:
                l, r = kids[i]
                q.in_len = Hd
                getattr(q, "in")[0], getattr(q, "in")[1] = V(l) + 4 * first * pitch, V(r) + 4 * first * pitch
                q.din[0], q.din[1] = G(l) + (0 if classify_cell else 4 * pitch), G(r) + (0 if classify_cell else 4 * pitch)
                second = 7 if classify_cell else 5
                q.cl, q.cr = V(l) + 4 * second * pitch, V(r) + 4 * second * pitch
                q.dcl, q.dcr = G(l) + (4 * pitch if classify_cell else 0), G(r) + (4 * pitch if classify_cell else 0)
                q.loss_l, q.loss_r = V(l) + 4 * (8 * pitch + 32), V(r) + 4 * (8 * pitch + 32)
                q.dloss_l, q.dloss_r = G(l) + 4 * 2 * pitch, G(r) + 4 * 2 * pitch
                for g in range(5):
                    bk = "bi%d" % (1 if g == 2 else g)
                    for k in (0, 1):
                        q.W[g][k], q.dW[g][k] = w["in%d%d" % (g, k)].x.ptr, w["in%d%d" % (g, k)].d.ptr
                    q.bias[g], q.dbias[g] = w[bk].x.ptr, w[bk].d.ptr
            q.Why, q.by, q.dWhy, q.dby, q.score = w["Why"].x.ptr, w["by"].x.ptr, w["Why"].d.ptr, w["by"].d.ptr, scores.ptr + 4 * i
            q.gates, q.c, q.tc, q.h = V(i), V(i) + 4 * 5 * pitch, V(i) + 4 * 6 * pitch, V(i) + 4 * 7 * pitch
            q.logp, q.loss = V(i) + 4 * 8 * pitch, V(i) + 4 * (8 * pitch + 32)
            q.dc, q.dh, q.dloss = G(i), G(i) + 4 * pitch, G(i) + 4 * 2 * pitch
        nbytes = ctypes.sizeof(arr)
        dev = lib.malloc_uninit(nbytes)
        lib.h2d(dev, ctypes.addressof(arr), nbytes)
        host = ctypes.addressof(arr)
        for lo, cnt in ((0, 4), (4, 2), (6, 1)):
            lib.tree_nodes_fwd(host, dev, lo, cnt)
        one = np.array([1.0], np.float32)
        lib.h2d(G(6) + 4 * 2 * pitch, one.ctypes.data, 4)                 # d(loss of the root) = 1
        for lo, cnt in ((6, 1), (4, 2), (0, 4)):
            lib.tree_nodes_bwd(host, dev, lo, cnt)
        out = {"vals": vals.toCPU()[:, 5 * pitch:8 * pitch + 64], "grads": grads.toCPU()}
        out.update({"d" + k: t.d.toCPU() for k, t in w.items()})
        return out
    check(f, ora, gpu)


@pytest.mark.parametrize("shape", [(128, 64, 16, 16), (128, 1024, 4, 4), (256, 64, 32, 32)])
def test_fusion_level_two_changes_no_result(gpu, shape):
    """ltb_set_fusion(2): the batch-norm backward / add gradient that absorbs a held in-place ReLU gradient applies the mask on
    load and does not write the masked gradient back into the (dead) buffer.  dx, dgamma, dbeta, da and db are those of level
    1, bit for bit -- for the register-resident kernels, the packed kernels and the two-sweep kernel of the largest maps --
    and only the dead buffer itself may differ."""
    b, lib = gpu, gpu.lib
    N, C, H, W = shape
    x0 = R(14).standard_normal(shape).astype(np.float32); dy0 = R(15).standard_normal(shape).astype(np.float32)
    res = []
    for level in (1, 2):
        lib.set_fusion(level)
        try:
            x = TensorR(b.fromNumpy(x0)); x.d = b.fill(shape, 0.0)
            gam, bet = TensorR(b.fill((C,), 1.5), b.fill((C,), 0.0)), TensorR(b.fill((C,), 0.1), b.fill((C,), 0.0))
            y, sm, si, _ = b.batchNormTraining(x.x, gam.x, bet.x, b.fill((C,), 0.0), b.fill((C,), 1.0))
            yr = TensorR(y, b.fromNumpy(dy0))
            b.relu(y, inPlace=True)
            b.relu_grad(yr, yr, inPlace=True)
            b.batchNorm_grad(x, yr, gam, bet, sm, si)
            # the add gradient absorbing the ReLU gradient of its output
            z = TensorR(b.fromNumpy(x0), b.fromNumpy(dy0)); a = TensorR(b.fromNumpy(x0), b.fill(shape, 0.0)); c = TensorR(b.fromNumpy(x0), b.fromNumpy(dy0 * 0.5))
            b.relu_grad(z, z, inPlace=True)
            sh = np.array(shape, np.int32)
            lib.ew_binary_grad(0, a.x.ptr, a.d.ptr, sh.ctypes.data, c.x.ptr, c.d.ptr, sh.ctypes.data, z.d.ptr, 4)
            lib.sync()
            res.append([x.d.toCPU(), gam.d.toCPU(), bet.d.toCPU(), a.d.toCPU(), c.d.toCPU()])
        finally:
            lib.set_fusion(0)
    for u, v in zip(res[0], res[1]):
        assert np.array_equal(u, v)


@pytest.mark.parametrize("shape", [(128, 64, 32, 32), (128, 256, 16, 16), (128, 128, 8, 8), (128, 1024, 4, 4), (64, 2048, 2, 2)])
@pytest.mark.parametrize("other_fresh", [False, True])
def test_bn_backward_absorbs_the_add_gradient(gpu, shape, other_fresh):
    """Fusion level 2, the end of a residual block backwards: in-place ReLU gradient of the block's output, gradient of the add
    (main path + shortcut), batch-norm backward of the main path's last layer.  When the main path's gradient buffer was
    declared unset, the add gradient is held once more and the batch-norm backward reads the masked gradient straight from
    the block output's gradient, writing the shortcut's share itself: dx, dgamma, dbeta and the shortcut gradient are those
    of level 1, bit for bit (two-sweep, register-resident and packed kernels; the shortcut's buffer unset or holding data)."""
    b, lib = gpu, gpu.lib
    N, C, H, W = shape
    x0 = R(21).standard_normal(shape).astype(np.float32); out0 = R(22).standard_normal(shape).astype(np.float32)
    d0 = R(23).standard_normal(shape).astype(np.float32); pre = R(24).standard_normal(shape).astype(np.float32)
    res = []
    for level in (1, 2):
        lib.set_fusion(level)
        try:
            l0 = lib.kernel_launches()
            x = TensorR(b.fromNumpy(x0)); x.d = b.fill(shape, 0.0)                          # the last convolution's output and its gradient
            gam, bet = TensorR(b.fill((C,), 1.5), b.fill((C,), 0.0)), TensorR(b.fill((C,), 0.1), b.fill((C,), 0.0))
            z, sm, si, _ = b.batchNormTraining(x.x, gam.x, bet.x, b.fill((C,), 0.0), b.fill((C,), 1.0))
            lib.sync()
            zr = TensorR(z, _poisoned(b, shape))                                             # main path: gradient buffer declared unset
            sc = TensorR(b.fromNumpy(x0), _poisoned(b, shape) if other_fresh else b.fromNumpy(pre))   # shortcut
            out = TensorR(b.fromNumpy(out0), b.fromNumpy(d0))                                # the block's output (after ReLU) and its gradient
            lib.sync(); l1 = lib.kernel_launches()
            b.relu_grad(out, out, inPlace=True)
            sh = np.array(shape, np.int32)
            lib.ew_binary_grad(0, zr.x.ptr, zr.d.ptr, sh.ctypes.data, sc.x.ptr, sc.d.ptr, sh.ctypes.data, out.d.ptr, 4)
            b.batchNorm_grad(x, zr, gam, bet, sm, si)
            lib.sync()
            res.append([x.d.toCPU(), gam.d.toCPU(), bet.d.toCPU(), sc.d.toCPU(), lib.kernel_launches() - l1])
        finally:
            lib.set_fusion(0)
    for u, v in zip(res[0][:4], res[1][:4]):
        assert np.isfinite(v).all() and np.array_equal(u, v)
    assert res[1][4] == res[0][4] - 1                                                        # one launch fewer: the add gradient went into the batch norm


@pytest.mark.parametrize("shape", [(128, 256, 16, 16), (128, 64, 32, 32), (128, 512, 8, 8), (128, 1024, 4, 4), (64, 2048, 2, 2), (8, 20, 6, 6), (4, 6, 5, 5)])
@pytest.mark.parametrize("order", ["bn_first", "shortcut_first"])
def test_bn_forward_absorbs_the_add_and_relu(gpu, shape, order):
    """Fusion level 3, the end of a residual block forwards: batch norm of the main path's last layer, its result plus the
    shortcut, ReLU in place on the sum.  One kernel does the three and never writes the batch norm's own result; the sum, the
    saved statistics and the running statistics are those of level 2, bit for bit (packed, register-resident and two-sweep
    kernels; either operand order).  When something other than the ReLU follows the add, the two operations are issued on
    their own and the batch norm's result is written as at level 2."""
    b, lib = gpu, gpu.lib
    N, C, H, W = shape
    x0 = R(31).standard_normal(shape).astype(np.float32) * 2 + 0.5; s0 = R(32).standard_normal(shape).astype(np.float32)
    res = []
    for level, then_relu in ((2, True), (3, True), (2, False), (3, False)):
        lib.set_fusion(level)
        try:
            x, sc = b.fromNumpy(x0), b.fromNumpy(s0)
            gam, bet, rm, rv = b.fill((C,), 1.5), b.fill((C,), 0.1), b.fill((C,), 0.0), b.fill((C,), 1.0)
            lib.sync(); l0 = lib.kernel_launches()
            z, sm, si, _ = b.batchNormTraining(x, gam, bet, rm, rv)
            out = (b.plus(z, sc) if order == "bn_first" else b.plus(sc, z))[0]
            if then_relu:
                b.relu(out, inPlace=True)
            else:
                out = b.mul(out, out)[0]                                                      # reads the sum: the held operations are issued first
            lib.sync()
            res.append([out.toCPU(), sm.toCPU(), si.toCPU(), rm.toCPU(), rv.toCPU(), z.toCPU() if not (level == 3 and then_relu) else None,
                        lib.kernel_launches() - l0])
        finally:
            lib.set_fusion(0)
    for u, v in ((res[0], res[1]), (res[2], res[3])):
        for p, q in zip(u[:5], v[:5]):
            assert np.isfinite(q).all() and np.array_equal(p, q)
    assert np.array_equal(res[2][5], res[3][5]) and np.array_equal(res[0][5], res[2][5])      # the batch norm's own result, wherever it is written
    vec = (H * W) % 4 == 0
    assert res[1][6] == (res[0][6] - 1 if vec else res[0][6])                                # one launch instead of two (the one-launch batch norm needs rows of whole float4)
    assert res[3][6] == res[2][6]


# ---------------------------------------------------------------------------------------------- deferred zero fill
def _poisoned(b, shape):
    """A gradient buffer full of NaN, declared unset: whatever adds into it without reading must leave no NaN behind."""
    t = b.fromNumpy(np.full(shape, np.nan, np.float32))
    b.lib.grad_unset(t.ptr, t.scalarCount)
    return t


@pytest.mark.parametrize("math", [0, 1])
@pytest.mark.parametrize("cfg", [(64, 64, 1, 1, 0, 16, 32), (64, 64, 3, 1, 1, 16, 32), (128, 128, 3, 2, 1, 16, 16), (256, 512, 1, 2, 0, 16, 16),
                                 (256, 1024, 1, 1, 0, 4, 32), (3, 64, 3, 1, 1, 32, 8), (20, 10, 5, 1, 0, 12, 4)],
                         ids=lambda c: "%dto%d_k%d_s%d_h%d" % (c[0], c[1], c[2], c[3], c[5]))
def test_conv_backward_into_an_unset_gradient_buffer(gpu, cfg, math):
    """ltb_grad_unset: the data gradient of a convolution written into a buffer declared unset (and poisoned with NaN) equals
    the data gradient added into a zero-filled buffer -- bit for bit in deterministic mode -- on every path: pointwise, tap
    loop, stride 2 (up-sampled taps and unfold + fold), in-kernel gather, FP32 fallback; and a second backward call into the
    same buffer adds, as always."""
    C, K, k, s, p, H, N = cfg
    b, lib = gpu, gpu.lib
    lib.set_math(math); lib.set_deterministic(1)
    try:
        x0 = R(1).standard_normal((N, C, H, H)).astype(np.float32)
        w0 = (R(2).standard_normal((K, C, k, k)) / np.sqrt(C * k * k)).astype(np.float32)
        Ho = (H + 2 * p - k) // s + 1
        dy0 = R(3).standard_normal((N, K, Ho, Ho)).astype(np.float32)
        res = []
        for unset in (False, True):
            x, w = TensorR(b.fromNumpy(x0)), TensorR(b.fromNumpy(w0))
            x.d = _poisoned(b, x0.shape) if unset else b.fill(x0.shape, 0.0)
            w.d = b.fill(w0.shape, 0.0)
            y = TensorR(b.empty(N, K, Ho, Ho), b.fromNumpy(dy0))
            b.conv2D_batch_grad(x, None, w, y, None, (p, p), (s, s))
            once = x.d.toCPU()
            b.conv2D_batch_grad(x, None, w, y, None, (p, p), (s, s))
            res.append((once, x.d.toCPU()))
        assert np.isfinite(res[1][0]).all()
        assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])
        assert np.abs(res[0][1]).max() > 1.5 * np.abs(res[0][0]).max() * 0.9          # the second call did add
    finally:
        lib.set_deterministic(0); lib.set_math(1)


@pytest.mark.parametrize("shape", [(128, 64, 16, 16), (128, 256, 8, 8), (128, 1024, 4, 4), (32, 2048, 2, 2), (8, 5, 3, 3)])
@pytest.mark.parametrize("with_relu", [False, True])
def test_batch_norm_backward_into_an_unset_gradient_buffer(gpu, shape, with_relu):
    """Batch-norm backward (cluster kernels, packed kernels, the three-kernel path for a pixel count that is no multiple of 4),
    alone and with the held in-place ReLU gradient fused into it: dx written into an unset (NaN-poisoned) buffer equals dx
    added into zeros, bit for bit; dgamma and dbeta unchanged."""
    b, lib = gpu, gpu.lib
    N, C, H, W = shape
    x0 = R(4).standard_normal(shape).astype(np.float32)
    dy0 = R(5).standard_normal(shape).astype(np.float32)
    res = []
    for unset in (False, True):
        lib.set_fusion(1 if with_relu else 0)
        try:
            x = TensorR(b.fromNumpy(x0))
            x.d = _poisoned(b, shape) if unset else b.fill(shape, 0.0)
            gam, bet = TensorR(b.fill((C,), 1.5), b.fill((C,), 0.0)), TensorR(b.fill((C,), 0.1), b.fill((C,), 0.0))
            rm, rv = b.fill((C,), 0.0), b.fill((C,), 1.0)
            y, sm, si, _ = b.batchNormTraining(x.x, gam.x, bet.x, rm, rv)
            yr = TensorR(y, b.fromNumpy(dy0))
            if with_relu:
                b.relu(y, inPlace=True)
                b.relu_grad(yr, yr, inPlace=True)                      # held: the batch-norm backward below applies it
            b.batchNorm_grad(x, yr, gam, bet, sm, si)
            lib.sync()
            res.append((x.d.toCPU(), gam.d.toCPU(), bet.d.toCPU(), yr.d.toCPU()))
        finally:
            lib.set_fusion(0)
    assert np.isfinite(res[1][0]).all()
    for a, c in zip(res[0], res[1]):
        assert np.array_equal(a, c)


@pytest.mark.parametrize("fused", [False, True])
def test_add_gradient_into_unset_gradient_buffers(gpu, fused):
    """The gradient of a same-shape add, plain and with the held in-place ReLU gradient fused in: one destination unset (written),
    the other holding data (added into); then both unset."""
    b, lib = gpu, gpu.lib
    n = (64, 32, 8, 8)
    y0 = R(6).standard_normal(n).astype(np.float32); d0 = R(7).standard_normal(n).astype(np.float32); pre = R(8).standard_normal(n).astype(np.float32)
    res = []
    for unset in (False, True):
        lib.set_fusion(1 if fused else 0)
        try:
            out = []
            for both in (False, True):
                y = TensorR(b.fromNumpy(y0), b.fromNumpy(d0))
                a = TensorR(b.fromNumpy(y0)); c = TensorR(b.fromNumpy(y0))
                a.d = _poisoned(b, n) if unset else b.fill(n, 0.0)
                c.d = (_poisoned(b, n) if unset else b.fill(n, 0.0)) if both else b.fromNumpy(pre)
                if fused:
                    b.relu_grad(y, y, inPlace=True)
                sh = np.array(n, np.int32)
                lib.ew_binary_grad(0, a.x.ptr, a.d.ptr, sh.ctypes.data, c.x.ptr, c.d.ptr, sh.ctypes.data, y.d.ptr, 4)
                lib.sync()
                out += [a.d.toCPU(), c.d.toCPU(), y.d.toCPU()]
            res.append(out)
        finally:
            lib.set_fusion(0)
    for a, c in zip(res[0], res[1]):
        assert np.isfinite(c).all() and np.array_equal(a, c)


def test_unset_buffers_are_zero_to_everything_else(gpu):
    """Entry points that cannot write instead of adding fill an unset block with zeros first: max-pool and average-pool
    backward, an activation's gradient, the transfers, ltb_grad_materialize; a part of a block is never taken as the whole;
    ltb_reset forgets declarations of blocks above the mark."""
    b, lib = gpu, gpu.lib
    x0 = R(9).standard_normal((4, 8, 8, 8)).astype(np.float32)
    x = b.fromNumpy(x0)
    y, idx = b.maxPool2D_batch(x, (2, 2), (2, 2))
    dy = b.fromNumpy(R(10).standard_normal((4, 8, 4, 4)).astype(np.float32))
    ref, got = TensorR(x, b.fill(x0.shape, 0.0)), TensorR(x, _poisoned(b, x0.shape))
    for t in (ref, got):
        b.maxPool2D_batch_grad(t, TensorR(y, dy), idx)
    assert np.array_equal(ref.d.toCPU(), got.d.toCPU())
    ref, got = TensorR(x, b.fill(x0.shape, 0.0)), TensorR(x, _poisoned(b, x0.shape))
    ya = b.averagePool2D_batch(x, (2, 2), (2, 2))
    for t in (ref, got):
        b.averagePool2D_batch_grad(t, TensorR(ya, dy), (2, 2), (2, 2))
    assert np.array_equal(ref.d.toCPU(), got.d.toCPU())
    ref, got = b.fill(x0.shape, 0.0), _poisoned(b, x0.shape)
    for d in (ref, got):
        lib.unary_grad(1, x.ptr, d.ptr, x.ptr, x.ptr, x.scalarCount, 0)            # tanh'(y) * dy added into d
    assert np.array_equal(ref.toCPU(), got.toCPU())
    assert not _poisoned(b, (1000,)).toCPU().any()                                  # a read-back sees zeros
    t = _poisoned(b, (1000,)); lib.grad_materialize(t.ptr, 1000)
    assert not t.toCPU().any()
    # a part of a declared block: conv backward into the first half of a buffer must not leave the second half unset and undefined
    big = _poisoned(b, (2, 4, 16, 8, 8))
    w = TensorR(b.fromNumpy((R(11).standard_normal((8, 16, 1, 1)) / 4).astype(np.float32))); w.d = b.fill((8, 16, 1, 1), 0.0)
    from lantern_b200.backend import Tensor
    half = Tensor(b, big.ptr, (4, 16, 8, 8))
    xin = TensorR(b.fromNumpy(R(12).standard_normal((4, 16, 8, 8)).astype(np.float32)), half)
    yout = TensorR(b.empty(4, 8, 8, 8), b.fromNumpy(R(13).standard_normal((4, 8, 8, 8)).astype(np.float32)))
    b.conv2D_batch_grad(xin, None, w, yout, None, (0, 0), (1, 1))
    whole = big.toCPU()
    assert np.isfinite(whole).all() and whole[0].any() and not whole[1].any()
    mark = lib.mark()
    t = _poisoned(b, (4096,))
    lib.reset(mark)
    t2 = b.fromNumpy(np.full((4096,), 3.0, np.float32))                              # the same address, now an ordinary tensor
    assert t2.ptr == t.ptr and np.array_equal(t2.toCPU(), np.full((4096,), 3.0, np.float32))


# ---------------------------------------------------------------------------------------------- branch regions
@pytest.mark.parametrize("replay", [False, True])
def test_branch_region_gives_the_results_of_program_order(gpu, replay):
    """A residual block's two paths (conv + BN + ReLU + 3x3 conv on one, 1x1 conv + BN on the other, then the sum) and their
    gradients, issued once in program order and once with the shortcut as a branch region on a second stream, eagerly and
    from a recorded step: every tensor bit-identical except the weight gradients, whose split-K partial sums are added
    atomically in any order (compared at 1e-5 of their largest element), and the arena back at its mark afterwards."""
    N, C, H, K = 128, 64, 16, 64
    x0 = R(1).standard_normal((N, C, H, H)).astype(np.float32)
    w10 = (R(2).standard_normal((K, C, 1, 1)) / 8).astype(np.float32)
    w20 = (R(3).standard_normal((K, K, 3, 3)) / 24).astype(np.float32)
    wd0 = (R(4).standard_normal((K, C, 1, 1)) / 8).astype(np.float32)
    dz0 = R(5).standard_normal((N, K, H, H)).astype(np.float32)
    b, lib = gpu, gpu.lib

    def run(branch):
        mark = lib.mark()
        x = TensorR(b.fromNumpy(x0)); x.d = b.fill(x0.shape, 0.0)
        w1, w2, wd = TensorR(b.fromNumpy(w10)), TensorR(b.fromNumpy(w20)), TensorR(b.fromNumpy(wd0))
        for w in (w1, w2, wd):
            w.d = b.fill(w.x.shape, 0.0)
        g, be = TensorR(b.fill((K,), 1.0)), TensorR(b.fill((K,), 0.0))
        gd, bd = TensorR(b.fill((K,), 1.0)), TensorR(b.fill((K,), 0.0))
        for t in (g, be, gd, bd):
            t.d = b.fill((K,), 0.0)
        rm, rv, rmd, rvd = b.fill((K,), 0.0), b.fill((K,), 1.0), b.fill((K,), 0.0), b.fill((K,), 1.0)
        dz = b.fromNumpy(dz0)
        lib.sync()
        inner = lib.mark()
        out = {}

        def step():
            if branch: lib.branch_mark()
            a, _, _ = b.conv2D_batch(x.x, w1.x, None, (1, 1), (0, 0, 0, 0))
            an, sm, si, _ = b.batchNormTraining(a, g.x, be.x, rm, rv)
            ar = TensorR(b.relu(an, True)); ar.d = b.fill(an.shape, 0.0)
            m, _, _ = b.conv2D_batch(ar.x, w2.x, None, (1, 1), (1, 1, 1, 1))
            if branch: lib.branch_begin()
            s, _, _ = b.conv2D_batch(x.x, wd.x, None, (1, 1), (0, 0, 0, 0))
            sn, smd, sid, _ = b.batchNormTraining(s, gd.x, bd.x, rmd, rvd)
            if branch: lib.branch_end(); lib.branch_join()
            z, _, _ = b.plus(m, sn)
            # backward: the sum's gradient reaches both paths; the shortcut's gradients run as a branch and are joined before
            # the first convolution's gradient, which accumulates into the same x.d
            mr, snr, sr, ac = TensorR(m, dz), TensorR(sn, dz), TensorR(s), TensorR(a)
            sr.d, ac.d = b.fill(s.shape, 0.0), b.fill(a.shape, 0.0)
            if branch: lib.branch_mark(); lib.branch_begin()
            b.batchNorm_grad(sr, snr, gd, bd, smd, sid)
            b.conv2D_batch_grad(x, None, wd, sr, None, (0, 0), (1, 1))
            if branch: lib.branch_end()
            b.conv2D_batch_grad(ar, None, w2, mr, None, (1, 1), (1, 1))
            b.relu_grad(ar, ar, True)
            b.batchNorm_grad(ac, ar, g, be, sm, si)
            if branch: lib.branch_join()
            b.conv2D_batch_grad(x, None, w1, ac, None, (0, 0), (1, 1))
            out["z"] = z
        if replay:
            assert lib.graph_begin() == 0
            step()
            graph = lib.graph_end()
            assert graph
            lib.graph_launch(graph); lib.sync(); lib.graph_destroy(graph)
        else:
            step()
        res = {"z": out["z"].toCPU(), "dx": x.d.toCPU(), "dw1": w1.d.toCPU(), "dw2": w2.d.toCPU(), "dwd": wd.d.toCPU(),
               "dg": g.d.toCPU(), "dgd": gd.d.toCPU(), "rm": rm.toCPU(), "rvd": rvd.toCPU()}
        lib.reset(inner)
        assert lib.mark() == inner          # staging blocks held during the regions went back with the reset
        lib.reset(mark)
        return res
    lib.set_fusion(1)
    try:
        plain, forked = run(False), run(True)
    finally:
        lib.set_fusion(0)
    for k in plain:
        assert np.isfinite(plain[k]).all() and np.abs(plain[k]).max() > 0, k
        if k.startswith("dw"):
            assert np.abs(plain[k] - forked[k]).max() <= 1e-5 * np.abs(plain[k]).max(), k
        else:
            assert np.array_equal(plain[k], forked[k]), k + ": branch region and program order differ"


def test_branch_region_misuse_is_reported(gpu):
    from lantern_b200._ffi import LanternError
    lib = gpu.lib
    with pytest.raises(LanternError):
        lib.branch_begin()                          # no mark
    with pytest.raises(LanternError):
        lib.branch_join()                           # no region
    lib.branch_mark()
    with pytest.raises(LanternError):
        lib.branch_mark()                           # one region at a time
    lib.branch_begin()
    with pytest.raises(LanternError):
        lib.branch_join()                           # the branch has not ended
    lib.branch_end()
    with pytest.raises(LanternError):
        lib.branch_begin()                          # one branch per region
    lib.branch_join()


# ---------------------------------------------------------------------------------------------- fused gate
@pytest.mark.parametrize("cfg", [(150, 150, 150, 2), (150, 300, 0, 1), (5, 150, 0, -1), (33, 70, 9, 2), (1, 1, 1, 1)])
def test_affine_act_and_gradient(ora, gpu, cfg):
    """out = act(W0.a + W1.b + bias) and its accumulating gradient against the oracle: the TreeLSTM gate sizes (two 150x150
    products; one 150x300 product of a leaf, whose input has no gradient; the 5-way output layer without activation)."""
    rows, c0, c1, act = cfg
    W00, a0 = R(1).standard_normal((rows, c0)).astype(np.float32) / np.sqrt(c0), R(2).standard_normal(c0).astype(np.float32)
    W10, b0 = R(3).standard_normal((rows, max(c1, 1))).astype(np.float32) / np.sqrt(max(c1, 1)), R(4).standard_normal(max(c1, 1)).astype(np.float32)
    bias0, dout0 = R(5).standard_normal(rows).astype(np.float32), R(6).standard_normal(rows).astype(np.float32)

    def f(b):
        lib = b.lib
        W0, a, W1, bb, bias, dout = (b.fromNumpy(v) for v in (W00, a0, W10, b0, bias0, dout0))
        dW0, da, dW1, db, dbias = (b.fromNumpy(v * 0.5) for v in (W00, a0, W10, b0, bias0))      # accumulate onto non-zero values
        out = b.fill((rows,), 0.0)
        two = c1 > 0
        leaf = c0 == 300                                                # the leaf's embedding is an input: no gradient for it
        lib.affine_act(W0, a, c0, W1 if two else 0, bb if two else 0, c1, bias, act, out, rows)
        lib.affine_act_grad(W0, dW0, a, 0 if leaf else da, c0, W1 if two else 0, dW1 if two else 0, bb if two else 0, db if two else 0, c1,
                            dbias, act, out, dout, rows)
        return {"out": out.toCPU(), "dW0": dW0.toCPU(), "da": da.toCPU(), "dW1": dW1.toCPU(), "db": db.toCPU(), "dbias": dbias.toCPU()}
    check(f, ora, gpu)


@pytest.mark.parametrize("inner", [True, False])
def test_lstm_cell_and_gradient(ora, gpu, inner):
    """cell = i*u (+ fl*cl + fr*cr), hidden = o*tanh(cell) and the accumulating gradient, inner node and leaf, against the oracle."""
    n = 150
    v = {k: R(10 + j).standard_normal(n).astype(np.float32) for j, k in enumerate(["i", "u", "fl", "cl", "fr", "cr", "o", "dc", "dh"])}

    def f(b):
        lib = b.lib
        t = {k: b.fromNumpy(a) for k, a in v.items()}
        d = {k: b.fromNumpy(v[k] * 0.25) for k in ["i", "u", "fl", "cl", "fr", "cr", "o"]}          # accumulate onto non-zero values
        c, tc, h = b.fill((n,), 0.0), b.fill((n,), 0.0), b.fill((n,), 0.0)
        kids = [t[k] if inner else 0 for k in ("fl", "cl", "fr", "cr")]
        lib.lstm_cell(t["i"], t["u"], kids[0], kids[1], kids[2], kids[3], t["o"], c, tc, h, n)
        g = lambda k: d[k] if inner else 0
        lib.lstm_cell_grad(t["i"], d["i"], t["u"], d["u"], kids[0], g("fl"), kids[1], g("cl"), kids[2], g("fr"), kids[3], g("cr"),
                           t["o"], d["o"], tc, t["dc"], t["dh"], n)
        out = {"c": c.toCPU(), "tc": tc.toCPU(), "h": h.toCPU()}
        out.update({"d" + k: d[k].toCPU() for k in d})
        return out
    check(f, ora, gpu)


@pytest.mark.parametrize("cfg", [(256, 80, 100, 100, 1), (1, 80, 100, 100, 1), (20, 26, 50, 50, 2), (256, 100, 0, 80, -1), (7, 5, 3, 130, 1)])
def test_affine_act_rows_and_gradient(ora, gpu, cfg):
    """out = act(x0 W0 + x1 W1 + bias) over a minibatch and its accumulating gradient against the oracle: the min-char-rnn
    cell (one-hot input without gradient) and its output layer (no activation, one product), at batch 1, 20 and 256."""
    batch, c0, c1, width, act = cfg
    x00 = R(1).standard_normal((batch, c0)).astype(np.float32)
    W00 = (R(2).standard_normal((c0, width)) / np.sqrt(c0)).astype(np.float32)
    x10 = R(3).standard_normal((batch, max(c1, 1))).astype(np.float32)
    W10 = (R(4).standard_normal((max(c1, 1), width)) / np.sqrt(max(c1, 1))).astype(np.float32)
    bias0, dout0 = R(5).standard_normal(width).astype(np.float32), R(6).standard_normal((batch, width)).astype(np.float32)

    def f(b):
        lib = b.lib
        x0, W0, x1, W1, bias, dout = (b.fromNumpy(v) for v in (x00, W00, x10, W10, bias0, dout0))
        dx0, dW0, dx1, dW1, dbias = (b.fromNumpy(v * 0.5) for v in (x00, W00, x10, W10, bias0))
        out = b.fill((batch, width), 0.0)
        two = c1 > 0
        onehot = c0 in (80, 26)                                         # the RNN's input: no gradient wanted
        lib.affine_act_rows(x0, W0, c0, x1 if two else 0, W1 if two else 0, c1, bias, act, out, batch, width)
        lib.affine_act_rows_grad(x0, 0 if onehot else dx0, W0, dW0, c0, x1 if two else 0, dx1 if two else 0, W1 if two else 0, dW1 if two else 0, c1,
                                 dbias, act, out, dout, batch, width)
        return {"out": out.toCPU(), "dx0": dx0.toCPU(), "dW0": dW0.toCPU(), "dx1": dx1.toCPU(), "dW1": dW1.toCPU(), "dbias": dbias.toCPU()}
    check(f, ora, gpu)
