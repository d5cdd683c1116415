"""Parity at the sizes the benchmark and the named configurations use, and the whole-step checks that are well conditioned.

What a whole ResNet-50 step can and cannot promise: the untrained 53-layer network with batch norm amplifies any
rounding-level difference in the forward pass by four to five orders of magnitude by the time it reaches the parameter
gradients.  The CPU oracle ALONE, fed the same batch plus Gaussian noise of relative size 4e-6 (the size of the per-operator
differences between two correct FP32 implementations: see test_conv_fwd_bwd_tf32_at_batch_128, worst 4.4e-6), moves its own
gradients by 4-6 % (FP32) and 40-60 % (TF32 emulation).  "Every gradient within 1e-4" is therefore not defined for this network,
at batch 8 or at batch 128.  The tests below hold the CUDA path to what IS defined:
  * every convolution of the network at batch 128, operator by operator, at the stated tolerances (the strict gate);
  * the loss of the whole step at the stated tolerances;
  * every gradient tensor no further from the oracle than twice the oracle's own movement under that 4e-6 perturbation;
  * every intermediate activation, in layer order, inside a band that a wrong stride, pad, layout or fusion would leave at once;
  * a shallow prefix of the network (stem + one bottleneck block) at batch 32, where the amplification is small;
  * arg-max predictions, bit for bit;
  * the TF32 step trains as the FP32 step does (loss trajectories over dozens of steps)."""
import ctypes
import os

import numpy as np
import pytest

import bench
from lantern_b200.backend import TensorR
from lantern_b200.hosts import HostPrograms, Model
from tests.parity import FP32_RTOL, TF32_RTOL, assert_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORA_HOSTS = os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so")
R = lambda seed: np.random.default_rng(seed)
libc = ctypes.CDLL(None)


# ------------------------------------------------------------------------------------------------ every conv of the bench, batch 128
@pytest.mark.parametrize("cfg", sorted(set(bench.resnet50_convs())), ids=lambda c: "%dto%d_k%d_s%d_h%d" % (c[0], c[1], c[2], c[3], c[5]))
def test_conv_fwd_bwd_tf32_at_batch_128(ora, gpu, cfg):
    """The 23 distinct convolutions of ResNet-50 (CIFAR shape) at the benchmark's batch of 128: forward, data-grad and
    weight-grad onto non-zero destinations.  Two gates: 2e-3 against the FP32 oracle, 1e-4 against the oracle emulating the
    tensor core's operand truncation.  Batch 128 takes other paths than small batches do: other tile counts and split
    factors, whole 128-byte rows of small images, the several-images-per-tile forms."""
    C, K, k, s, p, H = cfg
    N = 128
    x0 = R(1).standard_normal((N, C, H, H)).astype(np.float32)
    w0 = (R(2).standard_normal((K, C, k, k)) / np.sqrt(C * k * k)).astype(np.float32)
    Ho = (H + 2 * p - k) // s + 1
    dy0 = R(4).standard_normal((N, K, Ho, Ho)).astype(np.float32)

    def f(b, math):
        b.lib.set_math(math)
        x, w = TensorR(b.fromNumpy(x0)), TensorR(b.fromNumpy(w0))
        y, _, _ = b.conv2D_batch(x.x, w.x, None, (s, s), (p, p, p, p))
        x.d, w.d = b.fromNumpy(x0 * 0.25), b.fromNumpy(w0 * 0.5)
        b.conv2D_batch_grad(x, None, w, TensorR(y, b.fromNumpy(dy0)), None, (p, p), (s, s))
        return {"y": y.toCPU(), "dx": x.d.toCPU(), "dw": w.d.toCPU()}
    got, ref32, ref_tf = f(gpu, 1), f(ora, 0), f(ora, 1)
    for q in got:
        assert_close(ref32[q], got[q], TF32_RTOL, q + " vs FP32 oracle")
        assert_close(ref_tf[q], got[q], FP32_RTOL, q + " vs TF32-emulating oracle")
    gpu.lib.set_deterministic(1)                          # split-K sums combined in a fixed order: the same bits on every run
    try:
        d1, d2 = f(gpu, 1), f(gpu, 1)
    finally:
        gpu.lib.set_deterministic(0)
    for q in got:
        assert np.array_equal(d1[q], d2[q]), q + " differs between two runs in deterministic mode"
        assert_close(ref_tf[q], d1[q], FP32_RTOL, q + " (deterministic mode) vs TF32-emulating oracle")


# ------------------------------------------------------------------------------------------------ whole steps
def _pair(oracle_lib, cuda_lib, name, batch, math):
    cuda_lib.set_math(math); oracle_lib.set_math(math)
    mo = HostPrograms(oracle_lib, ORA_HOSTS, "orah_").model(name, batch, seed=42)
    mg = HostPrograms(cuda_lib).model(name, batch, seed=42)
    return mo, mg


def _grads(m):
    return [m.grad(i).astype(np.float64) for i in range(m.num_params)]


def _rel_l2(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(a), 1e-300))


@pytest.fixture()
def libs(oracle_lib, cuda_lib):
    mo, mg = oracle_lib.mark(), cuda_lib.mark()
    yield oracle_lib, cuda_lib
    cuda_lib.set_math(1); oracle_lib.set_math(0)
    oracle_lib.reset(mo); cuda_lib.reset(mg)


@pytest.mark.parametrize("batch", [8, 128])
@pytest.mark.parametrize("math", [0, 1])
def test_resnet50_gradients_within_the_oracles_own_sensitivity(libs, batch, math):
    """Loss at the stated tolerance; every gradient tensor no further from the oracle (relative L2) than twice the distance
    the oracle's own gradient moves when Gaussian noise of relative size 4e-6 is added to the batch.  math 1 compares the
    tensor-core path with the oracle emulating its operand truncation."""
    ora, lib = libs
    x = R(0).standard_normal(batch * 3072).astype(np.float32); y = R(1).integers(0, 10, batch).astype(np.int32)
    noisy = (x + np.float32(4e-6) * R(5).standard_normal(x.size).astype(np.float32)).astype(np.float32)

    def run(hp_lib, which, data):
        mo, mg = _pair(ora, lib, "resnet50", batch, math)
        m, other = (mo, mg) if which == "ora" else (mg, mo)
        other.close()
        loss = m.step(data, y, 0.0, update=False); g = _grads(m); m.close()
        return loss, g
    lo, go = run(ora, "ora", x)
    _, gp = run(ora, "ora", noisy)
    lg, gg = run(lib, "gpu", x)
    assert abs(lo - lg) <= (FP32_RTOL if math == 0 else TF32_RTOL) * abs(lo), (lo, lg)
    if math == 1:      # deterministic mode: the tensor-core path adds its split-K partial sums in a fixed order
        lib.set_deterministic(1)
        try:
            (l1, g1), (l2, g2) = run(lib, "gpu", x), run(lib, "gpu", x)
        finally:
            lib.set_deterministic(0)
        assert l1 == l2 and all(np.array_equal(a, b) for a, b in zip(g1, g2)), "two runs of the same step differ in deterministic mode"
        assert abs(lo - l1) <= TF32_RTOL * abs(lo), (lo, l1)
    worst = 0.0
    for i, (a, b, c) in enumerate(zip(go, gp, gg)):
        if not a.any():
            continue                                                  # running statistics: no gradient
        own, err = _rel_l2(a, b), _rel_l2(a, c)
        worst = max(worst, err / max(own, 1e-12))
        # the stated tolerance is the floor: a well-conditioned tensor (the classifier's bias) hardly moves under the noise
        assert err <= max(2.0 * own, FP32_RTOL if math == 0 else TF32_RTOL), "gradient %d: error %.3e, the oracle's own movement %.3e" % (i, err, own)
    print("resnet50 batch %d math %d: loss %.7f / %.7f, worst error / own movement %.2f" % (batch, math, lo, lg, worst))


@pytest.mark.parametrize("batch", [8, 128])
@pytest.mark.parametrize("math", [0, 1])
def test_resnet50_every_activation_in_layer_order(libs, batch, math):
    """The step's 128 operator outputs, in forward order, CUDA against oracle (estimated relative L2 distance from the
    trace's signed sums).  Rounding differences grow slowly with depth (measured: 1e-6 after the stem to 2e-4 (batch 8) and
    6e-4 (batch 128) at the classifier in FP32; 1e-4 to 6e-2 in TF32); a wrong stride, padding, layout, statistic or fused
    kernel puts its layer at order one.  The band grows quadratically with depth from the stated tolerance at the stem to ten
    (FP32) / fifty (TF32) times it at the classifier; the first layer outside it is reported."""
    ora, lib = libs
    x = R(0).standard_normal(batch * 3072).astype(np.float32); y = R(1).integers(0, 10, batch).astype(np.int32)
    mo, mg = _pair(ora, lib, "resnet50", batch, math)
    mg.close(); to = mo.trace(x, y); mo.close()
    mo, mg = _pair(ora, lib, "resnet50", batch, math)
    mo.close(); tg = mg.trace(x, y); mg.close()
    d = Model.trace_distance(to, tg)
    assert len(d) >= 120
    tol, late = (FP32_RTOL, 10.0) if math == 0 else (TF32_RTOL, 50.0)
    for k, (idx, shape, ex, ed) in enumerate(d):
        band = tol * (1.0 + (late - 1.0) * (k / float(len(d))) ** 2)       # the stated tolerance at the stem, `late` times it at the classifier
        assert ex <= band, "operator output %d %s is the first outside the band: %.3e > %.1e" % (idx, shape, ex, band)


@pytest.mark.parametrize("math,loss_tol,grad_l2", [(0, 1e-6, 1e-2), (1, 1e-5, 6e-2)])
def test_resnet50_prefix_at_batch_32(libs, math, loss_tol, grad_l2):
    """Stem, max pool, the first bottleneck block (with its shortcut convolution), average pool, classifier: the layer types
    and the issue order of the full program, shallow enough for a meaningful gradient comparison (measured: FP32 worst
    relative L2 2.7e-3, TF32 against the truncating oracle 1.9e-2, both dominated by single ReLU boundary elements)."""
    ora, lib = libs
    b = 32
    x = R(5).standard_normal(b * 3072).astype(np.float32); y = R(6).integers(0, 10, b).astype(np.int32)
    mo, mg = _pair(ora, lib, "resnet50_prefix", b, math)
    lo, lg = mo.step(x, y, 0.0, update=False), mg.step(x, y, 0.0, update=False)
    assert abs(lo - lg) <= loss_tol * abs(lo), (lo, lg)
    for i, (a, c) in enumerate(zip(_grads(mo), _grads(mg))):
        if a.any():
            assert _rel_l2(a, c) <= grad_l2, "prefix gradient %d: relative L2 %.3e" % (i, _rel_l2(a, c))
    assert np.array_equal(mo.logits().argmax(1), mg.logits().argmax(1))
    mo.close(); mg.close()


@pytest.mark.parametrize("math", [0, 1])
def test_squeezenet_at_batch_64(libs, math):
    """BASELINE configuration 4 at its stated batch: FP32 strict on every gradient tensor (1e-4, max-norm); TF32 loss within
    2e-3 and gradients within 10 % relative L2 of the truncating oracle (measured 1.2e-2 median); predictions equal."""
    ora, lib = libs
    b = 64
    x = R(7).standard_normal(b * 3072).astype(np.float32); y = R(8).integers(0, 10, b).astype(np.int32)
    mo, mg = _pair(ora, lib, "squeezenet", b, math)
    lo, lg = mo.step(x, y, 0.0, update=False), mg.step(x, y, 0.0, update=False)
    assert abs(lo - lg) <= (FP32_RTOL if math == 0 else TF32_RTOL) * abs(lo), (lo, lg)
    for i, (a, c) in enumerate(zip(_grads(mo), _grads(mg))):
        if not a.any():
            continue
        if math == 0:
            assert_close(a, c, FP32_RTOL, "squeezenet gradient %d" % i)
        else:
            assert _rel_l2(a, c) <= 0.1, "squeezenet gradient %d: relative L2 %.3e" % (i, _rel_l2(a, c))
    assert np.array_equal(mo.logits().argmax(1), mg.logits().argmax(1)), "predictions differ"
    mo.close(); mg.close()


def test_treelstm_on_trees_of_fifty_leaves(libs):
    """BASELINE configuration 3 at its largest tree (99 nodes): loss and all 22 gradient tensors at 1e-4."""
    from tests.test_gpu_models import _random_tree
    ora, lib = libs
    mo, mg = _pair(ora, lib, "treelstm", 1, 0)
    rng = R(17); x = np.zeros(1, np.float32)
    for leaves in (50, 50, 41):
        y = _random_tree(rng, leaves)
        lo, lg = mo.step(x, y, 0.0, update=False), mg.step(x, y, 0.0, update=False)
        assert abs(lo - lg) <= FP32_RTOL * abs(lo), (leaves, lo, lg)
        for i in range(mo.num_params):
            assert_close(mo.grad(i), mg.grad(i), FP32_RTOL, "treelstm gradient %d (%d leaves)" % (i, leaves))
        mo.step(x, y, 0.0); mg.step(x, y, 0.0)
    mo.close(); mg.close()


@pytest.mark.parametrize("math", [0, 1])
def test_predictions_are_bit_exact(libs, math):
    """Arg-max of the classifier output, oracle against CUDA, over five MNIST training steps at batch 100 (dropout masks from
    the same rand() stream on both sides)."""
    ora, lib = libs
    b = 100
    x = ((R(3).random(b * 784, dtype=np.float32) - np.float32(0.1307)) / np.float32(0.3081)); y = R(4).integers(0, 10, b).astype(np.int32)
    mo, mg = _pair(ora, lib, "mnist", b, math)
    for s in range(5):
        libc.srand(9 + s); mo.step(x, y, 0.0005)
        libc.srand(9 + s); mg.step(x, y, 0.0005)
        zo, zg = mo.logits(), mg.logits()
        assert np.array_equal(zo.argmax(1), zg.argmax(1)), "step %d: predictions differ" % s
        assert_close(zo, zg, FP32_RTOL if math == 0 else 1e-3, "logits")    # TF32: five updates carry the 1e-4 of one step forward (measured up to 1.6e-4)
    mo.close(); mg.close()


def test_the_tf32_step_trains_as_the_fp32_step_does(cuda_lib):
    """Loss trajectories on the GPU, TF32 against FP32 math, same weights and batches: SqueezeNet (batch 64, 40 steps, the
    configuration's lr 0.005) and ResNet-50 (batch 32, 30 steps, lr 0.002).  Per-step equality is not expected (see the module
    comment); both runs must bring the loss down, and to the same level.  The ResNet step size is one at which the loss falls
    from the first step on: at lr 0.02 on two batches the loss first climbs to 10-19 and the step at which it comes back down
    (25 to 35) differs from run to run within ONE math mode, so nothing about the two modes can be read off such a run; at
    0.002 repeated runs of either mode end within 0.46-0.53 of each other after 30 steps."""
    lib = cuda_lib
    mark = lib.mark()
    try:
        for name, b, steps, lr, batches, fall, apart in (("squeezenet", 64, 40, 0.005, 4, 0.8, 0.5), ("resnet50", 32, 30, 0.002, 2, 0.4, 0.1)):
            tr = {}
            for math in (0, 1):
                lib.set_math(math)
                m = HostPrograms(lib).model(name, b, seed=42); ls = []
                for s in range(steps):
                    rng = R(100 + s % batches)                      # a few batches, revisited: the loss must fall
                    ls.append(m.step(rng.standard_normal(b * 3072).astype(np.float32), rng.integers(0, 10, b).astype(np.int32), lr))
                tr[math] = np.array(ls); m.close(); lib.reset(mark)
            print(name, "fp32", np.round(tr[0][::5], 3), "tf32", np.round(tr[1][::5], 3))
            assert np.all(np.isfinite(tr[0])) and np.all(np.isfinite(tr[1]))
            first, end32, endtf = tr[0][0], tr[0][-6:].min(), tr[1][-6:].min()     # the two batches differ in loss: the best of the last steps
            # the first step is the same step; the tensor core TRUNCATES its operands to TF32 (a bias toward zero of up to 1e-3 per
            # product), which the large logits of an untrained SqueezeNet turn into 1 % of its loss of 6.7
            assert abs(tr[1][0] - first) <= 0.02 * first
            assert end32 < fall * first and endtf < fall * first, (first, end32, endtf)
            assert abs(endtf - end32) <= apart * first, (first, end32, endtf)
    finally:
        lib.set_math(1)
        lib.reset(mark)
