"""The recursive host programs (min-char-rnn, TreeLSTM) on the CPU oracle: sanity anchors that need no GPU.
An untrained classifier's loss is ln(classes) per prediction, and repeating one example must drive its loss down."""
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORA_HOSTS = os.path.join(ROOT, "oracle", "liblantern_oracle_hosts.so")


def _model(oracle_lib, name, batch):
    from lantern_b200.hosts import HostPrograms
    oracle_lib.set_math(0)
    return HostPrograms(oracle_lib, ORA_HOSTS, "orah_").model(name, batch, seed=42)


def test_rnn_untrained_loss_and_learning(oracle_lib):
    mark = oracle_lib.mark()
    T, V, B = 20, 80, 3
    m = _model(oracle_lib, "rnn", B)
    assert m.num_params == 5 and m.label_count == T * B and m.input_count == T * B * V
    ids = np.random.default_rng(0).integers(0, V, (T + 1, B))
    x = np.zeros((T, B, V), np.float32)
    x[np.arange(T)[:, None], np.arange(B)[None, :], ids[:T]] = 1.0
    y = ids[1:].astype(np.int32).ravel()
    first = m.step(x.ravel(), y, 0.01)
    assert abs(first - T * B * np.log(V)) < 0.02 * T * B * np.log(V)
    for _ in range(30):
        last = m.step(x.ravel(), y, 0.01)
    assert last < 0.5 * first
    m.close(); oracle_lib.reset(mark)


def test_treelstm_untrained_loss_and_learning(oracle_lib):
    from tests.test_gpu_models import _random_tree
    mark = oracle_lib.mark()
    m = _model(oracle_lib, "treelstm", 1)
    assert m.num_params == 22 and m.label_count == 1 + 4 * 99
    y = _random_tree(np.random.default_rng(4), 9)
    x = np.zeros(1, np.float32)
    first = m.step(x, y, 0.05)
    assert abs(first - 17 * np.log(5.0)) < 0.2
    for _ in range(8):
        last = m.step(x, y, 0.05)
    assert last < 0.1 * first
    m.close(); oracle_lib.reset(mark)


def test_treelstm_fused_gates_equal_operator_by_operator(oracle_lib):
    """One fused call per gate (affine_act) against the reference's operator-by-operator form on the oracle: same loss and
    the same 22 gradients up to the order of two float additions per gate."""
    from tests.test_gpu_models import _random_tree
    mark = oracle_lib.mark()
    y = _random_tree(np.random.default_rng(11), 7)
    x = np.zeros(1, np.float32)
    res = []
    for fused in (True, False):
        m = _model(oracle_lib, "treelstm", 1)
        m.use_fused_cells(fused)
        loss = m.step(x, y, 0.0, update=False)
        res.append((loss, [m.grad(i) for i in range(m.num_params)]))
        m.close(); oracle_lib.reset(mark)
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[1][0])
    for a, b in zip(res[0][1], res[1][1]):
        assert np.abs(a - b).max() <= 1e-5 * max(np.abs(b).max(), 1e-12)


@pytest.mark.parametrize("variant", ["treelstm", "treelstm_nips18"])
def test_treelstm_node_call_equals_operator_by_operator(oracle_lib, variant):
    """A whole tree node as one forward and one backward call (tree_node_fwd / tree_node_bwd) against the reference's
    operator-by-operator form, on the oracle, whose node entry points issue that operator sequence: same loss and the same 22
    gradients up to the order of a few float additions (both applications: exchanged roles with clipping, plain cell)."""
    from tests.test_gpu_models import _random_tree
    mark = oracle_lib.mark()
    x = np.zeros(1, np.float32)
    for leaves in (1, 2, 9, 30):
        y = _random_tree(np.random.default_rng(12 + leaves), leaves)
        res = []
        for level in (3, 2, 0):                      # a whole level of the tree per call, a whole node per call, operator by operator
            m = _model(oracle_lib, variant, 1)
            m.use_fused_cells(level)
            loss = m.step(x, y, 0.0, update=False)
            res.append((loss, [m.grad(i) for i in range(m.num_params)]))
            m.close(); oracle_lib.reset(mark)
        for r in res[:2]:
            assert abs(r[0] - res[2][0]) <= 1e-6 * abs(res[2][0]), (leaves, r[0], res[2][0])
            for i, (a, b) in enumerate(zip(r[1], res[2][1])):
                assert np.abs(a - b).max() <= 1e-5 * max(np.abs(b).max(), 1e-12), (leaves, i)


def test_rnn_fused_cell_equals_operator_by_operator(oracle_lib):
    """The recurrent cell and the output layer as one fused call each (affine_act_rows) against the operator-by-operator form."""
    mark = oracle_lib.mark()
    T, V, B = 20, 80, 3
    ids = np.random.default_rng(5).integers(0, V, (T + 1, B))
    x = np.zeros((T, B, V), np.float32)
    x[np.arange(T)[:, None], np.arange(B)[None, :], ids[:T]] = 1.0
    y = ids[1:].astype(np.int32).ravel()
    res = []
    for fused in (True, False):
        m = _model(oracle_lib, "rnn", B)
        m.use_fused_cells(fused)
        loss = m.step(x.ravel(), y, 0.0, update=False)
        res.append((loss, [m.grad(i) for i in range(m.num_params)]))
        m.close(); oracle_lib.reset(mark)
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[1][0])
    for a, b in zip(res[0][1], res[1][1]):
        assert np.abs(a - b).max() <= 2e-5 * max(np.abs(b).max(), 1e-12)


def test_rnn_whole_sequence_call_equals_operator_by_operator(oracle_lib):
    """The whole unrolled sequence as one forward and one backward call (rnn_seq_fwd / rnn_seq_bwd) against the
    operator-by-operator form, on the oracle, whose sequence entry points issue that very operator sequence: loss and the five
    gradients agree to the last bits of a few reordered float additions."""
    mark = oracle_lib.mark()
    T, V, B = 20, 80, 5
    ids = np.random.default_rng(6).integers(0, V, (T + 1, B))
    x = np.zeros((T, B, V), np.float32)
    x[np.arange(T)[:, None], np.arange(B)[None, :], ids[:T]] = 1.0
    y = ids[1:].astype(np.int32).ravel()
    res = []
    for level in (2, 0):
        m = _model(oracle_lib, "rnn", B)
        m.use_fused_cells(level)
        loss = m.step(x.ravel(), y, 0.0, update=False)
        res.append((loss, [m.grad(i) for i in range(m.num_params)]))
        m.close(); oracle_lib.reset(mark)
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[1][0])
    for a, b in zip(res[0][1], res[1][1]):
        assert np.abs(a - b).max() <= 2e-5 * max(np.abs(b).max(), 1e-12)


def test_deferred_zero_fill_is_invisible_on_the_oracle(oracle_lib):
    """The host programs declare large activation gradients unset (grad_unset) instead of taking them zero-filled; the CPU
    restatement keeps the reference's plain rule (it fills such a block with zeros at once), so a SqueezeNet step at batch 16
    (feature maps of 1.5 M floats and more) gives the same loss and the same gradients either way, bit for bit."""
    mark = oracle_lib.mark()
    rng = np.random.default_rng(3)
    x = rng.standard_normal(16 * 3072).astype(np.float32); y = rng.integers(0, 10, 16).astype(np.int32)
    res = []
    for deferred in (True, False):
        m = _model(oracle_lib, "squeezenet", 16)
        m.use_deferred_zero(deferred)
        loss = m.step(x, y, 0.0, update=False)
        res.append((loss, m.slab_grads()))
        m.use_deferred_zero(True)
        m.close(); oracle_lib.reset(mark)
    assert res[0][0] == res[1][0] and np.array_equal(res[0][1], res[1][1])
