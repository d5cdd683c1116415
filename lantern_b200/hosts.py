"""Binding of the host programs (lantern_b200/hosts/*.cpp): whole training steps of the reference's apps
issued through the C ABI from C++, the way Lantern's generated code would issue them."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

_SIGS = {
    "model_create": (ctypes.c_void_p, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]),
    "model_destroy": (None, [ctypes.c_void_p]),
    "model_num_params": (ctypes.c_int, [ctypes.c_void_p]),
    "model_param_count": (ctypes.c_int64, [ctypes.c_void_p, ctypes.c_int]),
    "model_param_is_state": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "model_param_ptr": (ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_int]),
    "model_grad_ptr": (ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_int]),
    "model_slab_count": (ctypes.c_int64, [ctypes.c_void_p]),
    "model_slab_params": (ctypes.c_void_p, [ctypes.c_void_p]),
    "model_slab_grads": (ctypes.c_void_p, [ctypes.c_void_p]),
    "model_input_count": (ctypes.c_int64, [ctypes.c_void_p]),
    "model_label_count": (ctypes.c_int64, [ctypes.c_void_p]),
    "model_set_table": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]),
    "model_use_graph": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "model_use_branches": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "model_use_deferred_zero": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "model_use_fused_cells": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "model_set_resident": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "model_step": (ctypes.c_float, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_int]),
    "model_step_async": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float]),
    "model_last_loss": (ctypes.c_float, [ctypes.c_void_p]),
    "model_logits": (ctypes.c_int64, [ctypes.c_void_p, ctypes.c_void_p]),
    "model_submit": (ctypes.c_int64, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float]),
    "model_collect": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_float)]),
    "model_train_epoch": (ctypes.c_int64, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64]),
    "model_save_params": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "model_load_params": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "loader_open_floats": (ctypes.c_void_p, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int64, ctypes.c_float, ctypes.c_float]),
    "loader_open_cifar": (ctypes.c_void_p, [ctypes.c_char_p, ctypes.c_int64]),
    "loader_error": (ctypes.c_char_p, [ctypes.c_void_p]),
    "loader_length": (ctypes.c_int64, [ctypes.c_void_p]),
    "loader_fill": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]),
    "loader_close": (None, [ctypes.c_void_p]),
    "model_trace": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]),
}


class HostPrograms:
    """`lib` is the BoundLibrary the programs compute with; `path`/`prefix` select the matching hosts build."""

    def __init__(self, lib, path=None, prefix="ltbh_"):
        self.lib = lib
        path = path or os.path.join(_HERE, "liblantern_b200_hosts.so")
        if not os.path.exists(path):
            raise ImportError("%s is not built" % path)
        self.cdll = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        self.fn = {}
        for name, (ret, args) in _SIGS.items():
            f = getattr(self.cdll, prefix + name)
            f.restype, f.argtypes = ret, args
            self.fn[name] = f

    def model(self, name, batch, seed=42):
        return Model(self, name, batch, seed)

    def float_loader(self, data_path, target_path, floats_per_sample, mean=0.0, std=1.0):
        """`<name>_train.bin` (raw float32) + `<name>_train_target.bin` (raw int32), samples used as (x - mean) / std."""
        return Loader(self, self.fn["loader_open_floats"](os.fsencode(data_path), os.fsencode(target_path), floats_per_sample, mean, std), floats_per_sample)

    def cifar_loader(self, path, bytes_per_sample=3072):
        """CIFAR binary records: one label byte + `bytes_per_sample` pixel bytes; x = byte / 255."""
        return Loader(self, self.fn["loader_open_cifar"](os.fsencode(path), bytes_per_sample), bytes_per_sample)


class Loader:
    def __init__(self, hp, handle, sample_count):
        self.hp, self.h, self.sample_count = hp, handle, sample_count
        err = hp.fn["loader_error"](handle).decode()
        if err:
            hp.fn["loader_close"](handle)
            self.h = None
            raise OSError(err)
        self.length = hp.fn["loader_length"](handle)

    def batch(self, index, batch):
        x = np.empty(batch * self.sample_count, dtype=np.float32)
        y = np.empty(batch, dtype=np.int32)
        if self.hp.fn["loader_fill"](self.h, index, batch, x.ctypes.data, y.ctypes.data):
            raise IndexError("batch %d of %d samples is outside the file" % (index, batch))
        return x, y

    def close(self):
        if self.h:
            self.hp.fn["loader_close"](self.h)
            self.h = None


class Model:
    def __init__(self, hp, name, batch, seed):
        self.hp, self.lib, self.name, self.batch = hp, hp.lib, name, batch
        self.h = hp.fn["model_create"](name.encode(), batch, seed)
        if not self.h:
            raise ValueError("unknown model %r" % name)
        self.num_params = hp.fn["model_num_params"](self.h)
        self.input_count = hp.fn["model_input_count"](self.h)
        self.label_count = hp.fn["model_label_count"](self.h)
        self.slab_count = hp.fn["model_slab_count"](self.h)

    def _arrs(self, x, y):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.ascontiguousarray(y, dtype=np.int32)
        assert x.size == self.input_count and y.size == self.label_count
        return x, y

    def step(self, x, y, lr, update=True):
        x, y = self._arrs(x, y)
        return float(self.hp.fn["model_step"](self.h, x.ctypes.data, y.ctypes.data, lr, int(update)))

    def step_async(self, x, y, lr):
        x, y = self._arrs(x, y)
        rc = self.hp.fn["model_step_async"](self.h, x.ctypes.data, y.ctypes.data, lr)
        if rc:
            raise RuntimeError("model_step_async failed: %d %s" % (rc, self.lib.error_message()))

    def submit(self, x, y, lr):
        """Queue one training step on host arrays and return its number without waiting (two steps stay in flight)."""
        x, y = self._arrs(x, y)
        k = self.hp.fn["model_submit"](self.h, x.ctypes.data, y.ctypes.data, lr)
        if k < 0:
            raise RuntimeError("model_submit failed: %s" % self.lib.error_message())
        return k

    def collect(self, step):
        """Wait for step `step` (one of the last two submitted) and return its loss."""
        out = ctypes.c_float()
        rc = self.hp.fn["model_collect"](self.h, step, ctypes.byref(out))
        if rc:
            raise RuntimeError("model_collect(%d) failed: %d %s" % (step, rc, self.lib.error_message()))
        return float(out.value)

    def train_epoch(self, loader, lr, max_batches=0):
        """One pass over `loader` with two steps in flight; returns the per-batch losses."""
        n = loader.length // self.batch
        if max_batches > 0:
            n = min(n, max_batches)
        losses = np.zeros(max(n, 1), dtype=np.float32)
        rc = self.hp.fn["model_train_epoch"](self.h, loader.h, lr, losses.ctypes.data, max_batches)
        if rc < 0:
            raise RuntimeError("model_train_epoch failed: %d %s" % (rc, self.lib.error_message()))
        return losses[:rc]

    def save_params(self, path):
        if self.hp.fn["model_save_params"](self.h, os.fsencode(path)):
            raise OSError("cannot write %s" % path)

    def load_params(self, path):
        if self.hp.fn["model_load_params"](self.h, os.fsencode(path)):
            raise ValueError("%s is not a parameter file of this model" % path)

    def last_loss(self):
        return float(self.hp.fn["model_last_loss"](self.h))

    def logits(self):
        """The classifier's output of the last step as [batch, classes] (CNN programs); predictions are its arg-max per row."""
        out = np.empty(self.batch * 10, dtype=np.float32)
        n = self.hp.fn["model_logits"](self.h, out.ctypes.data)
        if n != out.size:
            raise ValueError("this program keeps no classifier output")
        return out.reshape(self.batch, 10)

    def set_resident(self, x=None, y=None):
        """Keep one batch in device memory (steps then upload nothing); None switches back to per-step uploads."""
        if x is None:
            self.hp.fn["model_set_resident"](self.h, None, None)
            return
        x, y = self._arrs(x, y)
        self.hp.fn["model_set_resident"](self.h, x.ctypes.data, y.ctypes.data)

    def trace(self, x, y):
        """Debug: one row per operator output of one step without update, in forward order: (index, count, shape, sum|x|,
        sum|d|, non-zeros of x, of d, smallest non-zero |x|, sum x^2, sum d^2, eight signed sums of x, eight of d)."""
        x, y = self._arrs(x, y)
        buf = ctypes.create_string_buffer(1 << 22)
        self.hp.fn["model_trace"](self.h, x.ctypes.data, y.ctypes.data, buf, 1 << 22)
        rows = []
        for line in buf.value.decode().strip().split("\n"):
            p = line.split()
            rows.append((int(p[0]), int(p[1]), p[2], float(p[3]), float(p[4])) + tuple(float(v) for v in p[5:]))
        return rows

    @staticmethod
    def trace_distance(rows_a, rows_b):
        """Per operator output, the estimated relative L2 distance of value and gradient between two traces of the same
        program (from the signed sums: the mean of their squared differences estimates |a - b|^2): [(index, shape, ex, ed)]."""
        out = []
        for a, b in zip(rows_a, rows_b):
            assert a[:3] == b[:3], (a[:3], b[:3])
            xa, xb, da, db = np.array(a[10:18]), np.array(b[10:18]), np.array(a[18:26]), np.array(b[18:26])
            ex = float(np.sqrt(np.mean((xa - xb) ** 2) / max(a[8], 1e-300)))
            ed = float(np.sqrt(np.mean((da - db) ** 2) / max(a[9], 1e-300))) if a[9] > 0 else 0.0
            out.append((a[0], a[2], ex, ed))
        return out

    def set_table(self, table):
        """TreeLSTM: replace the embedding table by `table` (rows x 300 float32)."""
        t = np.ascontiguousarray(table, dtype=np.float32)
        rc = self.hp.fn["model_set_table"](self.h, t.ctypes.data, t.shape[0])
        if rc:
            raise ValueError("model_set_table failed: %d" % rc)

    def use_fused_cells(self, on=3):
        """Recursive models: 0 one call per operator, as the reference stages them; 1 one fused call per gate or cell; 2 in
        addition the vanilla RNN's whole unrolled sequence and a whole tree-LSTM node in one call; 3 (the default) a whole
        LEVEL of the tree in one call."""
        self.hp.fn["model_use_fused_cells"](self.h, int(on))

    def use_branches(self, on=True):
        """Issue independent runs of calls (shortcut convolutions) as branch regions (default) or all in program order."""
        self.hp.fn["model_use_branches"](self.h, int(on))

    def use_deferred_zero(self, on=True):
        """Large activation gradients are declared unset instead of zero-filled (default); off: every gradient buffer is zeroed
        when it is allocated, as the reference does.  Applies to every model of this library instance, from the next step on."""
        self.hp.fn["model_use_deferred_zero"](self.h, int(on))

    def use_graph(self, on=True):
        self.hp.fn["model_use_graph"](self.h, int(on))

    def _read(self, ptr, n):
        out = np.empty(n, dtype=np.float32)
        self.lib.d2h(out.ctypes.data, ptr, out.nbytes)
        return out

    def param(self, i):
        return self._read(self.hp.fn["model_param_ptr"](self.h, i), self.hp.fn["model_param_count"](self.h, i))

    def grad(self, i):
        return self._read(self.hp.fn["model_grad_ptr"](self.h, i), self.hp.fn["model_param_count"](self.h, i))

    def param_is_state(self, i):
        """True for a batch-norm running statistic: updated by each replica from its own batches, never trained or all-reduced."""
        return bool(self.hp.fn["model_param_is_state"](self.h, i))

    def trained_params(self):
        """Every trained parameter tensor (the running statistics left out), concatenated."""
        return np.concatenate([self.param(i) for i in range(self.num_params) if not self.param_is_state(i)])

    def slab_params(self):
        return self._read(self.hp.fn["model_slab_params"](self.h), self.slab_count)

    def slab_grads(self):
        return self._read(self.hp.fn["model_slab_grads"](self.h), self.slab_count)

    def slab_ptrs(self):
        return self.hp.fn["model_slab_params"](self.h), self.hp.fn["model_slab_grads"](self.h)

    def set_slab_params(self, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        assert arr.size == self.slab_count
        self.lib.h2d(self.hp.fn["model_slab_params"](self.h), arr.ctypes.data, arr.nbytes)

    def close(self):
        if self.h:
            self.hp.fn["model_destroy"](self.h)
            self.h = None
