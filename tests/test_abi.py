"""CPU-only checks of the boundary: the product library loads without a GPU, exports every symbol the header
declares, refuses to initialise without a device (no CPU fallback), and the oracle exports the same ABI."""
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_declares_the_hot_path():
    from lantern_b200 import parse_header
    decls = parse_header()
    for name in ("init", "malloc", "reset", "gemm", "gemm_grad", "conv2d_fwd", "conv2d_bwd", "maxpool_fwd", "bn_train_fwd",
                 "bn_bwd", "ew_binary", "unary", "log_softmax", "nll", "sum", "mean", "concat", "dropout", "sgd_step",
                 "adagrad_update", "momentum_update", "allreduce_sgd_step"):
        assert name in decls, name
    assert len(decls) >= 80


def test_product_library_exports_every_declared_symbol():
    import lantern_b200
    lib = lantern_b200.load()          # raises ImportError listing any missing symbol
    assert set(lib.decls) == set(lib._fns)


def test_oracle_exports_the_same_abi(oracle_lib):
    assert set(oracle_lib.decls) == set(oracle_lib._fns)


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present; the refusal path is exercised on CPU-only machines")
    import lantern_b200
    lib = lantern_b200.load()
    with pytest.raises(lantern_b200.LanternError) as e:
        lib.init(0, 1 << 20)
    assert "no CUDA device" in str(e.value) or "CUDA" in str(e.value)
    with pytest.raises(lantern_b200.LanternError):
        lib.fill(0, 1.0, 4)            # every op refuses before init


def test_product_sources_never_reference_the_oracle():
    bad = []
    for base in ("lantern_b200", "include"):
        for dp, _, fs in os.walk(os.path.join(ROOT, base)):
            if "build" in dp.split(os.sep):
                continue
            for f in fs:
                if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                    text = open(os.path.join(dp, f), errors="replace").read()
                    if "liblantern_oracle" in text or "ora_" in text.replace("ora_##", ""):
                        bad.append(os.path.join(dp, f))
    # the header documents the oracle prefix in a comment; nothing else may mention it
    assert [b for b in bad if not b.endswith("lantern_b200.h")] == []


def test_ctypes_mirror_of_the_tree_node_struct_has_the_c_layout(tmp_path):
    """`parse_struct` builds the ctypes mirror of `ltb_tree_node` from the header text; a C program compiled against the same
    header must report the same size and the same offset for every field."""
    import ctypes
    import subprocess
    from lantern_b200 import parse_struct
    node = parse_struct("ltb_tree_node")
    names = [n for n, _ in node._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "lantern_b200.h"\nint main(void) {\n  printf("%zu\\n", sizeof(ltb_tree_node));\n'
                   + "".join('  printf("%%zu\\n", offsetof(ltb_tree_node, %s));\n' % n for n in names) + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    assert got[0] == ctypes.sizeof(node)
    assert got[1:] == [getattr(node, n).offset for n in names]
