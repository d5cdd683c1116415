"""lantern_b200 -- B200-native tensor backend for Lantern's staged programs.

The product is the C-ABI shared library `liblantern_b200.so` (sources under csrc/, declarations in
include/lantern_b200.h).  This package is the Python host-side mirror used by tests, the benchmark
harness and scripting: `load()` binds the library, `Backend` mirrors the reference's Scala `Backend`
trait method by method.  There is no CPU fallback: if the CUDA library is missing, load() raises.
"""
import os

from ._ffi import BoundLibrary, LanternError, parse_header, parse_struct  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblantern_b200.so")
HOSTS_PATH = os.path.join(_HERE, "liblantern_b200_hosts.so")
_lib = None


def load():
    """Bind liblantern_b200.so. Raises ImportError when it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("liblantern_b200.so is not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
        _lib = BoundLibrary(LIB_PATH, "ltb_")
    return _lib


from .backend import Backend, Tensor, TensorR  # noqa: E402,F401
