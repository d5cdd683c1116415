"""ctypes binding generated from include/lantern_b200.h.

The header is the single source of truth for the C ABI: this module parses its declarations and sets
argtypes/restype for every entry point, so a library that lacks a declared symbol fails at load time.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(_HERE), "include", "lantern_b200.h")

_CTYPES = {
    "int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t, "int64_t": ctypes.c_int64,
    "void": None,
}


def _ctype(decl):
    """Map one C parameter/return declaration (without the name) to a ctypes type."""
    d = decl.replace("const", " ").strip()
    d = re.sub(r"\s+", " ", d).replace(" *", "*").replace("* ", "*")
    if d.endswith("*"):
        return ctypes.c_void_p          # every pointer crosses as a raw address
    if d not in _CTYPES:
        raise ValueError("unsupported C type in header: %r" % decl)
    return _CTYPES[d]


def parse_header(path=HEADER):
    """Return {name: (restype, [(argtype, argname), ...])} for every LTB_FN declaration."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out = {}
    for m in re.finditer(r"([A-Za-z_0-9\s\*]+?)\s*LTB_FN\((\w+)\)\s*\(([^;]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                mm = re.match(r"(.*?)(\w+)$", a)
                params.append((_ctype(mm.group(1)), mm.group(2)))
        out[name] = (_ctype(ret), params)
    return out


def parse_struct(name, path=HEADER):
    """ctypes.Structure mirroring `typedef struct <name> { ... } <name>;` of the header: int fields, and pointers (arrays of
    pointers) that cross as raw addresses."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    m = re.search(r"typedef\s+struct\s+%s\s*\{(.*?)\}\s*%s\s*;" % (name, name), text, flags=re.S)
    if not m:
        raise ValueError("no struct %s in the header" % name)
    fields = []
    for decl in m.group(1).split(";"):
        decl = decl.strip()
        if not decl:
            continue
        mm = re.match(r"(.*?)(\w+)((?:\[\d+\])*)$", decl)
        ctype = _ctype(mm.group(1))
        for dim in reversed(re.findall(r"\[(\d+)\]", mm.group(3))):
            ctype = ctype * int(dim)
        fields.append((mm.group(2), ctype))
    return type(name, (ctypes.Structure,), {"_fields_": fields})


class LanternError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("lantern backend error %d: %s" % (code, msg))
        self.code = code


class BoundLibrary:
    """A loaded backend library (prefix `ltb_` = the CUDA product; tests bind their CPU checker under its own prefix).

    Attribute access gives the entry point without its prefix; integer-returning entry points raise
    LanternError on a negative status (the library is switched to non-fatal mode at load)."""

    _NO_CHECK = {"last_error", "comm_world", "device_status", "kernel_launches", "arena_used"}

    def __init__(self, path, prefix):
        self.path, self.prefix = path, prefix
        self.cdll = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        self.decls = parse_header()
        self._fns = {}
        missing = []
        for name, (ret, params) in self.decls.items():
            try:
                f = getattr(self.cdll, prefix + name)
            except AttributeError:
                missing.append(prefix + name)
                continue
            f.restype = ret
            f.argtypes = [t for t, _ in params]
            self._fns[name] = f
        if missing:
            raise ImportError("%s lacks declared symbols: %s" % (path, ", ".join(missing)))
        self._fns["set_fatal"](0)

    def raw(self, name):
        return self._fns[name]

    def error_message(self):
        buf = ctypes.create_string_buffer(512)
        self._fns["last_error"](buf, 512)
        return buf.value.decode(errors="replace")

    def __getattr__(self, name):
        fns = self.__dict__.get("_fns", {})
        if name not in fns:
            raise AttributeError(name)
        f, ret = fns[name], self.decls[name][0]

        def call(*args):
            args = [a.ptr if hasattr(a, "ptr") else a for a in args]
            r = f(*args)
            if ret is ctypes.c_int and name not in self._NO_CHECK and r < 0:
                raise LanternError(r, self.error_message())
            if ret is ctypes.c_void_p and name in ("malloc", "malloc_uninit") and not r:
                raise LanternError(-3, self.error_message())
            return r
        call.__name__ = name
        return call
