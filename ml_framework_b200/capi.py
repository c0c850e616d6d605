"""ctypes view of the C ABI declared in include/seera_b200.h.

The signatures are read from the header itself, so the Python side cannot drift from the
declarations: `declared_functions()` lists (name, return type, argument types) and `load()`
binds every one of them on libseera_b200.so, raising if the library or a symbol is missing.
There is no fallback: without the compiled CUDA library nothing here computes.
"""
import ctypes
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(PKG), "include", "seera_b200.h")
LIB_PATH = os.path.join(PKG, "libseera_b200.so")

_CT = {
    "int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t, "uint64_t": ctypes.c_uint64,
    "long long": ctypes.c_longlong, "void": None,
}


def _ctype(t):
    t = t.replace("const", "").strip()
    if t.endswith("*"):
        return ctypes.c_char_p if t.replace(" ", "") == "char*" else ctypes.c_void_p
    return _CT[t]


def declared_functions(header=HEADER):
    src = open(header).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(seera_\w+)\s*\(([^)]*)\)\s*;", src):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        argt = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                # drop the parameter name: the type is everything up to the last identifier
                mm = re.match(r"(.*?[\*\s])(\w+)$", a)
                argt.append((mm.group(1) if mm else a).strip())
        out.append((name, ret, argt))
    return out


_lib = None


def load():
    """Bind the library; raises OSError / AttributeError when it or a declared symbol is absent."""
    global _lib
    if _lib is not None:
        return _lib
    lib = ctypes.CDLL(LIB_PATH)
    for name, ret, argt in declared_functions():
        fn = getattr(lib, name)
        fn.restype = _ctype(ret)
        fn.argtypes = [_ctype(a) for a in argt]
    _lib = lib
    return lib


def default_device():
    """Device index for this process: SEERA_DEVICE, else LOCAL_RANK (one process per GPU), else 0."""
    return int(os.environ.get("SEERA_DEVICE", os.environ.get("LOCAL_RANK", "0")))


class SeeraError(RuntimeError):
    pass


def check(status):
    if status:
        raise SeeraError(load().seera_last_error().decode())
    return status
