"""Loader for the reference's own CPU engine (`seera_cpp`), compiled unmodified by
`make -C oracle ref` into oracle/_ref/.  Test infrastructure only.

`load()` returns the module or None when it has not been built; callers that need it
skip (tests) or fall back to the C restatement (the benchmark's CPU-baseline leg).
"""
import glob
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_cached = []


def load():
    if _cached:
        return _cached[0]
    mod = None
    hits = sorted(glob.glob(os.path.join(_HERE, "_ref", "seera_cpp*.so")))
    if hits:
        try:
            spec = importlib.util.spec_from_file_location("seera_cpp", hits[0])
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        except Exception:  # wrong ABI or a missing BLAS on this host
            mod = None
    _cached.append(mod)
    return mod


def sgemm_kind():
    """'openblas <file>' or 'naive': which sgemm the engine in oracle/_ref was linked against."""
    try:
        with open(os.path.join(_HERE, "_ref", "SGEMM")) as f:
            return f.read().strip()
    except OSError:
        return "absent"
