"""B200-native engine for the Seera training hot path.

  ml_framework_b200.seera_cuda   pybind11 module with the reference binding's 60 function names
  ml_framework_b200.cuTen        the raw-pointer device tensor (`cuten`) the reference's Python layer uses
  ml_framework_b200.seera        Sequential / layers / Loss / SGD / Adam / autograd on top of the engine
  ml_framework_b200.capi         ctypes view of the C ABI (include/seera_b200.h)
  ml_framework_b200.workloads    the seeded synthetic training configurations

Importing the compute modules without the compiled CUDA library raises: there is no CPU fallback.
`install_dropin()` registers `seera_cuda` and `cuTen` under their top-level names, which is what
the reference's `Seera.py`, `Seera_init.py` and `Seera_Engine.py` import.
"""
import importlib
import sys


def install_dropin():
    sc = importlib.import_module("ml_framework_b200.seera_cuda")
    sys.modules.setdefault("seera_cuda", sc)
    ct = importlib.import_module("ml_framework_b200.cuTen")
    sys.modules.setdefault("cuTen", ct)
    return sc, ct
