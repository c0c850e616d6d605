"""Builds the engine in-tree for sm_100a:

  ml_framework_b200/libseera_b200.so         the C ABI (include/seera_b200.h): CUDA kernels + runtime
  ml_framework_b200/seera_cuda<EXT_SUFFIX>   the pybind11 shim module over it

    python -m ml_framework_b200.build [--force] [-v]

nvcc cross-compiles without a GPU.  Objects are cached under ml_framework_b200/build/ and
rebuilt when their source (or a header) is newer.
"""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libseera_b200.so")
EXT = os.path.join(PKG, "seera_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build(force=False, verbose=False, ptxas_info=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    jobs, objs = [], []
    for src in cus:
        o = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [src] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", o])
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    if force or jobs or _newer(LIB, objs):
        _run([NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"], verbose)
    shim = os.path.join(CSRC, "seera_cuda_module.cpp")
    if force or _newer(EXT, [shim, LIB] + headers):
        import pybind11
        _run(["g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-fvisibility=hidden",
              "-I" + os.path.join(ROOT, "include"), "-I" + pybind11.get_include(),
              "-I" + sysconfig.get_paths()["include"], shim, "-o", EXT,
              "-L" + PKG, "-lseera_b200", "-Wl,-rpath,$ORIGIN"], verbose)
    return LIB, EXT


if __name__ == "__main__":
    lib, ext = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print("built", lib)
    print("built", ext)
