"""NumPy-facing wrapper over the C restatement of the reference's CPU arithmetic
(oracle/seera_oracle.c).  TEST INFRASTRUCTURE ONLY: imported by tests, by the smoke
check and by the benchmark's CPU-baseline leg, never by the product package.

Function names and argument orders follow the reference's CPU engine bindings
(engine/src/bindings.cpp:14-248) so a check written against `seera_cpp` reads the
same against this module: matmul, relu ... clip_act, softmax, softmax_vjp,
conv2d_forward/backward, maxpool2d_forward/backward, unpooling_forward/backward,
conv_transpose2d_forward/backward.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libseera_oracle.so")
_lib = None

_F = ctypes.POINTER(ctypes.c_float)
_I = ctypes.POINTER(ctypes.c_int32)


def build():
    """Compile seera_oracle.c if the shared object is missing or older than the source."""
    src = os.path.join(_HERE, "seera_oracle.c")
    if (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", _LIB_PATH, src, "-lm"])


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(_F)


def _pi(a):
    return a.ctypes.data_as(_I)


def _cf(x):
    return ctypes.c_float(float(x))


# ---- GEMM -------------------------------------------------------------------
def matmul(A, B):
    A, B = _f(A), _f(B)
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), np.float32)
    lib().so_matmul(_p(A), _p(B), _p(C), M, K, N)
    return C


def matmul_backward(A, B, dC):
    A, B, dC = _f(A), _f(B), _f(dC)
    M, K = A.shape
    N = B.shape[1]
    dA = np.empty_like(A)
    dB = np.empty_like(B)
    lib().so_matmul_bwd(_p(A), _p(B), _p(dC), _p(dA), _p(dB), M, K, N)
    return dA, dB


# ---- unary ------------------------------------------------------------------
def _unary(name):
    def fn(X):
        X = _f(X)
        o = np.empty_like(X)
        g = np.empty_like(X)
        getattr(lib(), name)(_p(X), _p(o), _p(g), X.size)
        return o, g
    return fn


relu = _unary("so_relu")
sigmoid = _unary("so_sigmoid")
tanh_act = _unary("so_tanh")
log_act = _unary("so_log")
exp_act = _unary("so_exp")
abs_act = _unary("so_abs")
sqrt_act = _unary("so_sqrt")


def pow_act(X, e):
    X = _f(X)
    o = np.empty_like(X)
    g = np.empty_like(X)
    lib().so_pow(_p(X), _cf(e), _p(o), _p(g), X.size)
    return o, g


def clip_act(X, lo, hi):
    X = _f(X)
    o = np.empty_like(X)
    g = np.empty_like(X)
    lib().so_clip(_p(X), _cf(lo), _cf(hi), _p(o), _p(g), X.size)
    return o, g


def softmax(X):
    X = _f(X)
    C = X.shape[-1]
    o = np.empty_like(X)
    lib().so_softmax(_p(X), _p(o), X.size // C, C)
    return o


def softmax_vjp(S, dout):
    S, dout = _f(S), _f(dout)
    C = S.shape[-1]
    dx = np.empty_like(S)
    lib().so_softmax_vjp(_p(S), _p(dout), _p(dx), S.size // C, C)
    return dx


# ---- convolution ------------------------------------------------------------
def conv2d_forward(X, W, sh, sw, ph, pw):
    X, W = _f(X), _f(W)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    OH = (H + 2 * ph - KH) // sh + 1
    OW = (Wi + 2 * pw - KW) // sw + 1
    out = np.empty((N, F, OH, OW), np.float32)
    lib().so_conv2d_fwd(_p(X), _p(W), _p(out), N, C, H, Wi, F, KH, KW, sh, sw, ph, pw)
    return out


def conv2d_backward(dout, X, W, sh, sw, ph, pw):
    dout, X, W = _f(dout), _f(X), _f(W)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    dX = np.empty_like(X)
    dW = np.empty_like(W)
    lib().so_conv2d_bwd(_p(dout), _p(X), _p(W), _p(dX), _p(dW), N, C, H, Wi, F, KH, KW, sh, sw, ph, pw)
    return dX, dW


def conv_transpose2d_forward(X, W, sh, sw, ph, pw):
    X, W = _f(X), _f(W)
    N, Cin, H, Wi = X.shape
    _, Cout, KH, KW = W.shape
    Ho = (H - 1) * sh - 2 * ph + KH
    Wo = (Wi - 1) * sw - 2 * pw + KW
    out = np.empty((N, Cout, Ho, Wo), np.float32)
    lib().so_convT_fwd(_p(X), _p(W), _p(out), N, Cin, H, Wi, Cout, KH, KW, sh, sw, ph, pw)
    return out


def conv_transpose2d_backward(dout, X, W, sh, sw, ph, pw):
    dout, X, W = _f(dout), _f(X), _f(W)
    N, Cin, H, Wi = X.shape
    _, Cout, KH, KW = W.shape
    dX = np.empty_like(X)
    dW = np.empty_like(W)
    lib().so_convT_bwd(_p(dout), _p(X), _p(W), _p(dX), _p(dW), N, Cin, H, Wi, Cout, KH, KW, sh, sw, ph, pw)
    return dX, dW


# ---- pooling ----------------------------------------------------------------
def maxpool2d_forward(X, KH, KW, sh, sw, ph, pw):
    X = _f(X)
    N, C, H, W = X.shape
    OH = (H + 2 * ph - KH) // sh + 1
    OW = (W + 2 * pw - KW) // sw + 1
    out = np.empty((N, C, OH, OW), np.float32)
    mask = np.empty((N, C, OH, OW), np.int32)
    lib().so_maxpool_fwd(_p(X), _p(out), _pi(mask), N, C, H, W, KH, KW, sh, sw, ph, pw)
    return out, mask


def maxpool2d_backward(dout, mask, N, C, H, W, KH, KW, sh, sw, ph, pw):
    dout = _f(dout)
    mask = np.ascontiguousarray(mask, dtype=np.int32)
    OH, OW = dout.shape[2], dout.shape[3]
    dX = np.empty((N, C, H, W), np.float32)
    lib().so_maxpool_bwd(_p(dout), _pi(mask), _p(dX), N, C, H, W, OH, OW, KH, KW, sh, sw, ph, pw)
    return dX


def unpooling_forward(X, sh, sw):
    X = _f(X)
    N, C, H, W = X.shape
    out = np.empty((N, C, H * sh, W * sw), np.float32)
    lib().so_unpool_fwd(_p(X), _p(out), N, C, H, W, sh, sw)
    return out


def unpooling_backward(dout, N, C, H, W, sh, sw):
    dout = _f(dout)
    dx = np.empty((N, C, H, W), np.float32)
    lib().so_unpool_bwd(_p(dout), _p(dx), N, C, H, W, sh, sw)
    return dx


# ---- reductions (NumPy semantics on the reference's CPU path) ---------------
def _split(shape, dim):
    dim = dim % len(shape)
    outer = int(np.prod(shape[:dim], dtype=np.int64))
    inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
    return dim, outer, shape[dim], inner


def reduce(A, dim, op):
    """op in {'sum','mean','max','min'}; the axis is removed from the shape."""
    A = _f(A)
    dim, outer, n, inner = _split(A.shape, dim)
    out_shape = tuple(d for i, d in enumerate(A.shape) if i != dim) or (1,)
    out = np.empty(out_shape, np.float32)
    lib().so_reduce(_p(A), _p(out), outer, n, inner, {"sum": 0, "mean": 1, "max": 2, "min": 3}[op])
    return out


def argreduce(A, dim, want_max=True):
    A = _f(A)
    dim, outer, n, inner = _split(A.shape, dim)
    out_shape = tuple(d for i, d in enumerate(A.shape) if i != dim) or (1,)
    out = np.empty(out_shape, np.int32)
    lib().so_argreduce(_p(A), _pi(out), outer, n, inner, 1 if want_max else 0)
    return out


def reduce_backward(dout, in_shape, dim, scale=1.0):
    dout = _f(dout)
    dim, outer, n, inner = _split(tuple(in_shape), dim)
    dA = np.empty(tuple(in_shape), np.float32)
    lib().so_reduce_bwd(_p(dout), _p(dA), outer, n, inner, _cf(scale))
    return dA


# ---- optimizers (in place on w, m, v / vel) ---------------------------------
def adam_scalars(lr, b1, b2, eps, t):
    """The fp32 scalars NumPy forms from Python doubles in Seera.py:1069-1081."""
    f = np.float32
    return dict(lr=f(lr), b1=f(b1), omb1=f(1 - b1), b2=f(b2), omb2=f(1 - b2), eps=f(eps),
                c1=f(1 - b1 ** t), c2=f(1 - b2 ** t))


def adam_step(w, g, m, v, lr, b1, b2, eps, t):
    s = adam_scalars(lr, b1, b2, eps, t)
    for a in (w, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _f(g)
    lib().so_adam(_p(w), _p(g), _p(m), _p(v), w.size, _cf(s["lr"]), _cf(s["b1"]), _cf(s["omb1"]),
                  _cf(s["b2"]), _cf(s["omb2"]), _cf(s["eps"]), _cf(s["c1"]), _cf(s["c2"]))


def sgd_step(w, g, vel, lr, mu):
    for a in (w, vel):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _f(g)
    lib().so_sgd(_p(w), _p(g), _p(vel), w.size, _cf(lr), _cf(mu))


# ---- flat element-wise (engine/src/bindings.cpp:24-40) ------------------------
def add(A, B):
    A, B = _f(A), _f(B)
    o = np.empty_like(A)
    lib().so_add(_p(A), _p(B), _p(o), A.size)
    return o


def mul(A, B):
    A, B = _f(A), _f(B)
    o = np.empty_like(A)
    lib().so_mul(_p(A), _p(B), _p(o), A.size)
    return o


# ---- batch normalisation ---------------------------------------------------------
def batchnorm_forward(X, gamma, beta, running_mean, running_var, momentum, eps, training):
    """Returns (y, x_hat, mean, std_inv); running_mean / running_var (fp32 arrays) are updated in place when training."""
    X = _f(X)
    N, C = X.shape[0], X.shape[1]
    S = int(np.prod(X.shape[2:])) if X.ndim > 2 else 1
    out, xh = np.empty_like(X), np.empty_like(X)
    mean, si = np.empty(C, np.float32), np.empty(C, np.float32)
    assert running_mean.dtype == np.float32 and running_var.dtype == np.float32
    lib().so_batchnorm_fwd(_p(X), _p(_f(gamma)), _p(_f(beta)), _p(running_mean), _p(running_var), _p(out), _p(xh), _p(mean), _p(si),
                           N, C, S, _cf(momentum), _cf(eps), int(bool(training)))
    return out, xh, mean, si


def batchnorm_backward(dout, x_hat, std_inv, gamma):
    dout, x_hat = _f(dout), _f(x_hat)
    N, C = dout.shape[0], dout.shape[1]
    S = int(np.prod(dout.shape[2:])) if dout.ndim > 2 else 1
    dx, dg, db = np.empty_like(dout), np.empty(C, np.float32), np.empty(C, np.float32)
    lib().so_batchnorm_bwd(_p(dout), _p(x_hat), _p(_f(std_inv)), _p(_f(gamma)), _p(dx), _p(dg), _p(db), N, C, S)
    return dx, dg, db
