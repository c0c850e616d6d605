"""NumPy-in / NumPy-out calls into the device engine through the C ABI.

Function names and argument orders are those of the reference's CPU engine binding
(engine/src/bindings.cpp:14-248: matmul, relu, ..., conv2d_forward, conv2d_backward,
maxpool2d_forward, ...), so the parity tests read like calls into `seera_cpp`
with host arrays: each call uploads its operands, enqueues the device kernels of
include/seera_b200.h, and downloads the result.  Meant for checks and small experiments;
training keeps tensors resident (see ml_framework_b200.seera).
"""
import ctypes

import numpy as np

from ml_framework_b200 import capi


class _Dev:
    """Device buffers owned for the duration of one call."""

    def __init__(self):
        self.L = capi.load()
        capi.check(self.L.seera_init(capi.default_device()))
        self.bufs = []

    def up(self, a, dtype=np.float32):
        a = np.ascontiguousarray(a, dtype=dtype)
        p = self.L.seera_to_device(a.ctypes.data_as(ctypes.c_void_p), a.nbytes)
        if not p:
            raise capi.SeeraError(self.L.seera_last_error().decode())
        self.bufs.append(p)
        return p

    def new(self, n_elems, itemsize=4):
        p = self.L.seera_cuda_malloc(max(1, int(n_elems)) * itemsize)
        if not p:
            raise capi.SeeraError(self.L.seera_last_error().decode())
        self.bufs.append(p)
        return p

    def down(self, p, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        if out.size:
            capi.check(self.L.seera_to_host(out.ctypes.data_as(ctypes.c_void_p), p, out.nbytes))
        return out

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for p in self.bufs:
            self.L.seera_cuda_free(p)
        return False


def _cf(x):
    return ctypes.c_float(float(x))


def matmul(A, B):
    A = np.asarray(A, np.float32)
    B = np.asarray(B, np.float32)
    nb = A.shape[0] if A.ndim == 3 else 1
    M, K = A.shape[-2:]
    N = B.shape[1]
    with _Dev() as d:
        c = d.new(nb * M * N)
        capi.check(d.L.seera_cuda_matmul(d.up(A), d.up(B), c, M, N, K, nb))
        return d.down(c, (M, N) if A.ndim == 2 else (nb, M, N))


def matmul_backward(A, B, dC):
    A = np.asarray(A, np.float32)
    nb = A.shape[0] if A.ndim == 3 else 1
    M, K = A.shape[-2:]
    N = np.asarray(B).shape[1]
    with _Dev() as d:
        da, db = d.new(A.size), d.new(K * N)
        capi.check(d.L.seera_cuda_matmul_bwd(d.up(A), d.up(B), d.up(dC), da, db, M, N, K, nb))
        return d.down(da, A.shape), d.down(db, (K, N))


def _unary(sym):
    def fn(X, *scalars):
        X = np.asarray(X, np.float32)
        with _Dev() as d:
            o, g = d.new(X.size), d.new(X.size)
            f = getattr(d.L, sym)
            if sym == "seera_cuda_pow_fwd":
                capi.check(f(d.up(X), _cf(scalars[0]), o, g, X.size))
            elif sym == "seera_cuda_clip_fwd":
                capi.check(f(d.up(X), _cf(scalars[0]), _cf(scalars[1]), o, g, X.size))
            else:
                capi.check(f(d.up(X), o, g, X.size))
            return d.down(o, X.shape), d.down(g, X.shape)
    return fn


relu = _unary("seera_cuda_relu_fwd")
sigmoid = _unary("seera_cuda_sigmoid_fwd")
tanh_act = _unary("seera_cuda_tanh_fwd")
log_act = _unary("seera_cuda_log_fwd")
exp_act = _unary("seera_cuda_exp_fwd")
abs_act = _unary("seera_cuda_abs_fwd")
sqrt_act = _unary("seera_cuda_sqrt_fwd")
pow_act = _unary("seera_cuda_pow_fwd")
clip_act = _unary("seera_cuda_clip_fwd")


def _binary(sym):
    def fn(A, B):
        A = np.asarray(A, np.float32)
        with _Dev() as d:
            c = d.new(A.size)
            capi.check(getattr(d.L, sym)(d.up(A), d.up(B), c, A.size))
            return d.down(c, A.shape)
    return fn


add = _binary("seera_cuda_elemadd_gputogpu")
mul = _binary("seera_cuda_elemmult_gputogpu")
sub = _binary("seera_cuda_elemsub_gputogpu")
div = _binary("seera_cuda_elemdiv_gputogpu")


def softmax(X):
    X = np.asarray(X, np.float32)
    C = X.shape[-1]
    with _Dev() as d:
        o = d.new(X.size)
        capi.check(d.L.seera_cuda_softmax_fwd(d.up(X), o, X.size // C, C))
        return d.down(o, X.shape)


def softmax_vjp(S, dout):
    S = np.asarray(S, np.float32)
    C = S.shape[-1]
    with _Dev() as d:
        o = d.new(S.size)
        capi.check(d.L.seera_cuda_softmax_vjp(d.up(S), d.up(dout), o, S.size // C, C))
        return d.down(o, S.shape)


def conv2d_forward(X, W, sh, sw, ph, pw):
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    OH, OW = (H + 2 * ph - KH) // sh + 1, (Wi + 2 * pw - KW) // sw + 1
    with _Dev() as d:
        o = d.new(N * F * OH * OW)
        capi.check(d.L.seera_cuda_conv2d_fwd(d.up(X), d.up(W), o, N, C, H, Wi, F, KH, KW, ph, pw, sh, sw))
        return d.down(o, (N, F, OH, OW))


def conv2d_bias_act(X, W, bias, sh, sw, ph, pw, act):
    """act(conv2d(X, W) + bias[f]) in one call; bias may be None, act is a SEERA_ACT_* code."""
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    OH, OW = (H + 2 * ph - KH) // sh + 1, (Wi + 2 * pw - KW) // sw + 1
    with _Dev() as d:
        o = d.new(N * F * OH * OW)
        b = d.up(np.asarray(bias, np.float32).ravel()) if bias is not None else None
        capi.check(d.L.seera_conv2d_bias_act_fwd(d.up(X), d.up(W), b, o, N, C, H, Wi, F, KH, KW, ph, pw, sh, sw, act))
        return d.down(o, (N, F, OH, OW))


def conv2d_layer_roundtrip(X, W, bias, sh, sw, ph, pw, act, g=None, gp=None, need_dx=True, keep=True, pass_pooled=True):
    """Forward y = act(conv2d(X, W) + bias) with the input's copies kept, then seera_conv2d_act_bwd from g (gradient of
    y) or gp (gradient of maxpool2x2(y); the pool runs here to get its mask).  Returns y, pooled, dX, dW, dbias."""
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    OH, OW = (H + 2 * ph - KH) // sh + 1, (Wi + 2 * pw - KW) // sw + 1
    with _Dev() as d:
        L = d.L
        xd, wd, bd = d.up(X), d.up(W), d.up(np.asarray(bias, np.float32).ravel())
        y = d.new(N * F * OH * OW)
        kept = ctypes.c_void_p()
        capi.check(L.seera_conv2d_bias_act_fwd_s(xd, wd, bd, y, N, C, H, Wi, F, KH, KW, ph, pw, sh, sw, act, None,
                                                 ctypes.byref(kept) if keep else None))
        pooled = mask = None
        if gp is not None:
            pooled, mask = d.new(N * F * (OH // 2) * (OW // 2)), d.new(N * F * OH * OW)
            capi.check(L.seera_cuda_maxpool_fwd(y, pooled, mask, N, F, OH, OW, 2, 2, 0, 0, 2, 2))
        dx = d.new(X.size) if need_dx else None
        dw, db = d.new(W.size), d.new(F)
        try:
            capi.check(L.seera_conv2d_act_bwd(wd, xd, y, d.up(g) if g is not None else None, d.up(gp) if gp is not None else None,
                                              mask, pooled if pass_pooled else None, dx, dw, db, N, C, H, Wi, F, KH, KW, sh, sw,
                                              ph, pw, act, kept))
        finally:
            L.seera_shadow_free(kept)
        return (d.down(y, (N, F, OH, OW)), d.down(pooled, (N, F, OH // 2, OW // 2)) if gp is not None else None,
                d.down(dx, X.shape) if need_dx else None, d.down(dw, W.shape), d.down(db, (F,)))


def conv_transpose2d_bias_act(X, W, bias, sh, sw, ph, pw, act):
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, Ci, H, Wi = X.shape
    _, Co, KH, KW = W.shape
    Ho, Wo = (H - 1) * sh - 2 * ph + KH, (Wi - 1) * sw - 2 * pw + KW
    with _Dev() as d:
        o = d.new(N * Co * Ho * Wo)
        b = d.up(np.asarray(bias, np.float32).ravel()) if bias is not None else None
        capi.check(d.L.seera_conv2DTranspose_bias_act_fwd(d.up(X), d.up(W), b, o, N, Ci, H, Wi, Co, KH, KW, sh, sw, ph, pw, act))
        return d.down(o, (N, Co, Ho, Wo))


def matmul_bias_act(A, B, bias, act):
    A, B = np.asarray(A, np.float32), np.asarray(B, np.float32)
    M, K = A.shape
    N = B.shape[1]
    with _Dev() as d:
        o = d.new(M * N)
        b = d.up(np.asarray(bias, np.float32).ravel()) if bias is not None else None
        capi.check(d.L.seera_matmul_bias_act_fwd(d.up(A), d.up(B), b, o, M, N, K, act))
        return d.down(o, (M, N))


def conv2d_backward(dout, X, W, sh, sw, ph, pw):
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, C, H, Wi = X.shape
    F, _, KH, KW = W.shape
    with _Dev() as d:
        dx, dw = d.new(X.size), d.new(W.size)
        capi.check(d.L.seera_cuda_conv2d_bwd(d.up(W), d.up(X), d.up(dout), dx, dw, N, C, H, Wi, F, KH, KW, sh, sw, ph, pw))
        return d.down(dx, X.shape), d.down(dw, W.shape)


def conv_transpose2d_forward(X, W, sh, sw, ph, pw):
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, Cin, H, Wi = X.shape
    _, Cout, KH, KW = W.shape
    Ho, Wo = (H - 1) * sh - 2 * ph + KH, (Wi - 1) * sw - 2 * pw + KW
    with _Dev() as d:
        o = d.new(N * Cout * Ho * Wo)
        capi.check(d.L.seera_cuda_conv2DTranpose_fwd(d.up(X), d.up(W), o, N, Cin, H, Wi, Cout, KH, KW, sh, sw, ph, pw))
        return d.down(o, (N, Cout, Ho, Wo))


def conv_transpose2d_backward(dout, X, W, sh, sw, ph, pw):
    X, W = np.asarray(X, np.float32), np.asarray(W, np.float32)
    N, Cin, H, Wi = X.shape
    _, Cout, KH, KW = W.shape
    with _Dev() as d:
        dx, dw = d.new(X.size), d.new(W.size)
        capi.check(d.L.seera_cuda_conv2DTranspose_bwd(d.up(W), d.up(X), d.up(dout), dx, dw, N, Cin, H, Wi, Cout, KH, KW,
                                                      sh, sw, ph, pw))
        return d.down(dx, X.shape), d.down(dw, W.shape)


def maxpool2d_forward(X, KH, KW, sh, sw, ph, pw):
    X = np.asarray(X, np.float32)
    N, C, H, W = X.shape
    OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
    with _Dev() as d:
        o, m = d.new(N * C * OH * OW), d.new(X.size)          # mask buffer sized like the input, as the caller of the reference does
        capi.check(d.L.seera_cuda_maxpool_fwd(d.up(X), o, m, N, C, H, W, KH, KW, ph, pw, sh, sw))
        return d.down(o, (N, C, OH, OW)), d.down(m, (N, C, OH, OW), np.int32)


def maxpool2d_backward(dout, mask, N, C, H, W, KH, KW, sh, sw, ph, pw):
    with _Dev() as d:
        dx = d.new(N * C * H * W)
        mk = np.zeros(N * C * H * W, np.int32)
        mk[:np.asarray(mask).size] = np.asarray(mask, np.int32).ravel()
        capi.check(d.L.seera_cuda_maxpool_bwd(d.up(dout), d.up(mk, np.int32), dx, N, C, H, W, KH, KW, ph, pw, sh, sw))
        return d.down(dx, (N, C, H, W))


def unpooling_forward(X, sh, sw):
    X = np.asarray(X, np.float32)
    N, C, H, W = X.shape
    with _Dev() as d:
        o = d.new(X.size * sh * sw)
        capi.check(d.L.seera_cuda_unpooling_fwd(d.up(X), o, N, C, H, W, sh, sw))
        return d.down(o, (N, C, H * sh, W * sw))


def unpooling_backward(dout, N, C, H, W, sh, sw):
    with _Dev() as d:
        o = d.new(N * C * H * W)
        capi.check(d.L.seera_cuda_unpooling_bwd(d.up(dout), o, N, C, H, W, sh, sw))
        return d.down(o, (N, C, H, W))


def reduce(A, dim, op):
    A = np.asarray(A, np.float32)
    dim = dim % A.ndim
    shp = tuple(s for i, s in enumerate(A.shape) if i != dim) or (1,)
    da = np.array(A.shape, np.int32)
    with _Dev() as d:
        o = d.new(int(np.prod(shp)))
        f = getattr(d.L, "seera_cuda_%s_fwd" % op)
        capi.check(f(d.up(A), o, A.ndim, dim, da.ctypes.data_as(ctypes.c_void_p)))
        return d.down(o, shp, np.int32 if op.startswith("arg") else np.float32)


def reduce_backward(dout, in_shape, dim, op, fwd_in=None, fwd_out=None):
    in_shape = tuple(in_shape)
    dim = dim % len(in_shape)
    da = np.array(in_shape, np.int32)
    n = int(np.prod(in_shape))
    with _Dev() as d:
        o = d.new(n)
        dap = da.ctypes.data_as(ctypes.c_void_p)
        if op in ("sum", "mean"):
            capi.check(getattr(d.L, "seera_cuda_%s_bwd" % op)(d.up(dout), o, len(in_shape), dim, dap))
        else:
            capi.check(d.L.seera_cuda_memset(o, 0, n * 4))
            capi.check(getattr(d.L, "seera_cuda_%s_bwd" % op)(d.up(dout), d.up(fwd_in), d.up(fwd_out), o, len(in_shape), dim, dap))
        return d.down(o, in_shape)
