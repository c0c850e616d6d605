"""A host-memory stand-in for the `seera_cuda` binding, FOR CPU TESTS OF THE PYTHON HOST LOGIC ONLY.

It lets the tensor class, the layer-level autograd and the optimizers run in a container without a
GPU: "device addresses" are integers into a table of NumPy buffers (byte arithmetic on addresses
works, as callers do it), and every entry computes with the CPU oracle or NumPy.  The product never
imports this file; tests install it as `ml_framework_b200.seera_cuda` before importing the package's
Python modules.
"""
import bisect

import numpy as np

from oracle import cpu_oracle as co

_bases = []          # sorted base addresses
_bufs = {}           # base -> np.uint8 buffer
_next = [1 << 20]
CALLS = {}
LIVE = set()


def _count(name):
    CALLS[name] = CALLS.get(name, 0) + 1


def reset():
    _bases.clear(); _bufs.clear(); CALLS.clear(); LIVE.clear(); _next[0] = 1 << 20


def _alloc(nbytes):
    nbytes = max(int(nbytes), 1)
    p = _next[0]
    _next[0] += (nbytes + 511) // 512 * 512 + 512
    bisect.insort(_bases, p)
    _bufs[p] = np.zeros(nbytes, np.uint8)
    LIVE.add(p)
    return p


def _view(ptr, n, dtype=np.float32):
    i = bisect.bisect_right(_bases, ptr) - 1
    assert i >= 0, "bad device address %r" % ptr
    base = _bases[i]
    buf = _bufs[base]
    off = ptr - base
    nbytes = int(n) * np.dtype(dtype).itemsize
    assert base in LIVE, "use after free at %r" % ptr
    assert off + nbytes <= buf.size, "out-of-bounds device access: %d + %d > %d" % (off, nbytes, buf.size)
    return buf[off:off + nbytes].view(dtype)


def F(ptr, shape):
    return _view(ptr, int(np.prod(shape)), np.float32).reshape(shape)


# ---- memory / transfers ---------------------------------------------------------------------
def cuda_malloc(n): _count("cuda_malloc"); return _alloc(n)
def cuda_malloc_f16(n): _count("cuda_malloc"); return _alloc(n * 4)
def cuda_malloc_f32(n): _count("cuda_malloc"); return _alloc(n * 4)
def cuda_malloc_i32(n): _count("cuda_malloc"); return _alloc(n * 4)
def cuda_malloc_i16(n): _count("cuda_malloc"); return _alloc(n * 2)


def cuda_free(p):
    _count("cuda_free")
    assert p in LIVE, "free of a non-live block %r" % p
    LIVE.discard(p)


def cuda_memcopy_devicetodevice(d, s, n): _count("d2d"); _view(d, n)[:] = _view(s, n)
def cuda_memset(p, v, nbytes): _count("memset"); _view(p, nbytes, np.uint8)[:] = v


def _to_dev(a, dt):
    _count("to_device")
    a = np.ascontiguousarray(a, dtype=dt)
    p = _alloc(a.nbytes)
    _view(p, a.size, dt)[:] = a.ravel()
    return p


def to_device_f32(a): return _to_dev(a, np.float32)
to_device_f16 = to_device_f32
def to_device_i32(a): return _to_dev(a, np.int32)
def to_device_i16(a): return _to_dev(a, np.int16)
def to_host_f32(p, shape): _count("to_host"); return _view(p, int(np.prod(shape)), np.float32).reshape(shape).copy()
to_host_f16 = to_host_f32
def to_host_i32(p, shape): _count("to_host"); return _view(p, int(np.prod(shape)), np.int32).reshape(shape).copy()
def to_host_i16(p, shape): _count("to_host"); return _view(p, int(np.prod(shape)), np.int16).reshape(shape).copy()
def upload_f32(dst, a): a = np.ascontiguousarray(a, np.float32); _view(dst, a.size)[:] = a.ravel()


# ---- unary ---------------------------------------------------------------------------------------
def _unary(fn):
    def k(x, *rest):
        _count("unary")
        *sc, o, g, n = rest
        out, grad = fn(_view(x, n).copy(), *sc)
        _view(o, n)[:] = out
        _view(g, n)[:] = grad
    return k


cuda_relu_fwd = _unary(co.relu)
cuda_sigmoid_fwd = _unary(co.sigmoid)
cuda_tanh_fwd = _unary(co.tanh_act)
cuda_log_fwd = _unary(co.log_act)
cuda_exp_fwd = _unary(co.exp_act)
cuda_abs_fwd = _unary(co.abs_act)
cuda_sqrt_fwd = _unary(co.sqrt_act)
cuda_pow_fwd = _unary(co.pow_act)
cuda_clip_fwd = _unary(co.clip_act)


def cuda_softmax_fwd(x, o, N, C): _count("softmax"); F(o, (N, C))[:] = co.softmax(F(x, (N, C)))
def cuda_softmax_vjp(s, d, dx, N, C): _count("softmax_vjp"); F(dx, (N, C))[:] = co.softmax_vjp(F(s, (N, C)), F(d, (N, C)))


# ---- GEMM ------------------------------------------------------------------------------------------
def cuda_matmul(A, B, C, M, N, K, nb):
    _count("matmul")
    F(C, (nb * M, N))[:] = co.matmul(F(A, (nb * M, K)), F(B, (K, N)))


def cuda_matmul_bwd(A, B, dC, dA, dB, M, N, K, nb):
    _count("matmul_bwd")
    a, b = co.matmul_backward(F(A, (nb * M, K)), F(B, (K, N)), F(dC, (nb * M, N)))
    if dA: F(dA, (nb * M, K))[:] = a
    if dB: F(dB, (K, N))[:] = b


def cuda_transpose_2d(i, o, r, c): _count("transpose"); F(o, (c, r))[:] = F(i, (r, c)).T
def cuda_transpose_3d(i, o, nb, M, K): _count("transpose"); F(o, (nb, K, M))[:] = F(i, (nb, M, K)).transpose(0, 2, 1)


# ---- convolutions ------------------------------------------------------------------------------------
def cuda_conv2d_fwd(x, w, o, N, C, H, W, Fo, R, S, ph, pw, sh, sw):
    _count("conv_fwd")
    y = co.conv2d_forward(F(x, (N, C, H, W)), F(w, (Fo, C, R, S)), sh, sw, ph, pw)
    F(o, y.shape)[:] = y


def cuda_conv2d_bwd(w, x, dy, dx, dw, N, C, H, W, Fo, R, S, sh, sw, ph, pw):
    _count("conv_bwd")
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    a, b = co.conv2d_backward(F(dy, (N, Fo, OH, OW)), F(x, (N, C, H, W)), F(w, (Fo, C, R, S)), sh, sw, ph, pw)
    if dx: F(dx, a.shape)[:] = a
    if dw: F(dw, b.shape)[:] = b


def cuda_conv2DTranpose_fwd(x, w, o, N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw):
    _count("convT_fwd")
    y = co.conv_transpose2d_forward(F(x, (N, Ci, H, W)), F(w, (Ci, Co, KH, KW)), sh, sw, ph, pw)
    F(o, y.shape)[:] = y


def cuda_conv2DTranspose_bwd(w, x, dy, dx, dw, N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw):
    _count("convT_bwd")
    Ho, Wo = (H - 1) * sh - 2 * ph + KH, (W - 1) * sw - 2 * pw + KW
    a, b = co.conv_transpose2d_backward(F(dy, (N, Co, Ho, Wo)), F(x, (N, Ci, H, W)), F(w, (Ci, Co, KH, KW)), sh, sw, ph, pw)
    if dx: F(dx, a.shape)[:] = a
    if dw: F(dw, b.shape)[:] = b


# ---- pooling -----------------------------------------------------------------------------------------
def cuda_maxpool_fwd(x, o, m, N, C, H, W, R, S, ph, pw, sh, sw):
    _count("maxpool_fwd")
    y, mk = co.maxpool2d_forward(F(x, (N, C, H, W)), R, S, sh, sw, ph, pw)
    F(o, y.shape)[:] = y
    _view(m, mk.size, np.int32)[:] = mk.ravel()


def cuda_maxpool_bwd(d, m, dx, N, C, H, W, R, S, ph, pw, sh, sw):
    _count("maxpool_bwd")
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    mk = _view(m, N * C * OH * OW, np.int32).reshape(N, C, OH, OW)
    F(dx, (N, C, H, W))[:] = co.maxpool2d_backward(F(d, (N, C, OH, OW)), mk, N, C, H, W, R, S, sh, sw, ph, pw)


def cuda_unpooling_fwd(i, o, N, C, H, W, sh, sw): _count("unpool_fwd"); F(o, (N, C, H * sh, W * sw))[:] = co.unpooling_forward(F(i, (N, C, H, W)), sh, sw)
def cuda_unpooling_bwd(d, dx, N, C, H, W, sh, sw): _count("unpool_bwd"); F(dx, (N, C, H, W))[:] = co.unpooling_backward(F(d, (N, C, H * sh, W * sw)), N, C, H, W, sh, sw)


# ---- reductions ----------------------------------------------------------------------------------------
def _red(op):
    def k(A, o, nd, dim, da):
        _count("reduce")
        shape = tuple(int(v) for v in da[:nd])
        r = co.reduce(F(A, shape), dim, op)
        _view(o, r.size)[:] = r.ravel()
    return k


cuda_sum_fwd, cuda_mean_fwd, cuda_max_fwd, cuda_min_fwd = _red("sum"), _red("mean"), _red("max"), _red("min")


def _argred(mx):
    def k(A, o, nd, dim, da):
        shape = tuple(int(v) for v in da[:nd])
        r = co.argreduce(F(A, shape), dim, mx)
        _view(o, r.size, np.int32)[:] = r.ravel()
    return k


cuda_argmax_fwd, cuda_argmin_fwd = _argred(True), _argred(False)


def _red_bwd(mean):
    def k(d, dA, nd, dim, da):
        _count("reduce_bwd")
        shape = tuple(int(v) for v in da[:nd])
        dim_ = dim % nd
        oshape = tuple(s for i, s in enumerate(shape) if i != dim_) or (1,)
        F(dA, shape)[:] = co.reduce_backward(F(d, oshape), shape, dim_, 1.0 / shape[dim_] if mean else 1.0)
    return k


cuda_sum_bwd, cuda_mean_bwd = _red_bwd(False), _red_bwd(True)


def _ext_bwd(d, fi, fo, dA, nd, dim, da):
    shape = tuple(int(v) for v in da[:nd])
    dim_ = dim % nd
    A = F(fi, shape)
    oshape = tuple(s for i, s in enumerate(shape) if i != dim_) or (1,)
    hit = (A == np.expand_dims(F(fo, oshape).reshape([s for i, s in enumerate(shape) if i != dim_] or [1]), dim_))
    first = hit & (np.cumsum(hit, axis=dim_) == 1)
    F(dA, shape)[:] += first * np.expand_dims(F(d, oshape).reshape([s for i, s in enumerate(shape) if i != dim_] or [1]), dim_)


cuda_max_bwd = cuda_min_bwd = _ext_bwd


# ---- scalar / fills / binary / broadcast ----------------------------------------------------------------
def cuda_scaler_multiply_f(a, k, n): _count("scalar"); v = _view(a, n); v[:] = v * np.float32(k)
def cuda_scaler_add_f(a, k, n): _count("scalar"); v = _view(a, n); v[:] = v + np.float32(k)
def cuda_power_of(a, k, n): _count("scalar"); v = _view(a, n); v[:] = np.power(v, np.float32(k))
def cuda_ones_f(n): _count("fill"); p = _alloc(n * 4); _view(p, n)[:] = 1; return p
def cuda_zeros_f(n): _count("fill"); return _alloc(n * 4)
def cuda_elemadd(A, B, C, n): _count("elemadd"); _view(C, n)[:] = _view(A, n) + _view(B, n)
def cuda_elemsub(A, B, C, n): _count("elemsub"); _view(C, n)[:] = _view(A, n) - _view(B, n)
def cuda_elemmult(A, B, C, n): _count("elemmult"); _view(C, n)[:] = _view(A, n) * _view(B, n)
def cuda_elemdiv(A, B, C, n): _count("elemdiv"); _view(C, n)[:] = _view(A, n) / _view(B, n)


def _bcast(op):
    def k(A, B, C, aN, aC, aH, aW, bN, bC, bH, bW):
        _count("broadcast")
        r = op(F(A, (aN, aC, aH, aW)), F(B, (bN, bC, bH, bW)))
        F(C, r.shape)[:] = r
    return k


broadcast_add_4d, broadcast_mul_4d = _bcast(np.add), _bcast(np.multiply)


# ---- additive entries ---------------------------------------------------------------------------------------
def init(dev): pass
def stream_synchronize(): pass
def launch_count(): return sum(CALLS.values())
def set_precision(m): pass
def get_precision(): return 0
def mse_partials(n): return 64


def _act(z, code):
    return [lambda v: v, lambda v: np.maximum(v, 0) * (v > 0), lambda v: co.sigmoid(v)[0], lambda v: co.tanh_act(v)[0]][code](z)


def _dact(y, code):
    return [lambda v: np.ones_like(v), lambda v: (v > 0).astype(np.float32), lambda v: v * (1 - v), lambda v: 1 - v * v][code](y)


def bias_act_fwd(z, b, y, n, ch, inner, act):
    _count("bias_act_fwd")
    zz = _view(z, n).reshape(-1, ch, inner)
    bb = _view(b, ch).reshape(1, ch, 1) if b else 0
    _view(y, n)[:] = _act((zz + bb).astype(np.float32), act).ravel()


def matmul_bias_act_fwd(A, B, b, C, M, N, K, act):
    cuda_matmul(A, B, C, M, N, K, 1)
    bias_act_fwd(C, b, C, M * N, N, 1, act)


def conv2d_bias_act_fwd(x, w, b, o, N, C, H, W, Fo, R, S, ph, pw, sh, sw, act):
    cuda_conv2d_fwd(x, w, o, N, C, H, W, Fo, R, S, ph, pw, sh, sw)
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    bias_act_fwd(o, b, o, N * Fo * OH * OW, Fo, OH * OW, act)


def conv2DTranspose_bias_act_fwd(x, w, b, o, N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw, act):
    cuda_conv2DTranpose_fwd(x, w, o, N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw)
    Ho, Wo = (H - 1) * sh - 2 * ph + KH, (W - 1) * sw - 2 * pw + KW
    bias_act_fwd(o, b, o, N * Co * Ho * Wo, Co, Ho * Wo, act)


def conv2d_bias_act_fwd_s(x, w, b, o, N, C, H, W, Fo, R, S, ph, pw, sh, sw, act, x_in):
    conv2d_bias_act_fwd(x, w, b, o, N, C, H, W, Fo, R, S, ph, pw, sh, sw, act)
    return 0


def maxpool2x2_fwd_s(x, o, mask, N, C, H, W):
    cuda_maxpool_fwd(x, o, mask, N, C, H, W, 2, 2, 0, 0, 2, 2)
    return 0


def conv2d_pool_fusable(N, C, H, W, Fo, R, S, sh, sw, ph, pw):
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    return OH % 2 == 0 and OW % 2 == 0 and (OW in (2, 4, 8, 16) or C * R * S <= 64)


def conv2d_bias_act_pool_fwd_s(x, w, b, pooled, mask, N, C, H, W, Fo, R, S, ph, pw, sh, sw, act, x_in, want_copies):
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    tmp = _alloc(N * Fo * OH * OW * 4)
    conv2d_bias_act_fwd(x, w, b, tmp, N, C, H, W, Fo, R, S, ph, pw, sh, sw, act)
    cuda_maxpool_fwd(tmp, pooled, mask, N, Fo, OH, OW, 2, 2, 0, 0, 2, 2)
    cuda_free(tmp)
    return 0, 0


def shadow_free(h): pass


def rows_free(h): pass


def matmul_bias_act_fwd_s(A, B, b, C, M, N, K, act, a_in, want_c_copies):
    matmul_bias_act_fwd(A, B, b, C, M, N, K, act)
    return 0, 0, 0


def matmul_act_bwd(A, B, y, g, dA, dB, dbias, M, N, K, act, a_keep, w_keep):
    dz = _alloc(4 * M * N)
    act_bias_bwd(g, y, dz, dbias, M * N, N, 1, act)
    cuda_matmul_bwd(A, B, dz, dA, dB, M, N, K, 1)


# transfers: the stand-in has one "stream", so the copy-stream calls are plain copies and the fences do nothing
def host_alloc_pinned(n):
    return _alloc(n)


def host_free_pinned(p):
    cuda_free(p)


def host_view(p, nbytes):
    return _view(p, nbytes, np.uint8)


def copy_upload(dst, host, nbytes):
    _view(dst, nbytes, np.uint8)[:] = _view(host, nbytes, np.uint8)


def copy_download(host, src, nbytes):
    _view(host, nbytes, np.uint8)[:] = _view(src, nbytes, np.uint8)


def copy_wait_compute(): pass
def compute_wait_copy(): pass
def copy_synchronize(): pass


def batchnorm_fwd(x, g, b, rm, rv, y, mean, si, N, C, S, momentum, eps, training):
    _count("batchnorm_fwd")
    shape = (N, C, S)
    rmv, rvv = _view(rm, C).copy(), _view(rv, C).copy()
    yy, _, mu, s = co.batchnorm_forward(F(x, shape), _view(g, C), _view(b, C), rmv, rvv, momentum, eps, training)
    F(y, shape)[:] = yy
    _view(mean, C)[:] = mu
    _view(si, C)[:] = s
    _view(rm, C)[:] = rmv
    _view(rv, C)[:] = rvv


def batchnorm_bwd(dy, x, mean, si, g, dx, dg, db, N, C, S):
    _count("batchnorm_bwd")
    shape = (N, C, S)
    xh = ((F(x, shape) - _view(mean, C).reshape(1, C, 1)) * _view(si, C).reshape(1, C, 1)).astype(np.float32)
    a, b, c = co.batchnorm_backward(F(dy, shape), xh, _view(si, C), _view(g, C))
    F(dx, shape)[:] = a
    _view(dg, C)[:] = b
    _view(db, C)[:] = c


# one rank in this stand-in: the cross-rank forms are the local ones
batchnorm_fwd_sync = batchnorm_fwd
batchnorm_bwd_sync = batchnorm_bwd
def dp_world(): return 1
def dp_rank(): return 0


def concat_fwd(a, b, out, N, n1, n2):
    _count("concat_fwd")
    F(out, (N, n1 + n2))[:] = np.concatenate([F(a, (N, n1)), F(b, (N, n2))], axis=1)


def concat_bwd(dout, da, db, N, n1, n2):
    _count("concat_bwd")
    d = F(dout, (N, n1 + n2))
    F(da, (N, n1))[:] = d[:, :n1]
    F(db, (N, n2))[:] = d[:, n1:]


def onehot_f32(labels, out, n, classes):
    lab = _view(labels, n, np.int32)
    F(out, (n, classes))[:] = (lab[:, None] == np.arange(classes)[None, :]).astype(np.float32)


def conv2d_act_bwd(w, x, y, g, gp, mask, yp, dx, dw, db, N, C, H, W, Fo, R, S, sh, sw, ph, pw, act, x_shadow):
    OH, OW = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
    n = N * Fo * OH * OW
    ytmp = 0
    if not y and act:            # only the pool's output is at hand: it is y wherever the routed gradient is not zero
        ytmp = y = _alloc(n * 4)
        up = np.repeat(np.repeat(F(yp, (N, Fo, OH // 2, OW // 2)), 2, axis=2), 2, axis=3)
        _view(y, n)[:] = up.ravel()
    full = np.empty(n, np.float32)
    if gp:
        tmp = _alloc(n * 4)
        cuda_maxpool_bwd(gp, mask, tmp, N, Fo, OH, OW, 2, 2, 0, 0, 2, 2)
        full[:] = _view(tmp, n)
        cuda_free(tmp)
    else:
        full[:] = _view(g, n)
    tmp = _alloc(n * 4)
    _view(tmp, n)[:] = full
    act_bias_bwd(tmp, y, tmp, db, n, Fo, OH * OW, act)
    cuda_conv2d_bwd(w, x, tmp, dx, dw, N, C, H, W, Fo, R, S, sh, sw, ph, pw)
    cuda_free(tmp)
    if ytmp:
        cuda_free(ytmp)


def act_bias_bwd(dy, y, dz, db, n, ch, inner, act):
    _count("act_bias_bwd")
    g = _view(dy, n).reshape(-1, ch, inner)
    r = g * (_dact(_view(y, n).reshape(-1, ch, inner), act) if act else 1.0)
    r = r.astype(np.float32)
    _view(dz, n)[:] = r.ravel()
    if db:
        _view(db, ch)[:] = r.sum(axis=(0, 2))


def softmax_cce_fwd_bwd(z, y, p, rows, loss, dz, N, C, eps, inv):
    _count("softmax_cce")
    P = co.softmax(F(z, (N, C)))
    Y = F(y, (N, C))
    F(p, (N, C))[:] = P
    pc, gclip = co.clip_act(P, eps, 1.0 - eps)
    lg, glog = co.log_act(pc)
    per = (-Y * lg).sum(-1)
    _view(rows, N)[:] = per
    _view(loss, 1)[:] = per.sum() * np.float32(inv)
    dP = gclip * glog * (-Y * np.float32(inv))
    F(dz, (N, C))[:] = co.softmax_vjp(P, dP.astype(np.float32))


def mse_fwd_bwd(p, y, part, loss, dp, n, inv):
    _count("mse")
    d = _view(p, n) - _view(y, n)
    _view(loss, 1)[:] = (d * d).sum() * np.float32(inv)
    _view(dp, n)[:] = 2 * d * np.float32(inv)


def grad_scale_update(g, n): _count("grad_scale")


def mae_fwd_bwd(p, y, part, loss, dp, n, inv):
    _count("mae")
    d = _view(p, n) - _view(y, n)
    _view(loss, 1)[:] = np.abs(d).sum() * np.float32(inv)
    _view(dp, n)[:] = np.sign(d) * np.float32(inv)


def bce_fwd_bwd(p, y, part, loss, dp, n, inv, eps):
    _count("bce")
    P, Y, e = _view(p, n), _view(y, n), np.float32(eps)
    a, b = P + e, (np.float32(1) - P) + e
    _view(loss, 1)[:] = (-Y * np.log(a) - (1 - Y) * np.log(b)).sum() * np.float32(inv)
    _view(dp, n)[:] = (-Y / a + (1 - Y) / b) * np.float32(inv)


def cuda_adam_step(w, g, m, v, n, lr, b1, omb1, b2, omb2, eps, c1, c2, gs):
    _count("adam")
    f = np.float32
    W, G, M, V = _view(w, n), _view(g, n) * f(gs), _view(m, n), _view(v, n)
    M[:] = f(b1) * M + f(omb1) * G
    V[:] = f(b2) * V + f(omb2) * (G * G)
    W[:] = W - (f(lr) * (M / f(c1))) / (np.sqrt(V / f(c2)) + f(eps))


def is_capturing(): return False


def cuda_adam_step_dev(w, g, m, v, n, h):
    hv = _view(h, 9)
    cuda_adam_step(w, g, m, v, n, *[float(x) for x in hv])


def cuda_sgd_step_dev(w, g, vel, n, h):
    hv = _view(h, 3)
    cuda_sgd_step(w, g, vel, n, *[float(x) for x in hv])


def cuda_sgd_step(w, g, vel, n, lr, mu, gs):
    _count("sgd")
    f = np.float32
    W, G, Ve = _view(w, n), _view(g, n) * f(gs), _view(vel, n)
    Ve[:] = f(mu) * Ve + f(lr) * G
    W[:] = W - Ve
