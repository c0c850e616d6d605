"""GPU parity, op by op, through the C ABI (tests/engine_np.py -> ctypes -> libseera_b200.so)
against the CPU oracle and the golden vectors of the unmodified reference engine.
Integer results (max-pool masks, argmax/argmin) and pure data movement must be bit-exact; floating
point contractions must agree to rel-L2 <= 2e-5 in fp32 mode (summation order only)."""
import ctypes

import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co
from oracle import ref_engine
import cases

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-5


@pytest.fixture(scope="module")
def E():
    from ml_framework_b200 import capi
    import engine_np
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    capi.check(L.seera_set_precision(0))
    return engine_np


def test_known_answers(E):
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    assert np.array_equal(E.matmul(A, B), np.array([[19, 22], [43, 50]], np.float32))
    X = np.random.RandomState(0).standard_normal((6, 6)).astype(np.float32)
    assert np.array_equal(E.matmul(X, np.eye(6, dtype=np.float32)), X)


def test_ops_against_reference_golden(E, golden_dir):
    gold = np.load(golden_dir + "/ops.npz")
    got = cases.op_cases(E, np.random.RandomState(7))
    for k in gold.files:
        if k in ("pool_mask", "pool_out", "pool_dX", "unpool_fwd", "relu_o", "relu_g", "abs_act_o", "abs_act_g", "clip_o", "clip_g"):
            assert np.array_equal(np.asarray(got[k]), gold[k]), k
        else:
            assert rel_l2(got[k], gold[k]) < FP32_TOL, (k, rel_l2(got[k], gold[k]))


# (M, K, N) including the reference's odd-size diagnostics (Testing/diagnose_sizes.py:17-47)
MATMUL_SHAPES = [(1, 3, 2), (5, 7, 3), (17, 33, 65), (32, 400, 256), (64, 784, 10), (129, 130, 131), (300, 10, 1024), (256, 1024, 1024)]


@pytest.mark.parametrize("M,K,N", MATMUL_SHAPES)
def test_matmul_and_backward(E, M, K, N):
    rs = np.random.RandomState(M * 7 + N)
    A, B, dC = (rs.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (M, N)))
    assert rel_l2(E.matmul(A, B), co.matmul(A, B)) < FP32_TOL
    dA, dB = E.matmul_backward(A, B, dC)
    rA, rB = co.matmul_backward(A, B, dC)
    assert rel_l2(dA, rA) < FP32_TOL and rel_l2(dB, rB) < FP32_TOL


def test_batched_matmul_shared_rhs(E):
    rs = np.random.RandomState(3)
    A, B, dC = rs.standard_normal((4, 9, 11)).astype(np.float32), rs.standard_normal((11, 6)).astype(np.float32), \
        rs.standard_normal((4, 9, 6)).astype(np.float32)
    assert rel_l2(E.matmul(A, B), A @ B) < FP32_TOL
    dA, dB = E.matmul_backward(A, B, dC)
    assert rel_l2(dA, dC @ B.T) < FP32_TOL
    assert rel_l2(dB, np.einsum("bmk,bmn->kn", A, dC)) < FP32_TOL


# (N, C, H, W, F, KH, KW, sh, sw, ph, pw): shapes in the spirit of Testing/test_1.py:225-302 and test_3.py:51-93
CONV_SHAPES = [(1, 1, 5, 5, 1, 3, 3, 1, 1, 0, 0), (2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1), (3, 5, 9, 7, 6, 3, 3, 2, 1, 1, 2),
               (2, 4, 11, 13, 7, 5, 3, 2, 2, 2, 1), (4, 8, 14, 14, 16, 1, 1, 1, 1, 0, 0), (2, 16, 16, 16, 32, 3, 3, 2, 2, 1, 1),
               (8, 32, 32, 32, 64, 3, 3, 2, 2, 1, 1), (2, 130, 6, 6, 70, 3, 3, 1, 1, 1, 1), (5, 2, 7, 7, 3, 7, 7, 1, 1, 3, 3)]


@pytest.mark.parametrize("shape", CONV_SHAPES)
def test_conv2d_forward_backward(E, shape):
    N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape))
    X, Wt = rs.standard_normal((N, C, H, W)).astype(np.float32), rs.standard_normal((F, C, KH, KW)).astype(np.float32)
    Y = E.conv2d_forward(X, Wt, sh, sw, ph, pw)
    R = co.conv2d_forward(X, Wt, sh, sw, ph, pw)
    assert Y.shape == R.shape and rel_l2(Y, R) < FP32_TOL
    dY = rs.standard_normal(R.shape).astype(np.float32)
    dX, dW = E.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    rX, rW = co.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    assert rel_l2(dX, rX) < FP32_TOL and rel_l2(dW, rW) < FP32_TOL


# (N, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw), cf. Testing/test_1.py:397-468, test_3.py:96-136
CONVT_SHAPES = [(1, 1, 4, 4, 1, 3, 3, 1, 1, 0, 0), (2, 4, 5, 6, 3, 4, 3, 2, 2, 1, 0), (2, 8, 8, 8, 4, 4, 4, 2, 2, 1, 1),
                (3, 6, 7, 5, 5, 3, 3, 1, 1, 1, 1), (8, 64, 16, 16, 32, 4, 4, 2, 2, 1, 1), (2, 3, 6, 6, 2, 2, 2, 2, 2, 0, 0),
                (2, 5, 5, 5, 7, 3, 5, 3, 2, 1, 2)]


@pytest.mark.parametrize("shape", CONVT_SHAPES)
def test_conv_transpose2d_forward_backward(E, shape):
    N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape) + 1)
    X, Wt = rs.standard_normal((N, Ci, H, W)).astype(np.float32), rs.standard_normal((Ci, Co, KH, KW)).astype(np.float32)
    Y = E.conv_transpose2d_forward(X, Wt, sh, sw, ph, pw)
    R = co.conv_transpose2d_forward(X, Wt, sh, sw, ph, pw)
    assert Y.shape == R.shape and rel_l2(Y, R) < FP32_TOL
    dY = rs.standard_normal(R.shape).astype(np.float32)
    dX, dW = E.conv_transpose2d_backward(dY, X, Wt, sh, sw, ph, pw)
    rX, rW = co.conv_transpose2d_backward(dY, X, Wt, sh, sw, ph, pw)
    assert rel_l2(dX, rX) < FP32_TOL and rel_l2(dW, rW) < FP32_TOL


# (N, C, H, W, KH, KW, sh, sw, ph, pw), cf. Testing/test_1.py:309-390
POOL_SHAPES = [(2, 3, 8, 8, 2, 2, 2, 2, 0, 0), (2, 3, 9, 8, 3, 2, 2, 2, 1, 1), (1, 1, 7, 7, 3, 3, 1, 1, 0, 0), (4, 16, 28, 28, 2, 2, 2, 2, 0, 0),
               (3, 5, 10, 12, 3, 3, 2, 2, 1, 1), (2, 2, 6, 6, 2, 2, 1, 1, 0, 0), (2, 4, 13, 11, 2, 3, 2, 3, 0, 1), (8, 64, 32, 32, 2, 2, 2, 2, 0, 0)]


@pytest.mark.parametrize("shape", POOL_SHAPES)
@pytest.mark.parametrize("post_relu", [False, True])
def test_maxpool_mask_bit_exact(E, shape, post_relu):
    N, C, H, W, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape))
    X = rs.standard_normal((N, C, H, W)).astype(np.float32)
    if post_relu:
        X = np.maximum(X, 0)                              # ties: whole windows of zeros
    out, mask = E.maxpool2d_forward(X, KH, KW, sh, sw, ph, pw)
    ro, rm = co.maxpool2d_forward(X, KH, KW, sh, sw, ph, pw)
    assert np.array_equal(mask, rm) and np.array_equal(out, ro)
    d = rs.standard_normal(ro.shape).astype(np.float32)
    dX = E.maxpool2d_backward(d, mask, N, C, H, W, KH, KW, sh, sw, ph, pw)
    rX = co.maxpool2d_backward(d, rm, N, C, H, W, KH, KW, sh, sw, ph, pw)
    if sh >= KH and sw >= KW:
        assert np.array_equal(dX, rX)                     # disjoint windows: pure data movement
    else:
        assert rel_l2(dX, rX) < 1e-6


def test_maxpool_all_negative_with_padding(E):
    X = -np.ones((1, 1, 2, 2), np.float32)
    o, m = E.maxpool2d_forward(X, 2, 2, 2, 2, 1, 1)
    ro, rm = co.maxpool2d_forward(X, 2, 2, 2, 2, 1, 1)
    assert np.array_equal(o, ro) and np.array_equal(m, rm) and np.all(o == 0)
    d = E.maxpool2d_backward(np.ones_like(o), m, 1, 1, 2, 2, 2, 2, 2, 2, 1, 1)
    assert np.all(d == 0)


@pytest.mark.parametrize("shape,s", [((2, 3, 4, 5), (2, 3)), ((4, 32, 32, 32), (2, 2)), ((1, 1, 3, 3), (1, 1)), ((2, 2, 5, 7), (3, 1))])
def test_unpooling(E, shape, s):
    rs = np.random.RandomState(1)
    X = rs.standard_normal(shape).astype(np.float32)
    sh, sw = s
    assert np.array_equal(E.unpooling_forward(X, sh, sw), co.unpooling_forward(X, sh, sw))
    N, C, H, W = shape
    d = rs.standard_normal((N, C, H * sh, W * sw)).astype(np.float32)
    assert rel_l2(E.unpooling_backward(d, N, C, H, W, sh, sw), co.unpooling_backward(d, N, C, H, W, sh, sw)) < 1e-6


@pytest.mark.parametrize("shape", [(7,), (5, 10), (4096, 10), (3, 5, 7), (64, 8, 14, 14), (512, 37), (2, 3, 4, 5), (1000, 33)])
def test_reductions_and_arg_reductions(E, shape):
    rs = np.random.RandomState(len(shape) * 11 + shape[0])
    A = rs.standard_normal(shape).astype(np.float32)
    for dim in range(len(shape)):
        for op, f in (("sum", np.sum), ("mean", np.mean), ("max", np.max), ("min", np.min)):
            got = E.reduce(A, dim, op)
            want = f(A.astype(np.float64), axis=dim)
            if op in ("max", "min"):
                assert np.array_equal(got.reshape(-1), want.astype(np.float32).reshape(-1))
            else:
                assert np.allclose(got.reshape(-1), want.reshape(-1), rtol=2e-5, atol=2e-5)
        assert np.array_equal(E.reduce(A, dim, "argmax").reshape(-1), np.argmax(A, dim).astype(np.int32).reshape(-1))
        assert np.array_equal(E.reduce(A, dim, "argmin").reshape(-1), np.argmin(A, dim).astype(np.int32).reshape(-1))
        oshape = tuple(s for i, s in enumerate(shape) if i != dim) or (1,)
        d = rs.standard_normal(oshape).astype(np.float32)
        assert np.array_equal(E.reduce_backward(d, shape, dim, "sum"), co.reduce_backward(d, shape, dim, 1.0))
        assert np.allclose(E.reduce_backward(d, shape, dim, "mean"), co.reduce_backward(d, shape, dim, 1.0 / shape[dim]), rtol=1e-6)
        mx = np.max(A, axis=dim).reshape(oshape)
        got = E.reduce_backward(d, shape, dim, "max", A, mx)
        want = np.zeros(shape, np.float32)
        idx = np.expand_dims(np.argmax(A, dim), dim)
        np.put_along_axis(want, idx, np.expand_dims(d.reshape(np.argmax(A, dim).shape), dim), dim)
        assert np.array_equal(got, want)


def test_argmax_ties_take_first_index(E):
    A = np.array([[1, 3, 3, 0], [2, 2, 1, 1]], np.float32)
    assert E.reduce(A, 1, "argmax").tolist() == [1, 0]     # the reference GPU kernel would give [2, 1]
    assert E.reduce(A, 1, "argmin").tolist() == [3, 2]


def _dev_call(fn_name, arrays, scalars, outs):
    """Runs a raw C-ABI entry on uploaded arrays; `outs` lists (index, shape, dtype) to download."""
    from ml_framework_b200 import capi
    from engine_np import _Dev
    with _Dev() as d:
        ptrs = [None if a is None else d.up(a, a.dtype) for a in arrays]
        capi.check(getattr(d.L, fn_name)(*ptrs, *scalars))
        return [d.down(ptrs[i], shp, dt) for i, shp, dt in outs]


@pytest.mark.parametrize("rows,ch,inner", [(64, 10, 1), (4096, 1024, 1), (33, 7, 1), (8, 16, 196), (5, 3, 49), (64, 8, 784), (2, 1, 4096)])
@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_fused_bias_activation_forward_and_backward(E, rows, ch, inner, act):
    rs = np.random.RandomState(rows + ch + inner + act)
    f = ctypes.c_float
    z = rs.standard_normal((rows, ch, inner)).astype(np.float32)
    b = rs.standard_normal(ch).astype(np.float32)
    y, = _dev_call("seera_bias_act_fwd", [z, b, np.empty_like(z)], [z.size, ch, inner, act], [(2, z.shape, np.float32)])
    pre = z + b.reshape(1, ch, 1)
    ref = [lambda v: (v, None), co.relu, co.sigmoid, co.tanh_act][act](pre)[0]
    assert rel_l2(y, ref) < 1e-6
    dy = rs.standard_normal(z.shape).astype(np.float32)
    dz, db = _dev_call("seera_act_bias_bwd", [dy, y, np.empty_like(z), np.empty(ch, np.float32)], [z.size, ch, inner, act],
                       [(2, z.shape, np.float32), (3, (ch,), np.float32)])
    g = [np.ones_like(y), (y > 0).astype(np.float32), y * (1 - y), 1 - y * y][act]
    assert rel_l2(dz, dy * g) < 1e-6
    assert rel_l2(db, (dy * g).astype(np.float64).sum(axis=(0, 2))) < 1e-5


@pytest.mark.parametrize("N,C", [(64, 10), (4096, 10), (7, 3), (33, 100), (5, 1000)])
def test_softmax_and_fused_cross_entropy(E, N, C):
    rs = np.random.RandomState(N + C)
    f = ctypes.c_float
    z = (rs.standard_normal((N, C)) * 3).astype(np.float32)
    Y = np.eye(C, dtype=np.float32)[rs.randint(0, C, N)]
    s = E.softmax(z)
    assert rel_l2(s, co.softmax(z)) < 1e-6
    d = rs.standard_normal((N, C)).astype(np.float32)
    assert rel_l2(E.softmax_vjp(s, d), co.softmax_vjp(co.softmax(z), d)) < 1e-5
    eps, inv = 1e-7, np.float32(1.0 / N)
    p, rows, loss, dz = _dev_call("seera_softmax_cce_fwd_bwd",
                                  [z, Y, np.empty_like(z), np.empty(N, np.float32), np.empty(1, np.float32), np.empty_like(z)],
                                  [N, C, f(eps), f(inv)],
                                  [(2, (N, C), np.float32), (3, (N,), np.float32), (4, (1,), np.float32), (5, (N, C), np.float32)])
    P = co.softmax(z)
    pc, gclip = co.clip_act(P, eps, 1 - eps)
    lg, glog = co.log_act(pc)
    per = (-Y * lg).sum(-1)
    assert rel_l2(p, P) < 1e-6 and rel_l2(rows, per) < 1e-5
    assert abs(float(loss[0]) - float(per.mean())) < 1e-5 * max(1.0, abs(float(per.mean())))
    ref_dz = co.softmax_vjp(P, (gclip * glog * (-Y * inv)).astype(np.float32))
    assert rel_l2(dz, ref_dz) < 1e-5


def test_fused_mse(E):
    rs = np.random.RandomState(5)
    f = ctypes.c_float
    from ml_framework_b200 import capi
    p, y = rs.uniform(0, 1, 100003).astype(np.float32), rs.uniform(0, 1, 100003).astype(np.float32)
    nparts = capi.load().seera_mse_partials(p.size)
    _, loss, dp = _dev_call("seera_mse_fwd_bwd", [p, y, np.empty(nparts, np.float32), np.empty(1, np.float32), np.empty_like(p)],
                            [p.size, f(1.0 / p.size)], [(2, (nparts,), np.float32), (3, (1,), np.float32), (4, p.shape, np.float32)])
    assert abs(float(loss[0]) - float(np.mean((p.astype(np.float64) - y) ** 2))) < 1e-6
    assert rel_l2(dp, 2 * (p - y) / p.size) < 1e-6


@pytest.mark.parametrize("n", [1, 7, 1000, 9098, 1 << 20])
def test_fused_optimizers_match_the_oracle(E, n):
    rs = np.random.RandomState(n % 1000)
    f = ctypes.c_float
    w, g = rs.standard_normal(n).astype(np.float32), rs.standard_normal(n).astype(np.float32)
    w_ref, m_ref, v_ref = w.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    wd, md, vd = w.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in (1, 2, 3):
        co.adam_step(w_ref, g, m_ref, v_ref, 1e-3, 0.9, 0.999, 1e-8, t)
        s = co.adam_scalars(1e-3, 0.9, 0.999, 1e-8, t)
        wd, md, vd = _dev_call("seera_adam_step", [wd, g, md, vd],
                               [n] + [f(s[k]) for k in ("lr", "b1", "omb1", "b2", "omb2", "eps", "c1", "c2")] + [f(1.0)],
                               [(0, (n,), np.float32), (2, (n,), np.float32), (3, (n,), np.float32)])
        assert rel_l2(md, m_ref) < 1e-6 and rel_l2(vd, v_ref) < 1e-6 and rel_l2(wd, w_ref) < 1e-6
    ws_ref, vel_ref = w.copy(), np.zeros(n, np.float32)
    ws, vel = w.copy(), np.zeros(n, np.float32)
    for _ in range(3):
        co.sgd_step(ws_ref, g, vel_ref, 0.01, 0.9)
        ws, vel = _dev_call("seera_sgd_step", [ws, g, vel], [n, f(0.01), f(0.9), f(1.0)], [(0, (n,), np.float32), (2, (n,), np.float32)])
        assert rel_l2(ws, ws_ref) < 1e-6 and rel_l2(vel, vel_ref) < 1e-6


def test_elementwise_on_unaligned_addresses(E):
    """Callers do byte arithmetic on device addresses (concatenate); kernels must accept 4-byte alignment."""
    from ml_framework_b200 import capi
    from engine_np import _Dev
    a = np.arange(1001, dtype=np.float32)
    with _Dev() as d:
        pa, pc = d.up(a), d.new(1001)
        capi.check(d.L.seera_cuda_elemadd_gputogpu(pa + 4, pa + 4, pc + 4, 1000))
        out = d.down(pc + 4, (1000,))
    assert np.array_equal(out, 2 * a[1:])


def test_bad_arguments_return_status_not_crash(E):
    from ml_framework_b200 import capi
    L = capi.load()
    L.seera_clear_status()
    assert L.seera_cuda_matmul(None, None, None, 4, 4, 4, 1) == 2
    assert L.seera_last_status() == 2 and b"cuda_matmul" in L.seera_last_error()
    assert L.seera_broadcast_add_4d(1, 1, 1, 1, 2, 3, 4, 1, 5, 3, 4) == 2
    L.seera_clear_status()
    assert L.seera_last_status() == 0


@pytest.mark.parametrize("shape", [(7, 5), (64, 300), (4, 6, 3, 5), (16, 33, 14, 14), (3, 1, 1, 1), (512, 64), (6, 10, 16, 16), (3, 5, 32, 24),
                                   (70, 3, 20, 20)])
def test_batchnorm_forward_and_backward(shape):
    """seera_batchnorm_fwd / _bwd against the oracle (training and inference statistics, running-statistics update)."""
    import ctypes
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    rs = np.random.RandomState(sum(shape))
    X = (rs.standard_normal(shape) * 2 + 1).astype(np.float32)
    N, C = shape[0], shape[1]
    S = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    g, b = rs.standard_normal(C).astype(np.float32), rs.standard_normal(C).astype(np.float32)
    d = rs.standard_normal(shape).astype(np.float32)
    up = lambda a: L.seera_to_device(np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p), a.nbytes)
    def down(p, shp):
        a = np.empty(shp, np.float32)
        capi.check(L.seera_to_host(a.ctypes.data_as(ctypes.c_void_p), p, a.nbytes))
        return a
    for training in (1, 0):
        rm, rv = rs.standard_normal(C).astype(np.float32), (rs.rand(C) + 0.5).astype(np.float32)
        rm0, rv0 = rm.copy(), rv.copy()
        y_ref, xh_ref, mu_ref, si_ref = co.batchnorm_forward(X, g, b, rm0, rv0, 0.1, 1e-5, training)
        dx_ref, dg_ref, db_ref = co.batchnorm_backward(d, xh_ref, si_ref, g)
        xd, gd, bd, rmd, rvd, dd = up(X), up(g), up(b), up(rm), up(rv), up(d)
        yd, mud, sid = L.seera_cuda_malloc(X.nbytes), L.seera_cuda_malloc(4 * C), L.seera_cuda_malloc(4 * C)
        dxd, dgd, dbd = L.seera_cuda_malloc(X.nbytes), L.seera_cuda_malloc(4 * C), L.seera_cuda_malloc(4 * C)
        capi.check(L.seera_batchnorm_fwd(xd, gd, bd, rmd, rvd, yd, mud, sid, N, C, S, 0.1, 1e-5, training))
        capi.check(L.seera_batchnorm_bwd(dd, xd, mud, sid, gd, dxd, dgd, dbd, N, C, S))
        assert rel_l2(down(yd, shape), y_ref) < 1e-5 and rel_l2(down(sid, (C,)), si_ref) < 1e-5
        assert np.allclose(down(mud, (C,)), mu_ref, rtol=1e-5, atol=1e-6)
        assert np.allclose(down(rmd, (C,)), rm0, rtol=1e-5, atol=1e-6) and np.allclose(down(rvd, (C,)), rv0, rtol=1e-5, atol=1e-6)
        assert rel_l2(down(dxd, shape), dx_ref) < 2e-5
        assert np.allclose(down(dgd, (C,)), dg_ref, rtol=1e-4, atol=1e-4) and np.allclose(down(dbd, (C,)), db_ref, rtol=1e-4, atol=1e-4)
        for p in (xd, gd, bd, rmd, rvd, dd, yd, mud, sid, dxd, dgd, dbd):
            L.seera_cuda_free(p)


@pytest.mark.parametrize("shape", [(256, 40), (32, 8, 16, 16)])
def test_batchnorm_statistics_of_data_far_from_zero(shape):
    """The one-pass statistics (sums around a sample of the data, Chan merges) on inputs whose mean is 1000 standard deviations
    from zero: mean and 1 / std as close to the fp64 values as the CPU engine's two-pass form, or closer."""
    import ctypes
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    rs = np.random.RandomState(5)
    X = (rs.standard_normal(shape) * 0.05 + 50.0).astype(np.float32)
    N, C = shape[0], shape[1]
    S = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    g, b = np.ones(C, np.float32), np.zeros(C, np.float32)
    rm, rv = np.zeros(C, np.float32), np.ones(C, np.float32)
    _, _, mu_ref, si_ref = co.batchnorm_forward(X, g, b, rm.copy(), rv.copy(), 0.1, 1e-5, True)
    axes = (0,) + tuple(range(2, X.ndim))
    X64 = X.astype(np.float64)
    mu64, si64 = X64.mean(axis=axes), 1.0 / np.sqrt(X64.var(axis=axes) + 1e-5)
    up = lambda a: L.seera_to_device(np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p), a.nbytes)
    xd, gd, bd, rmd, rvd = up(X), up(g), up(b), up(rm), up(rv)
    yd, mud, sid = L.seera_cuda_malloc(X.nbytes), L.seera_cuda_malloc(4 * C), L.seera_cuda_malloc(4 * C)
    capi.check(L.seera_batchnorm_fwd(xd, gd, bd, rmd, rvd, yd, mud, sid, N, C, S, 0.1, 1e-5, 1))
    mu, si = np.empty(C, np.float32), np.empty(C, np.float32)
    capi.check(L.seera_to_host(mu.ctypes.data_as(ctypes.c_void_p), mud, 4 * C))
    capi.check(L.seera_to_host(si.ctypes.data_as(ctypes.c_void_p), sid, 4 * C))
    for p in (xd, gd, bd, rmd, rvd, yd, mud, sid):
        L.seera_cuda_free(p)
    assert np.max(np.abs(mu - mu64)) <= 2 * np.max(np.abs(mu_ref - mu64)) + 8e-6         # a few ulp of 50
    assert rel_l2(si, si64) <= 2 * rel_l2(si_ref, si64) + 2e-5


@pytest.mark.parametrize("N,n1,n2", [(1, 1, 1), (5, 7, 3), (16, 64 * 14 * 14, 32 * 14 * 14), (3, 4, 13), (257, 1000, 24)])
def test_concatenate_forward_and_backward(N, n1, n2):
    """seera_concat_fwd / _bwd (vector and scalar paths, offset pointers) against NumPy."""
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    rs = np.random.RandomState(N + n1 + n2)
    A, B = rs.standard_normal((N, n1)).astype(np.float32), rs.standard_normal((N, n2)).astype(np.float32)
    up = lambda a: L.seera_to_device(np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p), a.nbytes)
    def down(p, shp):
        a = np.empty(shp, np.float32)
        capi.check(L.seera_to_host(a.ctypes.data_as(ctypes.c_void_p), p, a.nbytes))
        return a
    ad, bd = up(A), up(B)
    od = L.seera_cuda_malloc(4 * N * (n1 + n2))
    capi.check(L.seera_concat_fwd(ad, bd, od, N, n1, n2))
    J = np.concatenate([A, B], axis=1)
    assert np.array_equal(down(od, (N, n1 + n2)), J)
    da, db = L.seera_cuda_malloc(4 * N * n1), L.seera_cuda_malloc(4 * N * n2)
    capi.check(L.seera_concat_bwd(od, da, db, N, n1, n2))
    assert np.array_equal(down(da, (N, n1)), A) and np.array_equal(down(db, (N, n2)), B)
    for p in (ad, bd, od, da, db):
        L.seera_cuda_free(p)


@pytest.mark.parametrize("n", [(7,), (64, 10), (256, 1, 64, 64)])
def test_mae_and_binary_cross_entropy_losses(E, n):
    """Loss.mae and Loss.binary_cross_entropy (Seera.py:947-953) with their gradients in one pass, against the formulas
    evaluated in double precision; |d| has gradient 0 at d = 0 (engine/src/activation_ops.cpp:50-56)."""
    from ml_framework_b200 import seera as S
    rs = np.random.RandomState(len(n))
    p = rs.uniform(0.02, 0.98, n).astype(np.float32)
    y = (rs.uniform(0, 1, n) > 0.5).astype(np.float32)
    p.ravel()[0] = y.ravel()[0]                              # one exact zero difference
    P, Y = p.astype(np.float64), y.astype(np.float64)
    for name, want, grad in (("mae", np.abs(P - Y).mean(), np.sign(P - Y) / P.size),
                             ("binary_cross_entropy", (-Y * np.log(P + 1e-15) - (1 - Y) * np.log(1 - P + 1e-15)).mean(),
                              (-Y / (P + 1e-15) + (1 - Y) / (1 - P + 1e-15)) / P.size)):
        pt, yt = S.Tensor(p, is_leaf=True), S.Tensor(y, is_leaf=True)
        loss = getattr(S.Loss(), name)(pt, yt)
        S.autograd4nn(loss)
        assert abs(loss.item() - want) < 2e-6 * max(1.0, abs(want)), name
        assert rel_l2(pt.grad.to_host_f32(), grad) < 1e-6, name
