"""Pins the CPU oracle: the C restatement (oracle/seera_oracle.c) and the step driver
(oracle/train_oracle.py) against the reference's known-answer vectors, against golden
vectors produced by the unmodified reference, and - when it has been compiled into
oracle/_ref - against the reference's own CPU engine."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co
from oracle import ref_engine
from oracle.train_oracle import RefNet
from ml_framework_b200 import workloads as wl
import cases

REF = ref_engine.load()
ENGINES = [("restatement", co)] + ([("reference-engine", REF)] if REF is not None else [])


# ---- the reference's own known answers (Testing/test_14.py:984-1011) -----------
@pytest.mark.parametrize("name,E", ENGINES)
def test_known_answer_matmul(name, E):
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    assert np.array_equal(E.matmul(A, B), np.array([[19, 22], [43, 50]], np.float32))
    X = np.random.RandomState(0).standard_normal((6, 6)).astype(np.float32)
    assert np.array_equal(E.matmul(X, np.eye(6, dtype=np.float32)), X)


# ---- per-op golden vectors from the reference engine -----------------------------
INT_KEYS = {"pool_mask"}
EXACT_KEYS = {"pool_out", "pool_dX", "unpool_fwd", "relu_o", "relu_g", "abs_act_o", "abs_act_g", "clip_o", "clip_g"}


@pytest.mark.parametrize("name,E", ENGINES)
def test_ops_against_golden(name, E, golden_dir):
    gold = np.load(golden_dir + "/ops.npz")
    got = cases.op_cases(E, np.random.RandomState(7))
    assert set(got) == set(gold.files)
    for k in gold.files:
        if k in INT_KEYS or k in EXACT_KEYS:
            assert np.array_equal(np.asarray(got[k]), gold[k]), k
        else:
            assert rel_l2(got[k], gold[k]) < 2e-6, (k, rel_l2(got[k], gold[k]))


def test_maxpool_tie_and_padding_semantics():
    # all-zero window: first tap wins (index 0); negative input with padding: the padded 0.0 wins
    X = np.zeros((1, 1, 4, 4), np.float32)
    o, m = co.maxpool2d_forward(X, 2, 2, 2, 2, 0, 0)
    assert np.all(m == 0) and np.all(o == 0)
    Xn = -np.ones((1, 1, 2, 2), np.float32)
    o, m = co.maxpool2d_forward(Xn, 2, 2, 2, 2, 1, 1)
    assert np.all(o == 0.0)
    d = co.maxpool2d_backward(np.ones_like(o), m, 1, 1, 2, 2, 2, 2, 2, 2, 1, 1)
    assert np.all(d == 0.0)       # gradient routed to padding is dropped


def test_argreduce_first_index_on_ties():
    A = np.array([[1, 3, 3, 0], [2, 2, 1, 1]], np.float32)
    assert co.argreduce(A, 1, True).tolist() == np.argmax(A, 1).tolist() == [1, 0]
    assert co.argreduce(A, 1, False).tolist() == np.argmin(A, 1).tolist() == [3, 2]
    R = np.random.RandomState(3).standard_normal((3, 5, 7)).astype(np.float32)
    for d in range(3):
        assert np.array_equal(co.argreduce(R, d, True), np.argmax(R, d).astype(np.int32))
        assert np.array_equal(co.argreduce(R, d, False), np.argmin(R, d).astype(np.int32))
        for op, f in (("sum", np.sum), ("mean", np.mean), ("max", np.max), ("min", np.min)):
            assert np.allclose(co.reduce(R, d, op), f(R, axis=d), rtol=1e-5, atol=1e-6)


def test_optimizer_restatement_matches_numpy_formulas():
    rs = np.random.RandomState(4)
    w = rs.standard_normal(1000).astype(np.float32)
    g = rs.standard_normal(1000).astype(np.float32)
    w2, m2, v2 = w.copy(), np.zeros_like(w), np.zeros_like(w)
    wn, mn, vn = w.copy(), np.zeros_like(w), np.zeros_like(w)
    for t in (1, 2, 3):
        co.adam_step(w2, g, m2, v2, 1e-3, 0.9, 0.999, 1e-8, t)
        mn = 0.9 * mn + (1 - 0.9) * g
        vn = 0.999 * vn + (1 - 0.999) * (g ** 2)
        wn = wn - (1e-3 * (mn / (1 - 0.9 ** t))) / ((vn / (1 - 0.999 ** t)) ** 0.5 + 1e-8)
        assert wn.dtype == np.float32
        assert np.array_equal(m2, mn) and np.array_equal(v2, vn)
        assert np.max(np.abs(w2 - wn)) <= 2.4e-7 * np.max(np.abs(wn))
    ws, vel = w.copy(), np.zeros_like(w)
    wn, veln = w.copy(), np.zeros_like(w)
    for _ in range(3):
        co.sgd_step(ws, g, vel, 0.01, 0.9)
        veln = 0.9 * veln + 0.01 * g
        wn = wn - veln
        assert np.array_equal(vel, veln) and np.array_equal(ws, wn)


# ---- whole training steps against the unmodified reference ------------------------
def _check_steps(work, n, seed, gold, E, tol):
    net = RefNet(work.layers, work.params(seed), work.loss, work.opt, E)
    X, Y = work.batch(n, seed)
    for s in range(2):
        P = net.forward(X)
        loss, dP = net.loss_and_grad(P, Y)
        grads = net.backward(dP)
        assert abs(float(loss) - float(gold["loss%d" % s])) <= tol * max(1.0, abs(float(gold["loss%d" % s])))
        if s == 0:
            assert rel_l2(P, gold["pred0"]) < tol
            k = 0
            for G in grads:
                if G is not None:
                    assert rel_l2(G[0], gold["dW%d" % k]) < tol, ("dW", k)
                    assert rel_l2(G[1], gold["db%d" % k]) < tol, ("db", k)
                    k += 1
        net.apply(grads)
        k = 0
        for Pm in net.params:
            if Pm is not None:
                assert rel_l2(Pm[0], gold["W%d_s%d" % (k, s)]) < tol, ("W", k, s)
                assert rel_l2(Pm[1].reshape(-1), gold["b%d_s%d" % (k, s)].reshape(-1)) < tol * 50 + 1e-9, ("b", k, s)
                k += 1


@pytest.mark.parametrize("name,E", ENGINES)
def test_c1_two_steps_against_reference(name, E, golden_dir):
    _check_steps(wl.c1_small_cnn(), 64, 1, np.load(golden_dir + "/c1_two_steps.npz"), E, 2e-5)


@pytest.mark.parametrize("name,E", ENGINES)
@pytest.mark.parametrize("case", ["c2s", "c3s", "c4s"])
def test_small_configs_two_steps_against_reference(name, E, case, golden_dir):
    work, n = cases.small_cases()[case]
    _check_steps(work, n, 2, np.load(golden_dir + "/%s_two_steps.npz" % case), E, 2e-5)


def test_batchnorm_restatement_matches_the_reference_engine_and_numpy():
    """so_batchnorm_fwd / _bwd against the compiled reference engine (bit for bit, same loops) and against the NumPy
    formulas of the reference's fallback (Seera_init.py:893-912, Seera_Engine.py:401-412)."""
    rs = np.random.RandomState(0)
    for shape in [(7, 5), (4, 6, 3, 5), (1, 3, 2, 2)]:
        X = (rs.standard_normal(shape) * 2 + 1).astype(np.float32)
        C = shape[1]
        g, b = rs.standard_normal(C).astype(np.float32), rs.standard_normal(C).astype(np.float32)
        axes = (0, 2, 3) if len(shape) == 4 else (0,)
        bs = (1, -1, 1, 1) if len(shape) == 4 else (1, -1)
        for training in (True, False):
            rm, rv = rs.standard_normal(C).astype(np.float32), (rs.rand(C) + 0.5).astype(np.float32)
            rm0, rv0 = rm.copy(), rv.copy()
            y, xh, mu, si = co.batchnorm_forward(X, g, b, rm, rv, 0.1, 1e-5, training)
            m_np, v_np = (X.mean(axis=axes), X.var(axis=axes)) if training else (rm0, rv0)
            xh_np = (X - m_np.reshape(bs)) / np.sqrt(v_np.reshape(bs) + 1e-5)
            assert np.allclose(xh, xh_np, rtol=2e-5, atol=2e-5) and np.allclose(y, g.reshape(bs) * xh_np + b.reshape(bs), rtol=2e-5, atol=2e-5)
            if training:
                assert np.allclose(rm, 0.9 * rm0 + 0.1 * m_np, atol=1e-6) and np.allclose(rv, 0.9 * rv0 + 0.1 * v_np, atol=1e-6)
            else:
                assert np.array_equal(rm, rm0) and np.array_equal(rv, rv0)
            d = rs.standard_normal(shape).astype(np.float32)
            dx, dg, db = co.batchnorm_backward(d, xh, si, g)
            M = X.size // C
            dxh = d * g.reshape(bs)
            dx_np = (1.0 / M) * si.reshape(bs) * (M * dxh - dxh.sum(axis=axes).reshape(bs) - xh * (dxh * xh).sum(axis=axes).reshape(bs))
            assert np.allclose(dx, dx_np, rtol=1e-4, atol=1e-5) and np.allclose(dg, (d * xh).sum(axis=axes), rtol=1e-4, atol=1e-5)
            assert np.allclose(db, d.sum(axis=axes), rtol=1e-4, atol=1e-5)
            if REF is not None:
                rm2, rv2 = rm0.copy(), rv0.copy()
                y2, xh2, si2 = REF.batchnorm_forward(X, g, b, rm2, rv2, 0.1, 1e-5, training, len(shape) == 4)
                assert np.array_equal(y, y2) and np.array_equal(xh, xh2) and np.array_equal(si, si2)
                assert np.array_equal(rm, rm2) and np.array_equal(rv, rv2)
                r = REF.batchnorm_backward(d, xh2, si2, g, M, len(shape) == 4)
                assert all(np.array_equal(p, q) for p, q in zip((dx, dg, db), r))
