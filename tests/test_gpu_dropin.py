"""The drop-in claim on the device: the reference's OWN Python layer (Seera.py, Seera_init.py, Seera_Engine.py,
byte-for-byte copies placed under oracle/_ref/py by `make -C oracle ref`) trains on this package's
`seera_cuda` module and `cuTen.cuten` class after `install_dropin()`.

Checked: two Adam steps of configuration C1 through the reference's `Sequential` / `Loss` / `autograd4nn` /
`Adam` (device="cuda") against the golden file written by the unmodified reference on its CPU path, in exact
fp32 mode and on the tensor cores; the `cuten` operator semantics the reference's own scripts pin
(Testing/test_9.py:39-77 value semantics, Testing/test_7.py:592-626 `_reduce_grad_gpu` shapes,
Testing/diagnose_sizes.py:17-47 odd matmul sizes); views keep their owner's memory alive.
The boundary calls and the time of one step of that path are printed (run with -s to see them)."""
import os
import sys
import time
import types

import numpy as np
import pytest

from conftest import rel_l2
from ml_framework_b200 import workloads as wl

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REF_PY = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "py")
have_ref = all(os.path.isfile(os.path.join(REF_PY, f)) for f in ("Seera.py", "Seera_init.py", "Seera_Engine.py"))


@pytest.fixture(scope="module")
def ref():
    """The reference's modules imported over this engine; sys.modules restored afterwards."""
    if not have_ref:
        pytest.skip("oracle/_ref/py is absent: run `make -C oracle ref` where the reference checkout is")
    import ml_framework_b200 as pkg
    names = ("seera_cuda", "cuTen", "matplotlib", "matplotlib.pyplot", "Seera", "Seera_init", "Seera_Engine", "seera_cpp")
    saved = {k: sys.modules.get(k) for k in names}
    for k in ("Seera", "Seera_init", "Seera_Engine", "seera_cuda", "cuTen"):
        sys.modules.pop(k, None)
    sc, ct = pkg.install_dropin()
    sc.init(0)
    if "matplotlib" not in sys.modules:                 # Seera.py:4 imports pyplot, nothing on the training path uses it
        mpl = types.ModuleType("matplotlib")
        mpl.pyplot = types.ModuleType("matplotlib.pyplot")
        sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot
    sys.modules["seera_cpp"] = None                     # no CPU engine on the table: every op must come from seera_cuda
    sys.path.insert(0, REF_PY)
    try:
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            import Seera as RS
            import Seera_Engine as RE
        yield types.SimpleNamespace(S=RS, E=RE, sc=sc, cuten=ct.cuten)
    finally:
        sc.set_precision(0)
        sys.path.remove(REF_PY)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _c1_model(ref, seed):
    RS = ref.S
    work = wl.c1_small_cnn()
    layers = [RS.Input((1, 28, 28))]
    for L, P in zip(work.layers, work.params(seed)):
        lay = {"conv": lambda: RS.Conv2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"]),
               "maxpool": lambda: RS.MaxPool2D(L["k"], stride=L["stride"], padding=L["pad"]),
               "flatten": lambda: RS.Flatten(),
               "dense": lambda: RS.Dense(L["in"], L["out"], activation=L["act"])}[L["type"]]()
        if P is not None:
            lay.set_weights(P[0].copy(), P[1].copy())
        layers.append(lay)
    return work, RS.Sequential(layers, device="cuda")


def _step(ref, model, opt, X, Y, precision):
    RT = ref.E.Tensor
    if precision is not None:
        ref.sc.set_precision(precision[0])
    yp = model.forward(RT(X, is_leaf=True, device="cuda"))
    loss = ref.S.Loss().categorical_cross_entropy(yp, RT(Y, device="cuda"))
    lv = float(loss.value.to_host_f32().ravel()[0])
    model.zero_grad()
    if precision is not None:
        ref.sc.set_precision(precision[1])
    ref.E.autograd4nn(loss)
    return lv


@pytest.mark.parametrize("precision,tol", [((0, 0), 5e-5), ((3, 2), 2e-3)])
def test_reference_python_layer_trains_c1_on_this_engine(ref, golden_dir, precision, tol):
    """Two steps of C1 through the unmodified reference driver: loss, every gradient, every updated weight against the
    reference's CPU path.  Exact-fp32 mode agrees to summation order; the tensor-core policy to the 2e-3 gate."""
    work, model = _c1_model(ref, 1)
    X, Y = work.batch(64, 1)
    opt = ref.S.Adam(model, lr=1e-3)
    gold = np.load(golden_dir + "/c1_two_steps.npz")
    for s in range(2):
        lv = _step(ref, model, opt, X, Y, precision)
        assert abs(lv - float(gold["loss%d" % s])) < tol * max(1.0, abs(float(gold["loss%d" % s])))
        plist = [lay for lay in model.model if hasattr(lay, "update_params")]
        if s == 0:
            for k, lay in enumerate(plist):
                assert rel_l2(lay.weights.node.cp.to_host_f32(), gold["dW%d" % k]) < tol, ("dW", k)
                assert rel_l2(lay.bais.node.cp.to_host_f32().ravel(), gold["db%d" % k].ravel()) < tol, ("db", k)
        opt.step()
        for k, lay in enumerate(plist):
            assert rel_l2(lay.weights.value.to_host_f32(), gold["W%d_s%d" % (k, s)]) < tol, ("W", k, s)
    assert ref.sc.tc_device_status() == 0


def test_boundary_calls_and_time_of_one_dropin_step(ref, capsys):
    """What the unmodified path costs per step on this engine: boundary calls (every `seera_cuda` function the
    reference's Python layer invokes), kernel launches, wall time with a synchronise at the end."""
    work, model = _c1_model(ref, 2)
    X, Y = work.batch(64, 2)
    opt = ref.S.Adam(model, lr=1e-3)
    sc = ref.sc
    for _ in range(3):
        _step(ref, model, opt, X, Y, (0, 0))
        opt.step()
    calls = {"n": 0}
    mod = sys.modules["seera_cuda"]
    originals = {k: getattr(mod, k) for k in dir(mod) if callable(getattr(mod, k)) and not k.startswith("_")}

    def counted(fn):
        def inner(*a, **kw):
            calls["n"] += 1
            return fn(*a, **kw)
        return inner
    try:
        for k, fn in originals.items():
            setattr(mod, k, counted(fn))
        l0 = originals["launch_count"]()
        _step(ref, model, opt, X, Y, (0, 0))
        opt.step()
        originals["stream_synchronize"]()
        n_calls, n_launch = calls["n"], originals["launch_count"]() - l0
    finally:
        for k, fn in originals.items():
            setattr(mod, k, fn)
    sc.stream_synchronize()
    t0 = time.perf_counter()
    for _ in range(5):
        _step(ref, model, opt, X, Y, (0, 0))
        opt.step()
    sc.stream_synchronize()
    ms = (time.perf_counter() - t0) / 5 * 1e3
    with capsys.disabled():
        print("\n[drop-in C1 b64] boundary calls/step %d, kernel launches/step %d, %.2f ms/step (unmodified Seera.py + "
              "Seera_Engine.py + composed Adam over this engine)" % (n_calls, n_launch, ms))
    out = os.environ.get("SEERA_TEST_REPORT_DIR")
    if out and os.path.isdir(out):
        with open(os.path.join(out, "dropin_c1.txt"), "w") as f:
            f.write("calls_per_step %d launches_per_step %d ms_per_step %.3f\n" % (n_calls, n_launch, ms))
    assert n_calls > 100 and n_launch > 0


# ---- cuten semantics the reference's own scripts pin ------------------------------------------------------------
def test_operators_have_value_semantics(ref):
    """g*5, g+10, g**2, -g, g-1, g/2 and the reflected forms leave g untouched and return the right values."""
    cuten = ref.cuten
    data = np.array([[1.0, 2.0, 3.0], [-4.0, 0.5, 6.0]], np.float32)
    other = np.array([[2.0, 0.5, -1.0], [3.0, 4.0, 0.25]], np.float32)
    ops = [(lambda g: g * 5.0, data * 5.0), (lambda g: g + 10.0, data + 10.0), (lambda g: g ** 2.0, data ** 2.0),
           (lambda g: -g, -data), (lambda g: g - 1.5, data - 1.5), (lambda g: g / 2.0, data / 2.0),
           (lambda g: 5.0 * g, 5.0 * data), (lambda g: 10.0 + g, 10.0 + data), (lambda g: 1.5 - g, 1.5 - data),
           (lambda g: g + cuten(other), data + other), (lambda g: g * cuten(other), data * other),
           (lambda g: g - cuten(other), data - other), (lambda g: g / cuten(other), data / other),
           (lambda g: cuten.zeros_like(g) + g, data), (lambda g: g * cuten.ones_like(g), data)]
    for i, (op, want) in enumerate(ops):
        g = cuten(data.copy())
        res = op(g)
        assert np.array_equal(g.to_host_f32(), data), ("operand changed", i)
        assert np.allclose(res.to_host_f32(), want, rtol=1e-6, atol=0), ("value", i)
    # a result that aliases its operand (0 + g) must not be changed by later arithmetic on either
    g = cuten(data.copy())
    alias = cuten.zeros_like(g) + g
    h = alias * 3.0
    assert np.array_equal(alias.to_host_f32(), data) and np.array_equal(g.to_host_f32(), data)
    assert np.allclose(h.to_host_f32(), data * 3.0)


def test_reduce_grad_gpu_shapes_and_values(ref):
    AG = ref.E.autograd4nn
    rs = np.random.RandomState(11)
    for src, tgt in [((8, 16), (1, 16)), ((4, 8, 16), (8, 16)), ((4, 1, 16), (1, 1, 16)), ((8,), (1,)),
                     ((6, 5, 4, 3), (1, 5, 1, 1))]:
        a = rs.standard_normal(src).astype(np.float32)
        r = AG._reduce_grad_gpu(ref.cuten(a), tgt)
        assert tuple(r.shape) == tgt, (src, tgt, r.shape)
        pad = (1,) * (len(src) - len(tgt)) + tgt
        want = a.sum(axis=tuple(i for i, s in enumerate(pad) if s == 1)).reshape(tgt)
        assert rel_l2(r.to_host_f32().reshape(tgt), want) < 1e-5


@pytest.mark.parametrize("M,K,N", [(1, 3, 2), (2, 5, 7), (7, 13, 3), (17, 33, 65), (32, 400, 256), (31, 17, 2)])
def test_cuten_matmul_small_and_odd_sizes(ref, M, K, N):
    rs = np.random.RandomState(M * 100 + N)
    A, B = rs.standard_normal((M, K)).astype(np.float32), rs.standard_normal((K, N)).astype(np.float32)
    got = (ref.cuten(A) @ ref.cuten(B)).to_host_f32()
    assert got.shape == (M, N) and rel_l2(got, A.astype(np.float64) @ B) < 2e-5
    # batched form: A 3-D (Nbatch, M, K), B shared
    A3 = rs.standard_normal((3, M, K)).astype(np.float32)
    got3 = ref.cuten(A3).matmul(ref.cuten(B)).to_host_f32()
    assert got3.shape == (3, M, N) and rel_l2(got3, A3.astype(np.float64) @ B) < 2e-5


def test_views_transposes_and_reductions(ref):
    cuten = ref.cuten
    rs = np.random.RandomState(5)
    a = rs.standard_normal((4, 6, 5)).astype(np.float32)
    t = cuten(a)
    v = t.reshape((24, 5))
    f = t.flatten()
    del t                                   # the views must keep the memory alive
    junk = [cuten(rs.standard_normal(120).astype(np.float32)) for _ in range(8)]      # would recycle a freed block
    assert np.array_equal(v.to_host_f32(), a.reshape(24, 5)) and np.array_equal(f.to_host_f32().ravel(), a.ravel())
    del junk
    m = rs.standard_normal((7, 9)).astype(np.float32)
    assert np.array_equal(cuten(m).T.to_host_f32(), m.T)
    b3 = rs.standard_normal((3, 4, 5)).astype(np.float32)
    assert np.array_equal(cuten(b3).T.to_host_f32(), b3.transpose(0, 2, 1))
    for dim in range(3):
        assert rel_l2(cuten(a).sum(dim).to_host_f32(), a.sum(axis=dim)) < 1e-6
        assert rel_l2(cuten(a).mean(dim).to_host_f32(), a.mean(axis=dim)) < 1e-6
        assert np.array_equal(cuten(a).max(dim).to_host_f32().reshape(a.max(axis=dim).shape), a.max(axis=dim))
        assert np.array_equal(cuten(a).min(dim).to_host_f32().reshape(a.min(axis=dim).shape), a.min(axis=dim))
    s = cuten(m).softmax().to_host_f32()
    e = np.exp(m - m.max(axis=1, keepdims=True))
    assert rel_l2(s, e / e.sum(axis=1, keepdims=True)) < 1e-6


def test_cuten_layer_methods_against_the_cpu_engine(ref):
    """conv2d, maxpool2d, unpool, conv2d_transpose as methods of the tensor class, against the CPU oracle."""
    from oracle import cpu_oracle as co
    cuten = ref.cuten
    rs = np.random.RandomState(8)
    x = rs.standard_normal((2, 3, 8, 8)).astype(np.float32)
    w = rs.standard_normal((4, 3, 3, 3)).astype(np.float32)
    y = cuten(x).conv2d(cuten(w), 1, 1, 1, 1)
    assert rel_l2(y.to_host_f32(), co.conv2d_forward(x, w, 1, 1, 1, 1)) < 2e-5
    out, mask = cuten(x).maxpool2d(2, 2, 2, 2, 0, 0)
    ro, rm = co.maxpool2d_forward(x, 2, 2, 2, 2, 0, 0)
    assert np.array_equal(out.to_host_f32(), ro)
    assert np.array_equal(mask.to_host_i32().ravel()[:ro.size], np.asarray(rm, np.int32).ravel())
    up = cuten(ro).unpool(2, 2)
    assert np.array_equal(up.to_host_f32(), co.unpooling_forward(ro, 2, 2))
    wt = rs.standard_normal((3, 5, 4, 4)).astype(np.float32)
    yt = cuten(x).conv2d_transpose(cuten(wt), 2, 2, 1, 1)
    assert rel_l2(yt.to_host_f32(), co.conv_transpose2d_forward(x, wt, 2, 2, 1, 1)) < 2e-5
