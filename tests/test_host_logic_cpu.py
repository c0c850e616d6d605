"""CPU tests of the Python host logic (tensor class, layer autograd, arenas, optimizers) on a
host-memory stand-in for the device binding (tests/fake_seera_cuda.py).  No GPU, no product
fallback: the stand-in is installed by a fixture for these tests only."""
import importlib
import os
import sys
import types

import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co
from oracle.train_oracle import RefNet
import cases

REFERENCE = os.environ.get("SEERA_REFERENCE", "/root/reference")


@pytest.fixture(scope="module")
def host():
    """Package modules re-imported over the fake binding; restored afterwards."""
    import fake_seera_cuda as fake
    import ml_framework_b200 as pkg
    names = ["ml_framework_b200.seera_cuda", "ml_framework_b200.cuTen", "ml_framework_b200.seera", "ml_framework_b200.train"]
    saved = {n: sys.modules.pop(n, None) for n in names}
    saved_attr = getattr(pkg, "seera_cuda", None)
    sys.modules["ml_framework_b200.seera_cuda"] = fake
    pkg.seera_cuda = fake
    ns = types.SimpleNamespace(fake=fake,
                               cuTen=importlib.import_module("ml_framework_b200.cuTen"),
                               seera=importlib.import_module("ml_framework_b200.seera"),
                               train=importlib.import_module("ml_framework_b200.train"))
    yield ns
    for n in names:
        sys.modules.pop(n, None)
        if saved[n] is not None:
            sys.modules[n] = saved[n]
    if saved_attr is not None:
        pkg.seera_cuda = saved_attr
    elif hasattr(pkg, "seera_cuda"):
        del pkg.seera_cuda


def test_lazy_constants_allocate_nothing(host):
    host.fake.reset()
    ct = host.cuTen.cuten
    x = ct(np.arange(6, dtype=np.float32).reshape(2, 3))
    before = dict(host.fake.CALLS)
    z, o = ct.zeros_like(x), ct.ones_like(x)
    s = (z + x)
    m = (o * x)
    assert host.fake.CALLS == before                      # no allocation, no kernel
    assert s.main_ptr == x.main_ptr and m.main_ptr == x.main_ptr and s is not x
    assert np.array_equal(z.to_host_f32(), np.zeros((2, 3), np.float32))
    assert np.array_equal((o * 3.0).to_host_f32(), np.full((2, 3), 3, np.float32))
    assert z.main_ptr is not None                         # materialises on demand
    assert np.array_equal(host.fake.to_host_f32(z.main_ptr, (2, 3)), np.zeros((2, 3), np.float32))


def test_operators_have_value_semantics(host):
    ct = host.cuTen.cuten
    g = ct(np.array([[1.0, -2.0], [3.0, 4.0]], np.float32))
    ref = g.to_host_f32()
    assert np.allclose((g * 5.0).to_host_f32(), ref * 5)
    assert np.allclose((g + 10.0).to_host_f32(), ref + 10)
    assert np.allclose((g ** 2.0).to_host_f32(), ref ** 2)
    assert np.allclose((-g).to_host_f32(), -ref)
    assert np.allclose((g - g).to_host_f32(), 0)
    assert np.allclose((1.0 - g).to_host_f32(), 1 - ref)
    assert np.allclose((g / g).to_host_f32(), 1)
    assert np.array_equal(g.to_host_f32(), ref)           # g untouched
    b = ct(np.array([[10.0, 20.0]], np.float32))
    assert np.allclose((g + b).to_host_f32(), ref + [[10, 20]])
    assert np.allclose((g * b).to_host_f32(), ref * [[10, 20]])
    assert (g @ ct(np.eye(2, dtype=np.float32))).shape == (2, 2)
    assert np.allclose(g.T.to_host_f32(), ref.T)
    with pytest.raises(ValueError):
        g + ct(np.ones((3, 3), np.float32))
    with pytest.raises(ValueError):
        g.reshape((3,))
    with pytest.raises(ValueError):
        ct(np.ones(2), dtype="float64")


def test_views_keep_owner_alive_and_memory_is_returned(host):
    host.fake.reset()
    ct = host.cuTen.cuten
    a = ct(np.ones((4, 3), np.float32))
    p = a.main_ptr
    v = a.flatten().reshape((3, 4))
    del a
    assert p in host.fake.LIVE and v.main_ptr == p
    assert np.array_equal(v.to_host_f32(), np.ones((3, 4), np.float32))
    del v
    assert p not in host.fake.LIVE


def _run_trainer(host, work, n, seed, steps=2):
    tr = host.train.Trainer(work, seed=seed)
    X, Y = work.batch(n, seed)
    ref = RefNet(work.layers, work.params(seed), work.loss, work.opt, co)
    for s in range(steps):
        loss = tr.forward_backward(X, Y)
        got_grads = tr.host_grads()
        tr.opt.step()
        P = ref.forward(X)
        rl, dP = ref.loss_and_grad(P, Y)
        rg = ref.backward(dP)
        ref.apply(rg)
        assert abs(float(loss.value.to_host_f32()[0]) - float(rl)) < 1e-5 * max(1, abs(float(rl)))
        assert rel_l2(tr.pred.to_numpy(), P) < 1e-5
        for G, R in zip(got_grads, rg):
            if R is not None:
                assert rel_l2(G[0], R[0]) < 2e-5 and rel_l2(G[1].ravel(), R[1].ravel()) < 2e-5
        for Pm, Rm in zip(tr.host_params(), ref.params):
            if Rm is not None:
                assert rel_l2(Pm[0], Rm[0]) < 1e-5 and rel_l2(Pm[1].ravel(), Rm[1].ravel()) < 1e-3 + 1e-9
    return tr


@pytest.mark.parametrize("case", ["c2s", "c3s", "c4s"])
def test_layer_autograd_matches_step_oracle(host, case):
    work, n = cases.small_cases()[case]
    _run_trainer(host, work, n, seed=2)


def test_gradients_accumulate_without_zero_grad_and_addresses_are_stable(host):
    work, n = cases.small_cases()["c2s"]
    tr = host.train.Trainer(work, seed=2)
    X, Y = work.batch(n, 2)
    w_ptr = tr.model.param_layers[0].weights.value.main_ptr
    tr.forward_backward(X, Y)
    g1 = tr.host_grads()[0][0].copy()
    S = host.seera
    pred = tr.model.forward(S.Tensor(X, is_leaf=True))
    loss = tr.lossf(pred, S.Tensor(Y, is_leaf=True))
    S.autograd4nn(loss)                                   # no zero_grad: must add
    g2 = tr.host_grads()[0][0]
    assert rel_l2(g2, 2 * g1) < 1e-6
    tr.opt.step()
    assert tr.model.param_layers[0].weights.value.main_ptr == w_ptr


def test_api_errors_match_the_reference(host):
    S = host.seera
    with pytest.raises(ValueError):
        S.Dense(4, 4, activation="gelu")
    with pytest.raises(ValueError):
        S.Dense(4, 4, activation="relu", kernel_initializer="nope")
    with pytest.raises(TypeError):
        S.Sequential((S.Input((4,)),))
    with pytest.raises(TypeError):
        S.Sequential([S.Dense(4, 4, activation="relu")])
    with pytest.raises(TypeError):
        S.SGD(object(), lr=0.1)
    with pytest.raises(ValueError):
        S.MaxPool2D(pool_size=2)
    with pytest.raises(ValueError):
        S.Sequential([S.Input((4,)), S.Dense(4, 4, activation="relu")], device="cpu")


def test_save_load_round_trip(host, tmp_path):
    work, n = cases.small_cases()["c3s"]
    tr = host.train.Trainer(work, seed=2)
    f = str(tmp_path / "m.pkl")
    tr.model.save(f)
    m2 = host.seera.Sequential.load(f)
    X, _ = work.batch(n, 2)
    a = tr.model.forward(host.seera.Tensor(X, is_leaf=True)).to_numpy()
    b = m2.forward(host.seera.Tensor(X, is_leaf=True)).to_numpy()
    assert np.array_equal(a, b)


def _bn_model_against_golden(S, golden_dir, tol):
    """Two SGD steps and an evaluation-mode prediction of the BatchNorm model against the unmodified reference."""
    sys.path.insert(0, golden_dir)
    import bn_case
    gold = np.load(os.path.join(golden_dir, "bn_two_steps.npz"))
    lays = bn_case.layers(S)
    for i, (W, B) in bn_case.weights().items():
        lays[i].set_weights(W, B)
    model = S.Sequential(lays, device="cuda")
    opt = S.SGD(model, lr=bn_case.LR, momentum=bn_case.MOMENTUM)
    lossf = S.Loss().categorical_cross_entropy
    X, Y = bn_case.data()
    rel = lambda a, b: float(np.linalg.norm(np.asarray(a, np.float64).ravel() - np.asarray(b, np.float64).ravel()) /
                             max(np.linalg.norm(np.asarray(b, np.float64).ravel()), 1e-12))
    plist = [l for l in model.model if isinstance(l, S._ParamLayer)]
    for s in range(bn_case.STEPS):
        yp = model.forward(S.Tensor(X, is_leaf=True))
        loss = lossf(yp, S.Tensor(Y, is_leaf=True))
        model.zero_grad()
        S.autograd4nn(loss)
        assert abs(float(loss.value.to_host_f32().ravel()[0]) - float(gold["loss%d" % s])) < tol * max(1.0, float(gold["loss%d" % s]))
        if s == 0:
            assert rel(yp.to_numpy(), gold["pred0"]) < tol
            model.gather_grads()
            for k, l in enumerate(plist):
                assert rel(l.weights.grad.to_host_f32(), gold["dW%d" % k]) < tol, ("dW", k)
                assert rel(l.bais.grad.to_host_f32(), gold["db%d" % k]) < tol, ("db", k)
        opt.step()
        for k, l in enumerate(plist):
            assert rel(l.weights.to_numpy(), gold["W%d_s%d" % (k, s)]) < tol, ("W", k, s)
            assert rel(l.bais.to_numpy(), gold["b%d_s%d" % (k, s)]) < tol, ("b", k, s)
    assert rel(lays[2].running_mean, gold["rm2"]) < tol and rel(lays[2].running_var, gold["rv2"]) < tol
    assert rel(lays[6].running_mean, gold["rm6"]) < tol and rel(lays[6].running_var, gold["rv6"]) < tol
    assert rel(model.predict(S.Tensor(X, is_leaf=True)).to_numpy(), gold["pred_eval"]) < tol
    assert lays[2].training and lays[6].training                      # predict() restores training mode


def test_batchnorm_layers_against_reference_golden(host, golden_dir):
    _bn_model_against_golden(host.seera, golden_dir, 2e-5)


def test_batchnorm_with_cross_rank_statistics_is_the_plain_layer_on_one_rank(host, golden_dir):
    """`sync=True` routes the layer through the cross-rank entries; with a single rank they are the plain ones, so the model
    still reproduces the reference's golden (the two-rank case runs on two GPUs: tests/test_gpu_dp_batchnorm.py)."""
    S = host.seera
    plain1d, plain2d = S.BatchNorm1d, S.BatchNorm2d

    class Sync1d(plain1d):
        def __init__(self, *a, **k):
            super().__init__(*a, sync=True, **k)

    class Sync2d(plain2d):
        def __init__(self, *a, **k):
            super().__init__(*a, sync=True, **k)
    S.BatchNorm1d, S.BatchNorm2d = Sync1d, Sync2d
    try:
        _bn_model_against_golden(S, golden_dir, 2e-5)
    finally:
        S.BatchNorm1d, S.BatchNorm2d = plain1d, plain2d


@pytest.mark.parametrize("kind", ["adam", "sgd"])
def test_checkpoint_with_optimizer_state_resumes_exactly(host, tmp_path, kind):
    """Two steps, save with the optimizer, load, one more step == three steps straight (weights bit-equal); a non-zero
    rank writes nothing."""
    S = host.seera
    work, n = cases.small_cases()["c3s"]
    X, Y = work.batch(n, 4)

    def make():
        m = host.train.build_model(work, work.params(6))
        return m, (S.Adam(m, lr=1e-3) if kind == "adam" else S.SGD(m, lr=1e-2, momentum=0.9))

    def step(m, o):
        loss = S.Loss().categorical_cross_entropy(m.forward(S.Tensor(X, is_leaf=True)), S.Tensor(Y, is_leaf=True))
        m.zero_grad()
        S.autograd4nn(loss)
        o.step()
    a, oa = make()
    for _ in range(3):
        step(a, oa)
    b, ob = make()
    for _ in range(2):
        step(b, ob)
    f = str(tmp_path / "ck.pkl")
    b.save(str(tmp_path / "none.pkl"), optimizer=ob, rank=1)
    assert not os.path.exists(str(tmp_path / "none.pkl"))
    b.save(f, optimizer=ob)
    c, oc = S.Sequential.load(f, with_optimizer=True)
    assert type(oc) is type(ob)
    step(c, oc)
    for la, lc in zip(a.param_layers, c.param_layers):
        assert np.array_equal(la.weights.to_numpy(), lc.weights.to_numpy()) and np.array_equal(la.bais.to_numpy(), lc.bais.to_numpy())
    assert S.Sequential.load(f).n_arena == a.n_arena                   # plain load ignores the optimizer record


def test_concatenate_layer_joins_and_splits(host):
    """Concatenate of two branches (4-D and 2-D): forward equals np.concatenate along axis 1, backward hands each branch
    its slice of the gradient; one concat launch per direction."""
    S, ct = host.seera, host.cuTen.cuten
    rs = np.random.RandomState(0)
    for sa, sb in (((3, 2, 4, 4), (3, 5, 4, 4)), ((6, 7), (6, 3))):
        A, B = rs.standard_normal(sa).astype(np.float32), rs.standard_normal(sb).astype(np.float32)
        la, lb = S.Input(sa[1:]), S.Input(sb[1:])
        la.inputs, lb.inputs = S.Tensor(A), S.Tensor(B)          # not leaves: they take gradients
        la.forward(); lb.forward()
        cat = S.Concatenate()(la, lb)
        before = dict(host.fake.CALLS)
        out = cat.forward()
        assert np.array_equal(out.to_numpy(), np.concatenate([A, B], axis=1))
        G = rs.standard_normal(out.shape).astype(np.float32)
        out._backward(ct(G))
        assert np.array_equal(la.outputs.grad.to_host_f32(), G[:, :sa[1]]) and np.array_equal(lb.outputs.grad.to_host_f32(), G[:, sa[1]:])
        assert host.fake.CALLS.get("concat_fwd", 0) - before.get("concat_fwd", 0) == 1
        assert host.fake.CALLS.get("concat_bwd", 0) - before.get("concat_bwd", 0) == 1
    with pytest.raises(ValueError):
        S.Concatenate()(la)


def test_fit_pipeline_matches_the_synchronous_loop(host):
    """Sequential.fit (double-buffered staging, loss read one step late, last batch ragged) gives the history and the
    weights of the synchronous loop; integer labels expanded on the device give the same as host one-hot rows."""
    S = host.seera
    rs = np.random.RandomState(3)
    X = rs.standard_normal((37, 1, 6, 6)).astype(np.float32)
    lab = rs.randint(0, 5, 37).astype(np.int32)
    Y = np.eye(5, dtype=np.float32)[lab]

    def make():
        np.random.seed(11)
        m = S.Sequential([S.Input((1, 6, 6)), S.Conv2D(4, 1, (3, 3), "relu", stride=1, zero_padding=1), S.MaxPool2D((2, 2), stride=2),
                          S.Flatten(), S.Dense(36, 5, activation="softmax")], device="cuda")
        return m, S.Adam(m, lr=1e-2), S.Loss().categorical_cross_entropy
    runs = []
    for mode in ("sync", "pipe", "labels"):
        m, opt, loss = make()
        np.random.seed(5)                               # the epoch shuffles
        if mode == "sync":
            h = m._fit_unpipelined(X, Y, opt, loss, Epochs=2, batch_size=8)
        elif mode == "pipe":
            h = m.fit(X, Y, opt, loss, Epochs=2, batch_size=8, Loss_interval=100)
        else:
            h = m.fit(X, lab, opt, loss, Epochs=2, batch_size=8, Loss_interval=100, num_classes=5)
        runs.append((h, [(l.weights.to_numpy(), l.bais.to_numpy()) for l in m.model if isinstance(l, S._ParamLayer)]))
    for h, ws in runs[1:]:
        assert np.array_equal(h, runs[0][0])
        for (w, b), (w0, b0) in zip(ws, runs[0][1]):
            assert np.array_equal(w, w0) and np.array_equal(b, b0)


def test_fit_history_matches_the_reference_fit(host, golden_dir):
    """`Sequential.fit` against the loss history of the reference's own `fit` (Seera.py:729-788) on the same data, initial
    weights and shuffling seed (tests/golden/make_golden_fit.py)."""
    import fit_case
    gold = np.load(golden_dir + "/fit_c1.npz")
    S = host.seera
    m = fit_case.build(S, device="cuda")
    X, Y = fit_case.data()
    np.random.seed(fit_case.SHUFFLE_SEED)
    h = m.fit(X, Y, S.Adam(m, lr=fit_case.LR), S.Loss().categorical_cross_entropy, Epochs=fit_case.EPOCHS,
              batch_size=fit_case.BATCH, Loss_interval=100)
    assert np.max(np.abs(h - gold["history"])) < 1e-4, (h, gold["history"])
    assert rel_l2(m.forward(X[:fit_case.BATCH]).to_numpy(), gold["pred"]) < 1e-4


def test_checkpoint_written_by_the_reference_loads_and_predicts(host, golden_dir):
    """A pickle written by the reference's `Sequential.save` (Seera.py:790-860) loads unchanged and predicts what the
    reference's trained model predicted."""
    import fit_case
    gold = np.load(golden_dir + "/fit_c1.npz")
    S = host.seera
    m = S.Sequential.load(golden_dir + "/ref_c1_checkpoint.pkl")
    X, _ = fit_case.data()
    assert [l.__class__.__name__ for l in m.model] == ["Input", "Conv2D", "MaxPool2D", "Conv2D", "MaxPool2D", "Flatten", "Dense"]
    assert rel_l2(m.predict(X[:fit_case.BATCH]).to_numpy(), gold["pred"]) < 1e-5


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="reference checkout not present")
def test_unmodified_reference_python_layer_runs_on_this_cuten(host, golden_dir):
    """Drop-in check of the tensor class: the reference's own Seera.py / Seera_init.py /
    Seera_Engine.py, device="cuda", over this package's cuTen and the stand-in binding."""
    from ml_framework_b200 import workloads as wl
    saved = {k: sys.modules.get(k) for k in ("seera_cuda", "cuTen", "matplotlib", "matplotlib.pyplot",
                                             "Seera", "Seera_init", "Seera_Engine", "seera_cpp")}
    try:
        for k in ("Seera", "Seera_init", "Seera_Engine"):
            sys.modules.pop(k, None)
        sys.modules["seera_cuda"] = host.fake
        sys.modules["cuTen"] = host.cuTen
        mpl = types.ModuleType("matplotlib"); mpl.pyplot = types.ModuleType("matplotlib.pyplot")
        sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot
        sys.modules["seera_cpp"] = None                   # force the reference's own NumPy path off the table
        sys.path.insert(0, REFERENCE)
        import Seera as RS
        from Seera_Engine import Tensor as RT, autograd4nn as rauto
        work = wl.c1_small_cnn()
        params = work.params(1)
        layers = [RS.Input((1, 28, 28))]
        for L, P in zip(work.layers, params):
            t = L["type"]
            lay = {"conv": lambda: RS.Conv2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"]),
                   "maxpool": lambda: RS.MaxPool2D(L["k"], stride=L["stride"], padding=L["pad"]),
                   "flatten": lambda: RS.Flatten(),
                   "dense": lambda: RS.Dense(L["in"], L["out"], activation=L["act"])}[t]()
            if P is not None:
                lay.set_weights(P[0].copy(), P[1].copy())
            layers.append(lay)
        model = RS.Sequential(layers, device="cuda")
        X, Y = work.batch(64, 1)
        opt = RS.Adam(model, lr=1e-3)
        gold = np.load(golden_dir + "/c1_two_steps.npz")
        host.fake.reset_calls = host.fake.CALLS.clear()
        for s in range(2):
            yp = model.forward(RT(X, is_leaf=True, device="cuda"))
            loss = RS.Loss().categorical_cross_entropy(yp, RT(Y, device="cuda"))
            lv = float(loss.value.to_host_f32().ravel()[0])
            model.zero_grad()
            rauto(loss)
            assert abs(lv - float(gold["loss%d" % s])) < 2e-5
            if s == 0:
                k = 0
                for lay in model.model:
                    if hasattr(lay, "update_params"):
                        assert rel_l2(lay.weights.node.cp.to_host_f32(), gold["dW%d" % k]) < 2e-5
                        assert rel_l2(lay.bais.node.cp.to_host_f32().ravel(), gold["db%d" % k].ravel()) < 2e-5
                        k += 1
            opt.step()
            k = 0
            for lay in model.model:
                if hasattr(lay, "update_params"):
                    assert rel_l2(lay.weights.value.to_host_f32(), gold["W%d_s%d" % (k, s)]) < 2e-5
                    k += 1
        # the lazy constants keep host->device uploads to the real inputs
        assert host.fake.CALLS.get("to_device", 0) < 40
    finally:
        if REFERENCE in sys.path:
            sys.path.remove(REFERENCE)
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v
