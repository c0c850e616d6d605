"""GPU parity of whole training steps (forward, loss, backward, optimizer) through the Python front
end, against golden vectors of the unmodified reference and against the CPU step oracle at the
configurations' full sizes.

Gates (relative L2 per tensor): loss, every gradient and every updated weight within 2e-3 after one
step; loss within 1e-2 after 100 steps.  In fp32 mode the observed errors are ~1e-6."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co
from oracle import ref_engine
from oracle.train_oracle import RefNet
from ml_framework_b200 import workloads as wl
import cases

pytestmark = pytest.mark.gpu

GATE = 2e-3


@pytest.fixture(scope="module")
def T():
    from ml_framework_b200 import train, seera_cuda as sc
    sc.init(0)
    sc.set_precision(0)
    return train


def _against_golden(T, work, n, seed, gold, tol):
    tr = T.Trainer(work, seed=seed)
    X, Y = work.batch(n, seed)
    for s in range(2):
        loss = tr.forward_backward(X, Y)
        lv = float(loss.value.to_host_f32()[0])
        assert abs(lv - float(gold["loss%d" % s])) <= tol * max(1.0, abs(float(gold["loss%d" % s])))
        if s == 0:
            assert rel_l2(tr.pred.to_numpy(), gold["pred0"]) < tol
            k = 0
            for G in tr.host_grads():
                if G is not None:
                    assert rel_l2(G[0], gold["dW%d" % k]) < tol, ("dW", k)
                    assert rel_l2(G[1].ravel(), gold["db%d" % k].ravel()) < tol, ("db", k)
                    k += 1
        tr.opt.step()
        k = 0
        for P in tr.host_params():
            if P is not None:
                assert rel_l2(P[0], gold["W%d_s%d" % (k, s)]) < tol, ("W", k, s)
                assert np.max(np.abs(P[1].ravel() - gold["b%d_s%d" % (k, s)].ravel())) < 1e-5, ("b", k, s)
                k += 1


def test_c1_two_steps_against_reference_golden(T, golden_dir):
    _against_golden(T, wl.c1_small_cnn(), 64, 1, np.load(golden_dir + "/c1_two_steps.npz"), 5e-5)


@pytest.mark.parametrize("case", ["c2s", "c3s", "c4s"])
def test_small_configs_against_reference_golden(T, case, golden_dir):
    work, n = cases.small_cases()[case]
    _against_golden(T, work, n, 2, np.load(golden_dir + "/%s_two_steps.npz" % case), 5e-5)


def _engine():
    return ref_engine.load() or co


@pytest.mark.parametrize("name,n", [("c1", 64), ("c2", 512), ("c3", 32), ("c4", 16)])
def test_one_step_at_config_shapes_against_step_oracle(T, name, n):
    """Full layer shapes of each configuration, batch reduced so the CPU oracle finishes in seconds."""
    work = wl.WORKLOADS[name]()
    tr = T.Trainer(work, seed=3)
    X, Y = work.batch(n, 3)
    ref = RefNet(work.layers, work.params(3), work.loss, work.opt, _engine())
    loss = tr.forward_backward(X, Y)
    grads = tr.host_grads()
    tr.opt.step()
    rl = ref.step(X, Y)
    assert abs(float(loss.value.to_host_f32()[0]) - rl) <= GATE * max(1.0, abs(rl))
    for G, R in zip(grads, ref.grads):
        if R is not None:
            assert rel_l2(G[0], R[0]) < GATE and rel_l2(G[1].ravel(), R[1].ravel()) < GATE
    for P, R in zip(tr.host_params(), ref.params):
        if R is not None:
            assert rel_l2(P[0], R[0]) < GATE


def test_c1_loss_after_100_steps(T):
    work = wl.c1_small_cnn()
    tr = T.Trainer(work, seed=4)
    ref = RefNet(work.layers, work.params(4), work.loss, work.opt, _engine())
    X, Y = work.batch(64, 4)
    for _ in range(100):
        loss = tr.step(X, Y)
        rl = ref.step(X, Y)
    lv = float(loss.value.to_host_f32()[0])
    assert abs(lv - rl) <= 1e-2 and lv < 2.0              # and it has actually learned the batch


def test_full_size_properties(T):
    """At the bench configuration's full batch the oracle is too slow; check size-independent properties:
    the step is deterministic run to run, and gradients are additive over a split of the batch."""
    work = wl.c3_vgg()
    X, Y = work.batch(512, 9)
    outs = []
    for _ in range(2):
        tr = T.Trainer(work, seed=9)
        tr.forward_backward(X, Y)
        outs.append(tr.host_grads())
    for A, B in zip(*outs):
        if A is not None:
            assert np.array_equal(A[0], B[0]) and np.array_equal(A[1], B[1])
    halves = []
    for sl in (slice(0, 256), slice(256, 512)):
        tr = T.Trainer(work, seed=9)
        tr.forward_backward(X[sl], Y[sl])
        halves.append(tr.host_grads())
    for F, A, B in zip(outs[0], *halves):
        if F is not None:
            assert rel_l2(F[0], 0.5 * (A[0] + B[0])) < 1e-4   # each half's loss is a mean over 256


@pytest.mark.parametrize("name,n,mode", [("c1", 64, 0), ("c2", 256, 1), ("c3", 16, 2)])
def test_captured_step_graph_replays_like_eager_steps(T, name, n, mode):
    """A CUDA graph of the whole step, replayed k times, gives the weights k eager steps give (bit for bit:
    same kernels, same order, deterministic reductions)."""
    from ml_framework_b200 import seera as S, seera_cuda as sc
    sc.set_precision(mode)
    work = wl.WORKLOADS[name]()
    X, Y = work.batch(n, 5)
    a, b = T.Trainer(work, seed=5), T.Trainer(work, seed=5)
    Xa, Ya = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)
    Xb, Yb = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)
    for _ in range(2):
        a.step(Xa, Ya)
        b.step(Xb, Yb)
    for _ in range(4):
        la = a.step(Xa, Ya)
    lb = b.capture(Xb, Yb)          # recording executes nothing
    for _ in range(4):
        lb = b.replay()
    assert float(la.value.to_host_f32()[0]) == float(lb.value.to_host_f32()[0])
    for Pa, Pb in zip(a.host_params(), b.host_params()):
        if Pa is not None:
            assert np.array_equal(Pa[0], Pb[0]) and np.array_equal(Pa[1], Pb[1])
    b.release_graph()
    sc.set_precision(0)
    assert sc.tc_device_status() == 0


def test_streamed_batches_match_step_by_step_uploads(T):
    """fit_stream (next batch uploaded and previous loss read back on the copy stream while a step runs) gives the
    losses and weights of upload -> replay -> read, batch by batch, bit for bit."""
    import ctypes
    from ml_framework_b200 import seera as S, seera_cuda as sc
    sc.set_precision(2)
    work = wl.WORKLOADS["c1"]()
    batches = [work.batch(32, 20 + i) for i in range(5)]
    a, b = T.Trainer(work, seed=3), T.Trainer(work, seed=3)
    dev = []
    for tr in (a, b):
        Xd, Yd = S.Tensor(batches[0][0], is_leaf=True), S.Tensor(batches[0][1], is_leaf=True)
        for _ in range(2):
            tr.step(Xd, Yd)
        tr.capture(Xd, Yd)
        dev.append((Xd, Yd))
    want = []
    for X, Y in batches:
        sc.upload_f32(dev[0][0].value.main_ptr, np.ascontiguousarray(X, np.float32))
        sc.upload_f32(dev[0][1].value.main_ptr, np.ascontiguousarray(Y, np.float32))
        want.append(float(a.replay().value.to_host_f32()[0]))
    pinned = []
    for X, Y in batches:
        X, Y = np.ascontiguousarray(X, np.float32), np.ascontiguousarray(Y, np.float32)
        hx, hy = sc.host_alloc_pinned(X.nbytes), sc.host_alloc_pinned(Y.nbytes)
        ctypes.memmove(hx, X.ctypes.data, X.nbytes)
        ctypes.memmove(hy, Y.ctypes.data, Y.nbytes)
        pinned.append((hx, hy))
    got = b.fit_stream(pinned)
    assert got == want
    for Pa, Pb in zip(a.host_params(), b.host_params()):
        if Pa is not None:
            assert np.array_equal(Pa[0], Pb[0]) and np.array_equal(Pa[1], Pb[1])
    for hx, hy in pinned:
        sc.host_free_pinned(hx); sc.host_free_pinned(hy)
    a.release_graph(); b.release_graph()
    sc.set_precision(0)


def test_step_recorded_in_segments_at_the_gradient_buckets(T):
    """capture_data_parallel with buckets cuts the recording where backward has finished a bucket of the gradient arena;
    with a do-nothing collective (one rank) the replayed weights equal eager steps bit for bit, and the cuts and the
    reduce calls come in arena order (last layers first)."""
    from ml_framework_b200 import seera as S, seera_cuda as sc, dp
    sc.set_precision(2)
    work = wl.WORKLOADS["c3"]()
    X, Y = work.batch(16, 9)
    a, b = T.Trainer(work, seed=4), T.Trainer(work, seed=4)
    Xa, Ya = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)
    Xb, Yb = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)
    for _ in range(2):
        a.step(Xa, Ya)
        b.step(Xb, Yb)
    for _ in range(3):
        la = a.step(Xa, Ya)
    buckets = dp.plan_buckets(b.model, 4)
    assert len(buckets) >= 2 and buckets[0][1] == b.model.n_arena and buckets[-1][0] == 0
    calls = []
    b.capture_data_parallel(Xb, Yb, buckets=buckets, reduce_range=lambda lo, hi: calls.append((lo, hi)), wait=lambda w: None)
    kinds = [item[0] for item in b._graph_plan]
    assert kinds.count("graph") == len(buckets) and kinds[0] == "graph" and kinds[-1] == "reduce"
    for _ in range(3):
        lb = b.replay_data_parallel()
    assert calls == list(buckets) * 3
    assert float(la.value.to_host_f32()[0]) == float(lb.value.to_host_f32()[0])
    for Pa, Pb in zip(a.host_params(), b.host_params()):
        if Pa is not None:
            assert np.array_equal(Pa[0], Pb[0]) and np.array_equal(Pa[1], Pb[1])
    b.release_graph()
    sc.set_precision(0)


def test_fit_pipeline_matches_the_synchronous_loop_on_the_device(T):
    """Sequential.fit with staging buffers, copy-stream uploads and late loss reads equals the synchronous loop bit for
    bit (history and weights), with host one-hot targets and with integer labels expanded by seera_onehot_f32."""
    from ml_framework_b200 import seera as S, seera_cuda as sc
    sc.set_precision(0)
    rs = np.random.RandomState(3)
    X = rs.standard_normal((150, 1, 12, 12)).astype(np.float32)
    lab = rs.randint(0, 7, 150).astype(np.int32)
    Y = np.eye(7, dtype=np.float32)[lab]

    def make():
        np.random.seed(11)
        m = S.Sequential([S.Input((1, 12, 12)), S.Conv2D(8, 1, (3, 3), "relu", stride=1, zero_padding=1), S.MaxPool2D((2, 2), stride=2),
                          S.Flatten(), S.Dense(288, 7, activation="softmax")], device="cuda")
        return m, S.Adam(m, lr=1e-2), S.Loss().categorical_cross_entropy
    runs = []
    for mode in ("sync", "pipe", "labels"):
        m, opt, loss = make()
        np.random.seed(5)
        if mode == "sync":
            h = m._fit_unpipelined(X, Y, opt, loss, Epochs=2, batch_size=32)
        elif mode == "pipe":
            h = m.fit(X, Y, opt, loss, Epochs=2, batch_size=32, Loss_interval=100)
        else:
            h = m.fit(X, lab, opt, loss, Epochs=2, batch_size=32, Loss_interval=100, num_classes=7)
        runs.append((h, [(l.weights.to_numpy(), l.bais.to_numpy()) for l in m.model if isinstance(l, S._ParamLayer)]))
    assert runs[0][0][-1] < runs[0][0][0]                       # it trains
    for h, ws in runs[1:]:
        assert np.array_equal(h, runs[0][0])
        for (w, b), (w0, b0) in zip(ws, runs[0][1]):
            assert np.array_equal(w, w0) and np.array_equal(b, b0)


@pytest.mark.parametrize("kind", ["adam", "sgd"])
def test_checkpoint_with_optimizer_state_resumes_exactly_on_the_device(T, tmp_path, kind):
    """fit two epochs, save with the optimizer, load, fit one more == three epochs straight, bit for bit (weights,
    BatchNorm running statistics, Adam moments / SGD velocity and the step count)."""
    from ml_framework_b200 import seera as S, seera_cuda as sc
    sc.set_precision(0)
    rs = np.random.RandomState(3)
    X = rs.standard_normal((96, 1, 12, 12)).astype(np.float32)
    Y = np.eye(7, dtype=np.float32)[rs.randint(0, 7, 96)]

    def make():
        np.random.seed(11)
        m = S.Sequential([S.Input((1, 12, 12)), S.Conv2D(8, 1, (3, 3), "relu", stride=1, zero_padding=1), S.BatchNorm2d(8),
                          S.MaxPool2D((2, 2), stride=2), S.Flatten(), S.Dense(288, 7, activation="softmax")], device="cuda")
        return m, (S.Adam(m, lr=1e-2) if kind == "adam" else S.SGD(m, lr=1e-2, momentum=0.9))
    loss = S.Loss().categorical_cross_entropy
    f = str(tmp_path / "ck.pkl")
    a, oa = make()
    b, ob = make()
    for e in range(3):                                          # fit shuffles from numpy's global stream: seed per epoch
        np.random.seed(100 + e)
        a.fit(X, Y, oa, loss, Epochs=1, batch_size=32, Loss_interval=100)
    for e in range(2):
        np.random.seed(100 + e)
        b.fit(X, Y, ob, loss, Epochs=1, batch_size=32, Loss_interval=100)
    b.save(f, optimizer=ob)
    c, oc = S.Sequential.load(f, with_optimizer=True)
    np.random.seed(102)
    c.fit(X, Y, oc, loss, Epochs=1, batch_size=32, Loss_interval=100)
    assert type(oc) is type(oa)
    pa = [l for l in a.model if isinstance(l, S._ParamLayer)]
    pc = [l for l in c.model if isinstance(l, S._ParamLayer)]
    assert len(pa) == len(pc) > 0
    for la, lc in zip(pa, pc):
        assert np.array_equal(la.weights.to_numpy(), lc.weights.to_numpy()) and np.array_equal(la.bais.to_numpy(), lc.bais.to_numpy())
    bna = [l for l in a.model if isinstance(l, S.BatchNorm2d)][0]
    bnc = [l for l in c.model if isinstance(l, S.BatchNorm2d)][0]
    assert np.array_equal(np.asarray(bna.running_mean), np.asarray(bnc.running_mean))
    assert np.array_equal(np.asarray(bna.running_var), np.asarray(bnc.running_var))
    sa, sb = oa.state_dict(), oc.state_dict()
    for k in sa:
        assert np.array_equal(sa[k], sb[k]), k


def test_batchnorm_model_against_reference_golden(T, golden_dir):
    """BatchNorm2d / BatchNorm1d on the device inside a small CNN: two SGD steps (loss, predictions, every gradient and
    weight, running statistics) and an evaluation-mode prediction against the unmodified reference (host BatchNorm)."""
    from ml_framework_b200 import seera as S, seera_cuda as sc
    from test_host_logic_cpu import _bn_model_against_golden
    sc.set_precision(0)
    _bn_model_against_golden(S, golden_dir, 2e-4)


def test_fit_history_matches_the_reference_fit_on_the_device(T, golden_dir):
    """`Sequential.fit` on the device against the loss history of the reference's own `fit` (Seera.py:729-788): same data,
    initial weights and shuffling seed; golden written by tests/golden/make_golden_fit.py."""
    from ml_framework_b200 import seera as S
    import fit_case
    gold = np.load(golden_dir + "/fit_c1.npz")
    m = fit_case.build(S, device="cuda")
    X, Y = fit_case.data()
    np.random.seed(fit_case.SHUFFLE_SEED)
    h = m.fit(X, Y, S.Adam(m, lr=fit_case.LR), S.Loss().categorical_cross_entropy, Epochs=fit_case.EPOCHS,
              batch_size=fit_case.BATCH, Loss_interval=100)
    assert np.max(np.abs(h - gold["history"])) < 1e-4, (h, gold["history"])
    assert rel_l2(m.forward(X[:fit_case.BATCH]).to_numpy(), gold["pred"]) < 1e-4


def test_checkpoint_written_by_the_reference_loads_and_predicts_on_the_device(T, golden_dir):
    """A pickle written by the reference's `Sequential.save` (Seera.py:790-860) loads unchanged on the device and predicts
    what the reference's trained model predicted."""
    from ml_framework_b200 import seera as S
    import fit_case
    gold = np.load(golden_dir + "/fit_c1.npz")
    m = S.Sequential.load(golden_dir + "/ref_c1_checkpoint.pkl")
    X, _ = fit_case.data()
    assert rel_l2(m.predict(X[:fit_case.BATCH]).to_numpy(), gold["pred"]) < 1e-5
