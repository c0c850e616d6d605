"""BatchNorm with cross-rank statistics on two GPUs against the UNMODIFIED reference on the joined batch.

Two child processes, one GPU each (skipped on a box with fewer than two).  Each trains the small BatchNorm model of
tests/golden/bn_case.py on its half of the 12 samples for two SGD steps with `sync_batchnorm`; the weights after each step, the
running statistics and the evaluation-mode prediction must be what the reference's CPU path produced on all 12 samples
(tests/golden/bn_two_steps.npz, written by make_golden_bn.py) - the statistics of the joined batch, not of a shard.  With
per-rank statistics (the default) the same run must NOT match: the check has teeth."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path[:0] = [%(root)r, os.path.join(%(root)r, "tests"), os.path.join(%(root)r, "tests", "golden")]
import numpy as np
from ml_framework_b200 import dp, seera as S, seera_cuda as sc
import bn_case
rank = int(os.environ["RANK"])
rv = dp.init_from_env(timeout_s=60.0, directory=%(rdv)r)
sc.set_precision(0)
gold = np.load(os.path.join(%(root)r, "tests", "golden", "bn_two_steps.npz"))
rel = lambda a, b: float(np.linalg.norm(np.asarray(a, np.float64).ravel() - np.asarray(b, np.float64).ravel()) /
                         max(np.linalg.norm(np.asarray(b, np.float64).ravel()), 1e-12))
X, Y = bn_case.data()
half = slice(rank * bn_case.N // 2, (rank + 1) * bn_case.N // 2)
worst = {}
for sync in (True, False):
    lays = bn_case.layers(S)
    for i, (W, B) in bn_case.weights().items():
        lays[i].set_weights(W, B)
    model = S.Sequential(lays, device="cuda")
    opt = S.SGD(model, lr=bn_case.LR, momentum=bn_case.MOMENTUM)
    dp.attach_nccl(model, 2, optimizer=opt, sync_batchnorm=sync)
    lossf = S.Loss().categorical_cross_entropy
    plist = [l for l in model.model if isinstance(l, S._ParamLayer)]
    w = 0.0
    for s in range(bn_case.STEPS):
        yp = model.forward(S.Tensor(X[half], is_leaf=True))
        loss = lossf(yp, S.Tensor(Y[half], is_leaf=True))
        model.zero_grad()
        S.autograd4nn(loss)
        opt.step()
        sc.dp_wait_host(20000)
        for k, l in enumerate(plist):
            w = max(w, rel(l.weights.to_numpy(), gold["W%%d_s%%d" %% (k, s)]), rel(l.bais.to_numpy(), gold["b%%d_s%%d" %% (k, s)]))
    w = max(w, rel(lays[2].running_mean, gold["rm2"]), rel(lays[2].running_var, gold["rv2"]),
            rel(lays[6].running_mean, gold["rm6"]), rel(lays[6].running_var, gold["rv6"]),
            rel(model.predict(S.Tensor(X, is_leaf=True)).to_numpy(), gold["pred_eval"]))
    assert dp.replicas_differ_by(model) == 0.0
    worst[sync] = w
    if sync:
        # the same sharded step as ONE recorded graph (the layer's small sums over the ranks ride on the compute stream inside it):
        # replays keep the replicas identical and match the same number of eager steps on a second model
        from ml_framework_b200 import train
        Xd, Yd = S.Tensor(X[half], is_leaf=True), S.Tensor(Y[half], is_leaf=True)
        def one_step():
            yp = model.forward(Xd)
            loss = lossf(yp, Yd)
            model.zero_grad()
            S.autograd4nn(loss)
            opt.step()
            return loss
        before = model.params.to_host_f32()[:model.n_arena].copy()
        sc.graph_begin()
        loss_t = one_step()
        g = sc.graph_end()
        for _ in range(2):
            opt.advance()
            sc.graph_launch(g)
        sc.dp_wait_host(20000)
        after = model.params.to_host_f32()[:model.n_arena].copy()
        assert np.all(np.isfinite(after)) and not np.array_equal(before, after)
        assert dp.replicas_differ_by(model) == 0.0
        sc.graph_destroy(g)
print("RESULT rank %%d sync %%.3e local %%.3e" %% (rank, worst[True], worst[False]), flush=True)
dp.finalize()                                   # before the checks: a rank that raised would leave its peer waiting here
assert worst[True] < 2e-4, worst
assert worst[False] > 1e-3 and worst[False] > 10 * worst[True], worst
print("DONE rank %%d" %% rank, flush=True)
'''


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_cross_rank_batchnorm_equals_the_reference_on_the_joined_batch(tmp_path):
    code = CHILD % {"root": ROOT, "rdv": str(tmp_path / "rdv")}
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=120)[0])
    except subprocess.TimeoutExpired:
        for p in procs:                                   # a rank that failed leaves its peer waiting in a collective: end both
            p.kill()
        outs = [p.communicate()[0] for p in procs]
        raise AssertionError("timed out; rank outputs:\n" + "\n----\n".join(o[-3000:] for o in outs))
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out[-3000:]
        assert "DONE rank %d" % rank in out, out[-3000:]
