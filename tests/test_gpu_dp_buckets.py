"""Data-parallel training on two GPUs with the optimizer's update enqueued bucket by bucket behind each bucket's sum
(dp.attach_nccl(model, buckets, optimizer=...), seera_dp_side_begin / _end) against one update of the whole arena after the
last sum: the same weights, bit for bit, eagerly and as a replayed CUDA graph, and the same on both ranks.

Two child processes, one GPU each (skipped on a box with fewer than two)."""
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
from ml_framework_b200 import dp, train, workloads as wl, seera_cuda as sc
from ml_framework_b200 import seera as S
rank = int(os.environ["RANK"])
rv = dp.init_from_env(timeout_s=60.0, directory=%(rdv)r)
out = {}
for wname, work in (("c1", wl.c1_small_cnn()), ("c2", wl.c2_mlp())):
    X, Y = work.batch(64, 20 + rank)
    for mode in ("whole", "buckets"):
        tr = train.Trainer(work, seed=3, precision=train.policy_for(work))
        nb = dp.attach_nccl(tr.model, 3, optimizer=tr.opt if mode == "buckets" else None)
        for i in range(3):                               # eager steps
            tr.step(X, Y)
        Xd, Yd = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)
        tr.capture(Xd, Yd)                               # then the same step recorded once and replayed
        for i in range(3):
            tr.replay()
        sc.dp_wait_host(20000)
        out[(wname, mode)] = tr.model.params.to_host_f32()[:tr.model.n_arena].copy()
        assert dp.replicas_differ_by(tr.model) == 0.0
        launches = len(nb)
    assert np.array_equal(out[(wname, "whole")], out[(wname, "buckets")]), wname
    assert np.all(np.isfinite(out[(wname, "buckets")]))
dp.finalize()
print("RESULT rank %%d ok" %% rank, flush=True)
'''


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_bucket_by_bucket_update_equals_the_whole_arena_update_on_two_gpus(tmp_path):
    code = CHILD % {"root": ROOT, "rdv": str(tmp_path / "rdv")}
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=150)[0])
    except subprocess.TimeoutExpired:
        for p in procs:                                   # a rank that failed leaves its peer waiting in a collective: end both
            p.kill()
        outs = [p.communicate()[0] for p in procs]
        raise AssertionError("timed out; rank outputs:\n" + "\n----\n".join(o[-3000:] for o in outs))
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out[-3000:]
        assert "RESULT rank %d ok" % rank in out, out[-3000:]
