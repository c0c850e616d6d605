"""A rank that leaves a data-parallel job between steps, on real GPUs with the engine's NCCL data plane.

Two child processes, one GPU each (skipped on a box with fewer than two).  Both train a few sharded steps; rank 1 then
finishes its work (stream synchronised: none of its kernels or collectives in flight), tells the others through the host-side
rendezvous that it is leaving, drops its communicator and exits.  Rank 0 checks the rendezvous before enqueueing its next
step, gets a RendezvousError instead of entering a collective nobody would join, drops its communicator with ncclCommAbort and
goes on alone: a plain single-GPU step still works in the same process.  Nothing on a GPU is made to fault, trap or hang; NVLS
is switched off for the run (a rank that dies while bound to an NVLink multicast object has raised faults on its peers here)."""
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
rank = int(os.environ["RANK"])
rv = dp.init_from_env(timeout_s=60.0, directory=%(rdv)r)
work = wl.c1_small_cnn()
tr = train.Trainer(work, seed=3, precision=(0, 0))
dp.attach_nccl(tr.model, 2)
X, Y = work.batch(32, 10 + rank)
steps, outcome = 0, "finished"
try:
    for i in range(6):
        if rank == 1 and i == 3:
            sc.stream_synchronize()                 # nothing of this rank is in flight
            rv.leave()
            outcome = "left"
            break
        if rank == 0 and i >= 3:
            import time
            t0 = time.monotonic()
            while not rv.gone() and time.monotonic() - t0 < 30:
                time.sleep(0.01)
        rv.check()
        tr.step(X, Y)
        sc.dp_wait_host(20000)                      # host-side wait with a deadline: both streams drained, NCCL healthy
        steps += 1
except dp.RendezvousError as e:
    outcome = "peer left"
same = dp.replicas_differ_by(tr.model) if outcome == "finished" else None
dp.abort()
if rank == 0:
    # alone now: the engine and the GPU are still usable
    solo = train.Trainer(work, seed=3, precision=(0, 0))
    loss = float(solo.step(X, Y).value.to_host_f32()[0])
    assert np.isfinite(loss)
print("RESULT rank %%d steps %%d outcome %%s" %% (rank, steps, outcome), flush=True)
'''


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_a_rank_that_leaves_between_steps_on_two_gpus(tmp_path):
    code = CHILD % {"root": ROOT, "rdv": str(tmp_path / "rdv")}
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", SEERA_DP_NO_WINDOW="1")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        out, _ = p.communicate(timeout=240)
        outs.append(out)
        assert p.returncode == 0, out[-2000:]
    assert "RESULT rank 0 steps 3 outcome peer left" in outs[0], outs[0][-2000:]
    assert "RESULT rank 1 steps 3 outcome left" in outs[1], outs[1][-2000:]
