"""Data-parallel host logic on CPU: two gloo ranks, each with its own host-memory stand-in for the device
binding, train on half of the batch; after one step every rank's weights must equal the single-process step
on the whole batch (gradients averaged over ranks == gradient of the global mean for equal shards)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, out_dir):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    import fake_seera_cuda as fake
    import ml_framework_b200 as pkg
    sys.modules["ml_framework_b200.seera_cuda"] = fake
    pkg.seera_cuda = fake
    from ml_framework_b200 import train, dp
    import cases
    dist.init_process_group("gloo", rank=rank, world_size=world)
    work, n = cases.small_cases()[case]
    X, Y = work.batch(n, 2)
    shard = slice(rank * n // world, (rank + 1) * n // world)
    tr = train.Trainer(work, seed=2)
    order = []

    def reduce_range(b, e):
        view = fake._view(tr.model.grads.main_ptr + 4 * b, e - b)       # host memory of the arena range
        t = torch.from_numpy(view)
        order.append((b, e))
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True)
    buckets = dp.attach(tr.model, world, reduce_range, lambda w: w.wait(), target_buckets=3)
    for _ in range(2):
        tr.step(X[shard], Y[shard])
    assert order[:len(buckets)] == buckets and len(order) == 2 * len(buckets)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), *[p for P in tr.host_params() if P is not None for p in P])
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["c2s", "c3s"])
def test_two_ranks_match_the_single_process_step(case, tmp_path):
    import torch.multiprocessing as mp
    from oracle import cpu_oracle as co
    from oracle.train_oracle import RefNet
    from conftest import rel_l2
    import cases
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, case, str(tmp_path)), nprocs=2, join=True)
    work, n = cases.small_cases()[case]
    X, Y = work.batch(n, 2)
    ref = RefNet(work.layers, work.params(2), work.loss, work.opt, co)
    for _ in range(2):
        ref.step(X, Y)
    want = [p for P in ref.params if P is not None for p in P]
    for r in range(2):
        got = np.load(str(tmp_path / ("rank%d.npz" % r)))
        for i, w in enumerate(want):
            g = got["arr_%d" % i]
            if np.linalg.norm(w) > 0:
                assert rel_l2(g.ravel(), w.ravel()) < 2e-5, (r, i)


def test_bucket_plan_covers_the_arena_back_to_front():
    sys.path[:0] = [os.path.join(ROOT, "tests")]
    from ml_framework_b200 import dp

    class T:
        def __init__(self, off): self._arena_off = off

    class M:
        n_arena = 1000
        def parameters(self): return [T(0), T(400), T(448), T(900), T(960)]
    b = dp.plan_buckets(M(), 3)
    assert b[0][1] == 1000 and b[-1][0] == 0
    assert all(b[i][0] == b[i + 1][1] for i in range(len(b) - 1))
