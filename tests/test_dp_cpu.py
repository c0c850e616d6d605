"""Data-parallel host logic on CPU: two gloo ranks, each with its own host-memory stand-in for the device
binding, train on half of the batch; after one step every rank's weights must equal the single-process step
on the whole batch (gradients averaged over ranks == gradient of the global mean for equal shards)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, out_dir, by_bucket=False):
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
    # by_bucket: the optimizer updates each bucket right after its sum (completed first: host memory has no stream order)
    after = dp.update_in_buckets(tr.opt, complete=lambda w: w.wait()) if by_bucket else None
    buckets = dp.attach(tr.model, world, reduce_range, lambda w: w.wait(), target_buckets=3, after_reduce=after)
    for _ in range(2):
        tr.step(X[shard], Y[shard])
    assert order[:len(buckets)] == buckets and len(order) == 2 * len(buckets)
    if by_bucket:
        n_updates = fake.CALLS.get("adam", 0) + fake.CALLS.get("sgd", 0)
        assert n_updates == 2 * len(buckets), (n_updates, len(buckets))
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), *[p for P in tr.host_params() if P is not None for p in P])
    dist.destroy_process_group()


@pytest.mark.parametrize("by_bucket", [False, True])
@pytest.mark.parametrize("case", ["c2s", "c3s"])
def test_two_ranks_match_the_single_process_step(case, by_bucket, tmp_path):
    import torch.multiprocessing as mp
    from oracle import cpu_oracle as co
    from oracle.train_oracle import RefNet
    from conftest import rel_l2
    import cases
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, case, str(tmp_path), by_bucket), nprocs=2, join=True)
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


# ---- failure handling on the host: no GPU, no collective is ever entered ------------------------------------------------
def _rank_that_arrives(directory, rank, world, timeout_s, q):
    sys.path[:0] = [ROOT]
    from ml_framework_b200 import dp
    try:
        rv = dp.Rendezvous(directory, rank, world, timeout_s=timeout_s)
        rv.arrive()
        q.put((rank, "arrived"))
    except dp.RendezvousError as e:
        q.put((rank, "error: %s" % e))


def test_a_rank_that_never_joins_is_reported_within_the_deadline(tmp_path):
    """World of 3, rank 2 never starts: ranks 0 and 1 raise RendezvousError naming rank 2 after the deadline, before any
    of them would have called into NCCL."""
    import multiprocessing as mp
    import time
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    t0 = time.monotonic()
    procs = [ctx.Process(target=_rank_that_arrives, args=(str(tmp_path / "job"), r, 3, 1.0, q)) for r in (0, 1)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=30) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert time.monotonic() - t0 < 20
    for r in (0, 1):
        assert got[r].startswith("error") and "[2]" in got[r], got


def test_the_id_of_rank_0_reaches_the_others_or_times_out(tmp_path):
    sys.path[:0] = [ROOT]
    from ml_framework_b200 import dp
    a = dp.Rendezvous(str(tmp_path / "j1"), 0, 2, timeout_s=1.0)
    b = dp.Rendezvous(str(tmp_path / "j1"), 1, 2, timeout_s=1.0)
    a.publish(b"\x01" * 128)
    assert b.fetch() == b"\x01" * 128
    c = dp.Rendezvous(str(tmp_path / "j2"), 1, 2, timeout_s=0.3)
    with pytest.raises(dp.RendezvousError, match="published no communicator id"):
        c.fetch()


def _train_until_peer_leaves(rank, world, port, directory, out_dir):
    """Two gloo ranks train; rank 1 leaves after its second step (between steps, nothing in flight).  Rank 0 learns of it on
    the host before enqueueing its next step and stops with an error instead of entering a collective nobody will join."""
    sys.path[:0] = [ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import torch
    import torch.distributed as dist
    import fake_seera_cuda as fake
    import ml_framework_b200 as pkg
    sys.modules["ml_framework_b200.seera_cuda"] = fake
    pkg.seera_cuda = fake
    from ml_framework_b200 import train, dp
    import cases
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    rv = dp.Rendezvous(directory, rank, world, timeout_s=10.0)
    rv.arrive()
    work, n = cases.small_cases()["c2s"]
    X, Y = work.batch(n, 2)
    tr = train.Trainer(work, seed=2)

    def reduce_range(b, e):
        return dist.all_reduce(torch.from_numpy(fake._view(tr.model.grads.main_ptr + 4 * b, e - b)), async_op=True)
    dp.attach(tr.model, world, reduce_range, lambda w: w.wait())
    steps, outcome = 0, "finished"
    try:
        for i in range(6):
            if rank == 1 and i == 2:
                rv.leave()
                outcome = "left"
                break
            if rank == 0 and i >= 2:
                import time
                deadline = time.monotonic() + 10
                while not rv.gone() and time.monotonic() < deadline:      # let the marker land: the point is what check() does with it
                    time.sleep(0.01)
            rv.check()
            tr.step(X, Y)
            steps += 1
    except dp.RendezvousError as e:
        outcome = "peer left: %s" % e
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %s" % (steps, outcome))
    dist.destroy_process_group()


def test_a_rank_that_leaves_between_steps_stops_the_other_with_an_error(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_train_until_peer_leaves, args=(2, port, str(tmp_path / "job"), str(tmp_path)), nprocs=2, join=True)
    r0 = open(str(tmp_path / "rank0.txt")).read()
    r1 = open(str(tmp_path / "rank1.txt")).read()
    assert r1 == "2 left"
    assert r0.startswith("2 peer left") and "[1]" in r0, r0
