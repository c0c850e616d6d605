"""Data-parallel training of a batch sharded over the GPUs of one node: one process per GPU, identical
weights on every rank, the gradient arena summed over the ranks in buckets while backward still runs.

Three parts:

  * the bucket plan and the hooks that launch a bucket's sum as soon as backward has written the last
    gradient of its range (`plan_buckets`, `attach`).  The collective is a pair of callables, so the same
    logic runs over NCCL on the GPU and over gloo on host memory in the CPU tests;
  * the NCCL data plane inside the engine (`init_from_env`, `attach_nccl`): the communicator, its
    high-priority stream and the registered gradient arena live in libseera_b200.so (csrc/dp.cu).  A bucket's
    sum and the final join are event edges between the engine's two streams, so a whole step - collectives
    included - records into one CUDA graph;
  * a host-side rendezvous (`Rendezvous`): the ranks meet through small files before any NCCL call, hand the
    communicator id from rank 0 to the others, and can tell each other that they are leaving.  A rank that
    never arrives or that left is therefore a Python exception within a stated deadline on the other ranks,
    found on the host before their next launch.

Gradients are averaged: every rank's loss is the mean over its own shard, the ranks' gradients are summed and
the optimizer multiplies by 1 / world.  The reference has no multi-GPU path."""
import os
import tempfile
import time


# ---- bucket plan and hooks ---------------------------------------------------------------------------------------
def plan_buckets(model, target_buckets=3):
    """Contiguous arena ranges, last layers first (their gradients are ready first in backward)."""
    params = model.parameters()
    if not params:
        return []
    target = max(1, model.n_arena // max(1, target_buckets))
    buckets, cur_end = [], model.n_arena
    for t in reversed(params):
        cur_beg = t._arena_off
        if cur_end - cur_beg >= target or t is params[0]:
            buckets.append((cur_beg, cur_end))
            cur_end = cur_beg
    return buckets


def attach(model, world, reduce_range, wait, target_buckets=3, join=None, after_reduce=None):
    """Installs the hooks on `model`; returns the bucket list.  `reduce_range(begin, end) -> handle` starts an in-place
    sum over the ranks of floats [begin, end) of the model's gradient arena; `wait(handle)` completes one; `join()`
    (optional) is called once after all waits.  `after_reduce(handle, begin, end)` (optional) runs right after a range's
    sum has been started - the place to enqueue the optimizer's update of that range behind the sum (see
    `update_in_buckets`)."""
    buckets = plan_buckets(model, target_buckets)
    state = {"works": [], "next": 0}

    def fire_upto(offset):
        while state["next"] < len(buckets) and offset <= buckets[state["next"]][0]:
            b, e = buckets[state["next"]]
            h = reduce_range(b, e)
            state["works"].append(h)
            if after_reduce is not None:
                after_reduce(h, b, e)
            state["next"] += 1

    def on_grad_ready(t):
        # backward runs from the last layer to the first, so once parameter t's gradient sits in the arena
        # every slot at or above t's offset is final
        fire_upto(t._arena_off)

    def finish(_grads):
        fire_upto(0)
        for w in state["works"]:
            wait(w)
        if join is not None:
            join()
        state["works"], state["next"] = [], 0

    model.world, model._allreduce, model._on_grad_ready = world, finish, on_grad_ready
    return buckets


# ---- host-side rendezvous ----------------------------------------------------------------------------------------
class RendezvousError(RuntimeError):
    pass


class Rendezvous:
    """The ranks of one job meet through files in `directory` (one node, a local file system).

    arrive()      announce this rank and wait until all `world` ranks have arrived, or raise RendezvousError after
                  `timeout_s` naming the ranks that never came
    publish(b) / fetch()   rank 0 hands a byte string (the communicator id) to the others; fetch raises after the deadline
    leave()       mark this rank as gone (call between steps, with nothing in flight)
    check()       raise RendezvousError if a peer has left - call before enqueueing a step's collectives"""

    def __init__(self, directory, rank, world, timeout_s=120.0, poll_s=0.01):
        self.dir, self.rank, self.world, self.timeout_s, self.poll_s = directory, int(rank), int(world), float(timeout_s), poll_s
        os.makedirs(directory, exist_ok=True)

    def _path(self, name, rank=None):
        return os.path.join(self.dir, name if rank is None else "%s.%d" % (name, rank))

    def _write(self, path, data=b""):
        fd, tmp = tempfile.mkstemp(dir=self.dir)
        with os.fdopen(fd, "wb") as f:
            f.write(data)
        os.replace(tmp, path)                      # readers see the whole file or none of it

    def arrive(self):
        self._write(self._path("here", self.rank))
        deadline = time.monotonic() + self.timeout_s
        while True:
            missing = [r for r in range(self.world) if not os.path.exists(self._path("here", r))]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise RendezvousError("rank %d: ranks %s did not arrive within %.1f s" % (self.rank, missing, self.timeout_s))
            time.sleep(self.poll_s)

    def publish(self, data):
        self._write(self._path("id"), bytes(data))

    def fetch(self):
        deadline = time.monotonic() + self.timeout_s
        path = self._path("id")
        while not os.path.exists(path):
            if time.monotonic() > deadline:
                raise RendezvousError("rank %d: rank 0 published no communicator id within %.1f s" % (self.rank, self.timeout_s))
            time.sleep(self.poll_s)
        with open(path, "rb") as f:
            return f.read()

    def leave(self):
        self._write(self._path("left", self.rank))

    def gone(self):
        return [r for r in range(self.world) if r != self.rank and os.path.exists(self._path("left", r))]

    def check(self):
        g = self.gone()
        if g:
            raise RendezvousError("rank %d: ranks %s have left the job" % (self.rank, g))

    def cleanup(self):
        """Rank 0, after every rank has joined the communicator: remove the files of this job."""
        for name in os.listdir(self.dir):
            try:
                os.unlink(os.path.join(self.dir, name))
            except OSError:
                pass
        try:
            os.rmdir(self.dir)
        except OSError:
            pass


def default_rendezvous_dir():
    """One directory per job: the launcher's process id (the ranks of a torchrun job share their parent) and port."""
    return os.path.join(tempfile.gettempdir(), "seera_dp_%d_%s" % (os.getppid(), os.environ.get("MASTER_PORT", "0")))


# ---- NCCL data plane inside the engine ---------------------------------------------------------------------------
_group = None


def init_from_env(timeout_s=120.0, directory=None):
    """Joins the job described by RANK / WORLD_SIZE / LOCAL_RANK (what `python -m torch.distributed.run` sets; any
    launcher that sets them works): selects the GPU, meets the other ranks on the host, creates the NCCL communicator
    inside the engine.  Returns the Rendezvous (its check() / leave() serve failure handling)."""
    global _group
    from . import seera_cuda as sc
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    sc.init(int(os.environ.get("LOCAL_RANK", str(rank))))
    rv = Rendezvous(directory or default_rendezvous_dir(), rank, world, timeout_s)
    rv.arrive()                                   # everyone is here before anyone blocks inside NCCL
    if rank == 0:
        uid = sc.dp_unique_id()
        rv.publish(uid)
    else:
        uid = rv.fetch()
    sc.dp_init(rank, world, uid)
    _group = rv
    return rv


def update_in_buckets(optimizer, complete=None):
    """An `after_reduce` callback that applies `optimizer`'s update to a bucket as soon as its sum is under way, instead of one
    update of the whole arena after the last sum.  `complete(handle)` makes the sum's result visible first where enqueueing
    order does not (host-memory collectives); with the engine's collectives the update is enqueued on the communication
    stream right behind the sum (seera_dp_side_begin / _end), so the weights of the late layers are updated while backward
    still runs through the early ones and only the last, small bucket's sum and update remain after backward."""
    optimizer.updates_by_bucket = True

    def after(handle, b, e):
        if complete is not None:
            complete(handle)
        optimizer.update_range(b, e)
    return after


def attach_nccl(model, target_buckets=3, optimizer=None, sync_batchnorm=False):
    """Moves the model's gradient arena into memory registered with the communicator and installs the bucket hooks over
    the engine's collectives.  With `optimizer`, each bucket is updated on the communication stream right behind its sum
    (`update_in_buckets`).  `sync_batchnorm`: the model's BatchNorm layers take their statistics over all ranks' shards
    (seera_batchnorm_fwd_sync / _bwd_sync) instead of each rank's own.  Returns the bucket list."""
    from . import seera_cuda as sc
    world = sc.dp_world()
    if sync_batchnorm:
        for layer in model.model:
            if hasattr(layer, "sync") and hasattr(layer, "_rm"):
                layer.sync = True
    ptr = sc.dp_alloc(4 * max(model.n_arena, 1))
    model.rehome_grads(ptr)
    arena = model.grads.main_ptr
    model._collectives_capturable = True
    after = None
    if optimizer is not None:
        inner = update_in_buckets(optimizer)

        def after(handle, b, e):
            sc.dp_side_begin()
            try:
                inner(handle, b, e)
            finally:
                sc.dp_side_end()
    return attach(model, world, reduce_range=lambda b, e: sc.dp_reduce_range(arena, b, e), wait=lambda h: None,
                  target_buckets=target_buckets, join=sc.dp_join, after_reduce=after)


def replicas_differ_by(model):
    """max over the parameter arena of (max over ranks - min over ranks): 0.0 when every rank holds the same weights."""
    import numpy as np
    from . import seera_cuda as sc
    n = model.n_arena
    hi, lo = sc.cuda_malloc_f32(n), sc.cuda_malloc_f32(n)
    try:
        sc.cuda_memcopy_devicetodevice(hi, model.params.main_ptr, n)
        sc.cuda_memcopy_devicetodevice(lo, model.params.main_ptr, n)
        sc.dp_allreduce(hi, n, 1)
        sc.dp_allreduce(lo, n, 2)
        d = sc.to_host_f32(hi, (n,)).astype(np.float64) - sc.to_host_f32(lo, (n,))
        return float(np.max(np.abs(d))) if n else 0.0
    finally:
        sc.cuda_free(hi)
        sc.cuda_free(lo)


def abort():
    """Leave the job without talking to the peers: for a rank that has learnt (Rendezvous.check) that one of them is gone."""
    global _group
    from . import seera_cuda as sc
    sc.dp_abort()
    _group = None


def finalize():
    global _group
    from . import seera_cuda as sc
    sc.dp_finalize()
    if _group is not None and _group.rank == 0:
        _group.cleanup()
    _group = None
