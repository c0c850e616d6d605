"""Data-parallel plumbing for the gradient arena: bucket plan and the hooks that launch a bucket's
all-reduce as soon as backward has written the last gradient of its range.

The collective itself is supplied by the caller as `reduce_range(begin, end) -> handle` (sum over ranks,
in place, on floats [begin, end) of the model's gradient arena) and `wait(handle)`: NCCL through
torch.distributed on the GPU (bench.py), gloo on host memory in the CPU tests.  Gradients are averaged:
the optimizer multiplies by 1/world (each rank's loss is the mean over its own shard)."""


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


def attach(model, world, reduce_range, wait, target_buckets=3):
    """Installs the hooks on `model`; returns the bucket list."""
    buckets = plan_buckets(model, target_buckets)
    state = {"works": [], "next": 0}

    def fire_upto(offset):
        while state["next"] < len(buckets) and offset <= buckets[state["next"]][0]:
            b, e = buckets[state["next"]]
            state["works"].append(reduce_range(b, e))
            state["next"] += 1

    def on_grad_ready(t):
        # backward runs from the last layer to the first, so once parameter t's gradient sits in the arena
        # every slot at or above t's offset is final
        fire_upto(t._arena_off)

    def finish(_grads):
        fire_upto(0)
        for w in state["works"]:
            wait(w)
        state["works"], state["next"] = [], 0

    model.world, model._allreduce, model._on_grad_ready = world, finish, on_grad_ready
    return buckets
