"""Builds a Sequential model, optimizer and loss from a workload record and runs training steps.

`Trainer.step(X, Y)` is one pass of the hot path: forward, loss, backward, optimizer update.
X / Y may be host arrays (uploaded each step: the end-to-end path) or device tensors already
resident (the kernel-only path).
"""
import numpy as np

from . import seera as S
from . import seera_cuda as sc
from .cuTen import cuten


# Precision policy (forward mode, backward mode) per kind of configuration: what the benchmark times and what the
# parity gates are checked at.  The forward pass always runs fp32-class split products: its results decide every ReLU
# slope and max-pool argmax, and a decision that differs from the reference's changes a gradient entry by O(1) - with
# forward values rounded to bf16 (2^-9) a few per mille of them would.  The backward products only add their own rounding:
# two-way split for the fp32 configurations, ONE bf16 pass for the bf16 configuration (its subject: dA = dC B^T, dB = A^T dC).
# Mode 4 is the two-way fp16 split: three products with the accuracy the three-way bf16 split (mode 3) needs six for.
POLICY = {"fp32": (4, 4), "bf16": (4, 5)}


def policy_for(work):
    return POLICY[work.precision]


def build_model(work, params=None):
    layers = [S.Input(tuple(work.in_shape))]
    for L in work.layers:
        t = L["type"]
        if t == "dense":
            layers.append(S.Dense(L["in"], L["out"], activation=L["act"]))
        elif t == "conv":
            layers.append(S.Conv2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"]))
        elif t == "convT":
            layers.append(S.ConvTranspose2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"]))
        elif t == "maxpool":
            layers.append(S.MaxPool2D(L["k"], stride=L["stride"], padding=L["pad"]))
        elif t == "unpool":
            layers.append(S.Unpool2D_Nearest(L["size"]))
        elif t == "flatten":
            layers.append(S.Flatten())
        else:
            raise ValueError(t)
    if params is not None:
        for lay, P in zip(layers[1:], params):
            if P is not None:
                lay.set_weights(P[0], P[1])
    return S.Sequential(layers, device="cuda")


class Trainer:
    """`precision`: None leaves the engine's current mode alone; an int sets it for the whole step; a pair
    (forward, backward) sets it per phase.  (3, 2) is the tensor-core policy for the fp32 configurations: the
    forward contractions decide every ReLU and max-pool mask, so they get the three-way split (fp32-class
    products), while the backward contractions only add ~5e-6 of rounding and run the cheaper two-way split."""

    def __init__(self, work, params=None, seed=0, precision=None):
        self.work = work
        self.precision = (precision, precision) if isinstance(precision, int) else precision
        self.model = build_model(work, work.params(seed) if params is None else params)
        o = work.opt
        if o["kind"] == "adam":
            self.opt = S.Adam(self.model, lr=o["lr"], beta1=o.get("beta1", 0.9), beta2=o.get("beta2", 0.999), eps=o.get("eps", 1e-8))
        else:
            self.opt = S.SGD(self.model, lr=o["lr"], momentum=o.get("momentum", 0))
        L = S.Loss()
        self.lossf = L.categorical_cross_entropy if work.loss == "cce" else L.mse
        self.pred = None

    def forward_backward(self, X, Y):
        x = X if isinstance(X, S.Tensor) else S.Tensor(X, is_leaf=True)
        y = Y if isinstance(Y, S.Tensor) else S.Tensor(Y, is_leaf=True)
        if self.precision:
            sc.set_precision(self.precision[0])
        self.pred = self.model.forward(x)
        loss = self.lossf(self.pred, y)
        self.model.zero_grad()
        if self.precision:
            sc.set_precision(self.precision[1])
        S.autograd4nn(loss)
        return loss

    def step(self, X, Y):
        self.opt.begin_step()
        loss = self.forward_backward(X, Y)
        self.opt.step()
        return loss

    # ---- whole-step CUDA graph -------------------------------------------------------------------
    def capture(self, X, Y):
        """Records forward + loss + backward + optimizer on the device tensors X, Y into a CUDA graph.  In a data-parallel
        run over the engine's own collectives (dp.attach_nccl) the bucket sums are part of the recording: they fork onto
        the communication stream and join before the optimizer, all inside the one graph.
        Run `step` eagerly at least twice first.  Afterwards `replay()` re-runs the recorded step on
        whatever X and Y hold at that moment; the loss tensor returned here is rewritten by every replay."""
        if not (isinstance(X, S.Tensor) and isinstance(Y, S.Tensor)):
            raise TypeError("capture needs device-resident Tensors")
        if self.model._allreduce is not None and not getattr(self.model, "_collectives_capturable", False):
            raise RuntimeError("capture needs collectives that can be recorded (dp.attach_nccl); with other collectives use "
                               "capture_data_parallel")
        sc.graph_begin()
        try:
            loss = self.step(X, Y)
        except Exception:
            try:
                sc.graph_end()
            except Exception:
                pass
            raise
        self._graph = sc.graph_end()
        self._graph_keep = (X, Y, loss, self.pred)
        return loss

    def replay(self):
        self.opt.advance()
        sc.graph_launch(self._graph)
        return self._graph_keep[2]

    def capture_data_parallel(self, X, Y, allreduce_arena=None, buckets=None, reduce_range=None, wait=None):
        """Data-parallel variant: records forward + loss + backward (gradients gathered in the arena) as CUDA graphs and
        leaves the collectives and the optimizer outside them.

        Without `buckets`: one graph, then `allreduce_arena()` (one in-place sum of the whole gradient arena over the ranks,
        enqueued on the engine's stream), then the optimizer.
        With `buckets` (arena ranges from dp.plan_buckets, last layers first), `reduce_range(begin, end) -> handle` (an
        asynchronous in-place sum) and `wait(handle)`: the recording is cut each time backward has written the last
        gradient of a bucket, so a replay is  graph 0, reduce(bucket 0), graph 1, reduce(bucket 1), ..., wait all,
        optimizer - the sums of the late layers' gradients (most of the parameters) travel while the early layers'
        backward still runs."""
        if not (isinstance(X, S.Tensor) and isinstance(Y, S.Tensor)):
            raise TypeError("capture needs device-resident Tensors")
        hook, self.model._on_grad_ready = self.model._on_grad_ready, None
        plan, nxt = [], [0]
        if buckets:
            def cut_at(t):
                # backward runs from the last layer to the first: once parameter t's gradient sits in the arena every
                # slot at or above its offset is final
                while nxt[0] < len(buckets) - 1 and t._arena_off <= buckets[nxt[0]][0]:
                    plan.append(("graph", sc.graph_end()))
                    plan.append(("reduce",) + tuple(buckets[nxt[0]]))
                    nxt[0] += 1
                    sc.graph_begin()
            self.model._on_grad_ready = cut_at
        sc.graph_begin()
        try:
            loss = self.forward_backward(X, Y)
            self.model.gather_grads()
        except Exception:
            try:
                sc.graph_end()
            except Exception:
                pass
            for item in plan:
                if item[0] == "graph":
                    sc.graph_destroy(item[1])
            self.model._on_grad_ready = hook
            raise
        plan.append(("graph", sc.graph_end()))
        if buckets:
            plan.extend(("reduce",) + tuple(bk) for bk in buckets[nxt[0]:])
        self.model._on_grad_ready = None
        self._graph = plan[0][1]
        self._graph_plan = plan
        self._graph_keep = (X, Y, loss, self.pred, hook)
        self._graph_allreduce = allreduce_arena
        self._graph_reduce = (reduce_range, wait)
        return loss

    def replay_data_parallel(self):
        reduce_range, wait = self._graph_reduce
        works = []
        for item in self._graph_plan:
            if item[0] == "graph":
                sc.graph_launch(item[1])
            else:
                works.append(reduce_range(item[1], item[2]))
        if not works:
            self._graph_allreduce()
        for w in works:
            wait(w)
        self.opt.advance()
        self.opt._enqueue()
        return self._graph_keep[2]

    def fit_stream(self, host_batches, data_parallel=False):
        """Runs the captured step once per host batch with the transfers on the copy stream: while step i runs, batch
        i+1 is uploaded and the loss of step i-1 is read back, so the compute stream never waits for PCIe.
        `host_batches` yields (x_ptr, y_ptr): addresses of page-locked host buffers (seera_cuda.host_alloc_pinned)
        holding float32 arrays of the captured shapes.  Returns the losses, one per batch, in order."""
        import ctypes
        X, Y, loss = self._graph_keep[:3]
        replay = self.replay_data_parallel if data_parallel else self.replay
        if getattr(self, "_stage", None) is None:
            self._stage = (S._new(X.value.shape), S._new(Y.value.shape), sc.host_alloc_pinned(8))
        sx, sy, hl = self._stage
        slots = (ctypes.c_float * 2).from_address(hl)
        nbx, nby = X.value.size * 4, Y.value.size * 4

        def upload(batch):
            sc.copy_upload(sx.main_ptr, batch[0], nbx)
            sc.copy_upload(sy.main_ptr, batch[1], nby)
        losses, it, i = [], iter(host_batches), 0
        batch = next(it, None)
        if batch is not None:
            sc.copy_wait_compute()                   # whatever still reads the staging buffers comes first
            upload(batch)
        while batch is not None:
            sc.compute_wait_copy()                   # batch i has landed in the staging buffers
            sc.cuda_memcopy_devicetodevice(X.value.main_ptr, sx.main_ptr, X.value.size)
            sc.cuda_memcopy_devicetodevice(Y.value.main_ptr, sy.main_ptr, Y.value.size)
            sc.copy_wait_compute()                   # the staging buffers are free again after those two copies
            replay()
            if i:                                    # loss of step i-1: the device is already busy with step i
                sc.copy_synchronize()
                losses.append(float(slots[(i - 1) & 1]))
            batch = next(it, None)
            if batch is not None:
                upload(batch)
            sc.copy_wait_compute()                   # the loss is final once step i has run
            sc.copy_download(hl + 4 * (i & 1), loss.value.main_ptr, 4)
            i += 1
        if i:
            sc.copy_synchronize()
            losses.append(float(slots[(i - 1) & 1]))
        return losses

    def release_graph(self):
        plan = getattr(self, "_graph_plan", None)
        if plan:
            for item in plan:
                if item[0] == "graph":
                    sc.graph_destroy(item[1])
            self._graph_plan, self._graph, self._graph_keep = None, None, None
            return
        g = getattr(self, "_graph", None)
        if g:
            sc.graph_destroy(g)
            self._graph, self._graph_keep = None, None

    def host_params(self):
        return [None if not isinstance(l, S._ParamLayer) else (l.weights.to_numpy(), l.bais.to_numpy())
                for l in self.model.model[1:]]

    def host_grads(self):
        self.model.gather_grads()
        out = []
        for l in self.model.model[1:]:
            if isinstance(l, S._ParamLayer):
                out.append((l.weights.grad.to_host_f32(), l.bais.grad.to_host_f32()))
            else:
                out.append(None)
        return out
