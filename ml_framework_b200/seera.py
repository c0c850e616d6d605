"""Training front end on the B200 engine: Sequential, layers, Loss, SGD, Adam, autograd4nn, Tensor.

Mirrors the user-facing API of the reference (Seera.py:26-1086, Seera_Engine.py:22-26) - same class
names, constructor arguments, method names (`forward`, `zero_grad`, `fit`, `step`, `set_weights`,
`get_weights`, the attribute spelled `bais`) and error behaviour - so a training script written for
the reference's `device="cuda"` path runs here with the import line changed.  What differs is the
machinery underneath:

  * autograd works per LAYER, not per scalar op.  A layer's forward enqueues its contraction plus
    ONE fused bias+activation pass, and records a backward closure that enqueues ONE fused
    activation-gradient+bias-gradient pass and the dX / dW contractions.  The reference builds a node
    per elementary op with five placeholder buffers each (Seera_init.py:75-80) and walks them in
    Seera_Engine.backward_step (Seera_Engine.py:259-598).
  * all parameters live in one contiguous device arena, with matching arenas for gradients and
    optimizer state: the optimizer is a single kernel launch over the arena (Seera.py:1038-1063 issues
    ~30 launches per tensor) and a data-parallel run all-reduces the gradient arena in place.
  * weights are updated in place; device addresses of parameters are stable across steps.
  * nothing blocks: calls enqueue on the engine's stream, the loss value is read when asked for.

There is no CPU path here: `device` must be "cuda" and the compiled engine must be present.
"""
from __future__ import annotations

import pickle

import numpy as np

from . import seera_cuda as sc
from .cuTen import cuten

_ACT = {None: 0, "relu": 1, "sigmoid": 2, "tanh": 3}
_ACTIVATIONS = ("relu", "sigmoid", "softmax", "tanh")
f32 = np.float32


def _numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def _new(shape):
    return cuten._wrap(sc.cuda_malloc_f32(_numel(shape)), shape)


# ─────────────────────────────────────────────────────────────────────────────────────────────
# Tensor: a device value, its gradient, and the closure that propagates the gradient
# ─────────────────────────────────────────────────────────────────────────────────────────────
class Tensor:
    def __init__(self, value, dtype="float32", is_leaf=False, device="cuda"):
        if isinstance(value, Tensor):
            value = value.value
        if not isinstance(value, cuten):
            value = cuten(np.ascontiguousarray(np.asarray(value, dtype=np.float32)))
        self.value = value
        self.dtype = dtype
        self.is_leaf = is_leaf
        self.grad = None                 # cuten, set by backward
        self._parents = ()
        self._backward = None            # fn(grad: cuten) -> None, deposits into parents via _accumulate
        self._softmax_logits = None      # for a softmax output: the Tensor of logits it came from
        self._grad_slot = None           # for a parameter: its view into the model's gradient arena

    # the reference reads gradients as `t.node.cp` (Seera_init.py:53-55)
    @property
    def node(self):
        return self

    @property
    def cp(self):
        return self.grad

    @cp.setter
    def cp(self, g):
        self.grad = g

    @property
    def shape(self):
        return self.value.shape

    def _grad_target(self):
        """Buffer a backward kernel should write this tensor's gradient contribution into: the arena
        slot when the gradient restarts from zero, otherwise a fresh buffer to be added."""
        if self.grad is None and self._grad_slot is not None:
            return self._grad_slot
        return _new(self.value.shape)

    def _accumulate(self, g):
        """Add a gradient contribution: a cuten of this tensor's shape, or a _PooledGrad (the gradient of a 2x2 max-pool
        of this tensor, still in pooled form) when it is the only contribution."""
        if self.grad is None:
            self.grad = g
        else:
            if isinstance(self.grad, _PooledGrad):
                self.grad = self.grad.materialize()
            if isinstance(g, _PooledGrad):
                g = g.materialize()
            out = _new(self.value.shape)
            sc.cuda_elemadd(self.grad.main_ptr, g.main_ptr, out.main_ptr, self.value.size)
            self.grad = out

    def to_numpy(self):
        return self.value.to_host_f32().copy()

    def item(self):
        a = self.value.to_host_f32()
        if a.size != 1:
            raise ValueError("Can only convert tensors with a single element to Python scalars")
        return a.item()

    def mean(self):
        if self.value.size == 1:
            return self
        raise NotImplementedError("Tensor.mean on a non-scalar: losses of this front end are already scalar")

    def detach(self):
        return Tensor(self.value, is_leaf=True)

    @classmethod
    def zeros(cls, shape, dtype="float32", device="cuda"):
        return cls(cuten.zeros(shape), is_leaf=True)

    @classmethod
    def ones(cls, shape, dtype="float32", device="cuda"):
        return cls(cuten.ones(shape), is_leaf=True)

    def __repr__(self):
        return f"Tensor(GPU)\n({self.value.to_host_f32()},\nshape={self.value.shape})"


tensor = Tensor


# Conv2D followed by a 2x2 / stride-2 MaxPool2D runs as one launch (pool in the convolution's epilogue) where the engine
# can do it; the convolution's own full-resolution output is then never materialised.  Set to False to keep every
# layer's output in memory.
FUSE_POOL = True
# A Dense layer that feeds another Dense layer can have its GEMM epilogue write the 16-bit copies of its output that the next
# layer's GEMM reads (seera_matmul_bias_act_fwd_s, c_copies).  Off: at the sizes measured (4096 x 1024 outputs, one tile per
# CTA) the two-byte stores lengthen an epilogue that nothing overlaps by more than the next layer's vectorised conversion
# launch costs (MLP configuration: step 0.317 ms with it, 0.287 ms without).
import os as _os
DENSE_EPILOGUE_COPIES = _os.environ.get("SEERA_DENSE_EPILOGUE_COPIES", "0") != "0"


class _PooledGrad:
    """Gradient of a 2x2 / stride-2 max-pool output, kept in pooled form with the pool's argmax mask.  A consumer that
    can route it itself (Conv2D backward: one kernel forms dz from it) takes it as is; anything else materialises the
    full-resolution gradient with cuda_maxpool_bwd."""
    __slots__ = ("gp", "mask", "shape", "pooled")

    def __init__(self, gp, mask, shape, pooled=None):
        self.gp, self.mask, self.shape, self.pooled = gp, mask, tuple(shape), pooled

    def materialize(self):
        N, C, H, W = self.shape
        dx = _new(self.shape)
        sc.cuda_maxpool_bwd(self.gp.main_ptr, self.mask.main_ptr, dx.main_ptr, N, C, H, W, 2, 2, 0, 0, 2, 2)
        return dx


class _KeptCopies:
    """Owner of the channels-last copies a forward call kept for its backward call (0: none kept)."""
    __slots__ = ("h",)

    def __init__(self):
        self.h = 0

    def release(self):
        if self.h:
            sc.shadow_free(self.h)
            self.h = 0

    __del__ = release


class _KeptRows:
    """Owner of row-major operand copies a Dense forward call kept or handed on (0: none)."""
    __slots__ = ("h",)

    def __init__(self):
        self.h = 0

    def release(self):
        if self.h:
            sc.rows_free(self.h)
            self.h = 0

    __del__ = release


class autograd4nn:
    """Reverse pass from a scalar loss: `autograd4nn(loss)` (same call shape as Seera_Engine.py:24-26)."""

    def __init__(self, hook):
        self.hook = hook
        self.backward()

    def backward(self):
        order, seen = [], set()
        stack = [(self.hook, False)]
        while stack:                                   # iterative DFS: no recursion limit on deep nets
            t, done = stack.pop()
            if done:
                order.append(t)
                continue
            if id(t) in seen:
                continue
            seen.add(id(t))
            stack.append((t, True))
            for p in t._parents:
                stack.append((p, False))
        for t in order:
            if not t.is_leaf:
                t.grad = None
        self.hook.grad = cuten.ones_like(self.hook.value)
        for t in reversed(order):
            if t._backward is not None and t.grad is not None:
                if isinstance(t.grad, _PooledGrad) and not getattr(t, "_takes_pooled", False):
                    t.grad = t.grad.materialize()
                t._backward(t.grad)


# ─────────────────────────────────────────────────────────────────────────────────────────────
# Layers
# ─────────────────────────────────────────────────────────────────────────────────────────────
class Layer:
    def __init__(self):
        self.inputs = []
        self.outputs = []
        self.activations = {a: a for a in _ACTIVATIONS}

    def __call__(self, input_layer):
        if not isinstance(input_layer, Layer):
            raise TypeError("The input should be a Layer")
        self.inpobj = input_layer
        return self


class Input(Layer):
    def __init__(self, shape):
        super().__init__()
        self.shape = shape
        self.weights = 0
        self.bais = 0
        self.inputs = None

    def forward(self):
        self.outputs = self.inputs
        return self.outputs

    def __repr__(self):
        return f"Input Layer with shape {self.shape}"


def _initial(kind_scale, shape):
    kind, scale = kind_scale
    if kind == "normal":
        return (np.random.randn(*shape) * scale).astype(np.float32)
    if kind == "uniform":
        return np.random.uniform(-scale, scale, shape).astype(np.float32)
    return (np.zeros if kind == "zeros" else np.ones)(shape, dtype=np.float32)


def _initializers(fan_in, fan_out):
    return {
        "zeros": ("zeros", 0), "ones": ("ones", 1), "random_normal": ("normal", 1), "random_uniform": ("uniform", 0.05),
        "he_normal": ("normal", np.sqrt(2 / fan_in)), "he_uniform": ("uniform", np.sqrt(6 / fan_in)),
        "glorot_normal": ("normal", np.sqrt(2 / (fan_in + fan_out))), "glorot_uniform": ("uniform", np.sqrt(6 / (fan_in + fan_out))),
        "lecun_normal": ("normal", np.sqrt(1 / fan_in)), "lecun_uniform": ("uniform", np.sqrt(3 / fan_in)),
    }


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class _ParamLayer(Layer):
    """Shared parameter handling: host initial values until the model places them in its arena."""

    def _check(self, activation, initializer, table):
        if activation not in self.activations:
            raise ValueError('Activation must be "relu", "sigmoid", "softmax", or "tanh"')
        if initializer not in table:
            raise ValueError(f"Initializer must be one of {list(table.keys())}")

    def set_weights(self, W, B):
        if isinstance(W, Tensor):
            W, B = W.to_numpy(), B.to_numpy()
        elif not isinstance(W, np.ndarray):
            raise TypeError("Weights must be Tensor or numpy array")
        W = np.ascontiguousarray(W, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        self._w_init, self._b_init = W, B
        if isinstance(self.weights, Tensor) and tuple(self.weights.value.shape) == W.shape:
            sc.upload_f32(self.weights.value.main_ptr, W)            # keeps the arena slot and its address
            sc.upload_f32(self.bais.value.main_ptr, B)
        else:
            self.weights = Tensor(W, is_leaf=True)
            self.bais = Tensor(B, is_leaf=True)

    def get_weights(self):
        return self.weights, self.bais

    def update_params(self, vW, vB):
        """w -= vW, b -= vB with device tensors (Seera.py:140-147), in place."""
        for t, v in ((self.weights, vW), (self.bais, vB)):
            neg = v * (-1)
            sc.cuda_elemadd(t.value.main_ptr, neg.main_ptr, t.value.main_ptr, t.value.size)

    # fused epilogue / prologue shared by Dense, Conv2D, ConvTranspose2D
    def _finish_forward(self, x, z, channels, inner, product, contraction_backward, fused_backward=None, takes_pooled=False):
        """product(bias_ptr, act_code) fills z with act(contraction + bias) in one call; this wraps z as the layer's
        output Tensor and attaches the backward closure."""
        act = self.layeract
        W, b = self.weights, self.bais
        if act == "softmax":
            if len(z.shape) != 2:
                raise ValueError("[Engine]: Softmax VJP requires at least 2D")
            product(b.value.main_ptr, 0)
            logits = Tensor(z)
            y = _new(z.shape)
            sc.cuda_softmax_fwd(z.main_ptr, y.main_ptr, z.shape[0], z.shape[1])
            out = Tensor(y)
            out._softmax_logits = logits
            out._parents = (logits,)

            def softmax_backward(g, y=y, logits=logits):
                dz = _new(y.shape)
                sc.cuda_softmax_vjp(y.main_ptr, g.main_ptr, dz.main_ptr, y.shape[0], y.shape[1])
                logits._accumulate(dz)
            out._backward = softmax_backward
            node, code = logits, 0
        else:
            code = _ACT[act]
            product(b.value.main_ptr, code)
            out = Tensor(z)
            node = out
        node._parents = (x, W, b)

        node._takes_pooled = takes_pooled and fused_backward is not None

        def layer_backward(g, y=node.value, code=code):
            db = b._grad_target()
            if fused_backward is not None:          # activation, bias and contraction gradients in one call
                dx, dw = fused_backward(g, y, code, db)
                b._accumulate(db)
                W._accumulate(dw)
                hook = getattr(getattr(self, "_model", None), "_on_grad_ready", None)
                if hook is not None and W.grad is W._grad_slot and b.grad is b._grad_slot:
                    hook(W)
                if dx is not None:
                    x._accumulate(dx)
                return
            if code == 0:
                dz = g
                sc.act_bias_bwd(g.main_ptr, 0, g.main_ptr, db.main_ptr, y.size, channels, inner, 0)
            else:
                dz = _new(y.shape)
                sc.act_bias_bwd(g.main_ptr, y.main_ptr, dz.main_ptr, db.main_ptr, y.size, channels, inner, code)
            b._accumulate(db)
            dx, dw = contraction_backward(dz)
            W._accumulate(dw)
            hook = getattr(getattr(self, "_model", None), "_on_grad_ready", None)
            if hook is not None and W.grad is W._grad_slot and b.grad is b._grad_slot:
                hook(W)                      # this layer's gradients sit in the arena: a bucket may go out
            if dx is not None:
                x._accumulate(dx)
        node._backward = layer_backward
        return out


class Dense(_ParamLayer):
    def __init__(self, in_units, out_units, activation=None, kernel_initializer="glorot_uniform",
                 bias_initializer="zeros", kernel_regularizer=None, bias_regularizer=None):
        super().__init__()
        table = _initializers(in_units, out_units)
        self._check(activation, kernel_initializer, table)
        self.layeract, self.in_units, self.out_units = activation, in_units, out_units
        self._w_init = _initial(table[kernel_initializer], (in_units, out_units))
        self._b_init = _initial(table[bias_initializer], (1, out_units))
        self.weights = Tensor(self._w_init, is_leaf=True)
        self.bais = Tensor(self._b_init, is_leaf=True)

    def __call__(self, input_layer):
        super().__call__(input_layer)
        input_layer._feeds_dense = True       # a Dense producer then also emits the row-major copies of its output this layer reads
        return self

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv, W = x.value, self.weights.value
        if len(xv.shape) != 2 or xv.shape[1] != self.in_units:
            raise ValueError(f"[cuTen]: matmul: inner dimensions must agree, got {xv.shape} @ {W.shape}")
        M, K, N = xv.shape[0], self.in_units, self.out_units
        z = _new((M, N))
        kept = {"a": _KeptRows(), "w": _KeptRows()}
        given = getattr(x, "_rows", None) if x.value is xv else None        # copies written by the Dense layer before
        out_rows = _KeptRows()
        want_out = DENSE_EPILOGUE_COPIES and bool(getattr(self, "_feeds_dense", False)) and self.layeract != "softmax"

        def product(bias, code):
            kept["a"].h, kept["w"].h, out_rows.h = sc.matmul_bias_act_fwd_s(xv.main_ptr, W.main_ptr, bias, z.main_ptr, M, N, K, code,
                                                                             given.h if given else 0, want_out)

        def fused_backward(g, y, code, db, need_dx=not x.is_leaf):
            # activation slope, bias gradient, dA and dB in one call; it reads the copies the forward call kept
            dw = self.weights._grad_target()
            dx = _new(xv.shape) if need_dx else None
            sc.matmul_act_bwd(xv.main_ptr, W.main_ptr, y.main_ptr if code else 0, g.main_ptr, dx.main_ptr if need_dx else 0, dw.main_ptr,
                              db.main_ptr, M, N, K, code, kept["a"].h or (given.h if given else 0), kept["w"].h)
            kept["a"].release(); kept["w"].release()
            if given:
                given.release()
            return dx, dw

        def contraction_backward(dz, need_dx=not x.is_leaf):
            dw = self.weights._grad_target()
            dx = _new(xv.shape) if need_dx else None
            sc.cuda_matmul_bwd(xv.main_ptr, W.main_ptr, dz.main_ptr, dx.main_ptr if need_dx else 0, dw.main_ptr, M, N, K, 1)
            return dx, dw
        self.outputs = self._finish_forward(x, z, N, 1, product, contraction_backward, fused_backward)
        if want_out:
            self.outputs._rows = out_rows
        return self.outputs

    def __repr__(self):
        return f"Dense({self.in_units}→{self.out_units}, act={self.layeract}, params={self.in_units * self.out_units + self.out_units})"


class Conv2D(_ParamLayer):
    def __init__(self, out_channels, in_channels, kernel_size, activation, stride=1, zero_padding=0,
                 kernel_initializer="he_normal", bias_initializer="zeros"):
        super().__init__()
        fan_in = in_channels * kernel_size[0] * kernel_size[1]
        table = _initializers(fan_in, out_channels * kernel_size[0] * kernel_size[1])
        self._check(activation, kernel_initializer, table)
        self.layeract, self.in_channels, self.out_channels = activation, in_channels, out_channels
        self.kernel_size, self.stride, self.zero_padding = tuple(kernel_size), _pair(stride), _pair(zero_padding)
        self._w_init = _initial(table[kernel_initializer], (out_channels, in_channels) + self.kernel_size)
        self._b_init = np.zeros((1, out_channels, 1, 1), np.float32)
        self.weights = Tensor(self._w_init, is_leaf=True)
        self.bais = Tensor(self._b_init, is_leaf=True)

    def __call__(self, input_layer):
        super().__call__(input_layer)
        input_layer._feeds_conv = True        # a pooling producer then also emits the channels-last copies this layer reads
        return self

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv, W = x.value, self.weights.value
        if len(xv.shape) == 3:
            xv = xv.reshape((1,) + tuple(xv.shape))
        if len(xv.shape) != 4:
            raise ValueError("[cuTen]: conv2d expects 4-D tensors (N,C,H,W) and (F,C,KH,KW)")
        N, C, H, Wd = xv.shape
        F, (KH, KW), (sh, sw), (ph, pw) = self.out_channels, self.kernel_size, self.stride, self.zero_padding
        OH, OW = (H + 2 * ph - KH) // sh + 1, (Wd + 2 * pw - KW) // sw + 1
        kept = _KeptCopies()
        given = getattr(x, "_copies", None) if x.value is xv else None       # copies made by the producer of x
        pool = getattr(self, "_pool_consumer", None)
        self._fused = None
        if (FUSE_POOL and pool is not None and self.layeract != "softmax"
                and sc.conv2d_pool_fusable(N, C, H, Wd, F, KH, KW, sh, sw, ph, pw)):
            # the pool is folded into this layer's epilogue: z stays a shape without memory
            z = cuten._wrap(0, (N, F, OH, OW))
            z._owns_memory = False
            pooled = _new((N, F, OH // 2, OW // 2))
            pmask = cuten._wrap(sc.cuda_malloc_i32(N * F * (OH // 2) * (OW // 2)), (N, F, OH // 2, OW // 2), "int32")
            pcopies = _KeptCopies()

            def product(bias, code):
                kept.h, pcopies.h = sc.conv2d_bias_act_pool_fwd_s(xv.main_ptr, W.main_ptr, bias, pooled.main_ptr, pmask.main_ptr, N, C, H,
                                                                  Wd, F, KH, KW, ph, pw, sh, sw, code, given.h if given else 0,
                                                                  bool(getattr(pool, "_feeds_conv", False)))
            self._fused = (pooled, pmask, pcopies)
        else:
            z = _new((N, F, OH, OW))

            def product(bias, code):
                kept.h = sc.conv2d_bias_act_fwd_s(xv.main_ptr, W.main_ptr, bias, z.main_ptr, N, C, H, Wd, F, KH, KW, ph, pw, sh, sw,
                                                  code, given.h if given else 0)

        def fused_backward(g, y, code, db, need_dx=not x.is_leaf):
            dw = self.weights._grad_target()
            dx = _new(xv.shape) if need_dx else None
            if isinstance(g, _PooledGrad):
                gptr, gpptr, mptr, ypptr = 0, g.gp.main_ptr, g.mask.main_ptr, g.pooled.main_ptr if g.pooled is not None else 0
            else:
                gptr, gpptr, mptr, ypptr = g.main_ptr, 0, 0, 0
            sc.conv2d_act_bwd(W.main_ptr, xv.main_ptr, y.main_ptr, gptr, gpptr, mptr, ypptr, dx.main_ptr if need_dx else 0, dw.main_ptr,
                              db.main_ptr, N, C, H, Wd, F, KH, KW, sh, sw, ph, pw, code, kept.h or (given.h if given else 0))
            kept.release()
            if given:
                given.release()
            return dx, dw

        def contraction_backward(dz, need_dx=not x.is_leaf):
            dw = self.weights._grad_target()
            dx = _new(xv.shape) if need_dx else None
            sc.cuda_conv2d_bwd(W.main_ptr, xv.main_ptr, dz.main_ptr, dx.main_ptr if need_dx else 0, dw.main_ptr,
                               N, C, H, Wd, F, KH, KW, sh, sw, ph, pw)
            return dx, dw
        self.outputs = self._finish_forward(x, z, F, OH * OW, product, contraction_backward, fused_backward, takes_pooled=True)
        return self.outputs

    def __repr__(self):
        return f"Conv2D({self.in_channels}→{self.out_channels}, kernel={self.kernel_size}, act={self.layeract})"


class ConvTranspose2D(_ParamLayer):
    def __init__(self, out_channels, in_channels, kernel_size, activation, stride=1, zero_padding=0,
                 kernel_initializer="he_normal"):
        super().__init__()
        fan_in = in_channels * kernel_size[0] * kernel_size[1]
        table = _initializers(fan_in, out_channels * kernel_size[0] * kernel_size[1])
        for k in ("lecun_normal", "lecun_uniform"):
            table.pop(k)
        self._check(activation, kernel_initializer, table)
        self.layeract, self.in_channels, self.out_channels = activation, in_channels, out_channels
        self.kernel_size, self.stride, self.zero_padding = tuple(kernel_size), _pair(stride), _pair(zero_padding)
        self._w_init = _initial(table[kernel_initializer], (in_channels, out_channels) + self.kernel_size)
        self._b_init = np.zeros((1, out_channels, 1, 1), np.float32)
        self.weights = Tensor(self._w_init, is_leaf=True)
        self.bais = Tensor(self._b_init, is_leaf=True)

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv, W = x.value, self.weights.value
        if len(xv.shape) != 4:
            raise ValueError("[cuTen]: conv2d_transpose expects 4-D tensors (N,Cin,H,W) and (Cin,Cout,KH,KW)")
        N, Cin, H, Wd = xv.shape
        Cout, (KH, KW), (sh, sw), (ph, pw) = self.out_channels, self.kernel_size, self.stride, self.zero_padding
        Ho, Wo = (H - 1) * sh - 2 * ph + KH, (Wd - 1) * sw - 2 * pw + KW
        z = _new((N, Cout, Ho, Wo))

        def product(bias, code):
            sc.conv2DTranspose_bias_act_fwd(xv.main_ptr, W.main_ptr, bias, z.main_ptr, N, Cin, H, Wd, Cout, KH, KW, sh, sw, ph, pw, code)

        def contraction_backward(dz, need_dx=not x.is_leaf):
            dw = self.weights._grad_target()
            dx = _new(xv.shape) if need_dx else None
            sc.cuda_conv2DTranspose_bwd(W.main_ptr, xv.main_ptr, dz.main_ptr, dx.main_ptr if need_dx else 0, dw.main_ptr,
                                        N, Cin, H, Wd, Cout, KH, KW, sh, sw, ph, pw)
            return dx, dw
        self.outputs = self._finish_forward(x, z, Cout, Ho * Wo, product, contraction_backward)
        return self.outputs

    def __repr__(self):
        return (f"ConvTranspose2D({self.in_channels}→{self.out_channels}, kernel={self.kernel_size}, "
                f"stride={self.stride}, act={self.layeract})")


class _BatchNorm(_ParamLayer):
    """Batch normalisation on the device (the reference computes it on the host even in its GPU path: Seera.py:511-623,
    Seera_init.py:870-921, Seera_Engine.py:381-415).  gamma / beta are the layer's `weights` / `bais` (as in the reference)
    and live in the model's parameter arena; the running statistics are device buffers, readable as NumPy arrays through
    `running_mean` / `running_var`.  In a data-parallel run each rank normalises with the statistics of its own shard, unless
    `sync` is set (also by `dp.attach_nccl(..., sync_batchnorm=True)`): then the statistics, and the sums of the backward
    formula, are those of all ranks' shards together, so that a sharded step equals the step on the joined batch."""

    def __init__(self, num, momentum=0.1, eps=1e-5, sync=False):
        super().__init__()
        self.momentum, self.eps, self.training, self.sync = momentum, eps, True, bool(sync)
        self._w_init = np.ones((num,), np.float32)
        self._b_init = np.zeros((num,), np.float32)
        self.weights = Tensor(self._w_init, is_leaf=True)
        self.bais = Tensor(self._b_init, is_leaf=True)
        self._rm = cuten(np.zeros(num, np.float32))
        self._rv = cuten(np.ones(num, np.float32))
        self._num = num

    gamma = property(lambda self: self.weights)
    beta = property(lambda self: self.bais)

    @property
    def running_mean(self):
        return self._rm.to_host_f32().copy()

    @running_mean.setter
    def running_mean(self, v):
        sc.upload_f32(self._rm.main_ptr, np.ascontiguousarray(v, np.float32).reshape(self._num))

    @property
    def running_var(self):
        return self._rv.to_host_f32().copy()

    @running_var.setter
    def running_var(self, v):
        sc.upload_f32(self._rv.main_ptr, np.ascontiguousarray(v, np.float32).reshape(self._num))

    def _shape_ok(self, shape):
        raise NotImplementedError

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv = x.value
        self._shape_ok(xv.shape)
        N, C = xv.shape[0], xv.shape[1]
        S = 1
        for d in xv.shape[2:]:
            S *= d
        g, b = self.weights, self.bais
        y, mean, si = _new(xv.shape), _new((C,)), _new((C,))
        fwd, bwd = (sc.batchnorm_fwd_sync, sc.batchnorm_bwd_sync) if self.sync else (sc.batchnorm_fwd, sc.batchnorm_bwd)
        fwd(xv.main_ptr, g.value.main_ptr, b.value.main_ptr, self._rm.main_ptr, self._rv.main_ptr, y.main_ptr,
                         mean.main_ptr, si.main_ptr, N, C, S, float(self.momentum), float(self.eps), bool(self.training))
        out = Tensor(y)
        out._parents = (x, g, b)

        def backward(dy, need_dx=not x.is_leaf):
            dg, db = g._grad_target(), b._grad_target()
            dx = _new(xv.shape)
            bwd(dy.main_ptr, xv.main_ptr, mean.main_ptr, si.main_ptr, g.value.main_ptr, dx.main_ptr, dg.main_ptr, db.main_ptr, N, C, S)
            g._accumulate(dg)
            b._accumulate(db)
            hook = getattr(getattr(self, "_model", None), "_on_grad_ready", None)
            if hook is not None and g.grad is g._grad_slot and b.grad is b._grad_slot:
                hook(g)
            if need_dx:
                x._accumulate(dx)
        out._backward = backward
        self.outputs = out
        return out


class BatchNorm1d(_BatchNorm):
    def __init__(self, num_features, momentum=0.1, eps=1e-5, sync=False):
        super().__init__(num_features, momentum, eps, sync)
        self.num_features = num_features

    def _shape_ok(self, shape):
        if len(shape) != 2 or shape[1] != self.num_features:
            raise ValueError(f"BatchNorm1d({self.num_features}) expects (N, {self.num_features}), got {tuple(shape)}")

    def __repr__(self):
        return f"BatchNorm1d({self.num_features})"


class BatchNorm2d(_BatchNorm):
    def __init__(self, num_channels, momentum=0.1, eps=1e-5, sync=False):
        super().__init__(num_channels, momentum, eps, sync)
        self.num_channels = num_channels

    def _shape_ok(self, shape):
        if len(shape) != 4 or shape[1] != self.num_channels:
            raise ValueError(f"BatchNorm2d({self.num_channels}) expects (N, {self.num_channels}, H, W), got {tuple(shape)}")

    def __repr__(self):
        return f"BatchNorm2d({self.num_channels})"


class Concatenate(Layer):
    """Joins the outputs of two layers along axis 1 (Seera.py:486-505); one strided-copy launch forward, one backward."""

    def __call__(self, *input_layers):
        if len(input_layers) != 2:
            raise ValueError("Only 2 layers supported for concatenation.")
        for l in input_layers:
            if not isinstance(l, Layer):
                raise TypeError("All inputs must be Layer instances.")
        self.input_layers = input_layers
        return self

    def forward(self):
        a, b = self.inputs = [l.outputs for l in self.input_layers]
        av, bv = a.value, b.value
        y = av.concatenate2D(bv) if len(av.shape) >= 4 else av.concatenate1D(bv)
        out = Tensor(y)
        out._parents = (a, b)

        def backward(g):
            da, db = cuten._concat_backward(g, av, bv)
            a._accumulate(da)
            b._accumulate(db)
        out._backward = backward
        self.outputs = out
        return out

    def __repr__(self):
        return "Concatenate Layer"


class MaxPool2D(Layer):
    def __init__(self, pool_size=(2, 2), stride=1, padding=0):
        super().__init__()
        if not isinstance(pool_size, tuple):
            raise ValueError("kernelsize should be a tuple (height, width)")
        self.pool_size, self.stride, self.padding = pool_size, _pair(stride), _pair(padding)

    def __call__(self, input_layer):
        if not isinstance(input_layer, Layer):
            raise TypeError("Input must be a Layer instance.")
        self.inpobj = input_layer
        if (tuple(self.pool_size), self.stride, self.padding) == ((2, 2), (2, 2), (0, 0)):
            input_layer._pool_consumer = self     # a Conv2D producer may fold this pool into its own launch
        return self

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv = x.value
        if len(xv.shape) != 4:
            raise ValueError("[cuTen]: maxpool2d expects 4-D tensor (N,C,H,W)")
        N, C, H, W = xv.shape
        (KH, KW), (sh, sw), (ph, pw) = self.pool_size, self.stride, self.padding
        OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
        if OH * OW > H * W:
            raise ValueError("[cuTen]: maxpool2d with more outputs than inputs is not supported")
        tiles_exactly = (KH, KW, sh, sw, ph, pw) == (2, 2, 2, 2, 0, 0) and H % 2 == 0 and W % 2 == 0
        fused = getattr(self.inpobj, "_fused", None)
        if fused is not None:                     # the producing convolution already pooled its output
            y, mask, copies = fused
            self.inpobj._fused = None
        else:
            y = _new((N, C, OH, OW))
            mask = cuten._wrap(sc.cuda_malloc_i32(N * C * OH * OW), (N, C, OH, OW), "int32")
            copies = _KeptCopies()
        if fused is not None:
            pass
        elif tiles_exactly and getattr(self, "_feeds_conv", False):   # also leaves the channels-last copies of y for that convolution
            copies.h = sc.maxpool2x2_fwd_s(xv.main_ptr, y.main_ptr, mask.main_ptr, N, C, H, W)
        else:
            sc.cuda_maxpool_fwd(xv.main_ptr, y.main_ptr, mask.main_ptr, N, C, H, W, KH, KW, ph, pw, sh, sw)
        out = Tensor(y)
        out._parents = (x,)
        out._copies = copies
        self.mask = mask

        def backward(g):
            if tiles_exactly and getattr(x, "_takes_pooled", False):
                x._accumulate(_PooledGrad(g, mask, xv.shape, y))   # the producer routes it through the mask itself
                return
            dx = _new(xv.shape)
            sc.cuda_maxpool_bwd(g.main_ptr, mask.main_ptr, dx.main_ptr, N, C, H, W, KH, KW, ph, pw, sh, sw)
            x._accumulate(dx)
        out._backward = backward
        self.outputs = out
        return out

    def __repr__(self):
        return f"MaxPool2D(pool={self.pool_size}, stride={self.stride})"


class Unpool2D_Nearest(Layer):
    def __init__(self, size=(2, 2)):
        super().__init__()
        self.size = size

    def __call__(self, input_layer):
        if not isinstance(input_layer, Layer):
            raise TypeError("Input must be a Layer instance.")
        self.inpobj = input_layer
        return self

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        xv = x.value
        if len(xv.shape) != 4:
            raise ValueError("[cuTen]:unpool expects 4-D tensor (N,C,H,W)")
        sw, sh = self.size                       # the reference unpacks (sw, sh) (Seera_init.py:793)
        N, C, H, W = xv.shape
        y = _new((N, C, H * sh, W * sw))
        sc.cuda_unpooling_fwd(xv.main_ptr, y.main_ptr, N, C, H, W, sh, sw)
        out = Tensor(y)
        out._parents = (x,)

        def backward(g):
            dx = _new(xv.shape)
            sc.cuda_unpooling_bwd(g.main_ptr, dx.main_ptr, N, C, H, W, sh, sw)
            x._accumulate(dx)
        out._backward = backward
        self.outputs = out
        return out

    def __repr__(self):
        return f"Unpool2D_Nearest(size={self.size})"


class Flatten(Layer):
    def __call__(self, input_layer):
        if not isinstance(input_layer, Layer):
            raise TypeError("Input must be a Layer instance.")
        self.inpobj = input_layer
        return self

    def forward(self):
        x = self.inputs = self.inpobj.outputs
        out = Tensor(x.value.flatten())
        out._parents = (x,)
        out._backward = lambda g: x._accumulate(g.reshape(x.value.shape))
        self.outputs = out
        return out

    def __repr__(self):
        return "Flatten Layer"


# ─────────────────────────────────────────────────────────────────────────────────────────────
# Sequential
# ─────────────────────────────────────────────────────────────────────────────────────────────
class Sequential:
    def __init__(self, layers, device="cuda"):
        if not isinstance(layers, list):
            raise TypeError("Layers must be a list")
        if not isinstance(layers[0], Input):
            raise TypeError("First layer must be an Input layer")
        if device != "cuda":
            raise ValueError("this engine has no CPU path: Sequential(..., device=\"cuda\")")
        self.device = device
        self.model = [layers[0]] + [layer(layers[i]) for i, layer in enumerate(layers[1:])]
        self.world, self._allreduce, self._on_grad_ready = 1, None, None
        self._build_arena()
        for l in self.param_layers:
            l._model = self

    # one contiguous block each for parameters and gradients; slots are 64-float aligned
    def _build_arena(self):
        self.param_layers = [l for l in self.model if isinstance(l, _ParamLayer)]
        offs, total = [], 0
        for l in self.param_layers:
            for init in (l._w_init, l._b_init):
                offs.append((total, init.shape, init.size))
                total += (init.size + 63) // 64 * 64
        self.n_arena = total
        host = np.zeros(max(total, 1), np.float32)
        for (o, _, n), init in zip(offs, [a for l in self.param_layers for a in (l._w_init, l._b_init)]):
            host[o:o + n] = init.ravel()
        self.params = cuten(host)
        self.grads = cuten._wrap(sc.cuda_zeros_f(max(total, 1)), (max(total, 1),))
        it = iter(offs)
        for l in self.param_layers:
            for name in ("weights", "bais"):
                o, shape, n = next(it)
                v = cuten._wrap(self.params.main_ptr + 4 * o, shape)
                v._owns_memory, v._base = False, self.params
                t = Tensor(v, is_leaf=True)
                t._arena_off, t._arena_n = o, n
                t._grad_slot = self._grad_view(t)
                setattr(l, name, t)
        self._grad_fresh = True

    def _grad_view(self, t):
        v = cuten._wrap(self.grads.main_ptr + 4 * t._arena_off, t.value.shape)
        v._owns_memory, v._base = False, self.grads
        return v

    def rehome_grads(self, ptr):
        """Use the caller's device block (at least n_arena floats, zeroed, kept alive by the caller) as the gradient arena
        from now on - e.g. memory registered with a communicator, so that collectives work on it in place."""
        g = cuten._wrap(int(ptr), (max(self.n_arena, 1),))
        g._owns_memory = False
        self.grads = g
        for t in self.parameters():
            t._grad_slot = self._grad_view(t)
            t.grad = None

    def parameters(self):
        return [t for l in self.param_layers for t in (l.weights, l.bais)]

    def forward(self, X=None):
        if X is not None:
            if isinstance(X, np.ndarray):
                X = Tensor(X, is_leaf=True)
            if not isinstance(X, Tensor):
                raise TypeError("Input must be a Tensor or numpy array.")
            self.model[0].inputs = X
        out = None
        for layer in self.model:
            out = layer.forward()
        return out

    def predict(self, X):
        """Forward in evaluation mode: BatchNorm layers normalise with their running statistics (Seera.py:690-700)."""
        self._set_mode(False)
        try:
            return self.forward(X)
        finally:
            self._set_mode(True)

    def _set_mode(self, training=True):
        for l in self.model:
            if hasattr(l, "training"):
                l.training = training

    def zero_grad(self):
        """Parameter gradients restart from zero: the next backward writes them instead of adding."""
        for t in self.parameters():
            t.grad = None

    def get_params(self):
        for l in self.param_layers:
            print(l.get_weights())

    def summary(self):
        print("=" * 60 + "\nModel Summary\n" + "=" * 60)
        for i, l in enumerate(self.model):
            print(f"  Layer {i}: {l}")
        print("=" * 60)

    def gather_grads(self):
        """Copy every parameter gradient into its slot of the gradient arena (no-op for slots already there)."""
        for t in self.parameters():
            g = t.grad
            dst = self.grads.main_ptr + 4 * t._arena_off
            if g is None:
                sc.cuda_memset(dst, 0, 4 * t._arena_n)
            elif g.main_ptr != dst:
                sc.cuda_memcopy_devicetodevice(dst, g.main_ptr, t._arena_n)
                t.grad = self._grad_view(t)

    def fit(self, X_train, y, Optimizer, Loss, Epochs, batch_size=1, Loss_interval=20, num_classes=None):
        """Training loop with the reference's signature, shuffling and history (Seera.py:715-788).  The input side is a
        pipeline: each batch is gathered straight into one of two page-locked staging buffers and uploaded on the copy
        stream while the previous step runs, and the loss of a step is read back one step later, so the compute stream
        never waits for a transfer.  `y` may be the reference's one-hot / target array, or, with `num_classes`, a 1-D
        integer label array: 4 bytes per sample cross PCIe and the one-hot rows are formed on the device."""
        X_train = np.ascontiguousarray(X_train, np.float32)
        labels = num_classes is not None and np.ndim(y) == 1
        y = np.ascontiguousarray(y, np.int32 if labels else np.float32)
        n = X_train.shape[0]
        bs = int(batch_size)
        xrow, yrow = int(np.prod(X_train.shape[1:])), int(np.prod(y.shape[1:]))
        # two sets of staging / device buffers, sized for a full batch
        stage = []
        for _ in range(2):
            hx, hy = sc.host_alloc_pinned(bs * xrow * 4), sc.host_alloc_pinned(bs * yrow * 4)
            stage.append({"hx": hx, "hy": hy, "vx": sc.host_view(hx, bs * xrow * 4).view(np.float32),
                          "vy": sc.host_view(hy, bs * yrow * 4).view(np.int32 if labels else np.float32),
                          "dx": _new((bs,) + X_train.shape[1:]), "dy": _new((bs,) + y.shape[1:]) if not labels else None,
                          "dl": cuten._wrap(sc.cuda_malloc_i32(bs), (bs,), "int32") if labels else None})
        hl = sc.host_alloc_pinned(8)
        slots = sc.host_view(hl, 8).view(np.float32)
        history = []
        try:
            for epoch in range(Epochs):
                perm = np.random.permutation(n)
                starts = list(range(0, n, bs))

                def upload(k):                      # batch k -> staging set k % 2 -> its device buffers (copy stream)
                    st, idx = stage[k & 1], perm[starts[k]:starts[k] + bs]
                    m = len(idx)
                    np.take(X_train.reshape(n, xrow), idx, axis=0, out=st["vx"][:m * xrow].reshape(m, xrow))
                    np.take(y.reshape(n, yrow), idx, axis=0, out=st["vy"][:m * yrow].reshape(m, yrow))
                    sc.copy_upload(st["dx"].main_ptr, st["hx"], m * xrow * 4)
                    sc.copy_upload((st["dl"] if labels else st["dy"]).main_ptr, st["hy"], m * yrow * 4)
                    return m
                total, pending = 0.0, None          # pending: loss tensor of the previous step, not read back yet
                sc.copy_wait_compute()              # whatever still reads the staging sets comes first
                sizes = {0: upload(0)}
                for k in range(len(starts)):
                    st, m = stage[k & 1], sizes[k]
                    sc.compute_wait_copy()          # batch k has landed
                    sc.copy_wait_compute()          # set (k + 1) % 2 is free once step k - 1 has run
                    xb = Tensor(cuten._wrap(st["dx"].main_ptr, (m,) + X_train.shape[1:]), is_leaf=True)
                    xb.value._owns_memory = False
                    if labels:
                        yv = _new((m, int(num_classes)))
                        sc.onehot_f32(st["dl"].main_ptr, yv.main_ptr, m, int(num_classes))
                    else:
                        yv = cuten._wrap(st["dy"].main_ptr, (m,) + y.shape[1:])
                        yv._owns_memory = False
                    loss = Loss(self.forward(xb), Tensor(yv, is_leaf=True))
                    self.zero_grad()
                    autograd4nn(loss)
                    Optimizer.step()
                    if pending is not None:         # the device is already busy with step k
                        sc.copy_synchronize()
                        total += float(slots[(k - 1) & 1])
                    if k + 1 < len(starts):
                        sizes[k + 1] = upload(k + 1)
                    sc.copy_wait_compute()          # the loss is final once step k has run
                    sc.copy_download(hl + 4 * (k & 1), loss.value.main_ptr, 4)
                    pending = loss
                sc.copy_synchronize()
                total += float(slots[(len(starts) - 1) & 1])
                history.append(total / len(starts))
                if epoch % Loss_interval == 0 or epoch == Epochs - 1:
                    print(f"Epoch {epoch + 1}/{Epochs} — Loss: {history[-1]:.6f}")
        finally:
            sc.stream_synchronize()
            sc.copy_synchronize()
            for st in stage:
                sc.host_free_pinned(st["hx"]); sc.host_free_pinned(st["hy"])
            sc.host_free_pinned(hl)
        return np.array(history)

    def _fit_unpipelined(self, X_train, y, Optimizer, Loss, Epochs, batch_size=1):
        """The same loop with a synchronous upload and loss read per step (the reference's structure); kept as the
        yardstick for fit()."""
        history = []
        n = X_train.shape[0]
        for epoch in range(Epochs):
            perm = np.random.permutation(n)
            Xs, ys = X_train[perm], y[perm]
            total, batches = 0.0, 0
            for s in range(0, n, batch_size):
                e = min(s + batch_size, n)
                ypred = self.forward(Tensor(Xs[s:e], is_leaf=True))
                loss = Loss(ypred, Tensor(ys[s:e], is_leaf=True))
                self.zero_grad()
                autograd4nn(loss)
                Optimizer.step()
                total += float(loss.value.to_host_f32().ravel()[0])
                batches += 1
            history.append(total / batches)
        return np.array(history)

    # checkpoint: layer configs + host copies of the weights (same record layout as Seera.py:790-860)
    def save(self, filepath, optimizer=None, rank=None):
        """Layer records as the reference writes them (Seera.py:790-860).  With `optimizer`, a last record of class
        "__optimizer__" carries its kind, hyper-parameters, step count and state arenas (Adam m / v, SGD velocity), so
        that training resumes exactly; the reference drops that state.  In a data-parallel run only rank 0 writes
        (`rank`, else the RANK environment variable): the ranks hold identical weights and optimizer state."""
        import os
        if int(os.environ.get("RANK", "0") if rank is None else rank) != 0:
            return
        data = []
        for l in self.model:
            info = {"class": l.__class__.__name__, "config": {}}
            if isinstance(l, Input):
                info["config"]["shape"] = l.shape
            elif isinstance(l, Dense):
                info["config"] = {"in_units": l.in_units, "out_units": l.out_units, "layeract": l.layeract}
            elif isinstance(l, (Conv2D, ConvTranspose2D)):
                info["config"] = {"out_channels": l.out_channels, "in_channels": l.in_channels, "kernel_size": l.kernel_size,
                                  "layeract": l.layeract, "stride": l.stride, "zero_padding": l.zero_padding}
            elif isinstance(l, MaxPool2D):
                info["config"] = {"pool_size": l.pool_size, "stride": l.stride, "padding": l.padding}
            elif isinstance(l, _BatchNorm):
                info["config"] = {"num_features" if isinstance(l, BatchNorm1d) else "num_channels": l._num, "momentum": l.momentum,
                                  "eps": l.eps, "running_mean": l.running_mean, "running_var": l.running_var}
            elif isinstance(l, Unpool2D_Nearest):
                info["config"] = {"size": l.size}
            if isinstance(l, _ParamLayer):
                info["weights"], info["bais"] = l.weights.to_numpy(), l.bais.to_numpy()
            data.append(info)
        if optimizer is not None:
            data.append({"class": "__optimizer__", "config": optimizer.state_dict()})
        with open(filepath, "wb") as f:
            pickle.dump(data, f)

    @classmethod
    def load(cls, filepath, with_optimizer=False):
        """Rebuilds the model; with_optimizer=True returns (model, optimizer) with the saved optimizer state restored
        (optimizer is None when the file holds none)."""
        with open(filepath, "rb") as f:
            data = pickle.load(f)
        layers, opt_state = [], None
        for info in data:
            c, k = info["config"], info["class"]
            if k == "__optimizer__":
                opt_state = c
                continue
            if k == "Input":
                l = Input(c["shape"])
            elif k == "Dense":
                l = Dense(c["in_units"], c["out_units"], activation=c["layeract"])
            elif k in ("Conv2D", "ConvTranspose2D"):
                l = (Conv2D if k == "Conv2D" else ConvTranspose2D)(c["out_channels"], c["in_channels"], c["kernel_size"],
                                                                 activation=c["layeract"], stride=c.get("stride", 1),
                                                                 zero_padding=c.get("zero_padding", 0))
            elif k == "MaxPool2D":
                l = MaxPool2D(pool_size=c["pool_size"], stride=c["stride"], padding=c["padding"])
            elif k in ("BatchNorm1d", "BatchNorm2d"):
                l = BatchNorm1d(c["num_features"], c["momentum"], c["eps"]) if k == "BatchNorm1d" else \
                    BatchNorm2d(c["num_channels"], c["momentum"], c["eps"])
                l.running_mean, l.running_var = c["running_mean"], c["running_var"]
            elif k in ("Unpool2D_Nearest", "UpSampling2D_Nearest"):
                l = Unpool2D_Nearest(size=c["size"])
            elif k == "Flatten":
                l = Flatten()
            elif k == "Concatenate":
                l = Concatenate()
            else:
                raise ValueError(f"Unknown layer type: {k}")
            if "weights" in info:
                l._w_init = np.ascontiguousarray(info["weights"], np.float32)
                l._b_init = np.ascontiguousarray(info["bais"], np.float32)
            layers.append(l)
        model = cls(layers)
        if not with_optimizer:
            return model
        return model, (_Optimizer.from_state(model, opt_state) if opt_state is not None else None)


# ─────────────────────────────────────────────────────────────────────────────────────────────
# Losses
# ─────────────────────────────────────────────────────────────────────────────────────────────
def _scale_gradients(g):
    """In the fp16 precision modes the backward pass scales its gradient copies by a power of two taken from the largest
    entry of the loss gradient (fp16's exponent range is 2^-14 .. 2^16; a converging run's gradients leave it downwards)."""
    if sc.get_precision() in (4, 5):
        sc.grad_scale_update(g.main_ptr, g.size)


class Loss:
    """Each loss is the mean over the batch THIS process holds.  In a data-parallel run the ranks' gradients are averaged
    by the optimizer (dp.attach sets the 1/world factor there), so no scale is applied here."""

    def categorical_cross_entropy(self, y_pred, y, epsilon=1e-7):
        """mean over the batch of -sum(y * log(clip(y_pred, eps, 1-eps)))  (Seera.py:955-969)."""
        if y_pred._softmax_logits is None:
            raise NotImplementedError("categorical_cross_entropy expects the output of a softmax layer")
        logits = y_pred._softmax_logits
        z, yv = logits.value, y.value
        N, C = z.shape
        if tuple(yv.shape) != (N, C):
            raise ValueError(f"[cuTen]: Shapes {tuple(yv.shape)} and {(N, C)} not broadcastable")
        rows, loss, dz = _new((N,)), _new((1,)), _new((N, C))
        sc.softmax_cce_fwd_bwd(z.main_ptr, yv.main_ptr, y_pred.value.main_ptr, rows.main_ptr, loss.main_ptr, dz.main_ptr,
                               N, C, float(epsilon), float(f32(1.0 / N)))
        out = Tensor(loss)
        out._parents = (logits,)
        out._keep = (rows, yv)
        out._backward = lambda g: (_scale_gradients(dz), logits._accumulate(dz))       # g is the all-ones seed of a scalar loss
        return out

    def _elementwise(self, kernel, y_pred, y, *extra):
        p, yv = y_pred.value, y.value
        if p.size != yv.size:
            raise ValueError(f"[cuTen]: Shapes {tuple(p.shape)} and {tuple(yv.shape)} not broadcastable")
        part, loss, dp = _new((sc.mse_partials(p.size),)), _new((1,)), _new(p.shape)
        kernel(p.main_ptr, yv.main_ptr, part.main_ptr, loss.main_ptr, dp.main_ptr, p.size,
               float(f32(1.0 / p.size)), *extra)
        out = Tensor(loss)
        out._parents = (y_pred,)
        out._keep = (part, yv)
        out._backward = lambda g: (_scale_gradients(dp), y_pred._accumulate(dp))
        return out

    def mse(self, y_pred, y):
        """mean((y_pred - y)^2) over all elements (Seera.py:943-945)."""
        return self._elementwise(sc.mse_fwd_bwd, y_pred, y)

    def mae(self, y_pred, y):
        """mean(|y_pred - y|) over all elements (Seera.py:947-949)."""
        return self._elementwise(sc.mae_fwd_bwd, y_pred, y)

    def binary_cross_entropy(self, y_pred, y, epsilon=1e-15):
        """mean(-y log(p + eps) - (1 - y) log(1 - p + eps)) over all elements (Seera.py:951-953)."""
        return self._elementwise(sc.bce_fwd_bwd, y_pred, y, float(epsilon))


# ─────────────────────────────────────────────────────────────────────────────────────────────
# Optimizers: one fused launch over the whole parameter arena
# ─────────────────────────────────────────────────────────────────────────────────────────────
class _Optimizer:
    """Keeps its step scalars in a small device buffer so that a captured step graph can be replayed: the
    update kernel reads them at run time, `advance()` refreshes them before each replay."""

    def __init__(self, model):
        if not isinstance(model, Sequential):
            raise TypeError("Model should be Sequential")
        self.model = model
        self.use_gpu = True
        self._hyper = cuten(np.zeros(16, np.float32))
        # data parallel: the bucket hooks apply the update range by range behind each bucket's sum (dp.update_in_buckets);
        # step() then only completes the sums
        self.updates_by_bucket = False
        self._advanced = False

    def _state(self):
        n = max(self.model.n_arena, 1)
        return cuten._wrap(sc.cuda_zeros_f(n), (n,))

    def _grads_ready(self):
        m = self.model
        m.gather_grads()
        if m._allreduce is not None:
            m._allreduce(m.grads)

    def _grad_scale(self):
        return 1.0 / self.model.world if self.model._allreduce is not None else 1.0

    def _upload(self, values):
        h = np.zeros(16, np.float32)
        h[:len(values)] = np.asarray(values, np.float32)
        sc.upload_f32(self._hyper.main_ptr, h)

    @staticmethod
    def from_state(model, state):
        if state["kind"] == "adam":
            o = Adam(model, lr=state["lr"], beta1=state["beta1"], beta2=state["beta2"], eps=state["eps"])
            o.t = state["t"]
            arenas = (("m", o.m), ("v", o.v))
        else:
            o = SGD(model, lr=state["lr"], momentum=state["momentum"])
            arenas = (("velocity", o.velocity),)
        for name, dst in arenas:
            a = np.ascontiguousarray(state[name], np.float32)
            if a.size != dst.size:
                raise ValueError(f"optimizer state '{name}' has {a.size} values, the model's arena {dst.size}")
            sc.upload_f32(dst.main_ptr, a)
        return o

    def begin_step(self):
        """Call before backward when the update runs bucket by bucket during it: the step's scalars must be on the device before
        the first bucket's update is enqueued.  A no-op otherwise and inside a capture (replays refresh the scalars themselves)."""
        if self.updates_by_bucket and not sc.is_capturing() and not self._advanced:
            self.advance()
            self._advanced = True

    def update_range(self, begin, end):
        """The update of arena slots [begin, end) alone (the same arithmetic as the whole-arena launch)."""
        if not sc.is_capturing() and not self._advanced:        # first range of a step whose caller did not call begin_step()
            self.advance()
            self._advanced = True
        if end > begin:
            self._enqueue(begin, end)

    def step(self):
        """One update.  Outside a capture this also refreshes the device scalars and advances the step count."""
        if not sc.is_capturing() and not self._advanced:
            self.advance()
        self._advanced = False
        self._grads_ready()
        if not (self.updates_by_bucket and self.model._allreduce is not None):
            self._enqueue()


class SGD(_Optimizer):
    """vel = momentum*vel + lr*g ; w -= vel   (Seera.py:986-1008)."""

    def __init__(self, model, lr, momentum=0):
        super().__init__(model)
        self.lr, self.momentum = lr, momentum
        self.velocity = self._state()

    def advance(self):
        self._upload([self.lr, self.momentum, self._grad_scale()])

    def state_dict(self):
        return {"kind": "sgd", "lr": self.lr, "momentum": self.momentum, "velocity": self.velocity.to_host_f32().copy()}

    def _enqueue(self, begin=0, end=None):
        m = self.model
        end = m.n_arena if end is None else end
        o = 4 * begin
        sc.cuda_sgd_step_dev(m.params.main_ptr + o, m.grads.main_ptr + o, self.velocity.main_ptr + o, end - begin, self._hyper.main_ptr)


class Adam(_Optimizer):
    """m, v exponential averages with bias correction, t starting at 1 (Seera.py:1014-1086)."""

    def __init__(self, model, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8):
        super().__init__(model)
        self.lr, self.beta1, self.beta2, self.eps, self.t = lr, beta1, beta2, eps, 1
        self.m, self.v = self._state(), self._state()

    def advance(self):
        b1, b2 = self.beta1, self.beta2
        self._upload([self.lr, b1, 1 - b1, b2, 1 - b2, self.eps, 1 - b1 ** self.t, 1 - b2 ** self.t, self._grad_scale()])
        self.t += 1

    def state_dict(self):
        return {"kind": "adam", "lr": self.lr, "beta1": self.beta1, "beta2": self.beta2, "eps": self.eps, "t": self.t,
                "m": self.m.to_host_f32().copy(), "v": self.v.to_host_f32().copy()}

    def _enqueue(self, begin=0, end=None):
        md = self.model
        end = md.n_arena if end is None else end
        o = 4 * begin
        sc.cuda_adam_step_dev(md.params.main_ptr + o, md.grads.main_ptr + o, self.m.main_ptr + o, self.v.main_ptr + o, end - begin,
                              self._hyper.main_ptr)
