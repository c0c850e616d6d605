"""One training step (forward, loss, backward, optimizer) on the CPU, op for op as the
reference's CPU path runs it.  TEST INFRASTRUCTURE ONLY.

`RefNet` replays, for a layer list from ml_framework_b200.workloads, the sequence of engine
calls the reference's Python layer issues when `device="cpu"`:

  Dense.forward            z = x.matmul(W) + b ; act(z)                 Seera.py:133-138
  Conv2D.forward           z = conv2d(x, W) + b ; act(z)                Seera.py:235-259
  ConvTranspose2D.forward  z = conv_transpose2d(x, W) + b ; act(z)      Seera.py:398-422
  MaxPool2D / Unpool2D_Nearest / Flatten                                Seera.py:471-477, 323-326, 300-303
  Loss.categorical_cross_entropy  clip -> log -> (-y * .) -> sum(-1) -> mean   Seera.py:955-969
  Loss.mse                        ((p - y) ** 2).mean()                         Seera.py:943-945
  autograd4nn.backward_step       Seera_Engine.py:259-598
  Adam.step / SGD.step (CPU)      Seera.py:1064-1086, 1002-1008

`engine` is any object with the function names of the reference's `seera_cpp` module
(engine/src/bindings.cpp): either that module itself (oracle.ref_engine.load()) or the C
restatement (oracle.cpu_oracle).  Bias gradients and the loss reductions are NumPy, as
on the reference's CPU path (Seera_Engine.py:30-39, Seera_init.py:476, :514).

`quant` (optional) is applied to every GEMM / convolution operand before the engine call:
with ml_framework_b200.workloads.bf16_round it gives the "matched quantisation" oracle for
the bf16 configurations - the arithmetic stays the engine's fp32, only its inputs carry
the rounding the tensor-core path applies.  With `quant_forward=False` only the backward products' operands are
rounded: the oracle of a policy that runs the forward pass in fp32-class split products and the backward GEMMs in
one bf16 pass.
"""
import numpy as np


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class RefNet:
    def __init__(self, layers, params, loss, opt, engine, quant=None, quant_forward=True):
        self.layers, self.loss_kind, self.opt, self.E = layers, loss, dict(opt), engine
        self.q = quant or (lambda a: a)
        self.qf = self.q if quant_forward else (lambda a: a)      # forward operands: rounded too, or left in fp32
        self.params = [None if p is None else [p[0].copy(), p[1].copy()] for p in params]
        self.state = [None if p is None else [np.zeros_like(p[0]), np.zeros_like(p[1]),
                                              np.zeros_like(p[0]), np.zeros_like(p[1])] for p in params]
        self.t = 1                     # Seera.py:1023
        self.first = True
        self.grads = None
        self.acts = None

    # ---- forward ---------------------------------------------------------
    def _act(self, z, kind):
        E = self.E
        if kind == "relu":
            return E.relu(z)
        if kind == "sigmoid":
            return E.sigmoid(z)
        if kind == "tanh":
            return E.tanh_act(z)
        if kind == "softmax":
            return E.softmax(z), None
        raise ValueError(kind)

    def forward(self, X):
        E, q = self.E, self.qf
        x = np.ascontiguousarray(X, dtype=np.float32)
        tape = []
        for L, P in zip(self.layers, self.params):
            t = L["type"]
            if t == "dense":
                z = E.matmul(q(x), q(P[0])) + P[1]
                y, g = self._act(z, L["act"])
                tape.append((x, y, g))
            elif t == "conv":
                z = E.conv2d_forward(q(x), q(P[0]), *L["stride"], *L["pad"]) + P[1]
                y, g = self._act(z, L["act"])
                tape.append((x, y, g))
            elif t == "convT":
                z = E.conv_transpose2d_forward(q(x), q(P[0]), *L["stride"], *L["pad"]) + P[1]
                y, g = self._act(z, L["act"])
                tape.append((x, y, g))
            elif t == "maxpool":
                y, mask = E.maxpool2d_forward(x, *L["k"], *L["stride"], *L["pad"])
                tape.append((x, y, np.array(mask, dtype=np.int32)))
            elif t == "unpool":
                sw, sh = L["size"]               # Seera_init.py:793
                y = E.unpooling_forward(x, sh, sw)
                tape.append((x, y, None))
            elif t == "flatten":
                y = x.reshape(x.shape[0], -1)
                tape.append((x, y, None))
            else:
                raise ValueError(t)
            x = np.ascontiguousarray(y, dtype=np.float32)
        self.tape = tape
        return x

    # ---- loss + its gradient w.r.t. the prediction --------------------------
    def loss_and_grad(self, P, Y):
        E = self.E
        Y = np.ascontiguousarray(Y, dtype=np.float32)
        if self.loss_kind == "cce":
            eps = 1e-7
            pc, gclip = E.clip_act(P, eps, 1.0 - eps)
            lg, glog = E.log_act(pc)
            negy = Y * np.float32(-1)
            per = (negy * lg).sum(axis=-1)
            loss = np.float32(np.mean(per))
            n = per.shape[0]
            d_per = np.full(per.shape, np.float32(1.0 / n), np.float32)           # mean backward
            d_prod = np.broadcast_to(d_per[:, None], P.shape).astype(np.float32)  # sum(-1) backward
            d_log = E.mul(negy, d_prod)                                           # mul backward
            d_clip = E.mul(glog, d_log)
            return loss, E.mul(gclip, d_clip)
        if self.loss_kind == "mse":
            diff = P + Y * np.float32(-1)
            sq, gsq = E.pow_act(diff, 2.0)
            loss = np.float32(np.mean(sq))
            d_sq = np.full(sq.shape, np.float32(1.0 / sq.size), np.float32)
            return loss, E.mul(gsq, d_sq)
        raise ValueError(self.loss_kind)

    # ---- backward ----------------------------------------------------------
    def backward(self, dY):
        E, q = self.E, self.q
        grads = [None] * len(self.layers)
        d = np.ascontiguousarray(dY, dtype=np.float32)
        for i in reversed(range(len(self.layers))):
            L, P = self.layers[i], self.params[i]
            x, y, aux = self.tape[i]
            t = L["type"]
            if t in ("dense", "conv", "convT"):
                if L["act"] == "softmax":
                    dz = E.softmax_vjp(y, d)                       # Seera_Engine.py:371-379
                else:
                    dz = E.mul(aux, d)                             # Seera_Engine.py:590-591
                dz = np.ascontiguousarray(dz, dtype=np.float32)
                if t == "dense":
                    db = dz.sum(axis=(0,), keepdims=True)          # Seera_Engine.py:30-39
                    dx = E.matmul(q(dz), q(np.ascontiguousarray(P[0].T)))       # :561
                    dW = E.matmul(q(np.ascontiguousarray(x.T)), q(dz))          # :563
                elif t == "conv":
                    db = dz.sum(axis=(0, 2, 3), keepdims=True)
                    dx, dW = E.conv2d_backward(q(dz), q(x), q(P[0]), *L["stride"], *L["pad"])
                else:
                    db = dz.sum(axis=(0, 2, 3), keepdims=True)
                    dx, dW = E.conv_transpose2d_backward(q(dz), q(x), q(P[0]), *L["stride"], *L["pad"])
                grads[i] = (np.asarray(dW, np.float32), np.asarray(db, np.float32))
                d = dx
            elif t == "maxpool":
                N, C, H, W = x.shape
                d = E.maxpool2d_backward(d, aux, N, C, H, W, *L["k"], *L["stride"], *L["pad"])
            elif t == "unpool":
                N, C, H, W = x.shape
                sw, sh = L["size"]
                d = E.unpooling_backward(d, N, C, H, W, sh, sw)
            elif t == "flatten":
                d = d.reshape(x.shape)
            d = np.ascontiguousarray(d, dtype=np.float32)
        self.grads = grads
        self.dX = d
        return grads

    # ---- optimizer -----------------------------------------------------------
    def apply(self, grads, grad_scale=1.0):
        o = self.opt
        for P, S, G in zip(self.params, self.state, grads):
            if P is None:
                continue
            for j in range(2):
                g = G[j] if grad_scale == 1.0 else (G[j] * np.float32(grad_scale))
                if o["kind"] == "adam":
                    b1, b2, eps, lr = o.get("beta1", 0.9), o.get("beta2", 0.999), o.get("eps", 1e-8), o["lr"]
                    m, v = S[j], S[2 + j]
                    m[...] = b1 * m + (1 - b1) * g                               # Seera.py:1069-1073
                    v[...] = b2 * v + (1 - b2) * (g ** 2)
                    mh = m / (1 - b1 ** self.t)
                    vh = v / (1 - b2 ** self.t)
                    P[j] -= (lr * mh) / (vh ** 0.5 + eps)                        # Seera.py:1081-1084
                else:
                    vel = S[j]
                    vel[...] = o.get("momentum", 0.0) * vel + o["lr"] * g       # Seera.py:1006-1007
                    P[j] -= vel
        self.t += 1

    def step(self, X, Y):
        """forward + loss + backward + optimizer; returns the loss before the update."""
        P = self.forward(X)
        loss, dP = self.loss_and_grad(P, Y)
        grads = self.backward(dP)
        self.apply(grads)
        return float(loss)
