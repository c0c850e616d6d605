"""Seeded synthetic workloads: the five training configurations the benchmark and the
parity tests run, as plain layer lists plus NumPy generators for inputs and weights.

Layer records (dicts):
  {"type": "conv",  "out": F, "in": C, "k": (KH, KW), "act": a, "stride": (sh, sw), "pad": (ph, pw)}
  {"type": "convT", "out": Cout, "in": Cin, "k": (KH, KW), "act": a, "stride": ..., "pad": ...}
  {"type": "dense", "in": K, "out": N, "act": a}
  {"type": "maxpool", "k": (KH, KW), "stride": (sh, sw), "pad": (ph, pw)}
  {"type": "unpool", "size": (sw, sh)}
  {"type": "flatten"}
Activations: "relu", "sigmoid", "tanh", "softmax".  Weight layouts follow the reference's
layers: Dense (in, out) with bias (1, out) (Seera.py:99-125); Conv2D (F, C, KH, KW) with bias
(1, F, 1, 1) (Seera.py:215-227); ConvTranspose2D (Cin, Cout, KH, KW) with bias (1, Cout, 1, 1)
(Seera.py:377-390).  Initial scales follow the layer defaults there: He-normal for the
convolutions, Glorot-uniform for Dense, zero biases.

No public data set is read: every input is drawn from a seeded RandomState with the shape
and value range the configuration states.
"""
import numpy as np


def conv(out, inp, k=3, act="relu", stride=1, pad=0):
    t = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    return {"type": "conv", "out": out, "in": inp, "k": t(k), "act": act, "stride": t(stride), "pad": t(pad)}


def convT(out, inp, k=3, act="relu", stride=1, pad=0):
    d = conv(out, inp, k, act, stride, pad)
    d["type"] = "convT"
    return d


def dense(inp, out, act="relu"):
    return {"type": "dense", "in": inp, "out": out, "act": act}


def maxpool(k=2, stride=2, pad=0):
    t = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    return {"type": "maxpool", "k": t(k), "stride": t(stride), "pad": t(pad)}


def unpool(size=2):
    return {"type": "unpool", "size": (size, size) if isinstance(size, int) else tuple(size)}


def flatten():
    return {"type": "flatten"}


def bf16_round(a):
    """Round fp32 values to the nearest bf16-representable fp32 (ties to even)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def init_params(layers, rng, round_bf16=False):
    """One (W, b) pair per parametrised layer, in layer order; None for the others."""
    params = []
    for L in layers:
        if L["type"] == "dense":
            lim = np.sqrt(6.0 / (L["in"] + L["out"]))
            W = rng.uniform(-lim, lim, (L["in"], L["out"])).astype(np.float32)
            b = np.zeros((1, L["out"]), np.float32)
        elif L["type"] == "conv":
            fan_in = L["in"] * L["k"][0] * L["k"][1]
            W = (rng.standard_normal((L["out"], L["in"]) + L["k"]) * np.sqrt(2.0 / fan_in)).astype(np.float32)
            b = np.zeros((1, L["out"], 1, 1), np.float32)
        elif L["type"] == "convT":
            fan_in = L["in"] * L["k"][0] * L["k"][1]
            W = (rng.standard_normal((L["in"], L["out"]) + L["k"]) * np.sqrt(2.0 / fan_in)).astype(np.float32)
            b = np.zeros((1, L["out"], 1, 1), np.float32)
        else:
            params.append(None)
            continue
        if round_bf16:
            W = bf16_round(W)
        params.append((W, b))
    return params


class Workload:
    """name, layers, loss ('cce' | 'mse'), optimizer record, precision ('fp32' | 'bf16'),
    and `batch(n, seed)` -> (X, Y) NumPy arrays for n samples."""

    def __init__(self, name, layers, loss, opt, in_shape, batch, precision, gen, flops_fwd):
        self.name, self.layers, self.loss, self.opt = name, layers, loss, opt
        self.in_shape, self.batch_size, self.precision = in_shape, batch, precision
        self._gen, self.flops_fwd = gen, flops_fwd

    def batch(self, n=None, seed=0):
        return self._gen(np.random.RandomState(seed), n or self.batch_size)

    def params(self, seed=0):
        return init_params(self.layers, np.random.RandomState(1000 + seed), self.precision == "bf16")

    def flops_per_sample(self):
        """Algorithmic FLOPs of one training step per sample: forward GEMM/conv work x3
        (forward, data gradient, weight gradient), padding taps counted."""
        return 3 * self.flops_fwd


def _onehot(rng, n, classes=10):
    return np.eye(classes, dtype=np.float32)[rng.randint(0, classes, n)]


def _fwd_flops(layers, in_shape):
    shp, fl = tuple(in_shape), 0
    for L in layers:
        if L["type"] == "conv":
            C, H, W = shp
            OH = (H + 2 * L["pad"][0] - L["k"][0]) // L["stride"][0] + 1
            OW = (W + 2 * L["pad"][1] - L["k"][1]) // L["stride"][1] + 1
            fl += 2 * L["out"] * OH * OW * C * L["k"][0] * L["k"][1]
            shp = (L["out"], OH, OW)
        elif L["type"] == "convT":
            C, H, W = shp
            Ho = (H - 1) * L["stride"][0] - 2 * L["pad"][0] + L["k"][0]
            Wo = (W - 1) * L["stride"][1] - 2 * L["pad"][1] + L["k"][1]
            fl += 2 * L["out"] * L["k"][0] * L["k"][1] * C * H * W
            shp = (L["out"], Ho, Wo)
        elif L["type"] == "dense":
            fl += 2 * L["in"] * L["out"]
            shp = (L["out"],)
        elif L["type"] == "maxpool":
            C, H, W = shp
            shp = (C, (H + 2 * L["pad"][0] - L["k"][0]) // L["stride"][0] + 1,
                   (W + 2 * L["pad"][1] - L["k"][1]) // L["stride"][1] + 1)
        elif L["type"] == "unpool":
            C, H, W = shp
            shp = (C, H * L["size"][1], W * L["size"][0])
        elif L["type"] == "flatten":
            shp = (int(np.prod(shp)),)
    return fl


def _make(name, layers, loss, opt, in_shape, batch, precision, gen):
    return Workload(name, layers, loss, opt, in_shape, batch, precision, gen, _fwd_flops(layers, in_shape))


def c1_small_cnn():
    layers = [conv(8, 1, 3, "relu", 1, 1), maxpool(2, 2), conv(16, 8, 3, "relu", 1, 1), maxpool(2, 2),
              flatten(), dense(784, 10, "softmax")]
    gen = lambda r, n: (r.uniform(0, 1, (n, 1, 28, 28)).astype(np.float32), _onehot(r, n))
    return _make("C1 small CNN 1x28x28 b64 fp32 Adam", layers, "cce", {"kind": "adam", "lr": 1e-3},
                 (1, 28, 28), 64, "fp32", gen)


def c2_mlp():
    layers = [dense(784, 1024, "relu"), dense(1024, 1024, "relu"), dense(1024, 10, "softmax")]
    gen = lambda r, n: (bf16_round(r.standard_normal((n, 784)).astype(np.float32)), _onehot(r, n))
    return _make("C2 MLP 784-1024-1024-10 b4096 bf16 SGD-momentum", layers, "cce",
                 {"kind": "sgd", "lr": 0.01, "momentum": 0.9}, (784,), 4096, "bf16", gen)


def c3_vgg():
    layers = [conv(64, 3, 3, "relu", 1, 1), maxpool(2, 2), conv(128, 64, 3, "relu", 1, 1), maxpool(2, 2),
              conv(256, 128, 3, "relu", 1, 1), maxpool(2, 2), conv(256, 256, 3, "relu", 1, 1), maxpool(2, 2),
              flatten(), dense(1024, 256, "relu"), dense(256, 10, "softmax")]
    gen = lambda r, n: (r.standard_normal((n, 3, 32, 32)).astype(np.float32), _onehot(r, n))
    return _make("C3 VGG-style CNN 3x32x32 b512 fp32 Adam", layers, "cce", {"kind": "adam", "lr": 1e-3},
                 (3, 32, 32), 512, "fp32", gen)


def c4_autoencoder():
    layers = [conv(32, 1, 3, "relu", 2, 1), conv(64, 32, 3, "relu", 2, 1),
              convT(32, 64, 4, "relu", 2, 1), unpool(2), convT(1, 32, 3, "sigmoid", 1, 1)]

    def gen(r, n):
        X = r.uniform(0, 1, (n, 1, 64, 64)).astype(np.float32)
        return X, X.copy()
    return _make("C4 conv autoencoder 1x64x64 b256 fp32 Adam", layers, "mse", {"kind": "adam", "lr": 1e-3},
                 (1, 64, 64), 256, "fp32", gen)


C5_SHAPES = [(64, 56), (128, 28), (256, 14), (512, 7)]   # (C = K, H = W), N = 256, 3x3 s1 p1


def c5_conv_bwd(ck, hw, n=256, seed=5):
    """Operands of one Conv2D-backward microbenchmark point: X, W, dY rounded to bf16."""
    r = np.random.RandomState(seed)
    X = bf16_round(r.standard_normal((n, ck, hw, hw)).astype(np.float32))
    W = bf16_round((r.standard_normal((ck, ck, 3, 3)) * 0.02).astype(np.float32))
    dY = bf16_round(r.standard_normal((n, ck, hw, hw)).astype(np.float32))
    return X, W, dY


WORKLOADS = {"c1": c1_small_cnn, "c2": c2_mlp, "c3": c3_vgg, "c4": c4_autoencoder}
