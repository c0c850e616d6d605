"""Generates tests/golden/*.npz from the UNMODIFIED reference (its Python layer on
device="cpu" over its own C++ engine compiled into oracle/_ref/).  Run in a container
that has the reference checkout; the GPU box never runs this.

    make -C oracle ref && python tests/golden/make_golden.py [/path/to/reference]

What is stored are OUTPUTS only (losses, gradients, updated weights, per-op results);
inputs and initial weights are regenerated at test time from the same seeds through
ml_framework_b200.workloads, so the files stay small.
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"

from oracle import ref_engine  # noqa: E402
from ml_framework_b200 import workloads as wl  # noqa: E402
sys.path.insert(0, HERE)
from cases import small_cases, op_cases  # noqa: E402

cpp = ref_engine.load()
assert cpp is not None, "build the reference engine first: make -C oracle ref"
sys.modules["seera_cpp"] = cpp
sys.modules["seera_cuda"] = types.ModuleType("seera_cuda")          # cuTen.py:3 imports it unconditionally
mpl = types.ModuleType("matplotlib"); mpl.pyplot = types.ModuleType("matplotlib.pyplot")
sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot   # Seera.py:4
sys.path.insert(0, REF)
import Seera as S  # noqa: E402
from Seera_Engine import Tensor, autograd4nn  # noqa: E402


def build_reference_model(work, params):
    layers = [S.Input(tuple(work.in_shape))]
    for L, P in zip(work.layers, params):
        t = L["type"]
        if t == "dense":
            lay = S.Dense(L["in"], L["out"], activation=L["act"])
        elif t == "conv":
            lay = S.Conv2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"])
        elif t == "convT":
            lay = S.ConvTranspose2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"])
        elif t == "maxpool":
            lay = S.MaxPool2D(L["k"], stride=L["stride"], padding=L["pad"])
        elif t == "unpool":
            lay = S.Unpool2D_Nearest(L["size"])
        elif t == "flatten":
            lay = S.Flatten()
        if P is not None:
            lay.set_weights(P[0].copy(), P[1].copy())
        layers.append(lay)
    return S.Sequential(layers)


def run_steps(work, n, steps, seed):
    params = work.params(seed)
    model = build_reference_model(work, params)
    X, Y = work.batch(n, seed)
    o = work.opt
    opt = S.Adam(model, lr=o["lr"]) if o["kind"] == "adam" else S.SGD(model, lr=o["lr"], momentum=o.get("momentum", 0))
    lossf = S.Loss().categorical_cross_entropy if work.loss == "cce" else S.Loss().mse
    out = {}
    for s in range(steps):
        yp = model.forward(Tensor(X, is_leaf=True))
        loss = lossf(yp, Tensor(Y))
        if loss.value.ndim > 0 and loss.value.size > 1:
            loss = loss.mean()
        model.zero_grad()
        autograd4nn(loss)
        out["loss%d" % s] = np.float32(np.asarray(loss.value).ravel()[0])
        if s == 0:
            out["pred0"] = np.asarray(yp.value, np.float32)
        k = 0
        for lay in model.model:
            if hasattr(lay, "update_params"):
                if s == 0:
                    out["dW%d" % k] = np.asarray(lay.weights.node.cp, np.float32).copy()
                    out["db%d" % k] = np.asarray(lay.bais.node.cp, np.float32).copy()
                k += 1
        opt.step()
        k = 0
        for lay in model.model:
            if hasattr(lay, "update_params"):
                out["W%d_s%d" % (k, s)] = np.asarray(lay.weights.value, np.float32).copy()
                out["b%d_s%d" % (k, s)] = np.asarray(lay.bais.value, np.float32).copy()
                k += 1
    return out


if __name__ == "__main__":
    c1 = wl.c1_small_cnn()
    np.savez_compressed(os.path.join(HERE, "c1_two_steps.npz"), **run_steps(c1, 64, 2, seed=1))
    for name, (work, n) in small_cases().items():
        np.savez_compressed(os.path.join(HERE, name + "_two_steps.npz"), **run_steps(work, n, 2, seed=2))
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **op_cases(cpp, np.random.RandomState(7)))
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith(".npz"):
            print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")
