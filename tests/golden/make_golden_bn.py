"""Generates tests/golden/bn_two_steps.npz from the UNMODIFIED reference Python layer on device="cpu" (its BatchNorm is
host-only in every mode): two SGD-with-momentum steps of the model in bn_case.py, then a prediction in evaluation mode.

    make -C oracle ref && python tests/golden/make_golden_bn.py [/path/to/reference]
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"

from oracle import ref_engine  # noqa: E402
import bn_case  # noqa: E402

cpp = ref_engine.load()
assert cpp is not None, "build the reference engine first: make -C oracle ref"
sys.modules["seera_cpp"] = cpp
sys.modules["seera_cuda"] = types.ModuleType("seera_cuda")
mpl = types.ModuleType("matplotlib"); mpl.pyplot = types.ModuleType("matplotlib.pyplot")
sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot
sys.path.insert(0, REF)
import Seera as S  # noqa: E402
from Seera_Engine import Tensor, autograd4nn  # noqa: E402

lays = bn_case.layers(S)
for i, (W, B) in bn_case.weights().items():
    if isinstance(lays[i], (S.BatchNorm1d, S.BatchNorm2d)):
        lays[i].gamma = Tensor(W.copy(), is_leaf=True); lays[i].beta = Tensor(B.copy(), is_leaf=True)
        lays[i].weights, lays[i].bais = lays[i].gamma, lays[i].beta
    else:
        lays[i].set_weights(W.copy(), B.copy())
model = S.Sequential(lays)
opt = S.SGD(model, lr=bn_case.LR, momentum=bn_case.MOMENTUM)
lossf = S.Loss().categorical_cross_entropy
X, Y = bn_case.data()
out = {}
for s in range(bn_case.STEPS):
    yp = model.forward(Tensor(X, is_leaf=True))
    loss = lossf(yp, Tensor(Y))
    if loss.value.ndim > 0 and loss.value.size > 1:
        loss = loss.mean()
    model.zero_grad()
    autograd4nn(loss)
    out["loss%d" % s] = np.float32(np.asarray(loss.value).ravel()[0])
    if s == 0:
        out["pred0"] = np.array(yp.value, np.float32, copy=True)
    k = 0
    for lay in model.model:
        if hasattr(lay, "update_params"):
            if s == 0:
                out["dW%d" % k] = np.array(lay.weights.node.cp, np.float32, copy=True)
                out["db%d" % k] = np.array(lay.bais.node.cp, np.float32, copy=True)
            k += 1
    opt.step()
    k = 0
    for lay in model.model:
        if hasattr(lay, "update_params"):
            out["W%d_s%d" % (k, s)] = np.array(lay.weights.value, np.float32, copy=True)
            out["b%d_s%d" % (k, s)] = np.array(lay.bais.value, np.float32, copy=True)
            k += 1
out["rm2"], out["rv2"] = lays[2].running_mean.copy(), lays[2].running_var.copy()
out["rm6"], out["rv6"] = lays[6].running_mean.copy(), lays[6].running_var.copy()
out["pred_eval"] = np.asarray(model.predict(Tensor(X, is_leaf=True)).value, np.float32)
np.savez_compressed(os.path.join(HERE, "bn_two_steps.npz"), **out)
print({k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items()})
