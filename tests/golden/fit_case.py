"""The `fit` / checkpoint case shared by make_golden_fit.py (reference side) and the tests (this package's side):
configuration C1's model on 160 seeded samples, 3 epochs of Adam at batch 32."""
import numpy as np

from ml_framework_b200 import workloads as wl

SEED, SHUFFLE_SEED, SAMPLES, BATCH, EPOCHS, LR = 6, 77, 160, 32, 3, 1e-3


def data():
    return wl.c1_small_cnn().batch(SAMPLES, SEED)


def build(S, **kw):
    """C1's layers from module S (the reference's Seera or this package's seera), with the seeded initial weights."""
    work = wl.c1_small_cnn()
    layers = [S.Input((1, 28, 28))]
    for L, P in zip(work.layers, work.params(SEED)):
        lay = {"conv": lambda: S.Conv2D(L["out"], L["in"], L["k"], L["act"], stride=L["stride"], zero_padding=L["pad"]),
               "maxpool": lambda: S.MaxPool2D(L["k"], stride=L["stride"], padding=L["pad"]),
               "flatten": lambda: S.Flatten(),
               "dense": lambda: S.Dense(L["in"], L["out"], activation=L["act"])}[L["type"]]()
        if P is not None:
            lay.set_weights(P[0].copy(), P[1].copy())
        layers.append(lay)
    return S.Sequential(layers, **kw)
