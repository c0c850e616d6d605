"""Generates tests/golden/fit_c1.npz and tests/golden/ref_c1_checkpoint.pkl from the UNMODIFIED reference Python layer on
device="cpu": `Sequential.fit` (Seera.py:729-788) on a small seeded data set of configuration C1's shapes, then the
reference's own `Sequential.save` (Seera.py:790-860) and a prediction of the trained model on a fixed batch.

    make -C oracle ref && python tests/golden/make_golden_fit.py [/path/to/reference]

Stored: the loss history of `fit`, the prediction, and the pickle file exactly as the reference wrote it.  The data set,
the initial weights and the shuffling order are regenerated at test time from the same seeds (fit_case.py)."""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SEERA_REFERENCE", "/root/reference")

from oracle import ref_engine  # noqa: E402
import fit_case  # noqa: E402

cpp = ref_engine.load()
assert cpp is not None, "build the reference engine first: make -C oracle ref"
sys.modules["seera_cpp"] = cpp
sys.modules["seera_cuda"] = types.ModuleType("seera_cuda")
mpl = types.ModuleType("matplotlib"); mpl.pyplot = types.ModuleType("matplotlib.pyplot")
sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot
sys.path.insert(0, REF)
import Seera as S  # noqa: E402
from Seera_Engine import Tensor  # noqa: E402

model = fit_case.build(S)
X, Y = fit_case.data()
opt = S.Adam(model, lr=fit_case.LR)
np.random.seed(fit_case.SHUFFLE_SEED)                       # fit() shuffles with the global NumPy generator
hist = model.fit(X, Y, opt, S.Loss().categorical_cross_entropy, Epochs=fit_case.EPOCHS, batch_size=fit_case.BATCH,
                 Loss_interval=100)
pred = np.asarray(model.forward(Tensor(X[:fit_case.BATCH], is_leaf=True)).value, np.float32)
model.save(os.path.join(HERE, "ref_c1_checkpoint.pkl"))
np.savez_compressed(os.path.join(HERE, "fit_c1.npz"), history=np.asarray(hist, np.float64), pred=pred)
print("history", hist)
for fn in ("fit_c1.npz", "ref_c1_checkpoint.pkl"):
    print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")
