"""Case tables shared by the golden-vector generator and the parity tests: reduced training
configurations and a per-op sweep on small, odd shapes.  `op_cases(engine, rs)` runs against any
object exposing the reference CPU engine's function names (engine/src/bindings.cpp): the
compiled reference engine, the C restatement, or the GPU adapter."""
import numpy as np

from ml_framework_b200 import workloads as wl


def small_cases():
    """Reduced versions of C2, C3, C4 that keep every layer kind and the optimizer of the full
    configuration (the full C1 is small enough to store whole)."""
    c2 = wl.c2_mlp(); c2.layers = [wl.dense(784, 32), wl.dense(32, 32), wl.dense(32, 10, "softmax")]
    c3 = wl.c3_vgg(); c3.layers = [wl.conv(8, 3, 3, "relu", 1, 1), wl.maxpool(), wl.conv(16, 8, 3, "relu", 1, 1), wl.maxpool(),
                                   wl.conv(16, 16, 3, "relu", 1, 1), wl.maxpool(), wl.conv(16, 16, 3, "relu", 1, 1), wl.maxpool(),
                                   wl.flatten(), wl.dense(64, 32), wl.dense(32, 10, "softmax")]
    c4 = wl.c4_autoencoder(); c4.in_shape = (1, 16, 16)
    c4.layers = [wl.conv(4, 1, 3, "relu", 2, 1), wl.conv(8, 4, 3, "relu", 2, 1), wl.convT(4, 8, 4, "relu", 2, 1),
                 wl.unpool(2), wl.convT(1, 4, 3, "sigmoid", 1, 1)]
    c4._gen = lambda r, n: (lambda X: (X, X.copy()))(r.uniform(0, 1, (n, 1, 16, 16)).astype(np.float32))
    return {"c2s": (c2, 32), "c3s": (c3, 8), "c4s": (c4, 4)}


def op_cases(cpp, rs):
    """Per-op outputs of the reference engine on small, odd shapes."""
    out = {}
    f = lambda *s: rs.standard_normal(s).astype(np.float32)
    A, B = f(7, 13), f(13, 5)
    out["matmul"] = cpp.matmul(A, B)
    X, W = f(3, 5, 9, 7), f(6, 5, 3, 3)
    Y = cpp.conv2d_forward(X, W, 2, 1, 1, 2)
    dY = f(*Y.shape)
    out["conv_fwd"] = Y
    out["conv_dX"], out["conv_dW"] = cpp.conv2d_backward(dY, X, W, 2, 1, 1, 2)
    Xt, Wt = f(2, 4, 5, 6), f(4, 3, 4, 3)
    Yt = cpp.conv_transpose2d_forward(Xt, Wt, 2, 2, 1, 0)
    dYt = f(*Yt.shape)
    out["convT_fwd"] = Yt
    out["convT_dX"], out["convT_dW"] = cpp.conv_transpose2d_backward(dYt, Xt, Wt, 2, 2, 1, 0)
    Xp = np.maximum(f(2, 3, 9, 8), 0)      # post-ReLU input: all-zero windows give ties
    o, m = cpp.maxpool2d_forward(Xp, 3, 2, 2, 2, 1, 1)
    out["pool_out"], out["pool_mask"] = o, np.asarray(m, np.int32)
    dO = f(*o.shape)
    out["pool_dX"] = cpp.maxpool2d_backward(dO, m, 2, 3, 9, 8, 3, 2, 2, 2, 1, 1)
    Xu = f(2, 3, 4, 5)
    out["unpool_fwd"] = cpp.unpooling_forward(Xu, 2, 3)
    out["unpool_bwd"] = cpp.unpooling_backward(f(2, 3, 8, 15), 2, 3, 4, 5, 2, 3)
    Z = f(6, 10)
    s = cpp.softmax(Z)
    out["softmax"] = s
    out["softmax_vjp"] = cpp.softmax_vjp(s, f(6, 10))
    U = f(50) * 2
    for name in ("relu", "sigmoid", "tanh_act", "exp_act", "abs_act"):
        o, g = getattr(cpp, name)(U)
        out[name + "_o"], out[name + "_g"] = o, g
    Up = np.abs(U) + 0.1
    for name in ("log_act", "sqrt_act"):
        o, g = getattr(cpp, name)(Up)
        out[name + "_o"], out[name + "_g"] = o, g
    o, g = cpp.pow_act(Up, 2.5); out["pow_o"], out["pow_g"] = o, g
    o, g = cpp.clip_act(U, -0.5, 0.75); out["clip_o"], out["clip_g"] = o, g
    return out
