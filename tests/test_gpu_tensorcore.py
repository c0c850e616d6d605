"""GPU parity of the tcgen05 tensor-core contraction (precision modes 1 and 2) through the C ABI.

Mode 1 (bf16 operands, fp32 accumulate) is compared with the CPU oracle fed the SAME bf16-rounded
operands ("matched quantisation": products of bf16 values are exact in fp32, so only the summation
order differs): rel-L2 <= 1e-5.  Mode 2 (bf16x3 split) is compared with the untouched fp32 oracle:
rel-L2 <= 2e-5 (observed ~5e-6), far inside the 2e-3 gate of the training configurations.  Mode 4 (fp16x3 split with
power-of-two scales) likewise against the fp32 oracle: rel-L2 <= 1e-5.  Its arithmetic would allow 7e-8 (the dropped lo*lo
term is 2^-22 of a product); observed on N(0,1) operands is 1e-7 for short contractions and 3.7e-6 at K = 1024 in one
accumulation chain - the tensor core keeps fewer low-order bits of a 22-bit fp16 product than of a 16-bit bf16 product when
it aligns the addends, and that truncation adds up along the chain."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co
from oracle.train_oracle import RefNet
from ml_framework_b200 import workloads as wl
import cases

pytestmark = pytest.mark.gpu

TOL = {1: 1e-5, 2: 2e-5, 4: 1e-5}


@pytest.fixture(scope="module")
def E():
    from ml_framework_b200 import capi
    import engine_np
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    capi.check(L.seera_set_option(b"wgrad_single", 0))        # mode 4 at its full three products, weight gradients included
    capi.check(L.seera_set_option(b"skinny_gemm", 0))         # products of few output columns on the tensor cores too
    yield engine_np
    capi.check(L.seera_set_option(b"wgrad_single", 1))
    capi.check(L.seera_set_option(b"skinny_gemm", 1))
    assert L.seera_tc_device_status() == 0            # no bounded wait ever expired
    L.seera_set_precision(0)


def _prep(mode, *arrays):
    from ml_framework_b200 import capi
    capi.load().seera_set_precision(mode)
    return [wl.bf16_round(a) if mode == 1 else a for a in arrays]


MATMUL = [(1, 3, 2), (5, 7, 3), (128, 64, 32), (129, 65, 33), (64, 784, 10), (300, 10, 1024), (257, 1000, 255), (4096, 1024, 1024)]


@pytest.mark.parametrize("mode", [1, 2, 4])
@pytest.mark.parametrize("M,K,N", MATMUL)
def test_matmul_and_backward(E, mode, M, K, N):
    rs = np.random.RandomState(M + K + N)
    A, B, dC = _prep(mode, *(rs.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (M, N))))
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert rel_l2(E.matmul(A, B), ref) < TOL[mode]
    dA, dB = E.matmul_backward(A, B, dC)
    assert rel_l2(dA, dC.astype(np.float64) @ B.T.astype(np.float64)) < TOL[mode]
    assert rel_l2(dB, A.T.astype(np.float64) @ dC.astype(np.float64)) < TOL[mode]


@pytest.mark.parametrize("mode", [1, 4])
@pytest.mark.parametrize("M,K,N,batch", [(1, 1, 1, 1), (5, 7, 3, 1), (64, 784, 10, 1), (512, 256, 10, 1), (4096, 1024, 10, 1), (33, 300, 16, 3),
                                         (1000, 513, 7, 1), (70000, 24, 2, 1), (64, 3136, 10, 1), (2000, 1500, 3, 1), (1300, 2100, 13, 1)])
def test_products_of_few_output_columns_are_exact_fp32_in_every_mode(E, mode, M, K, N, batch):
    """By default a product of at most 16 output columns (a classifier head) runs as fp32 on the CUDA cores whatever the precision
    mode: the plain entries, the fused forward and the one-call backward with its bias gradient all agree with double precision
    to fp32 rounding, the operands are NOT rounded to the mode's 16-bit type, and two runs give the same bits."""
    import ctypes
    from ml_framework_b200 import capi
    from engine_np import _Dev
    L = capi.load()
    L.seera_set_precision(mode)
    capi.check(L.seera_set_option(b"skinny_gemm", 1))
    try:
        rs = np.random.RandomState(M + K + N)
        A = rs.standard_normal((batch, M, K)).astype(np.float32)
        B = (rs.standard_normal((K, N)) * 0.1).astype(np.float32)
        bias, g = rs.standard_normal(N).astype(np.float32), rs.standard_normal((batch, M, N)).astype(np.float32)
        A64, B64, g64 = A.reshape(-1, K).astype(np.float64), B.astype(np.float64), g.reshape(-1, N).astype(np.float64)
        with _Dev() as d:
            pa, pb, pbias, pg = d.up(A), d.up(B), d.up(bias), d.up(g)
            c, da, db, dbias = d.new(batch * M * N), d.new(batch * M * K), d.new(K * N), d.new(N)
            capi.check(L.seera_cuda_matmul(pa, pb, c, M, N, K, batch))
            assert rel_l2(d.down(c, (batch * M, N)), A64 @ B64) < 2e-6
            capi.check(L.seera_cuda_matmul_bwd(pa, pb, pg, da, db, M, N, K, batch))
            first = d.down(db, (K, N)).copy()
            assert rel_l2(d.down(da, (batch * M, K)), g64 @ B64.T) < 2e-6
            assert rel_l2(first, A64.T @ g64) < 2e-6
            capi.check(L.seera_cuda_matmul_bwd(pa, pb, pg, da, db, M, N, K, batch))
            assert np.array_equal(first, d.down(db, (K, N)))
            if batch == 1:
                capi.check(L.seera_matmul_bias_act_fwd(pa, pb, pbias, c, M, N, K, 1))
                y = d.down(c, (M, N))
                assert rel_l2(y, np.maximum(A64 @ B64 + bias, 0)) < 2e-6
                ak, wk = ctypes.c_void_p(), ctypes.c_void_p()
                capi.check(L.seera_matmul_bias_act_fwd_s(pa, pb, pbias, c, M, N, K, 1, None, ctypes.byref(ak), ctypes.byref(wk), None))
                assert not ak.value and not wk.value and np.array_equal(y, d.down(c, (M, N)))
                for act, slope in ((0, np.ones((M, N))), (1, (y > 0).astype(np.float64))):
                    capi.check(L.seera_matmul_act_bwd(pa, pb, c, pg, da, db, dbias, M, N, K, act, None, None))
                    dz = g64 * slope
                    assert rel_l2(d.down(dbias, (N,)), dz.sum(axis=0)) < 1e-5
                    assert rel_l2(d.down(da, (M, K)), dz @ B64.T) < 2e-6
                    assert rel_l2(d.down(db, (K, N)), A64.T @ dz) < 2e-6
    finally:
        capi.check(L.seera_set_option(b"skinny_gemm", 0))


CONV = [(1, 1, 5, 5, 1, 3, 3, 1, 1, 0, 0), (2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1), (3, 5, 9, 7, 6, 3, 3, 2, 1, 1, 2),
        (2, 4, 11, 13, 7, 5, 3, 2, 2, 2, 1), (4, 8, 14, 14, 16, 1, 1, 1, 1, 0, 0), (8, 32, 32, 32, 64, 3, 3, 2, 2, 1, 1),
        (2, 130, 6, 6, 70, 3, 3, 1, 1, 1, 1), (16, 64, 16, 16, 300, 3, 3, 1, 1, 1, 1),
        (2, 3, 9, 9, 4, 1, 1, 2, 2, 0, 0), (2, 8, 32, 32, 8, 3, 3, 2, 2, 0, 0), (2, 16, 15, 17, 12, 4, 4, 3, 2, 2, 1)]


@pytest.mark.parametrize("mode", [1, 2, 4])
@pytest.mark.parametrize("shape", CONV)
def test_conv2d(E, mode, shape):
    N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape))
    X, Wt = _prep(mode, rs.standard_normal((N, C, H, W)).astype(np.float32), rs.standard_normal((F, C, KH, KW)).astype(np.float32))
    R = co.conv2d_forward(X, Wt, sh, sw, ph, pw)
    assert rel_l2(E.conv2d_forward(X, Wt, sh, sw, ph, pw), R) < TOL[mode]
    dY, = _prep(mode, rs.standard_normal(R.shape).astype(np.float32))
    dX, dW = E.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    rX, rW = co.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    assert rel_l2(dX, rX) < TOL[mode] and rel_l2(dW, rW) < TOL[mode]


# channels-last bf16 copy of the input = N*H*W*Cp*2 bytes: 64 KiB, 127.5 KiB (just below), 128 KiB (at) and 256 KiB (above)
# the size under which drivers up to CUDA 13.1 need one bit of the IM2COL descriptor cleared (conv_tma.cu, make_map_im2col)
@pytest.mark.parametrize("N,C,H,W", [(2, 64, 16, 16), (1, 8, 51, 160), (4, 64, 16, 16), (8, 64, 16, 16)])
def test_im2col_maps_of_tensors_below_128_kib(E, N, C, H, W):
    rs = np.random.RandomState(N * C + H)
    X, Wt = _prep(1, rs.standard_normal((N, C, H, W)).astype(np.float32), rs.standard_normal((64, C, 3, 3)).astype(np.float32))
    assert rel_l2(E.conv2d_forward(X, Wt, 1, 1, 1, 1), co.conv2d_forward(X, Wt, 1, 1, 1, 1)) < TOL[1]
    dY, = _prep(1, rs.standard_normal((N, 64, H, W)).astype(np.float32))
    dX, dW = E.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
    rX, rW = co.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
    assert rel_l2(dX, rX) < TOL[1] and rel_l2(dW, rW) < TOL[1]


@pytest.mark.parametrize("mode", [1, 4])
def test_cta_pair_tiles_give_the_same_results(E, mode):
    """The "pair_tiles" option (clusters of two CTAs on 256-row tiles, tcgen05 cta_group::2) against the single-CTA kernel:
    Dense forward / dA / dB and convolution forward / dX / dW, shapes with full, partial and odd tiles."""
    from ml_framework_b200 import capi
    L = capi.load()
    rs = np.random.RandomState(5 + mode)
    cases = []
    for (M, K, N) in ((512, 256, 256), (1000, 520, 130), (2048, 64, 64), (4096, 1024, 1024)):
        A, B, dC = _prep(mode, *(rs.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (M, N))))
        cases.append(lambda A=A, B=B, dC=dC: (E.matmul(A, B),) + tuple(E.matmul_backward(A, B, dC)))
    for shape in ((64, 64, 16, 16, 128, 3, 3, 1, 1, 1, 1), (32, 128, 8, 8, 256, 3, 3, 1, 1, 1, 1), (40, 32, 33, 31, 72, 3, 3, 2, 2, 1, 1)):
        N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
        X, Wt = _prep(mode, rs.standard_normal((N, C, H, W)).astype(np.float32), rs.standard_normal((F, C, KH, KW)).astype(np.float32))
        OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
        dY, = _prep(mode, rs.standard_normal((N, F, OH, OW)).astype(np.float32))
        cases.append(lambda X=X, Wt=Wt, dY=dY, g=(sh, sw, ph, pw): (E.conv2d_forward(X, Wt, *g),) + tuple(E.conv2d_backward(dY, X, Wt, *g)))
    try:
        for run in cases:
            capi.check(L.seera_set_option(b"pair_tiles", 0))
            want = run()
            capi.check(L.seera_set_option(b"pair_tiles", 1))
            got = run()
            for a, b in zip(got, want):
                assert rel_l2(a, b) < TOL[mode]     # same products; split-K chunking may differ, hence not bit-equal
    finally:
        capi.check(L.seera_set_option(b"pair_tiles", 0))


def test_mode_4_weight_gradients_from_one_fp16_copy(E):
    """The default of mode 4 ("wgrad_single"): dW / dB from the first fp16 copy of each operand - one product, 2^-12 rounding
    per operand (a few 1e-4 here, where nothing averages; 3e-5 and less on the training configurations) - while the data
    gradient keeps its three products."""
    from ml_framework_b200 import capi
    L = capi.load()
    rs = np.random.RandomState(77)
    A, B, dC = (rs.standard_normal(s).astype(np.float32) for s in ((512, 300), (300, 200), (512, 200)))
    X, Wt = rs.standard_normal((8, 64, 12, 12)).astype(np.float32), rs.standard_normal((96, 64, 3, 3)).astype(np.float32)
    dY = rs.standard_normal((8, 96, 12, 12)).astype(np.float32)
    _prep(4)
    try:
        capi.check(L.seera_set_option(b"wgrad_single", 1))
        dA, dB = E.matmul_backward(A, B, dC)
        assert rel_l2(dA, dC.astype(np.float64) @ B.T) < TOL[4]
        assert 1e-5 < rel_l2(dB, A.T.astype(np.float64) @ dC) < 5e-4
        dX, dW = E.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
        rX, rW = co.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
        assert rel_l2(dX, rX) < TOL[4] and 1e-5 < rel_l2(dW, rW) < 5e-4
    finally:
        capi.check(L.seera_set_option(b"wgrad_single", 0))


CONVT = [(1, 1, 4, 4, 1, 3, 3, 1, 1, 0, 0), (2, 4, 5, 6, 3, 4, 3, 2, 2, 1, 0), (8, 64, 16, 16, 32, 4, 4, 2, 2, 1, 1),
         (3, 6, 7, 5, 5, 3, 3, 1, 1, 1, 1), (2, 5, 5, 5, 7, 3, 5, 3, 2, 1, 2), (4, 32, 16, 16, 1, 3, 3, 1, 1, 1, 1),
         (2, 4, 5, 5, 3, 2, 2, 3, 3, 0, 0), (16, 128, 8, 8, 64, 4, 4, 2, 2, 1, 1)]


@pytest.mark.parametrize("mode", [1, 2, 4])
@pytest.mark.parametrize("shape", CONVT)
def test_conv_transpose2d(E, mode, shape):
    N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape) + 1)
    X, Wt = _prep(mode, rs.standard_normal((N, Ci, H, W)).astype(np.float32), rs.standard_normal((Ci, Co, KH, KW)).astype(np.float32))
    R = co.conv_transpose2d_forward(X, Wt, sh, sw, ph, pw)
    assert rel_l2(E.conv_transpose2d_forward(X, Wt, sh, sw, ph, pw), R) < TOL[mode]
    dY, = _prep(mode, rs.standard_normal(R.shape).astype(np.float32))
    dX, dW = E.conv_transpose2d_backward(dY, X, Wt, sh, sw, ph, pw)
    rX, rW = co.conv_transpose2d_backward(dY, X, Wt, sh, sw, ph, pw)
    assert rel_l2(dX, rX) < TOL[mode] and rel_l2(dW, rW) < TOL[mode]


def _act_ref(z, act):
    z = z.astype(np.float64)
    return [z, np.maximum(z, 0), 1 / (1 + np.exp(-z)), np.tanh(z)][act]


# Convolutions whose whole patch is at most 64 values (one 128-byte operand row): the patches are gathered and split
# inside the kernel.  Patches of 9, 25, 27, 48 and 64 values, strides, padding, filter counts that are not multiples
# of 8 or 64 and beyond 128 (CUDA-core variant), pixel counts that are not multiples of the tile.
SHORT = [(2, 1, 28, 28, 8, 3, 3, 1, 1, 1, 1), (3, 3, 32, 32, 64, 3, 3, 1, 1, 1, 1), (2, 1, 9, 11, 70, 5, 5, 2, 1, 2, 0),
         (2, 3, 13, 9, 5, 4, 4, 2, 3, 1, 2), (5, 4, 7, 7, 130, 4, 4, 1, 1, 0, 0), (64, 3, 32, 32, 64, 3, 3, 1, 1, 1, 1),
         (1, 2, 6, 6, 3, 1, 1, 1, 1, 0, 0), (9, 4, 10, 10, 100, 4, 4, 1, 1, 1, 1),
         (3, 1, 8, 64, 33, 3, 3, 1, 1, 1, 1), (2, 1, 10, 16, 5, 3, 3, 1, 1, 0, 1), (70, 1, 4, 4, 2, 3, 3, 1, 1, 2, 1)]
SHORT_TOL = {1: 1e-5, 2: 2e-5, 3: 5e-6}


@pytest.mark.parametrize("mode", [1, 2, 3])
@pytest.mark.parametrize("shape", SHORT)
def test_short_patch_conv_forward_and_weight_gradient(E, mode, shape):
    N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape) + 7)
    X, Wt = _prep(mode, rs.standard_normal((N, C, H, W)).astype(np.float32), rs.standard_normal((F, C, KH, KW)).astype(np.float32))
    Wt = (Wt / np.float32(np.sqrt(C * KH * KW))).astype(np.float32)
    if mode == 1:
        Wt = wl.bf16_round(Wt)
    b = rs.standard_normal(F).astype(np.float32)
    tol = SHORT_TOL[mode]
    R = co.conv2d_forward(X, Wt, sh, sw, ph, pw)
    assert rel_l2(E.conv2d_forward(X, Wt, sh, sw, ph, pw), R) < tol
    for act in (0, 1, 2, 3):
        want = _act_ref(R + b.reshape(1, F, 1, 1), act)
        assert rel_l2(E.conv2d_bias_act(X, Wt, b, sh, sw, ph, pw, act), want) < tol
    assert rel_l2(E.conv2d_bias_act(X, Wt, None, sh, sw, ph, pw, 1), np.maximum(R, 0)) < tol
    dY, = _prep(mode, rs.standard_normal(R.shape).astype(np.float32))
    dX, dW = E.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    rX, rW = co.conv2d_backward(dY, X, Wt, sh, sw, ph, pw)
    assert rel_l2(dW, rW) < tol and rel_l2(dX, rX) < max(tol, 2e-5)


FUSED_CONV = [(2, 70, 9, 9, 20, 3, 3, 1, 1, 1, 1), (4, 64, 16, 16, 128, 3, 3, 2, 2, 1, 1), (2, 130, 6, 6, 300, 3, 3, 1, 1, 1, 1)]
FUSED_CONVT = [(2, 64, 8, 8, 32, 4, 4, 2, 2, 1, 1), (3, 16, 7, 5, 20, 3, 3, 1, 1, 1, 1), (2, 8, 5, 5, 7, 2, 2, 3, 3, 0, 0)]


@pytest.mark.parametrize("mode", [2, 3])
def test_bias_and_activation_in_the_epilogue(E, mode):
    """The fused forward entries against product + bias + activation of the oracle, all activation codes."""
    rs = np.random.RandomState(mode)
    _prep(mode)
    for shape in FUSED_CONV:
        N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
        X, Wt, b = (rs.standard_normal(s).astype(np.float32) for s in ((N, C, H, W), (F, C, KH, KW), (F,)))
        R = co.conv2d_forward(X, Wt, sh, sw, ph, pw) + b.reshape(1, F, 1, 1)
        for act in (0, 1, 2, 3):
            assert rel_l2(E.conv2d_bias_act(X, Wt, b, sh, sw, ph, pw, act), _act_ref(R, act)) < 3e-5
    for shape in FUSED_CONVT:
        N, Ci, H, W, Co, KH, KW, sh, sw, ph, pw = shape
        X, Wt, b = (rs.standard_normal(s).astype(np.float32) for s in ((N, Ci, H, W), (Ci, Co, KH, KW), (Co,)))
        R = co.conv_transpose2d_forward(X, Wt, sh, sw, ph, pw) + b.reshape(1, Co, 1, 1)
        for act in (0, 1, 3):
            assert rel_l2(E.conv_transpose2d_bias_act(X, Wt, b, sh, sw, ph, pw, act), _act_ref(R, act)) < 3e-5
    for M, K, N in [(5, 7, 3), (300, 1024, 10), (64, 4096, 256), (257, 1000, 255)]:      # the last two also through split-K
        A, B, b = (rs.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (N,)))
        A /= np.float32(np.sqrt(K))                                   # keeps sigmoid and tanh off their flat ends
        R = A.astype(np.float64) @ B.astype(np.float64) + b
        for act in (0, 1, 2, 3):
            assert rel_l2(E.matmul_bias_act(A, B, b, act), _act_ref(R, act)) < 3e-5


def _dact_ref(y, act):
    y = y.astype(np.float64)
    return [np.ones_like(y), (y > 0).astype(np.float64), y * (1 - y), 1 - y * y][act]


# (N, C, H, W, F, KH, KW, sh, sw, ph, pw): tensor-core shapes (kept copies, dz never stored), short-patch shapes (the
# bias gradient rides in a spare patch column; none spare when C*KH*KW is 16), a strided one and tiny pooled images.
LAYER_BWD = [(4, 16, 8, 8, 24, 3, 3, 1, 1, 1, 1), (2, 70, 12, 12, 130, 3, 3, 1, 1, 1, 1), (3, 8, 16, 16, 16, 3, 3, 2, 2, 1, 1),
             (4, 3, 16, 16, 20, 3, 3, 1, 1, 1, 1), (2, 1, 12, 12, 6, 4, 4, 1, 1, 2, 2), (2, 1, 8, 8, 70, 3, 3, 1, 1, 1, 1),
             (3, 3, 16, 16, 64, 3, 3, 1, 1, 1, 1), (2, 1, 8, 12, 128, 3, 3, 1, 1, 1, 1), (70, 2, 6, 6, 64, 3, 3, 1, 1, 1, 1),
             # pooled images of 4, 1 and 8 windows: several whole images per tile of the pooled-gradient kernel, ragged at the end
             (13, 16, 4, 4, 130, 3, 3, 1, 1, 1, 1), (37, 16, 2, 2, 72, 3, 3, 1, 1, 1, 1), (3, 32, 4, 8, 24, 3, 3, 1, 1, 1, 1)]


@pytest.mark.parametrize("mode", [2, 3])
@pytest.mark.parametrize("shape", LAYER_BWD)
def test_conv_layer_backward_in_one_call(E, mode, shape):
    """seera_conv2d_act_bwd from a full-resolution gradient and from a pooled one, against the oracle's separate steps."""
    N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
    rs = np.random.RandomState(sum(shape) + 11)
    X, Wt, b = (rs.standard_normal(s).astype(np.float32) for s in ((N, C, H, W), (F, C, KH, KW), (F,)))
    Wt /= np.float32(np.sqrt(C * KH * KW))
    _prep(mode)
    Z = co.conv2d_forward(X, Wt, sh, sw, ph, pw) + b.reshape(1, F, 1, 1)
    OH, OW = Z.shape[2:]
    for act in (0, 1, 2, 3):
        for pooled in (False, True):
            for need_dx in (True, False):
                if pooled and (OH % 2 or OW % 2):
                    continue
                if pooled:
                    gp = rs.standard_normal((N, F, OH // 2, OW // 2)).astype(np.float32)
                    y, pool_out, dX, dW, db = E.conv2d_layer_roundtrip(X, Wt, b, sh, sw, ph, pw, act, gp=gp, need_dx=need_dx,
                                                                       pass_pooled=act != 3)      # tanh: slope read from y itself
                    ref_pool, mask = co.maxpool2d_forward(y, 2, 2, 2, 2, 0, 0)
                    assert np.array_equal(pool_out, ref_pool)
                    dy = co.maxpool2d_backward(gp, mask, N, F, OH, OW, 2, 2, 2, 2, 0, 0)
                else:
                    g = rs.standard_normal((N, F, OH, OW)).astype(np.float32)
                    y, _, dX, dW, db = E.conv2d_layer_roundtrip(X, Wt, b, sh, sw, ph, pw, act, g=g, need_dx=need_dx, keep=act != 2)
                    dy = g
                assert rel_l2(y, _act_ref(Z, act)) < 3e-5
                dz = (dy.astype(np.float64) * _dact_ref(y, act)).astype(np.float32)        # from the device's own y, as the kernel does
                rX, rW = co.conv2d_backward(dz, X, Wt, sh, sw, ph, pw)
                assert rel_l2(dW, rW) < 3e-5 and rel_l2(db, dz.astype(np.float64).sum(axis=(0, 2, 3))) < 3e-5
                if need_dx:
                    assert rel_l2(dX, rX) < 3e-5


# Unit-stride transposed convolutions with 1, 2 or 4 output channels run a direct fp32 stencil kernel (the last layer of the
# autoencoder configuration): 3x3 and other filter sizes, zero / full padding, widths that are no multiple of anything.
FEW_FILTER_CONVT = [(3, 32, 16, 16, 1, 3, 3, 1, 1), (2, 5, 9, 13, 1, 3, 3, 0, 0), (2, 7, 6, 10, 2, 3, 3, 2, 2), (2, 3, 7, 5, 4, 3, 3, 1, 0),
                    (2, 6, 8, 8, 1, 4, 4, 1, 2), (1, 4, 5, 11, 2, 5, 2, 2, 0), (2, 40, 12, 12, 4, 3, 3, 1, 1),
                    (2, 9, 8, 64, 2, 3, 3, 1, 1), (1, 8, 4, 4, 1, 3, 3, 1, 1), (3, 8, 5, 136, 1, 3, 3, 0, 1), (37, 3, 6, 8, 1, 3, 3, 2, 1)]


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_few_filter_transposed_convolution(E, mode):
    """Forward with bias and every activation against the oracle at fp32 accuracy (the kernel is exact fp32 in every tensor-core
    mode), and the layer's backward through the usual entry."""
    rs = np.random.RandomState(40 + mode)
    _prep(mode)
    for (N, Ci, H, W, Co, KH, KW, ph, pw) in FEW_FILTER_CONVT:
        X, Wt, b = (rs.standard_normal(s).astype(np.float32) for s in ((N, Ci, H, W), (Ci, Co, KH, KW), (Co,)))
        R = co.conv_transpose2d_forward(X, Wt, 1, 1, ph, pw)
        assert rel_l2(E.conv_transpose2d_forward(X, Wt, 1, 1, ph, pw), R) < 2e-6
        for act in (0, 1, 2, 3):
            got = E.conv_transpose2d_bias_act(X, Wt, b, 1, 1, ph, pw, act)
            assert got.shape == R.shape and rel_l2(got, _act_ref(R + b.reshape(1, Co, 1, 1), act)) < 2e-6
        if Co == 1 and KH * KW <= 9:      # the weight gradient of a one-channel output is a direct fp32 kernel as well
            dY = rs.standard_normal(R.shape).astype(np.float32)
            dX, dW = E.conv_transpose2d_backward(dY, X, Wt, 1, 1, ph, pw)
            rX, rW = co.conv_transpose2d_backward(dY, X, Wt, 1, 1, ph, pw)
            assert rel_l2(dW, rW) < 2e-6 and rel_l2(dX, rX) < 3e-3
        # the same kernel serves a unit-stride convolution with few filters (patch longer than 64, or it is a short-patch layer)
        if Ci * KH * KW > 64:
            Wc = rs.standard_normal((Co, Ci, KH, KW)).astype(np.float32)
            Rc = co.conv2d_forward(X, Wc, 1, 1, ph, pw) + b.reshape(1, Co, 1, 1)
            assert rel_l2(E.conv2d_bias_act(X, Wc, b, 1, 1, ph, pw, 2), _act_ref(Rc, 2)) < 2e-6
            dY = rs.standard_normal(Rc.shape).astype(np.float32)
            dX, dW = E.conv2d_backward(dY, X, Wc, 1, 1, ph, pw)
            rX, rW = co.conv2d_backward(dY, X, Wc, 1, 1, ph, pw)
            assert rel_l2(dX, rX) < 3e-3 and rel_l2(dW, rW) < 3e-3


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_pool_hands_its_copies_to_the_next_convolution(E, mode):
    """seera_maxpool2x2_fwd_s: pooled values and mask bit-equal to the oracle; a convolution fed the returned copies gives
    bit-equal results to one that makes its own."""
    import ctypes
    from ml_framework_b200 import capi
    L = capi.load()
    _prep(mode)
    rs = np.random.RandomState(mode)
    for (N, C, H, W, F) in [(3, 70, 12, 20, 40), (2, 16, 8, 8, 16), (5, 9, 6, 10, 7)]:
        Y = rs.standard_normal((N, C, H, W)).astype(np.float32)
        Wt = rs.standard_normal((F, C, 3, 3)).astype(np.float32)
        want_out, want_mask = co.maxpool2d_forward(Y, 2, 2, 2, 2, 0, 0)
        up = lambda a: L.seera_to_device(np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p), a.nbytes)
        yd, wd = up(Y), up(Wt)
        n_out = N * C * (H // 2) * (W // 2)
        od, md = L.seera_cuda_malloc(n_out * 4), L.seera_cuda_malloc(n_out * 4)
        h = ctypes.c_void_p()
        capi.check(L.seera_maxpool2x2_fwd_s(yd, od, md, N, C, H, W, ctypes.byref(h)))
        assert h.value
        out, mask = np.empty((N, C, H // 2, W // 2), np.float32), np.empty((N, C, H // 2, W // 2), np.int32)
        capi.check(L.seera_to_host(out.ctypes.data_as(ctypes.c_void_p), od, out.nbytes))
        capi.check(L.seera_to_host(mask.ctypes.data_as(ctypes.c_void_p), md, mask.nbytes))
        assert np.array_equal(out, want_out) and np.array_equal(mask, want_mask)
        res = []
        for x_in in (h, None):
            zd = L.seera_cuda_malloc(N * F * (H // 2) * (W // 2) * 4)
            keep = ctypes.c_void_p()
            capi.check(L.seera_conv2d_bias_act_fwd_s(od, wd, None, zd, N, C, H // 2, W // 2, F, 3, 3, 1, 1, 1, 1, 0, x_in, ctypes.byref(keep)))
            assert bool(keep.value) == (x_in is None)         # copies are made only when none were given
            z = np.empty((N, F, H // 2, W // 2), np.float32)
            capi.check(L.seera_to_host(z.ctypes.data_as(ctypes.c_void_p), zd, z.nbytes))
            res.append(z)
            L.seera_shadow_free(keep); L.seera_cuda_free(zd)
        assert np.array_equal(res[0], res[1])
        L.seera_shadow_free(h)
        for p in (yd, wd, od, md):
            L.seera_cuda_free(p)


POOL_FUSED = [(3, 16, 16, 16, 24, 3, 3, 1, 1, 1, 1), (2, 70, 8, 8, 130, 3, 3, 1, 1, 1, 1), (5, 8, 4, 4, 16, 3, 3, 1, 1, 1, 1),
              (4, 8, 8, 8, 8, 3, 3, 2, 2, 1, 1), (4, 3, 32, 32, 64, 3, 3, 1, 1, 1, 1), (3, 1, 28, 28, 20, 5, 5, 1, 1, 2, 2),
              (1, 2, 6, 6, 3, 1, 1, 1, 1, 0, 0)]


@pytest.mark.parametrize("mode", [2, 3])
@pytest.mark.parametrize("shape", POOL_FUSED)
def test_pool_folded_into_the_convolution_epilogue(E, mode, shape):
    """seera_conv2d_bias_act_pool_fwd_s against the separate calls: pooled values and mask bit-equal; the copies it returns
    feed the next convolution to a bit-equal result; backward from (gp, mask, pooled) with y = NULL equals backward with y."""
    import ctypes
    from ml_framework_b200 import capi
    L = capi.load()
    _prep(mode)
    N, C, H, W, F, KH, KW, sh, sw, ph, pw = shape
    OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
    short = C * KH * KW <= 64
    # 3 x 3 unit-stride short-patch layers with a multiple of 8 filters run an exact-fp32 kernel when the pool is folded in: the
    # separate calls (tensor-core products) then agree with it to rounding, not bit for bit
    exact = short and (KH, KW, sh, sw) == (3, 3, 1, 1) and C <= 7 and F % 8 == 0
    assert L.seera_conv2d_pool_fusable(N, C, H, W, F, KH, KW, sh, sw, ph, pw) == (0 if short and not exact else 1)
    capi.check(L.seera_set_option(b"pool_short_patch", 1))            # off by default (slower), still has to be right
    assert L.seera_conv2d_pool_fusable(N, C, H, W, F, KH, KW, sh, sw, ph, pw) == 1
    rs = np.random.RandomState(sum(shape) + mode)
    X, Wt, b = (rs.standard_normal(s).astype(np.float32) for s in ((N, C, H, W), (F, C, KH, KW), (F,)))
    W2 = rs.standard_normal((9, F, 3, 3)).astype(np.float32)
    gp = rs.standard_normal((N, F, OH // 2, OW // 2)).astype(np.float32)
    up = lambda a: L.seera_to_device(np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p), a.nbytes)
    def down(p, shape, dt=np.float32):
        a = np.empty(shape, dt)
        capi.check(L.seera_to_host(a.ctypes.data_as(ctypes.c_void_p), p, a.nbytes))
        return a
    xd, wd, bd, w2d, gpd = up(X), up(Wt), up(b), up(W2), up(gp)
    nq = N * F * (OH // 2) * (OW // 2)
    for act in (1, 2):
        # separate calls
        y = L.seera_cuda_malloc(N * F * OH * OW * 4)
        p1, m1 = L.seera_cuda_malloc(nq * 4), L.seera_cuda_malloc(nq * 4)
        capi.check(L.seera_conv2d_bias_act_fwd(xd, wd, bd, y, N, C, H, W, F, KH, KW, ph, pw, sh, sw, act))
        capi.check(L.seera_cuda_maxpool_fwd(y, p1, m1, N, F, OH, OW, 2, 2, 0, 0, 2, 2))
        # one call
        p2, m2 = L.seera_cuda_malloc(nq * 4), L.seera_cuda_malloc(nq * 4)
        keep, pc = ctypes.c_void_p(), ctypes.c_void_p()
        capi.check(L.seera_conv2d_bias_act_pool_fwd_s(xd, wd, bd, p2, m2, N, C, H, W, F, KH, KW, ph, pw, sh, sw, act, None,
                                                      ctypes.byref(keep), ctypes.byref(pc)))
        shp = (N, F, OH // 2, OW // 2)
        if exact:
            ref = _act_ref(co.conv2d_forward(X, Wt, sh, sw, ph, pw) + b.reshape(1, F, 1, 1), act).astype(np.float32)
            want, want_mask = co.maxpool2d_forward(ref, 2, 2, 2, 2, 0, 0)
            assert rel_l2(down(p2, shp), want) < 2e-6 and rel_l2(down(p2, shp), down(p1, shp)) < 2e-5
            assert (down(m2, shp, np.int32) == want_mask).mean() > 0.999          # ties within rounding may pick another tap
        else:
            assert np.array_equal(down(p1, shp), down(p2, shp)) and np.array_equal(down(m1, shp, np.int32), down(m2, shp, np.int32))
        # the returned copies of the pooled tensor feed the next convolution
        if F * 9 > 64:
            res = []
            for x_in in (pc, None):
                zd = L.seera_cuda_malloc(N * 9 * (OH // 2) * (OW // 2) * 4)
                capi.check(L.seera_conv2d_bias_act_fwd_s(p2, w2d, None, zd, N, F, OH // 2, OW // 2, 9, 3, 3, 1, 1, 1, 1, 0, x_in, None))
                res.append(down(zd, (N, 9, OH // 2, OW // 2)))
                L.seera_cuda_free(zd)
            assert np.array_equal(res[0], res[1])
        # backward without the full-resolution output
        outs = []
        for yy in (y, None):
            dw, db, dx = L.seera_cuda_malloc(Wt.size * 4), L.seera_cuda_malloc(F * 4), L.seera_cuda_malloc(X.size * 4)
            capi.check(L.seera_conv2d_act_bwd(wd, xd, yy, None, gpd, m2, p2, dx, dw, db, N, C, H, W, F, KH, KW, sh, sw, ph, pw, act, keep))
            outs.append((down(dw, Wt.shape), down(db, (F,)), down(dx, X.shape)))
            for p in (dw, db, dx):
                L.seera_cuda_free(p)
        for a, bb in zip(*outs):
            assert rel_l2(a, bb) < 1e-4 if exact else np.array_equal(a, bb)
        L.seera_shadow_free(keep); L.seera_shadow_free(pc)
        for p in (y, p1, m1, p2, m2):
            L.seera_cuda_free(p)
    for p in (xd, wd, bd, w2d, gpd):
        L.seera_cuda_free(p)
    capi.check(L.seera_set_option(b"pool_short_patch", 0))


def test_c5_conv_backward_point_bf16(E):
    """One point of the Conv2D-backward sweep at reduced batch (C = K = 64, 56x56, 3x3 s1 p1), bf16 operands."""
    X, Wt, dY = wl.c5_conv_bwd(64, 56, n=4)
    _prep(1)
    dX, dW = E.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
    rX, rW = co.conv2d_backward(dY, X, Wt, 1, 1, 1, 1)
    assert rel_l2(dX, rX) < 1e-5 and rel_l2(dW, rW) < 1e-5


# C3 at a reduced batch carries a looser bound on its first two layers: a handful of ReLU / max-pool decisions flip
# under ANY change of summation order (exact-fp32 mode 0 already differs from the CPU oracle by 2e-4..7e-4 there),
# and with few samples each flip weighs more.  The 2e-3 gate is checked at the configuration's full batch below.
@pytest.mark.parametrize("name,n,gate", [("c1", 64, 2e-3), ("c3", 32, 6e-3), ("c4", 16, 2e-3)])
def test_training_step_bf16x3_against_fp32_oracle(E, name, n, gate):
    """fp32 configurations on the tensor cores (mode 2) against the untouched fp32 step oracle."""
    from ml_framework_b200 import train, seera_cuda as sc
    sc.set_precision(2)
    work = wl.WORKLOADS[name]()
    tr = train.Trainer(work, seed=3)
    X, Y = work.batch(n, 3)
    ref = RefNet(work.layers, work.params(3), work.loss, work.opt, co)
    loss = tr.forward_backward(X, Y)
    grads = tr.host_grads()
    tr.opt.step()
    rl = ref.step(X, Y)
    assert abs(float(loss.value.to_host_f32()[0]) - rl) <= 2e-3 * max(1.0, abs(rl))
    worst = 0.0
    for G, R in zip(grads, ref.grads):
        if R is not None:
            worst = max(worst, rel_l2(G[0], R[0]), rel_l2(G[1].ravel(), R[1].ravel()))
    assert worst < gate, worst
    for P, R in zip(tr.host_params(), ref.params):
        if R is not None:
            assert rel_l2(P[0], R[0]) < 2e-3


def test_c3_full_batch_step_bf16x3_meets_the_gate(E):
    """C3 at its full batch of 512 on the tensor cores (forward three-way split, backward two-way split) against
    the reference CPU engine: loss, every gradient and every updated weight within rel-L2 2e-3 after one step.
    (With the two-way split in the forward pass as well, the first layer's dW lands at 2.7e-3.)"""
    from ml_framework_b200 import train, seera_cuda as sc
    from oracle import ref_engine
    work = wl.c3_vgg()
    tr = train.Trainer(work, seed=3, precision=(3, 2))
    X, Y = work.batch(512, 3)
    ref = RefNet(work.layers, work.params(3), work.loss, work.opt, ref_engine.load() or co)
    loss = tr.forward_backward(X, Y)
    grads = tr.host_grads()
    tr.opt.step()
    rl = ref.step(X, Y)
    assert abs(float(loss.value.to_host_f32()[0]) - rl) <= 2e-3 * max(1.0, abs(rl))
    errs = []
    for G, R in zip(grads, ref.grads):
        if R is not None:
            errs += [rel_l2(G[0], R[0]), rel_l2(G[1].ravel(), R[1].ravel())]
    assert max(errs) < 2e-3, errs
    for P, R in zip(tr.host_params(), ref.params):
        if R is not None:
            assert rel_l2(P[0], R[0]) < 2e-3


def test_training_step_bf16_against_matched_oracle(E):
    """C2 (bf16 inputs, fp32 accumulate) against the step oracle whose GEMM operands carry the same rounding."""
    from ml_framework_b200 import train, seera_cuda as sc
    sc.set_precision(1)
    work = wl.c2_mlp()
    tr = train.Trainer(work, seed=3)
    X, Y = work.batch(512, 3)
    ref = RefNet(work.layers, work.params(3), work.loss, work.opt, co, quant=wl.bf16_round)
    loss = tr.forward_backward(X, Y)
    grads = tr.host_grads()
    tr.opt.step()
    rl = ref.step(X, Y)
    assert abs(float(loss.value.to_host_f32()[0]) - rl) <= 2e-3 * max(1.0, abs(rl))
    for G, R in zip(grads, ref.grads):
        if R is not None:
            assert rel_l2(G[0], R[0]) < 2e-3 and rel_l2(G[1].ravel(), R[1].ravel()) < 2e-3
    for P, R in zip(tr.host_params(), ref.params):
        if R is not None:
            assert rel_l2(P[0], R[0]) < 2e-3


@pytest.mark.parametrize("mode", [0, 1, 2, 4])
@pytest.mark.parametrize("M,K,N,act", [(64, 784, 10, 0), (512, 1024, 256, 1), (300, 200, 130, 2), (4096, 784, 1024, 1), (33, 17, 9, 3)])
def test_dense_layer_entries_that_keep_their_copies(E, mode, M, K, N, act):
    """seera_matmul_bias_act_fwd_s / seera_matmul_act_bwd through the C ABI: forward with the copies of its output written by the
    epilogue, a second forward fed those copies, and the one-call backward (activation slope, bias gradient, dA, dB) reading the
    copies the forward kept - against the plain entries on the same inputs (bit-equal where the same kernels run) and against
    the formulas in double precision."""
    import ctypes
    from ml_framework_b200 import capi
    from engine_np import _Dev
    L = capi.load()
    L.seera_set_precision(mode)
    rs = np.random.RandomState(M + N + act)
    q = wl.bf16_round if mode == 1 else (lambda a: a)
    A, B = q(rs.standard_normal((M, K)).astype(np.float32)), q((rs.standard_normal((K, N)) * 0.1).astype(np.float32))
    bias = rs.standard_normal(N).astype(np.float32)
    g = q(rs.standard_normal((M, N)).astype(np.float32))
    B2 = q((rs.standard_normal((N, 24)) * 0.1).astype(np.float32))
    f = [lambda z: z, lambda z: np.maximum(z, 0), lambda z: 1 / (1 + np.exp(-z)), np.tanh][act]
    P = ctypes.POINTER(ctypes.c_void_p)
    tol = {0: 2e-5, 1: 1e-5, 2: 2e-5, 4: 1e-5}[mode]
    with _Dev() as d:
        pa, pb, pbias, pg, pb2 = d.up(A), d.up(B), d.up(bias), d.up(g), d.up(B2)
        c, c_ref, c2, c2_ref = d.new(M * N), d.new(M * N), d.new(M * 24), d.new(M * 24)
        ak, wk, cc = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        capi.check(L.seera_matmul_bias_act_fwd_s(pa, pb, pbias, c, M, N, K, act, None, ctypes.byref(ak), ctypes.byref(wk), ctypes.byref(cc)))
        capi.check(L.seera_matmul_bias_act_fwd(pa, pb, pbias, c_ref, M, N, K, act))
        y = d.down(c, (M, N))
        assert np.array_equal(y, d.down(c_ref, (M, N)))
        want = f(A.astype(np.float64) @ B + bias)
        assert rel_l2(y, want) < tol
        # the next layer, fed the copies the epilogue wrote, equals the next layer converting y itself
        capi.check(L.seera_matmul_bias_act_fwd_s(c, pb2, None, c2, M, 24, N, 0, cc, None, None, None))
        capi.check(L.seera_matmul_bias_act_fwd(c, pb2, None, c2_ref, M, 24, N, 0))
        assert np.array_equal(d.down(c2, (M, 24)), d.down(c2_ref, (M, 24)))
        assert (mode == 0) == (not cc.value)             # copies exist exactly in the tensor-core modes
        # backward in one call
        da, db, dbias = d.new(M * K), d.new(K * N), d.new(N)
        capi.check(L.seera_matmul_act_bwd(pa, pb, c, pg, da, db, dbias, M, N, K, act, ak, wk))
        slope = [np.ones_like(want), (y > 0).astype(np.float64), y.astype(np.float64) * (1 - y), 1 - y.astype(np.float64) ** 2][act]
        dz = g.astype(np.float64) * slope
        dz_q = q(dz.astype(np.float32)).astype(np.float64) if mode == 1 else dz
        assert rel_l2(d.down(dbias, (N,)), dz.sum(axis=0)) < 1e-5
        assert rel_l2(d.down(da, (M, K)), dz_q @ B.T.astype(np.float64)) < max(tol, 2e-5)
        assert rel_l2(d.down(db, (K, N)), A.T.astype(np.float64) @ dz_q) < max(tol, 2e-5)
        for h in (ak, wk, cc):
            L.seera_rows_free(h)
    assert L.seera_tc_device_status() == 0
