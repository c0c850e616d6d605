"""GPU parity of the flat, scalar, broadcast, fill, transpose and copy entries through the C ABI.

These carry gradient accumulation (`cp = cp + d`), the bias add of every layer and the composed optimizer on the
drop-in path (reference: engine_cuda/src/elemops.cu:46-80, cuTen_essentails.cu:80-147, broadcast.cu:95-154,
GEMM.cu:108-143, cuda_bindings.cpp:61-66).  fp32 add / subtract / multiply / divide of two values is one correctly
rounded IEEE operation on both sides, so the results must be BIT-EXACT against NumPy and against the CPU engine's
`add` / `mul` (engine/src/tensor_ops.cpp:18-31); `power` is compared to 2 ulp-class tolerance (powf)."""
import ctypes

import numpy as np
import pytest

from conftest import rel_l2
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu

f = ctypes.c_float


@pytest.fixture(scope="module")
def D():
    from ml_framework_b200 import capi
    import engine_np
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    capi.check(L.seera_set_precision(0))
    return engine_np._Dev, capi


SIZES = [1, 3, 4, 31, 1000, 1024, 65537, 1 << 20]


@pytest.mark.parametrize("n", SIZES)
def test_flat_binary_ops_are_bit_exact(D, n):
    Dev, capi = D
    rs = np.random.RandomState(n)
    a = rs.standard_normal(n).astype(np.float32)
    b = (rs.standard_normal(n) + 3.0).astype(np.float32)          # away from zero for the division
    want = {"seera_cuda_elemadd_gputogpu": a + b, "seera_cuda_elemsub_gputogpu": a - b,
            "seera_cuda_elemmult_gputogpu": a * b, "seera_cuda_elemdiv_gputogpu": a / b}
    with Dev() as d:
        pa, pb, pc = d.up(a), d.up(b), d.new(n)
        for name, w in want.items():
            capi.check(getattr(d.L, name)(pa, pb, pc, n))
            assert np.array_equal(d.down(pc, (n,)), w), name
        # operands untouched
        assert np.array_equal(d.down(pa, (n,)), a) and np.array_equal(d.down(pb, (n,)), b)
    assert np.array_equal(want["seera_cuda_elemadd_gputogpu"], co.add(a, b))
    assert np.array_equal(want["seera_cuda_elemmult_gputogpu"], co.mul(a, b))


@pytest.mark.parametrize("n", SIZES)
def test_scalar_ops_and_fills(D, n):
    Dev, capi = D
    rs = np.random.RandomState(n + 1)
    a = (np.abs(rs.standard_normal(n)) + 0.1).astype(np.float32)
    with Dev() as d:
        p = d.up(a)
        capi.check(d.L.seera_cuda_scaler_multiply_f(p, f(-2.5), n))
        assert np.array_equal(d.down(p, (n,)), a * np.float32(-2.5))
        capi.check(d.L.seera_cuda_scaler_add_f(p, f(0.75), n))
        assert np.array_equal(d.down(p, (n,)), a * np.float32(-2.5) + np.float32(0.75))
        q = d.up(a)
        capi.check(d.L.seera_cuda_scaler_power_f(q, f(2.0), n))
        assert rel_l2(d.down(q, (n,)), a.astype(np.float64) ** 2) < 1e-6
        q2 = d.up(a)
        capi.check(d.L.seera_cuda_scaler_power_f(q2, f(0.5), n))
        assert rel_l2(d.down(q2, (n,)), np.sqrt(a.astype(np.float64))) < 1e-6
        capi.check(d.L.seera_cuda_ones_f(p, n))
        assert np.array_equal(d.down(p, (n,)), np.ones(n, np.float32))
        capi.check(d.L.seera_cuda_zeros_f(p, n))
        assert np.array_equal(d.down(p, (n,)), np.zeros(n, np.float32))


def test_memset_and_device_copy_count_conventions(D):
    """cuda_memset counts BYTES and sets each to the value's low byte; cuda_memcopy_devicetodevice counts FLOAT elements
    (cuda_bindings.cpp:61-66)."""
    Dev, capi = D
    n = 1003
    a = np.arange(n, dtype=np.float32) + 0.5
    with Dev() as d:
        pa, pb = d.up(a), d.up(np.full(n, 7.0, np.float32))
        capi.check(d.L.seera_cuda_memcopy_devicetodevice(pb, pa, n - 3))            # n - 3 floats, not bytes
        got = d.down(pb, (n,))
        assert np.array_equal(got[:n - 3], a[:n - 3]) and np.array_equal(got[n - 3:], np.full(3, 7.0, np.float32))
        capi.check(d.L.seera_cuda_memset(pb, 0, 4 * 10))                             # the first ten floats only
        got = d.down(pb, (n,))
        assert np.array_equal(got[:10], np.zeros(10, np.float32)) and np.array_equal(got[10:n - 3], a[10:n - 3])
        capi.check(d.L.seera_cuda_memset(pb, 0x1FF, 8))                              # byte value 0xFF in 8 bytes
        raw = d.down(pb, (n,)).view(np.uint32)
        assert raw[0] == 0xFFFFFFFF and raw[1] == 0xFFFFFFFF and raw[2] == 0
        # addresses with 4-byte alignment only (callers add n*4 to a base address)
        capi.check(d.L.seera_cuda_memcopy_devicetodevice(pb + 4, pa + 12, 500))
        assert np.array_equal(d.down(pb + 4, (500,)), a[3:503])


@pytest.mark.parametrize("rows,cols", [(1, 1), (1, 7), (7, 1), (31, 33), (64, 64), (257, 1000), (1024, 784)])
def test_transpose_2d(D, rows, cols):
    Dev, capi = D
    a = np.random.RandomState(rows + cols).standard_normal((rows, cols)).astype(np.float32)
    with Dev() as d:
        pa, pb = d.up(a), d.new(a.size)
        capi.check(d.L.seera_cuda_transpose_2d(pa, pb, rows, cols))
        assert np.array_equal(d.down(pb, (cols, rows)), a.T)


@pytest.mark.parametrize("nb,m,k", [(1, 1, 1), (3, 5, 7), (2, 33, 31), (8, 64, 128), (64, 28, 28)])
def test_transpose_3d(D, nb, m, k):
    Dev, capi = D
    a = np.random.RandomState(nb + m + k).standard_normal((nb, m, k)).astype(np.float32)
    with Dev() as d:
        pa, pb = d.up(a), d.new(a.size)
        capi.check(d.L.seera_cuda_transpose_3d(pa, pb, nb, m, k))
        assert np.array_equal(d.down(pb, (nb, k, m)), a.transpose(0, 2, 1))


# every NumPy broadcast pattern of two 4-D shapes: each axis equal, or 1 on either side
BCAST = [((4, 8, 6, 5), (4, 8, 6, 5)), ((4, 8, 6, 5), (1, 8, 1, 1)), ((1, 8, 1, 1), (4, 8, 6, 5)),
         ((64, 16, 14, 14), (1, 16, 1, 1)), ((1, 1, 64, 10), (1, 1, 1, 10)), ((1, 1, 1, 10), (1, 1, 64, 10)),
         ((4, 1, 6, 1), (1, 8, 1, 5)), ((3, 1, 1, 1), (1, 2, 5, 7)), ((2, 3, 4, 5), (2, 1, 4, 1)),
         ((2, 3, 4, 5), (1, 1, 1, 1)), ((1, 1, 1, 1), (1, 1, 1, 1)), ((5, 1, 3, 1), (5, 4, 1, 6)),
         ((512, 64, 2, 2), (1, 64, 1, 1)), ((1, 1, 4096, 33), (1, 1, 1, 33))]


@pytest.mark.parametrize("sa,sb", BCAST)
def test_broadcast_add_and_mul_4d(D, sa, sb):
    Dev, capi = D
    rs = np.random.RandomState(sum(sa) + 3 * sum(sb))
    a, b = rs.standard_normal(sa).astype(np.float32), rs.standard_normal(sb).astype(np.float32)
    with Dev() as d:
        pa, pb = d.up(a), d.up(b)
        out_shape = np.broadcast_shapes(sa, sb)
        pc = d.new(int(np.prod(out_shape)))
        capi.check(d.L.seera_broadcast_add_4d(pa, pb, pc, *sa, *sb))
        assert np.array_equal(d.down(pc, out_shape), a + b)
        capi.check(d.L.seera_broadcast_mul_4d(pa, pb, pc, *sa, *sb))
        assert np.array_equal(d.down(pc, out_shape), a * b)


def test_broadcast_shape_mismatch_is_an_error_status(D):
    Dev, capi = D
    with Dev() as d:
        p = d.new(64)
        assert d.L.seera_broadcast_add_4d(p, p, p, 1, 2, 3, 4, 1, 5, 3, 4) == 2
        d.L.seera_clear_status()


def test_binding_level_conventions(D):
    """The Python binding's forms of the same entries: cuda_ones_f / cuda_zeros_f ALLOCATE and return an address
    (cuda_bindings.cpp:467-477); to_host_f32 takes a shape tuple (:107)."""
    from ml_framework_b200 import seera_cuda as sc
    sc.init(0)
    p1, p0 = sc.cuda_ones_f(37), sc.cuda_zeros_f(37)
    assert np.array_equal(sc.to_host_f32(p1, (37,)), np.ones(37, np.float32))
    assert np.array_equal(sc.to_host_f32(p0, (37,)), np.zeros(37, np.float32))
    sc.cuda_scaler_multiply_f(p1, 3.0, 37)
    sc.cuda_scaler_add_f(p1, -1.0, 37)
    sc.cuda_power_of(p1, 2.0, 37)
    assert np.array_equal(sc.to_host_f32(p1, (37,)), np.full(37, 4.0, np.float32))
    out = sc.cuda_malloc_f32(37)
    for fn, want in ((sc.cuda_elemadd, 4.0), (sc.cuda_elemsub, 4.0), (sc.cuda_elemmult, 0.0)):
        fn(p1, p0, out, 37)
        assert np.array_equal(sc.to_host_f32(out, (37,)), np.full(37, want, np.float32))
    sc.cuda_elemdiv(p0, p1, out, 37)
    assert np.array_equal(sc.to_host_f32(out, (37,)), np.zeros(37, np.float32))
    for p in (p1, p0, out):
        sc.cuda_free(p)
