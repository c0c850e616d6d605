"""The allocation-free activation-backward entry against the regular one, through the C ABI.

Who needs it: a host that owns all device memory itself and forbids the library to call cudaMalloc (a serving
process with a fixed budget, a plugin given its buffers up front), or one that is already recording a stream
and cannot afford a pool miss.  The entry keeps its partial-sum scratch in a fixed device array inside the
library, so the check here is that (a) it produces what seera_act_bias_bwd produces, twice in a row - the
array still holds the first call's sums when the second starts - and (b) on a trimmed pool and a shape no call
has seen, it takes nothing from the pool, while the regular entry on the same shape does.  Collected last so that a failure here cannot hide another test's result in a stop-at-first-failure run."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(L, entry, dy, y, channels, inner, act, want_bias=True):
    from ml_framework_b200 import capi
    n = dy.size
    V = ctypes.c_void_p

    def up(a):
        p = L.seera_to_device(a.ctypes.data_as(V), a.nbytes)
        assert p
        return p
    pdy, py = up(dy), up(y)
    pdz, pdb = L.seera_cuda_malloc(n * 4), L.seera_cuda_malloc(channels * 4)
    before = L.seera_pool_bytes_reserved()
    capi.check(getattr(L, entry)(pdy, py, pdz, pdb if want_bias else None, n, channels, inner, act))
    grew = L.seera_pool_bytes_reserved() - before
    dz, db = np.empty(n, np.float32), np.empty(channels, np.float32)
    capi.check(L.seera_to_host(dz.ctypes.data_as(V), pdz, n * 4))
    capi.check(L.seera_to_host(db.ctypes.data_as(V), pdb, channels * 4))
    for p in (pdy, py, pdz, pdb):
        L.seera_cuda_free(p)
    return dz, db, grew


@pytest.mark.parametrize("rows,channels,inner,act", [(512, 64, 1024, 1), (4096, 1024, 1, 1), (33, 7, 49, 2), (64, 10, 1, 0), (8, 3000, 16, 3),
                                                     (16, 65536, 1, 1), (2, 65536, 3, 2)])
def test_noalloc_entry_matches_regular_entry_twice_in_a_row(rows, channels, inner, act):
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    rs = np.random.RandomState(rows + channels)
    for call in range(2):                                # second call: the fixed array still holds the first call's sums
        dy = rs.standard_normal(rows * channels * inner).astype(np.float32)
        y = rs.uniform(-1, 1, dy.size).astype(np.float32)
        dz_ref, db_ref, _ = _run(L, "seera_act_bias_bwd", dy, y, channels, inner, act)
        dz, db, grew = _run(L, "seera_act_bias_bwd_noalloc", dy, y, channels, inner, act)
        assert np.array_equal(dz, dz_ref)
        scale = max(1.0, float(np.abs(db_ref).max()))
        assert np.max(np.abs(db - db_ref)) <= 1e-5 * scale, call


def test_noalloc_entry_takes_nothing_from_the_pool_where_the_regular_entry_does():
    """Inputs and outputs are allocated first; then the pool's cached blocks are released, so any scratch a call wants has
    to come from the driver and shows up in the reserved-bytes counter."""
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    V = ctypes.c_void_p
    rows, channels, inner = 96, 1536, 5                  # a shape no other test uses
    n = rows * channels * inner
    dy = np.random.RandomState(1).standard_normal(n).astype(np.float32)
    pdy = L.seera_to_device(dy.ctypes.data_as(V), dy.nbytes)
    pdz, pdb = L.seera_cuda_malloc(n * 4), L.seera_cuda_malloc(channels * 4)
    capi.check(L.seera_synchronize())
    capi.check(L.seera_pool_trim())
    before = L.seera_pool_bytes_reserved()
    capi.check(L.seera_act_bias_bwd_noalloc(pdy, pdy, pdz, pdb, n, channels, inner, 1))
    assert L.seera_pool_bytes_reserved() == before       # the fixed array served the partial sums
    capi.check(L.seera_act_bias_bwd(pdy, pdy, pdz, pdb, n, channels, inner, 1))
    assert L.seera_pool_bytes_reserved() > before        # the regular entry needed a block
    # a product channels * inner beyond 32 bits is an argument error, not a crash
    L.seera_clear_status()
    assert L.seera_act_bias_bwd_noalloc(pdy, pdy, pdz, pdb, n, 65536, 65536, 1) == 2
    L.seera_clear_status()
    for p in (pdy, pdz, pdb):
        L.seera_cuda_free(p)


def test_noalloc_entry_rejects_sizes_beyond_its_fixed_scratch():
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    L.seera_clear_status()
    n = 70000
    p = L.seera_cuda_malloc(n * 4)
    assert L.seera_act_bias_bwd_noalloc(p, p, p, p, n, n, 1, 0) == 5          # SEERA_E_LIMIT
    assert b"fixed scratch" in L.seera_last_error()
    L.seera_cuda_free(p)
    L.seera_clear_status()
