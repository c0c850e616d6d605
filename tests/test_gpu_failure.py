"""Failure handling of the tensor-core kernels on the device, in the one form that cannot hurt the GPU: a wait that runs
out.  Every wait inside the TMA-fed kernel (producer on a free stage, MMA issuer on a full stage, epilogue on a finished
accumulator) has a clock budget; when it runs out the kernel records which role gave up, the other roles see the flag and
stop, copies in flight are given a bounded time to land, TMEM is freed and the kernel RETURNS.  The test shortens the
budget to 50 ms and uses the engine's test hook to leave one stage unfilled in one launch - nothing faults, traps or
spins without a bound - then checks that the status word names the MMA issuer (code 2), that reading clears it, and that
the very next launch on the same context computes correctly."""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    from ml_framework_b200 import capi
    import engine_np as E
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    capi.check(L.seera_set_precision(1))
    assert L.seera_tc_device_status() == 0
    rs = np.random.RandomState(0)
    A, B = rs.standard_normal((128, 256)).astype(np.float32), rs.standard_normal((256, 128)).astype(np.float32)
    want = A.astype(np.float64) @ B
    try:
        capi.check(L.seera_set_option(b"tc_wait_ms", 50))
        capi.check(L.seera_set_option(b"tc_test_skip_load", 1))     # the second k-step of the next launch never arrives
        E.matmul(A, B)                                              # returns: the kernel unwound by itself
        assert L.seera_tc_device_status() == 2                      # the MMA issuer's wait for that stage ran out
        assert L.seera_tc_device_status() == 0                      # reading cleared it; the hook cleared itself
        got = E.matmul(A, B)                                        # same context, same stream, next launch
        assert rel_l2(got, want) < 1e-2
        assert L.seera_tc_device_status() == 0
        assert L.seera_last_status() == 0
    finally:
        L.seera_set_option(b"tc_test_skip_load", -1)
        L.seera_set_option(b"tc_wait_ms", 2000)
        L.seera_set_precision(0)


def test_wait_budget_option_is_validated():
    from ml_framework_b200 import capi
    L = capi.load()
    capi.check(L.seera_init(capi.default_device()))
    assert L.seera_set_option(b"tc_wait_ms", 0) == 2
    L.seera_clear_status()
