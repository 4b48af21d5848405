"""The failure path of the bounded device-side waits, exercised without faulting anything.

Every wait a kernel of this library performs on something another party has to raise (an
mbarrier another warp arrives on, a flag another GPU stores, a grid barrier) has a limit.  When it
runs out the kernel writes a code to the context's error word and returns; `cg_sync` turns the
code into CG_ERR_TIMEOUT and clears it.  The probe entry point waits on a flag that nothing ever
raises, with the limit lowered to a few milliseconds, so the wait expires by itself: no trap, no
bad address, no endless loop.
"""
import time

import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu

CG_ERR_TIMEOUT = 7


def test_a_wait_that_nothing_satisfies_expires_and_the_context_stays_usable():
    C = cg.CudaBackend(0, cg.PREC_F32)
    try:
        C.set_option("wait_limit_us", 5000)
        t0 = time.perf_counter()
        C.probe_wait_timeout()
        with pytest.raises(cg.BackendPanic) as e:
            C.sync()
        dt = time.perf_counter() - t0
        assert e.value.status == CG_ERR_TIMEOUT
        assert "wait expired" in e.value.message
        assert dt < 0.9, dt                      # gave up after ~5 ms, not after the default second
        # the word was cleared: the next sync is clean and kernels run as before
        C.sync()
        x = np.arange(12, dtype=np.float32).reshape(3, 4)
        got = C.to_numpy(C.add(C.from_numpy(x), C.from_numpy(x)))
        np.testing.assert_array_equal(got, x + x)
        # two probes in a row: the second sees the first one's report and gives up at once
        C.probe_wait_timeout()
        C.probe_wait_timeout()
        with pytest.raises(cg.BackendPanic) as e:
            C.sync()
        assert e.value.status == CG_ERR_TIMEOUT
        C.sync()
    finally:
        C.set_option("wait_limit_us", 1000000)
        C.close()
