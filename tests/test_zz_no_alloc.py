"""The allocation-free arg-max entry point against the regular one.

`cg_argmax_rows_noalloc` exists for hosts that may not allocate device memory when they need the
result (another stream of the process is under graph capture, a plugin with a fixed budget, a
latency-critical loop).  It keeps its per-row merge slots in an array inside the library, which
every call shares and which keeps the previous call's contents, so the check runs twice in a row
with different shapes: stale slots from the first call must not leak into the second.
Collected last on purpose: a failure here cannot hide other tests from a `-x` run.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu


def test_noalloc_argmax_matches_argmax_twice(cuda):
    import torch

    lib = cg.load_library()
    fn = lib.cg_argmax_rows_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_char_p, C.c_int64]
    fn.restype = C.c_int32
    rng = np.random.Generator(np.random.PCG64(11))
    cases = [rng.integers(0, 4, size=(37, 5000)).astype(np.float32),        # heavy ties: last index wins
             np.concatenate([rng.standard_normal((5, 130), dtype=np.float32),
                             np.float32([[-0.0, 0.0] * 65, [np.nan] + [1.0] * 129])])]  # fewer rows the second time
    for x in cases:
        want = cuda.to_numpy(cuda.argmax(cuda.from_numpy(x))).ravel()     # existing entry point
        dx = torch.from_numpy(x).cuda()
        dout = torch.full((x.shape[0],), 0xFFFFFFF, dtype=torch.int32, device="cuda")
        err = C.create_string_buffer(256)
        st = fn(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(dx.data_ptr()), x.shape[0], x.shape[1],
                C.c_void_p(dout.data_ptr()), err, 256)
        assert st == 0, err.value
        torch.cuda.synchronize()
        got = dout.cpu().numpy().astype(np.uint32)
        np.testing.assert_array_equal(got, want)   # index work: bit-exact


def test_noalloc_rejects_more_rows_than_its_scratch(cuda):
    lib = cg.load_library()
    fn = lib.cg_argmax_rows_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_char_p, C.c_int64]
    fn.restype = C.c_int32
    err = C.create_string_buffer(256)
    st = fn(None, C.c_void_p(16), 4097, 8, C.c_void_p(16), err, 256)   # rejected before any pointer is used
    assert st == 3 and b"exceed the fixed scratch" in err.value
