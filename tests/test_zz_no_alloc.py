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


def total_order_argmax(x: np.ndarray) -> np.ndarray:
    """Row-wise arg-max under f32::total_cmp, last index on ties, computed on the host with numpy
    only (no library code): -NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN."""
    bits = x.view(np.uint32).astype(np.uint64)
    key = np.where(bits & 0x80000000, (~bits) & 0xFFFFFFFF, bits | 0x80000000)
    n = x.shape[1]
    return (n - 1 - np.argmax(key[:, ::-1], axis=1)).astype(np.uint32)   # first maximum of the reversed row


def test_noalloc_argmax_matches_argmax_twice(cuda):
    import torch

    lib = cg.load_library()
    fn = lib.cg_argmax_rows_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_char_p, C.c_int64]
    fn.restype = C.c_int32
    rng = np.random.Generator(np.random.PCG64(11))
    neg_nan = np.uint32(0xFFC00000).view(np.float32)
    # long rows take the chunked reduction (64 chunks per row); one row holds nothing but -NaN and -inf
    # except a late -inf run, one has +NaN in the middle, one is all -NaN (the smallest key there is)
    long_rows = rng.standard_normal((4, 70000), dtype=np.float32)
    long_rows[1, :] = neg_nan
    long_rows[1, 123:60000] = -np.inf
    long_rows[2, 40000] = np.nan
    long_rows[3, :] = neg_nan
    cases = [rng.integers(0, 4, size=(37, 5000)).astype(np.float32),        # heavy ties: last index wins
             np.concatenate([rng.standard_normal((5, 130), dtype=np.float32),
                             np.float32([[-0.0, 0.0] * 65, [np.nan] + [1.0] * 129])]),  # fewer rows the second time
             long_rows]
    for x in cases:
        want = cuda.to_numpy(cuda.argmax(cuda.from_numpy(x))).ravel()     # existing entry point
        np.testing.assert_array_equal(want, total_order_argmax(x))        # ... which agrees with the host expectation
        dx = torch.from_numpy(x).cuda()
        dout = torch.full((x.shape[0],), 0xFFFFFFF, dtype=torch.int32, device="cuda")
        err = C.create_string_buffer(256)
        st = fn(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(dx.data_ptr()), x.shape[0], x.shape[1],
                C.c_void_p(dout.data_ptr()), err, 256)
        assert st == 0, err.value
        torch.cuda.synchronize()
        got = dout.cpu().numpy().astype(np.uint32)
        np.testing.assert_array_equal(got, want)                          # index work: bit-exact
        np.testing.assert_array_equal(got, total_order_argmax(x))         # and against numpy alone


def test_noalloc_rejects_more_rows_than_its_scratch(cuda):
    lib = cg.load_library()
    fn = lib.cg_argmax_rows_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_char_p, C.c_int64]
    fn.restype = C.c_int32
    err = C.create_string_buffer(256)
    st = fn(None, C.c_void_p(16), 4097, 8, C.c_void_p(16), err, 256)   # rejected before any pointer is used
    assert st == 3 and b"exceed the fixed scratch" in err.value
