"""Parity of every `Backend` trait method: CUDA library vs the CPU checker on the same
seeded inputs, through the C ABI.  Integer / index / byte-moving results must be
bit-exact; f32 arithmetic that only moves or compares values too; pow/sin/cos within one
ulp; sums and GEMMs within 1e-5 relative (summation order differs)."""
import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
F32, U32 = cg.F32, cg.U32
RNG = np.random.Generator(np.random.PCG64(1234))


def rand_f32(shape, scale=1.0):
    return (RNG.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def rand_u32(shape, hi=2 ** 32):
    return RNG.integers(0, hi, size=shape, dtype=np.uint64).astype(np.uint32)


def run_both(oracle, cuda, fn, *arrays):
    outs = []
    for B in (oracle, cuda):
        ts = [B.from_numpy(a) for a in arrays]
        r = fn(B, *ts)
        if not isinstance(r, (tuple, list)):
            r = (r,)
        outs.append([(t.dtype, t.shape, B.to_numpy(t)) for t in r])
    return outs


def assert_exact(outs):
    for (d0, s0, a0), (d1, s1, a1) in zip(*outs):
        assert d0 == d1 and s0 == s1
        np.testing.assert_array_equal(a0.view(np.uint32), a1.view(np.uint32))


def ulp_diff(a, b):
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def assert_ulp(outs, ulps):
    for (d0, s0, a0), (d1, s1, a1) in zip(*outs):
        assert d0 == d1 and s0 == s1
        both_nan = np.isnan(a0) & np.isnan(a1)
        d = ulp_diff(np.where(both_nan, 0, a0).astype(np.float32), np.where(both_nan, 0, a1).astype(np.float32))
        assert d.max(initial=0) <= ulps, d.max()


def assert_close(outs, rtol, atol=0.0):
    for (d0, s0, a0), (d1, s1, a1) in zip(*outs):
        assert d0 == d1 and s0 == s1
        np.testing.assert_allclose(a1, a0, rtol=rtol, atol=atol)


SHAPES = [(), (1,), (7,), (3, 5), (2, 1, 3), (4, 3, 2, 5), (2, 2, 2, 2, 3), (1031,), (64, 257)]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "lt", "eq"])
@pytest.mark.parametrize("shape", SHAPES)
def test_binary_f32_exact(oracle, cuda, op, shape):
    a, b = rand_f32(shape), rand_f32(shape)
    if a.size:
        b.flat[0] = a.flat[0]  # one equal pair for eq
    assert_exact(run_both(oracle, cuda, lambda B, x, y: getattr(B, op)(x, y), a, b))


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "pow", "lt", "eq"])
@pytest.mark.parametrize("shape", [(), (9,), (3, 4, 5), (1000,)])
def test_binary_u32_exact(oracle, cuda, op, shape):
    a = rand_u32(shape)
    b = rand_u32(shape, hi=40) + np.uint32(1)  # no zero divisors: Rust would panic
    assert_exact(run_both(oracle, cuda, lambda B, x, y: getattr(B, op)(x, y), a, b))


def test_special_values_f32(oracle, cuda):
    v = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 3.4e38, -1.0, 2.5], dtype=np.float32)
    a, b = np.meshgrid(v, v)
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    for op in ("add", "sub", "mul", "div", "lt", "eq"):
        outs = run_both(oracle, cuda, lambda B, x, y: getattr(B, op)(x, y), a, b)
        (_, _, r0), (_, _, r1) = outs[0][0], outs[1][0]
        np.testing.assert_array_equal(np.isnan(r0), np.isnan(r1))
        np.testing.assert_array_equal(np.where(np.isnan(r0), 0, r0).view(np.uint32), np.where(np.isnan(r1), 0, r1).view(np.uint32))


@pytest.mark.parametrize("shape", [(5,), (33, 17), (2, 3, 64)])
def test_pow_within_one_ulp(oracle, cuda, shape):
    base = np.abs(rand_f32(shape)) + np.float32(0.1)
    ex = rand_f32(shape, 3.0)
    assert_ulp(run_both(oracle, cuda, lambda B, x, y: B.pow(x, y), base, ex), 1)
    # the shapes the stdlib uses: E^x, x^0.5, x^3 with negative x (nn/mod.rs:117-160)
    x = rand_f32(shape, 4.0)
    e = np.full(shape, np.float32(np.e), dtype=np.float32)
    assert_ulp(run_both(oracle, cuda, lambda B, a, b: B.pow(a, b), e, x), 1)
    assert_ulp(run_both(oracle, cuda, lambda B, a, b: B.pow(a, b), np.abs(x), np.full(shape, 0.5, np.float32)), 1)
    assert_ulp(run_both(oracle, cuda, lambda B, a, b: B.pow(a, b), x, np.full(shape, 3.0, np.float32)), 1)


@pytest.mark.parametrize("op", ["sin", "cos", "neg"])
def test_unary_f32(oracle, cuda, op):
    x = np.concatenate([rand_f32((500,), 10.0), np.arange(0, 700, dtype=np.float32), np.float32([1e6, -1e6, 0.0])])
    outs = run_both(oracle, cuda, lambda B, t: getattr(B, op)(t), x)
    if op == "neg":
        assert_exact(outs)
    else:
        assert_ulp(outs, 1)


def test_neg_u32_and_dtype_errors(oracle, cuda):
    assert_exact(run_both(oracle, cuda, lambda B, t: B.neg(t), rand_u32((17,))))
    for B in (oracle, cuda):
        with pytest.raises(cg.BackendPanic):
            B.cos(B.from_numpy(rand_u32((3,))))
        with pytest.raises(cg.BackendPanic, match="Shape mismatch"):
            B.mul(B.from_numpy(rand_f32((2, 3))), B.from_numpy(rand_f32((3, 2))))
        with pytest.raises(cg.BackendError):
            B.ndarray_from_vec_u32([1, 2, 3], (2,))


def test_cast(oracle, cuda):
    x = np.concatenate([rand_f32((300,), 1e5), np.float32([np.nan, np.inf, -np.inf, 4294967296.0, 4294967040.0, -0.5, 0.99])])
    assert_exact(run_both(oracle, cuda, lambda B, t: B.cast(t, U32), x))
    u = np.concatenate([rand_u32((300,)), np.uint32([0, 16777217, 0xFFFFFFFF])])
    assert_exact(run_both(oracle, cuda, lambda B, t: B.cast(t, F32), u))
    assert_exact(run_both(oracle, cuda, lambda B, t: B.cast(t, F32), x))  # identity arm


@pytest.mark.parametrize("shape", [(), (1,), (5,), (4, 33), (3, 2, 129), (2, 1500), (6, 4097), (3, 0)])
def test_reductions(oracle, cuda, shape):
    x = rand_f32(shape)
    assert_close(run_both(oracle, cuda, lambda B, t: B.sum(t), x), rtol=2e-5, atol=1e-5)
    assert_exact(run_both(oracle, cuda, lambda B, t: B.max(t), x))
    u = rand_u32(shape)
    assert_exact(run_both(oracle, cuda, lambda B, t: B.sum(t), u))
    assert_exact(run_both(oracle, cuda, lambda B, t: B.max(t), u))
    if len(shape) == 0 or shape[-1] > 0:
        assert_exact(run_both(oracle, cuda, lambda B, t: B.argmax(t), x))
        assert_exact(run_both(oracle, cuda, lambda B, t: B.argmax(t), u))


def test_argmax_ties_last_and_total_order(oracle, cuda):
    x = RNG.integers(0, 4, size=(64, 300)).astype(np.float32)  # heavy ties
    assert_exact(run_both(oracle, cuda, lambda B, t: B.argmax(t), x))
    z = np.float32([[-0.0, 0.0, -0.0, 0.0, -1], [np.nan, 1, 2, np.nan, 0], [-np.inf] * 5, [5, 1, 5, 5, 2]])
    assert_exact(run_both(oracle, cuda, lambda B, t: B.argmax(t), z))
    # f32::max does not order -0.0 against +0.0, so the sign of a zero maximum is free
    (_, _, m0), (_, _, m1) = [o[0] for o in run_both(oracle, cuda, lambda B, t: B.max(t), z)]
    np.testing.assert_array_equal(m0, m1)
    big = RNG.integers(0, 3, size=(2, 128256)).astype(np.float32)
    assert_exact(run_both(oracle, cuda, lambda B, t: B.argmax(t), big))


@pytest.mark.parametrize("shape,k", [((2, 5), 2), ((7, 128), 8), ((3, 2, 40), 40), ((4, 1000), 3), ((5, 9), 0)])
def test_topk(oracle, cuda, shape, k):
    assert_exact(run_both(oracle, cuda, lambda B, t: B.topk(t, k), rand_f32(shape)))
    ties = RNG.integers(0, 3, size=shape).astype(np.float32)  # ties keep ascending index
    assert_exact(run_both(oracle, cuda, lambda B, t: B.topk(t, k), ties))


def test_topk_golden_and_errors(oracle, cuda):
    # catgrad/tests/test_interpreter.rs:175-226
    v, i = cuda.topk(cuda.from_numpy(np.float32([[0.1, 5, 3, 10, 5], [8, 9, 7, 6, 8]])), 2)
    np.testing.assert_array_equal(cuda.to_vec(v), np.float32([10, 5, 9, 8]))
    np.testing.assert_array_equal(cuda.to_vec(i), np.uint32([3, 1, 1, 0]))
    for B in (oracle, cuda):
        with pytest.raises(cg.BackendPanic):
            B.topk(B.from_numpy(rand_f32((2, 3))), 4)


def test_views_chain(oracle, cuda):
    src = rand_f32((2, 3, 4, 5))

    def chain(B, x):
        t = B.transpose(x, 1, 3)            # non-contiguous
        s = B.slice(t, 2, 1, 2)             # offset view of it
        r = B.reshape(s, (2, 10, 3))        # forces a gather
        b = B.broadcast(B.slice(r, 1, 0, 1), (2, 10, 3))
        return B.add(r, b), B.concat(t, t, 0), B.reshape(t, (10, 12)), B.neg(s)

    assert_exact(run_both(oracle, cuda, chain, src))


def test_broadcast_rules(oracle, cuda):
    assert_exact(run_both(oracle, cuda, lambda B, x: B.broadcast(x, (4, 3, 5)), rand_f32((3, 1))))
    assert_exact(run_both(oracle, cuda, lambda B, x: B.broadcast(x, (2, 2)), rand_f32(())))
    assert_exact(run_both(oracle, cuda, lambda B, x: B.mul(B.broadcast(x, (6, 7)), B.broadcast(x, (6, 7))), rand_f32((7,))))
    for B in (oracle, cuda):
        with pytest.raises(cg.BackendPanic):
            B.broadcast(B.from_numpy(rand_f32((3,))), (3, 2))


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_index(oracle, cuda, dim):
    x = rand_f32((6, 5, 4))
    idx = RNG.integers(0, (6, 5, 4)[dim], size=(3, 2)).astype(np.uint32)  # rank-2: flattened
    assert_exact(run_both(oracle, cuda, lambda B, t, i: B.index(t, dim, i), x, idx))
    assert_exact(run_both(oracle, cuda, lambda B, t, i: B.index(t, dim, i), rand_u32((6, 5, 4)), idx))


def test_index_out_of_bounds_is_reported(cuda):
    x = cuda.from_numpy(rand_f32((4, 3)))
    bad = cuda.from_numpy(np.uint32([1, 9]))
    with pytest.raises(cg.BackendPanic, match="index out of bounds"):
        cuda.to_vec(cuda.index(x, 0, bad))
    # the context stays usable
    np.testing.assert_array_equal(cuda.to_vec(cuda.arange(3)), np.uint32([0, 1, 2]))


def test_concat_slice_arange_zeros(oracle, cuda):
    a, b = rand_f32((2, 3, 4)), rand_f32((2, 5, 4))
    assert_exact(run_both(oracle, cuda, lambda B, x, y: B.concat(x, y, 1), a, b))
    assert_exact(run_both(oracle, cuda, lambda B, x: B.concat(x, x, 2), rand_u32((2, 2, 2))))
    assert_exact(run_both(oracle, cuda, lambda B, x: B.slice(x, 1, 2, 3), b))
    assert_exact(run_both(oracle, cuda, lambda B, x: B.slice(x, 0, 1, 0), a))  # empty slice
    for n in (0, 1, 17, 5000):
        assert_exact(run_both(oracle, cuda, lambda B: B.arange(n)))
    assert_exact(run_both(oracle, cuda, lambda B: (B.zeros((3, 4), F32), B.zeros((2, 0), U32), B.zeros((), U32))))


def test_compare(oracle, cuda):
    a = rand_f32((5, 6))
    for B in (oracle, cuda):
        x, y = B.from_numpy(a), B.from_numpy(a.copy())
        assert B.compare(x, y)
        assert B.compare(B.transpose(x, 0, 1), B.transpose(y, 0, 1))
        z = a.copy()
        z[4, 5] += 1
        assert not B.compare(x, B.from_numpy(z))
        assert not B.compare(x, B.from_numpy(a[:, :5].copy()))
        assert not B.compare(B.from_numpy(np.float32([np.nan])), B.from_numpy(np.float32([np.nan])))
        assert B.compare(B.from_numpy(np.float32([0.0])), B.from_numpy(np.float32([-0.0])))


@pytest.mark.parametrize("shape_a,shape_b", [((2, 2), (2, 1)), ((2, 3, 2, 2), (2, 3, 2, 1)), ((1, 70, 33), (1, 33, 129)),
                                             ((3, 5, 64, 16), (3, 5, 16, 64)), ((1, 1, 200), (1, 200, 1))])
def test_matmul_f32(oracle, cuda, shape_a, shape_b):
    a, b = rand_f32(shape_a), rand_f32(shape_b)
    assert_close(run_both(oracle, cuda, lambda B, x, y: B.matmul(x, y), a, b), rtol=2e-5, atol=2e-5)


def test_matmul_goldens_and_views(oracle, cuda):
    # ndarray.rs:630-674 through the CUDA library: small integers are exact
    lhs = np.arange(1, 25, dtype=np.float32).reshape(2, 3, 2, 2)
    rhs = np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2, 1)
    out = cuda.matmul(cuda.from_numpy(lhs), cuda.from_numpy(rhs))
    np.testing.assert_array_equal(cuda.to_vec(out), np.float32([5, 11, 39, 53, 105, 127, 203, 233, 333, 371, 495, 541]))
    # the linear layer's operand: transpose + reshape of a [out, in] weight (nn/mod.rs:174-199)
    w, x = rand_f32((37, 48)), rand_f32((1, 9, 48))
    assert_close(run_both(oracle, cuda, lambda B, xx, ww: B.matmul(xx, B.reshape(B.transpose(ww, 0, 1), (1, 48, 37))), x, w),
                 rtol=2e-5, atol=2e-5)
    # u32 matmul wraps
    assert_exact(run_both(oracle, cuda, lambda B, p, q: B.matmul(p, q), rand_u32((2, 5, 7)), rand_u32((2, 7, 3))))
    for B in (oracle, cuda):
        with pytest.raises(cg.BackendPanic):
            B.matmul(B.from_numpy(rand_f32((2, 3))), B.from_numpy(rand_f32((4, 2))))


def test_to_vec_and_shape_are_host_metadata(cuda):
    x = cuda.from_numpy(rand_f32((3, 4)))
    t = cuda.transpose(x, 0, 1)
    assert t.shape == (4, 3) and t.dtype == F32
    assert cuda.to_vec(t).shape == (12,)
    before = cuda.launch_count()
    _ = cuda.broadcast(cuda.slice(cuda.transpose(x, 0, 1), 0, 1, 2), (5, 2, 3)).shape
    assert cuda.launch_count() == before  # views launch nothing
