"""The CPU checker against every golden vector the reference's own tests hold at the
Backend boundary.  Citations are reference file:line."""
import numpy as np
import pytest

from conftest import cg

nn = cg.graphs.nn
H = cg.graphs.helpers
F32, U32 = cg.F32, cg.U32


def f32(a):
    return np.asarray(a, dtype=np.float32)


def u32(a):
    return np.asarray(a, dtype=np.uint32)


def test_batched_matmul_golden(oracle):
    # catgrad/src/interpreter/backend/ndarray.rs:630-674
    B = oracle
    lhs = B.from_numpy(np.arange(1, 25, dtype=np.float32).reshape(2, 3, 2, 2))
    rhs = B.from_numpy(np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2, 1))
    out = B.matmul(lhs, rhs)
    assert out.shape == (2, 3, 2, 1)
    np.testing.assert_array_equal(B.to_vec(out), f32([5, 11, 39, 53, 105, 127, 203, 233, 333, 371, 495, 541]))


def test_add_sub_golden(oracle):
    # ndarray.rs:676-716
    B = oracle
    x = B.from_numpy(f32([[1, 2], [3, 4]]))
    y = B.from_numpy(f32([[5, 6], [7, 8]]))
    np.testing.assert_array_equal(B.to_vec(B.add(x, y)), f32([6, 8, 10, 12]))
    a = B.from_numpy(f32([[10, 8], [6, 4]]))
    b = B.from_numpy(f32([[1, 2], [3, 4]]))
    np.testing.assert_array_equal(B.to_vec(B.sub(a, b)), f32([9, 6, 3, 0]))


def test_sum_max_golden(oracle):
    # ndarray.rs:718-821
    B = oracle
    s = B.sum(B.from_numpy(u32([[1, 2, 3], [4, 5, 6]])))
    assert s.shape == (2, 1) and s.dtype == U32
    np.testing.assert_array_equal(B.to_vec(s), u32([6, 15]))
    x3 = B.from_numpy(np.arange(1, 13, dtype=np.float32).reshape(2, 2, 3))
    s3 = B.sum(x3)
    assert s3.shape == (2, 2, 1)
    np.testing.assert_array_equal(B.to_vec(s3), f32([6, 15, 24, 33]))
    m = B.max(B.from_numpy(f32([[1, 5, 3], [2, 8, 4]])))
    assert m.shape == (2, 1)
    np.testing.assert_array_equal(B.to_vec(m), f32([5, 8]))
    np.testing.assert_array_equal(B.to_vec(B.max(B.from_numpy(u32([[1, 5], [3, 2]])))), u32([5, 3]))
    np.testing.assert_array_equal(B.to_vec(B.max(x3)), f32([3, 6, 9, 12]))


def test_interpreter_goldens(oracle):
    # catgrad/tests/test_interpreter.rs:85-226
    B = oracle
    a = B.from_numpy(u32([[[1, 2, 3]], [[4, 5, 6]]]))
    assert B.add(a, a).shape == (2, 1, 3)
    np.testing.assert_array_equal(B.to_vec(B.add(a, a)), u32([2, 4, 6, 8, 10, 12]))
    x0 = B.from_numpy(f32([1, 2, 3, 4, 5, 6, 7, 8]).reshape(2, 2, 2))
    x1 = B.from_numpy(f32([1, 2, 3, 4]).reshape(2, 2, 1))
    np.testing.assert_array_equal(B.to_vec(B.matmul(x0, x1)), f32([5, 11, 39, 53]))
    data = f32([[0, 1], [2, -1]])
    got = B.to_vec(nn.exp(B, B.from_numpy(data)))
    want = np.exp(data.astype(np.float64)).astype(np.float32).ravel()
    assert np.all(np.abs(got - want) <= 1e-8 + 1e-5 * np.abs(want))
    v, i = B.topk(B.from_numpy(f32([[0.1, 5, 3, 10, 5], [8, 9, 7, 6, 8]])), 2)
    np.testing.assert_array_equal(B.to_vec(v), f32([10, 5, 9, 8]))
    np.testing.assert_array_equal(B.to_vec(i), u32([3, 1, 1, 0]))  # ties -> first index


def test_from_vec_shapes(oracle):
    # catgrad/src/interpreter/tests.rs:7-18 and BackendError::ShapeError
    B = oracle
    assert B.ndarray_from_vec_f32([1, 2, 3, 4, 5, 6], (2, 3)).shape == (2, 3)
    assert B.ndarray_from_vec_u32([1, 2, 3, 4], (4,)).dtype == U32
    with pytest.raises(cg.BackendError):
        B.ndarray_from_vec_f32([1, 2, 3], (2, 2))


def test_activation_goldens(oracle):
    # same formulas through the legacy evaluator: catgrad-llm/src/legacy/nn/layers.rs:735-784
    B = oracle
    x = B.from_numpy(f32([1, 2, 3]))
    tol = dict(rtol=0, atol=2e-6)
    np.testing.assert_allclose(B.to_vec(nn.tanh(B, x)), [0.761594, 0.964028, 0.995055], **tol)
    np.testing.assert_allclose(B.to_vec(nn.gelu(B, x)), [0.841192, 1.954598, 2.996363], **tol)
    np.testing.assert_allclose(B.to_vec(nn.sigmoid(B, x)), [0.731059, 0.880797, 0.952574], **tol)
    np.testing.assert_allclose(B.to_vec(nn.silu(B, x)), [0.731059, 1.761594, 2.857722], **tol)
    np.testing.assert_allclose(B.to_vec(nn.softmax(B, x)), [0.090031, 0.244728, 0.665241], **tol)
    y = B.from_numpy(f32([100.1, 100.2, 100.3]))
    np.testing.assert_allclose(B.to_vec(nn.softmax(B, y)), [0.300609, 0.332224, 0.367167], **tol)


def test_norm_goldens(oracle):
    # layers.rs:735-784: rmsnorm_raw / layernorm_raw on {0..4}, eps 1e-5
    B = oracle
    x = B.from_numpy(np.arange(5, dtype=np.float32).reshape(1, 1, 5))
    np.testing.assert_allclose(B.to_vec(H.rmsnorm_raw(B, 1e-5, x)), [0, 0.408248, 0.816496, 1.224744, 1.632992],
                               rtol=0, atol=2e-6)
    np.testing.assert_allclose(B.to_vec(H.layernorm_raw(B, 1e-5, x)), [-1.414210, -0.707105, 0, 0.707105, 1.414210],
                               rtol=0, atol=2e-6)


def test_causal_mask_golden(oracle):
    # layers.rs:1191-1208: [0, MIN, MIN, 0, 0, MIN, 0, 0, 0]
    B = oracle
    m = B.to_vec(H.causal_mask(B, 3))
    mn = np.finfo(np.float32).min
    np.testing.assert_array_equal(m, f32([0, mn, mn, 0, 0, mn, 0, 0, 0]))


def test_repeat_kv_order(oracle):
    # layers.rs:1482-1515: head h of the output is kv head h // rep
    B = oracle
    x = B.from_numpy(np.arange(2 * 3 * 2, dtype=np.float32).reshape(1, 2, 3, 2))
    y = B.to_numpy(H.repeat_kv(B, 2, x))
    assert y.shape == (1, 4, 3, 2)
    src = np.arange(12, dtype=np.float32).reshape(1, 2, 3, 2)
    np.testing.assert_array_equal(y, np.repeat(src, 2, axis=1))


def test_legacy_argmax_topk_goldens(oracle):
    # catgrad-legacy/src/backend/cpu/eval.rs:1200-1255
    B = oracle
    np.testing.assert_array_equal(B.to_vec(B.argmax(B.from_numpy(f32([[1, 2], [4, 3]])))), u32([1, 0]))
    v, i = B.topk(B.from_numpy(f32([[1, 3, 2, 4], [8, 7, 5, 6]])), 2)
    np.testing.assert_array_equal(B.to_vec(i), u32([3, 1, 0, 1]))


def test_tie_rules_and_total_order(oracle):
    # ndarray.rs:469-520: argmax keeps the LAST maximum, topk the FIRST; order is total_cmp
    B = oracle
    x = B.from_numpy(f32([[5, 1, 5, 5, 2], [-0.0, 0.0, -0.0, 0.0, -1]]))
    np.testing.assert_array_equal(B.to_vec(B.argmax(x)), u32([3, 3]))  # +0 > -0 in total order
    _, i = B.topk(x, 3)
    np.testing.assert_array_equal(B.to_vec(i), u32([0, 2, 3, 1, 3, 0]))
    n = B.from_numpy(f32([[1, np.nan, 3]]))
    np.testing.assert_array_equal(B.to_vec(B.argmax(n)), u32([1]))  # +NaN is greatest
    np.testing.assert_array_equal(B.to_vec(B.max(n)), f32([3]))  # f32::max ignores NaN
    inf = B.from_numpy(f32([[-np.inf, -np.inf]]))
    np.testing.assert_array_equal(B.to_vec(B.max(inf)), f32([np.finfo(np.float32).min]))  # fold starts at f32::MIN


def test_cast_semantics(oracle):
    # ndarray.rs:97-114: Rust `as`
    B = oracle
    x = B.from_numpy(f32([1.9, -3.0, np.nan, 5e9, 0.0, 4294967040.0]))
    np.testing.assert_array_equal(B.to_vec(B.cast(x, U32)), u32([1, 0, 0, 0xFFFFFFFF, 0, 4294967040]))
    y = B.from_numpy(u32([0, 7, 16777217, 0xFFFFFFFF]))
    np.testing.assert_array_equal(B.to_vec(B.cast(y, F32)), f32([0, 7, 16777216, 4294967296]))


def test_lt_eq_keep_dtype(oracle):
    # ndarray.rs:164-198
    B = oracle
    a, b = B.from_numpy(f32([1, 2, 3])), B.from_numpy(f32([2, 2, 2]))
    r = B.lt(a, b)
    assert r.dtype == F32
    np.testing.assert_array_equal(B.to_vec(r), f32([1, 0, 0]))
    np.testing.assert_array_equal(B.to_vec(B.eq(a, b)), f32([0, 1, 0]))
    ua, ub = B.from_numpy(u32([1, 2, 3])), B.from_numpy(u32([2, 2, 2]))
    assert B.lt(ua, ub).dtype == U32
    np.testing.assert_array_equal(B.to_vec(B.lt(ua, ub)), u32([1, 0, 0]))


def test_u32_arith_wraps(oracle):
    B = oracle
    a, b = B.from_numpy(u32([0, 0xFFFFFFFF, 7, 3])), B.from_numpy(u32([1, 2, 2, 40]))
    np.testing.assert_array_equal(B.to_vec(B.sub(a, b)), u32([0xFFFFFFFF, 0xFFFFFFFD, 5, (3 - 40) & 0xFFFFFFFF]))
    np.testing.assert_array_equal(B.to_vec(B.add(a, b)), u32([1, 1, 9, 43]))
    np.testing.assert_array_equal(B.to_vec(B.div(a, b)), u32([0, 0x7FFFFFFF, 3, 0]))
    np.testing.assert_array_equal(B.to_vec(B.pow(a, b)), u32([0, 1, 49, pow(3, 40, 2 ** 32)]))
    np.testing.assert_array_equal(B.to_vec(B.neg(a)), u32([0, 1, (-7) & 0xFFFFFFFF, (-3) & 0xFFFFFFFF]))


def test_shape_errors(oracle):
    # candle.rs:413-415 "Shape mismatch in operation"; ndarray.rs:212,255,293,333
    B = oracle
    a, b = B.from_numpy(f32([[1, 2, 3]])), B.from_numpy(f32([[1, 2]]))
    with pytest.raises(cg.BackendPanic, match="Shape mismatch"):
        B.add(a, b)
    with pytest.raises(cg.BackendPanic):
        B.sin(B.from_numpy(u32([1])))
    with pytest.raises(cg.BackendPanic):
        B.topk(B.from_numpy(u32([[1, 2]])), 1)
    with pytest.raises(cg.BackendPanic):
        B.broadcast(a, (2, 2))
    with pytest.raises(cg.BackendPanic):
        B.index(a, 1, B.from_numpy(u32([3])))
    with pytest.raises(cg.BackendPanic):
        B.matmul(B.from_numpy(f32(np.zeros((2, 2, 3)))), B.from_numpy(f32(np.zeros((3, 3, 2)))))
    with pytest.raises(cg.BackendPanic):
        B.slice(a, 1, 2, 5)


def test_views_and_movement(oracle):
    B = oracle
    src = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    x = B.from_numpy(src)
    np.testing.assert_array_equal(B.to_numpy(B.transpose(x, 0, 2)), src.transpose(2, 1, 0))
    np.testing.assert_array_equal(B.to_numpy(B.reshape(B.transpose(x, 1, 2), (8, 3))), src.transpose(0, 2, 1).reshape(8, 3))
    np.testing.assert_array_equal(B.to_numpy(B.slice(x, 2, 1, 2)), src[:, :, 1:3])
    np.testing.assert_array_equal(B.to_numpy(B.concat(x, x, 1)), np.concatenate([src, src], 1))
    np.testing.assert_array_equal(B.to_numpy(B.broadcast(B.from_numpy(f32([1, 2, 3, 4])), (2, 3, 4))),
                                  np.broadcast_to(f32([1, 2, 3, 4]), (2, 3, 4)))
    idx = B.from_numpy(u32([[2], [0]]))  # rank-2 indices are flattened (ndarray.rs:378)
    np.testing.assert_array_equal(B.to_numpy(B.index(x, 1, idx)), src[:, [2, 0], :])
    np.testing.assert_array_equal(B.to_vec(B.arange(5)), u32([0, 1, 2, 3, 4]))
    assert B.arange(0).shape == (0,)
    z = B.zeros((2, 0, 3), F32)
    assert z.shape == (2, 0, 3)
    assert B.compare(x, B.from_numpy(src)) and not B.compare(x, B.from_numpy(src + 1))
    assert not B.compare(B.from_numpy(f32([np.nan])), B.from_numpy(f32([np.nan])))
