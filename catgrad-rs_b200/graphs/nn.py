"""catgrad/src/stdlib/nn/mod.rs:117-246 and catgrad/src/stdlib/ops.rs:61-70 as backend calls."""
from __future__ import annotations

import numpy as np

F32, U32 = 0, 1
E32 = float(np.float32(np.e))  # std::f32::consts::E = 2.7182817
SQRT_2_OVER_PI = float(np.sqrt(np.float32(2.0) / np.float32(np.pi), dtype=np.float32))


def constant(B, v, shape):
    """`constant` = broadcast(lit(v), shape) (stdlib/ops.rs:61-64)."""
    return B.broadcast(B.ndarray_from_vec_f32([v], ()), shape)


def inverse(B, x):
    """`inverse` = constant(1.0) / x (stdlib/ops.rs:66-70)."""
    return B.div(constant(B, 1.0, x.shape), x)


def sqrt(B, x):  # nn/mod.rs:117-121
    return B.pow(x, constant(B, 0.5, x.shape))


def exp(B, x):  # nn/mod.rs:123-128
    e = constant(B, E32, x.shape)
    e = B.cast(e, x.dtype)
    return B.pow(e, x)


def sigmoid(B, x):  # nn/mod.rs:130-136
    one = constant(B, 1.0, x.shape)
    one = B.cast(one, x.dtype)
    ex = exp(B, B.neg(x))
    return B.div(one, B.add(one, ex))


def tanh(B, x):  # nn/mod.rs:138-144
    one = constant(B, 1.0, x.shape)
    two = constant(B, 2.0, x.shape)
    s = sigmoid(B, B.mul(two, x))
    return B.sub(B.mul(two, s), one)


def silu(B, x):  # nn/mod.rs:146-148
    return B.mul(x, sigmoid(B, x))


def gelu(B, x):  # nn/mod.rs:151-160
    sh = x.shape
    c = constant(B, SQRT_2_OVER_PI, sh)
    one = constant(B, 1.0, sh)
    three = constant(B, 3.0, sh)
    half = constant(B, 0.5, sh)
    k = constant(B, 0.044715, sh)
    hx = B.mul(half, x)
    inner = B.add(x, B.mul(k, B.pow(x, three)))
    t = tanh(B, B.mul(c, inner))
    return B.mul(hx, B.add(one, t))


def softmax(B, x):  # nn/mod.rs:162-171
    sh = x.shape
    m = B.max(x)
    bmax = B.broadcast(m, sh)
    x = B.sub(x, bmax)
    ex = exp(B, x)
    s = B.sum(ex)
    bsum = B.broadcast(s, sh)
    return B.div(ex, bsum)


def linear_b_param(B, in_dim, out_dim, weight, bias, x):  # nn/mod.rs:174-199
    w_t = B.transpose(weight, 0, 1)
    batch = x.shape[0]
    w_t = B.reshape(w_t, (batch, in_dim, out_dim))  # only valid for batch == 1
    m = B.matmul(x, w_t)
    if bias is not None:
        bb = B.broadcast(bias, m.shape)
        return B.add(m, bb)
    return m


def linear_no_bias(B, in_dim, out_dim, params, path, x):  # nn/mod.rs:240-242
    return linear_b_param(B, in_dim, out_dim, params[path + ".weight"], None, x)


def linear(B, in_dim, out_dim, params, path, x):  # nn/mod.rs:244-246
    return linear_b_param(B, in_dim, out_dim, params[path + ".weight"], params[path + ".bias"], x)
