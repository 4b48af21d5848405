"""catgrad-llm/src/helpers.rs as backend calls (line ranges in each docstring)."""
from __future__ import annotations

import numpy as np

from . import nn

F32, U32 = 0, 1
F32_MIN = float(np.finfo(np.float32).min)  # f32::MIN, the mask value (helpers.rs:254)


def chunk(B, dim, chunks, chunk_size, x):
    """helpers.rs:45-53"""
    return [B.slice(x, dim, i * chunk_size, chunk_size) for i in range(chunks)]


def split(B, dim, sizes, x):
    """helpers.rs:55-65"""
    out, off = [], 0
    for s in sizes:
        out.append(B.slice(x, dim, off, s))
        off += s
    return out


def unsqueeze(B, dim, x):
    """helpers.rs:77-84"""
    s = list(x.shape)
    s.insert(dim, 1)
    return B.reshape(x, s)


def squeeze(B, dim, x):
    """helpers.rs:68-75"""
    s = list(x.shape)
    s.pop(dim)
    return B.reshape(x, s)


def layernorm_raw(B, eps, x):
    """helpers.rs:86-106"""
    x_shape = x.shape
    n = x_shape[2]
    s = B.sum(x)
    constn = B.cast(B.ndarray_from_vec_u32([n], ()), x.dtype)
    constn = B.broadcast(constn, s.shape)
    mean = B.div(s, constn)
    nom = B.sub(x, B.broadcast(mean, x_shape))
    var = B.div(B.sum(B.mul(nom, nom)), constn)
    epsilon = nn.constant(B, eps, var.shape)
    stddev = nn.sqrt(B, B.add(var, epsilon))
    denom = B.broadcast(stddev, x_shape)
    return B.div(nom, denom)


def layernorm(B, eps, params, path, x):
    """helpers.rs:108-118"""
    gamma = params[path + ".weight"]
    lr = layernorm_raw(B, eps, x)
    lr = B.mul(lr, B.broadcast(gamma, lr.shape))
    beta = B.broadcast(params[path + ".bias"], lr.shape)
    return B.add(lr, beta)


def rmsnorm_raw(B, eps, x):
    """helpers.rs:120-136"""
    x_shape = x.shape
    n = x_shape[-1]
    s = B.sum(B.mul(x, x))
    constn = B.cast(B.ndarray_from_vec_u32([n], ()), x.dtype)
    constn = B.broadcast(constn, s.shape)
    mean = B.div(s, constn)
    epsilon = nn.constant(B, eps, mean.shape)
    rms = nn.sqrt(B, B.add(mean, epsilon))
    denom = B.broadcast(rms, x_shape)
    return B.div(x, denom)


def rmsnorm(B, eps, params, path, x):
    """helpers.rs:139-145"""
    gamma = params[path + ".weight"]
    lr = rmsnorm_raw(B, eps, x)
    gamma = B.broadcast(gamma, lr.shape)
    return B.mul(lr, gamma)


def repeat_kv(B, rep, x):
    """helpers.rs:147-161: reshape -> broadcast -> reshape (torch.repeat_interleave on dim 1)"""
    b, nkv, s, d = x.shape
    x = B.reshape(x, (b, nkv, 1, s, d))
    x = B.broadcast(x, (b, nkv, rep, s, d))
    return B.reshape(x, (b, nkv * rep, s, d))


def rope_tables(B, theta, seq_len, head_dim):
    """helpers.rs:164-193"""
    half = head_dim // 2
    f = B.cast(B.arange(half), F32)
    two = nn.constant(B, float(np.float32(2.0) / np.float32(head_dim)), f.shape)
    f = B.mul(f, two)
    th = nn.constant(B, theta, f.shape)
    freq = B.pow(th, f)
    inv_freq = nn.inverse(B, freq)
    inv_freq = B.broadcast(inv_freq, (seq_len, half))
    pos = B.cast(B.arange(seq_len), F32)
    pos = B.reshape(pos, (seq_len, 1))
    pos = B.broadcast(pos, inv_freq.shape)
    pos = B.mul(pos, inv_freq)
    cos = B.cos(pos)
    sin = B.sin(pos)
    cos = B.concat(cos, cos, 1)
    sin = B.concat(sin, sin, 1)
    return cos, sin


def rotate_half(B, head_dim, x):
    """helpers.rs:195-199"""
    v = chunk(B, 3, 2, head_dim // 2, x)
    return B.concat(B.neg(v[1]), v[0], 3)


def apply_rope_embedding(B, pos, head_dim, cos, sin, x):
    """helpers.rs:202-221"""
    sh = x.shape
    seq_len = sh[2]
    cos = B.slice(cos, 0, pos, seq_len)
    sin = B.slice(sin, 0, pos, seq_len)
    cos = B.broadcast(cos, sh)
    sin = B.broadcast(sin, sh)
    rotated = rotate_half(B, head_dim, x)
    return B.add(B.mul(cos, x), B.mul(sin, rotated))


def rope(B, theta, pos, seq_len, head_dim, x):
    """helpers.rs:224-237"""
    cos, sin = rope_tables(B, theta, pos + seq_len, head_dim)
    return apply_rope_embedding(B, pos, head_dim, cos, sin, x)


def causal_mask(B, size):
    """helpers.rs:239-257: cast(lt(row, col)) * f32::MIN"""
    i = B.arange(size)
    i = B.broadcast(i, (size, size))
    j = B.arange(size)
    j = B.reshape(j, (size, 1))
    j = B.broadcast(j, (size, size))
    mask = B.lt(j, i)
    mask = B.cast(mask, F32)
    ninf = nn.constant(B, F32_MIN, mask.shape)
    return B.mul(mask, ninf)


def embeddings(B, params, path, x):
    """helpers.rs:259-271"""
    wte = params[path + ".weight"]
    b, s = x.shape
    x = B.reshape(x, (b * s,))
    te = B.index(wte, 0, x)
    return unsqueeze(B, 0, te)
