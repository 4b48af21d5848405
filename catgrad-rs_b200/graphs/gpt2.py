"""catgrad-llm/src/models/gpt2.rs as backend calls: learned position embeddings, LayerNorm with
bias, linear layers whose checkpoint weights are stored already transposed ([in, out]) and carry
a bias, one fused qkv projection split with `chunk`, tanh-GELU, tied head."""
from __future__ import annotations

import numpy as np

from . import helpers as H
from . import nn


def embeddings(B, params, p, x):
    """gpt2.rs:13-34: token rows plus rows 0..S of the position table (`p` is a name prefix, "" for
    a bare checkpoint)"""
    wte = params[p + "wte.weight"]
    b, s = x.shape
    te = B.index(wte, 0, B.reshape(x, (b * s,)))
    seq_len, hidden = te.shape
    sh = (1, seq_len, hidden)
    te = B.reshape(te, sh)
    wpe = params[p + "wpe.weight"]
    pe = B.index(wpe, 0, B.arange(seq_len))
    pe = B.reshape(pe, sh)
    return B.add(te, pe)


def gpt_linear(B, params, p, x):
    """gpt2.rs:36-56: x @ W + b with W stored [in, out]"""
    w = params[p + ".weight"]
    b = params[p + ".bias"]
    w_t = H.unsqueeze(B, 0, w)
    m = B.matmul(x, w_t)
    return B.add(m, B.broadcast(b, m.shape))


def mlp(B, cfg, params, p, x):
    """gpt2.rs:58-63"""
    x = gpt_linear(B, params, p + ".c_fc", x)
    x = nn.gelu(B, x)
    return gpt_linear(B, params, p + ".c_proj", x)


def attention(B, cfg, params, p, x):
    """gpt2.rs:65-114: multi-head attention without rotary embedding"""
    dim, nh = cfg.hidden_size, cfg.num_attention_heads
    hd = dim // nh
    b, s, _ = x.shape
    c_attn = gpt_linear(B, params, p + ".c_attn", x)
    q, k, v = H.chunk(B, 2, 3, dim, c_attn)
    sh = (b, s, nh, hd)
    q = B.transpose(B.reshape(q, sh), 1, 2)
    k = B.transpose(B.reshape(k, sh), 1, 2)
    v = B.transpose(B.reshape(v, sh), 1, 2)
    attn = B.matmul(q, B.transpose(k, 2, 3))
    sh = attn.shape
    attn = B.div(attn, nn.constant(B, float(np.sqrt(np.float32(hd), dtype=np.float32)), sh))
    attn = B.add(attn, B.broadcast(H.causal_mask(B, s), sh))
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.reshape(B.transpose(attn, 1, 2), (b, s, dim))
    return gpt_linear(B, params, p + ".c_proj", attn)


def layer(B, cfg, params, p, x):
    """gpt2.rs:116-134"""
    res = x
    x = H.layernorm(B, cfg.layer_norm_epsilon, params, p + ".ln_1", x)
    x = attention(B, cfg, params, p + ".attn", x)
    x = B.add(res, x)
    res = x
    x = H.layernorm(B, cfg.layer_norm_epsilon, params, p + ".ln_2", x)
    x = mlp(B, cfg, params, p + ".mlp", x)
    return B.add(x, res)


def forward(B, cfg, params, tokens, max_sequence_length, want_logits=False):
    """`GPT2Model::def` (gpt2.rs:137-171); parameter names are the checkpoint's (wte, wpe, h.N...)."""
    x = embeddings(B, params, "", tokens)
    for i in range(cfg.num_hidden_layers):
        x = layer(B, cfg, params, f"h.{i}", x)
    x = H.layernorm(B, cfg.layer_norm_epsilon, params, "ln_f", x)
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, "wte", x)
    out = B.argmax(logits)
    return (out, logits) if want_logits else out


def param_shapes(cfg) -> dict:
    """Checkpoint tensor names and shapes (weights of the linear layers are [in, out])."""
    H_, V, T = cfg.hidden_size, cfg.vocab_size, cfg.max_position_embeddings
    s = {"wte.weight": (V, H_), "wpe.weight": (T, H_), "ln_f.weight": (H_,), "ln_f.bias": (H_,)}
    for i in range(cfg.num_hidden_layers):
        p = f"h.{i}."
        for ln in ("ln_1", "ln_2"):
            s[p + ln + ".weight"] = (H_,)
            s[p + ln + ".bias"] = (H_,)
        s[p + "attn.c_attn.weight"] = (H_, 3 * H_)
        s[p + "attn.c_attn.bias"] = (3 * H_,)
        s[p + "attn.c_proj.weight"] = (H_, H_)
        s[p + "attn.c_proj.bias"] = (H_,)
        s[p + "mlp.c_fc.weight"] = (H_, 4 * H_)
        s[p + "mlp.c_fc.bias"] = (4 * H_,)
        s[p + "mlp.c_proj.weight"] = (4 * H_, H_)
        s[p + "mlp.c_proj.bias"] = (H_,)
    return s
