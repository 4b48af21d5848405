"""catgrad-llm/src/models/llama.rs as backend calls, plus the greedy driver loop of
catgrad-llm/examples/llama/main.rs:118-169."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import helpers as H
from . import nn


@dataclass
class Config:
    """The fields of catgrad-llm/src/legacy/models/utils.rs:52-112 that the Llama graph reads."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False

    def get_head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def mlp(B, cfg, params, p, x):
    """llama.rs:12-35"""
    gate = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".gate_proj", x)
    up = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".up_proj", x)
    x = B.mul(nn.silu(B, gate), up)
    return nn.linear_no_bias(B, cfg.intermediate_size, cfg.hidden_size, params, p + ".down_proj", x)


def attention(B, cfg, params, cache, pos, p, x):
    """llama.rs:37-115"""
    dim = cfg.hidden_size
    nh = cfg.num_attention_heads
    hd = dim // nh
    nkv = cfg.num_key_value_heads
    rep = nh // nkv
    b, s, _ = x.shape
    q = nn.linear_no_bias(B, dim, dim, params, p + ".q_proj", x)
    k = nn.linear_no_bias(B, dim, dim // rep, params, p + ".k_proj", x)
    v = nn.linear_no_bias(B, dim, dim // rep, params, p + ".v_proj", x)
    k = B.reshape(k, (b, s, nkv, hd))
    v = B.reshape(v, (b, s, nkv, hd))
    q = B.reshape(q, (b, s, nh, hd))
    q = B.transpose(q, 1, 2)
    k = B.transpose(k, 1, 2)
    v = B.transpose(v, 1, 2)
    k = H.repeat_kv(B, rep, k)
    v = H.repeat_kv(B, rep, v)
    cos, sin = cache
    q = H.apply_rope_embedding(B, pos, hd, cos, sin, q)
    k = H.apply_rope_embedding(B, pos, hd, cos, sin, k)
    tk = B.transpose(k, 2, 3)
    attn = B.matmul(q, tk)
    sh = attn.shape
    denom = nn.constant(B, float(np.sqrt(np.float32(hd), dtype=np.float32)), sh)
    attn = B.div(attn, denom)
    mask = H.causal_mask(B, s)
    mask = B.broadcast(mask, sh)
    attn = B.add(attn, mask)
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.transpose(attn, 1, 2)
    attn = B.reshape(attn, (b, s, dim))
    return nn.linear_no_bias(B, dim, dim, params, p + ".o_proj", attn)


def layer(B, cfg, params, cache, pos, p, x):
    """llama.rs:117-151"""
    res = x
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".input_layernorm", x)
    x = attention(B, cfg, params, cache, pos, p + ".self_attn", x)
    x = B.add(res, x)
    res = x
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_attention_layernorm", x)
    x = mlp(B, cfg, params, p + ".mlp", x)
    return B.add(x, res)


def forward(B, cfg, params, tokens, max_sequence_length, want_logits=False):
    """`LlamaModel::def` (llama.rs:159-204).  `tokens` is a U32 tensor [1, S].  Returns the
    argmax tensor [1, S, 1]; with want_logits also the logits [1, S, V] it was taken from."""
    cache = H.rope_tables(B, cfg.rope_theta, max_sequence_length, cfg.get_head_dim())  # Cache::init
    x = H.embeddings(B, params, "model.embed_tokens", tokens)
    for i in range(cfg.num_hidden_layers):
        x = layer(B, cfg, params, cache, 0, f"model.layers.{i}", x)
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, "model.norm", x)
    head = "model.embed_tokens" if cfg.tie_word_embeddings else "lm_head"
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, head, x)
    out = B.argmax(logits)
    return (out, logits) if want_logits else out


def generate(B, cfg, params, prompt, steps, max_sequence_length=None, forward_fn=forward):
    """The greedy loop of examples/llama/main.rs:118-169: one full forward over all tokens
    per generated token, next token = last element of the argmax output.  `prompt` is a 1-D
    sequence of token ids; returns the `steps` generated ids."""
    ids = [int(t) for t in prompt]
    if max_sequence_length is None:
        max_sequence_length = len(ids) + steps
    out = []
    for _ in range(steps):
        x = B.ndarray_from_vec_u32(np.asarray(ids, dtype=np.uint32), (1, len(ids)))
        y = forward_fn(B, cfg, params, x, max_sequence_length)
        nxt = int(B.to_vec(y)[-1])
        out.append(nxt)
        ids.append(nxt)
    return out
