"""The Llama graph with an explicit KV cache, and the runner that drives it.

catgrad-llm's serving runner (catgrad-llm/src/run.rs:149-262) builds, for every call, a graph
whose inputs are the new tokens plus one (k, v) pair per layer holding the keys and values of all
earlier positions, and whose outputs are the next token plus the grown pairs
(`Cache::update_kv_cache`, catgrad-llm/src/legacy/models/utils.rs:210-228: `concat` along the
position axis, after the rotation, before `repeat_kv`; catgrad-llm/src/legacy/models/llama.rs:100-130).
The prompt goes through in one call, then one token per call.  This module is that graph and
that loop as backend calls, on the trait path: the cache tensors are ordinary backend tensors
(device-resident on the CUDA backend) handed from one call to the next.
"""
from __future__ import annotations

import numpy as np

from . import helpers as H
from . import llama
from . import nn


def attention_kv(B, cfg, params, cache, pos, kv, p, x):
    """legacy/models/llama.rs:75-131 with `update_kv_cache`; returns (output, (k, v) grown)."""
    dim, nh, nkv = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads
    hd = dim // nh
    rep = nh // nkv
    b, s, _ = x.shape
    q = nn.linear_no_bias(B, dim, dim, params, p + ".q_proj", x)
    k = nn.linear_no_bias(B, dim, dim // rep, params, p + ".k_proj", x)
    v = nn.linear_no_bias(B, dim, dim // rep, params, p + ".v_proj", x)
    q = B.transpose(B.reshape(q, (b, s, nh, hd)), 1, 2)
    k = B.transpose(B.reshape(k, (b, s, nkv, hd)), 1, 2)
    v = B.transpose(B.reshape(v, (b, s, nkv, hd)), 1, 2)
    cos, sin = cache
    q = H.apply_rope_embedding(B, pos, hd, cos, sin, q)
    k = H.apply_rope_embedding(B, pos, hd, cos, sin, k)
    if kv is not None:                       # update_kv_cache (utils.rs:210-228)
        k = B.concat(kv[0], k, 2)
        v = B.concat(kv[1], v, 2)
    grown = (k, v)
    k = H.repeat_kv(B, rep, k)
    v = H.repeat_kv(B, rep, v)
    attn = B.matmul(q, B.transpose(k, 2, 3))
    sh = attn.shape
    attn = B.div(attn, nn.constant(B, float(np.sqrt(np.float32(hd), dtype=np.float32)), sh))
    # causal_mask(s) is [s, s]; it broadcasts to [b, nh, s, T] when the cache is empty (T = s) or
    # when one token is run (s = 1, a single zero): the two cases the runner produces
    if not (s == 1 or sh[3] == s):
        raise ValueError("the explicit-cache graph takes a whole prompt on an empty cache or one token at a time")
    attn = B.add(attn, B.broadcast(H.causal_mask(B, s), sh))
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.reshape(B.transpose(attn, 1, 2), (b, s, dim))
    return nn.linear_no_bias(B, dim, dim, params, p + ".o_proj", attn), grown


def forward_kv(B, cfg, params, tokens, pos, kv_cache, max_sequence_length, want_logits=False):
    """One call of the runner's graph (run.rs:149-217): tokens U32 [1, S] at positions
    [pos, pos + S), kv_cache a list of per-layer (k, v) or None.  Returns (argmax [1, S, 1],
    new kv_cache[, logits])."""
    cache = H.rope_tables(B, cfg.rope_theta, max_sequence_length, cfg.get_head_dim())
    x = H.embeddings(B, params, "model.embed_tokens", tokens)
    grown = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        res = x
        x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".input_layernorm", x)
        x, g = attention_kv(B, cfg, params, cache, pos, kv_cache[i] if kv_cache else None, p + ".self_attn", x)
        grown.append(g)
        x = B.add(res, x)
        res = x
        x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_attention_layernorm", x)
        x = llama.mlp(B, cfg, params, p + ".mlp", x)
        x = B.add(x, res)
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, "model.norm", x)
    head = "model.embed_tokens" if cfg.tie_word_embeddings else "lm_head"
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, head, x)
    out = B.argmax(logits)
    return (out, grown, logits) if want_logits else (out, grown)


class KVRunner:
    """`ModelRunner` with `use_kv_cache` (run.rs:219-262 and the Iterator / LM impls at :262-305):
    `set_context` then iterate; every step runs only the tokens not yet cached."""

    def __init__(self, B, cfg, params, max_sequence_length: int, eos_token_ids=()):
        self.B, self.cfg, self.params, self.max_len = B, cfg, params, max_sequence_length
        self.eos = set(int(t) for t in eos_token_ids)
        self.context: list[int] = []
        self.tokens: list[int] = []
        self.kv_cache = None
        self.total_tokens = 0

    def set_context(self, context):
        context = [int(t) for t in context]
        n = 0
        for a, b in zip(self.context, context):
            if a != b:
                break
            n += 1
        if n < len(self.context):       # run.rs:295-299: a changed context drops the cache
            self.kv_cache = None
            self.total_tokens = 0
        self.context = list(context)
        self.tokens = list(context) if self.total_tokens == 0 else context[self.total_tokens:]

    def __iter__(self):
        return self

    def __next__(self) -> int:
        tokens, self.tokens = self.tokens, []
        if not tokens:
            raise StopIteration
        x = self.B.ndarray_from_vec_u32(np.asarray(tokens, dtype=np.uint32), (1, len(tokens)))
        out, self.kv_cache = forward_kv(self.B, self.cfg, self.params, x, self.total_tokens, self.kv_cache, self.max_len)
        token = int(self.B.to_vec(out)[-1])
        self.total_tokens += len(tokens)
        if token in self.eos:
            raise StopIteration
        self.tokens.append(token)
        self.context.append(token)
        return token

    def complete(self, context):
        self.set_context(context)
        return self
