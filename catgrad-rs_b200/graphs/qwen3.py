"""catgrad-llm/src/models/qwen3.rs as backend calls: Llama plus per-head q/k RMSNorm before the
rotation, head_dim from the config, and the mixture-of-experts FFN on sparse layers."""
from __future__ import annotations

import numpy as np

from . import helpers as H
from . import nn


def rmsnorm(B, eps, params, path, x):
    """qwen3.rs:37-62 (any rank; same op chain as helpers.rmsnorm)"""
    return H.rmsnorm(B, eps, params, path, x)


def moe(B, cfg, params, p, x):
    """qwen3.rs:64-133: router softmax -> topk -> optional renorm, then per slot a whole
    expert matrix is gathered per token and applied by a batched matmul."""
    _, seq_len, _ = x.shape
    gate_all = params[p + ".experts.gate_proj.weight"]
    up_all = params[p + ".experts.up_proj.weight"]
    down_all = params[p + ".experts.down_proj.weight"]
    routed = nn.linear_no_bias(B, cfg.hidden_size, cfg.num_local_experts, params, p + ".gate", x)
    routed = nn.softmax(B, routed)
    values, indices = B.topk(routed, cfg.num_experts_per_tok)
    sh = (seq_len, cfg.num_experts_per_tok)
    indices = B.reshape(indices, sh)
    values = B.reshape(values, sh)
    if cfg.norm_topk_prob:
        sv = B.broadcast(B.sum(values), sh)
        values = B.div(values, sv)
    fullx = B.transpose(x, 0, 1)  # [S, 1, H]
    sumk = nn.constant(B, 0.0, fullx.shape)
    for i in range(cfg.num_experts_per_tok):
        idx = B.slice(indices, 1, i, 1)  # rank-2 ids: the backends flatten them (ndarray.rs:378)
        val = B.slice(values, 1, i, 1)
        gate = B.transpose(B.index(gate_all, 0, idx), 1, 2)
        up = B.transpose(B.index(up_all, 0, idx), 1, 2)
        down = B.transpose(B.index(down_all, 0, idx), 1, 2)
        g = B.matmul(fullx, gate)
        u = B.matmul(fullx, up)
        h = B.mul(nn.silu(B, g), u)
        y = B.matmul(h, down)
        v = H.unsqueeze(B, 2, val)
        v = B.broadcast(v, y.shape)
        sumk = B.add(sumk, B.mul(y, v))
    return B.transpose(sumk, 0, 1), indices


def attention(B, cfg, params, cache, pos, p, x):
    """qwen3.rs:135-262"""
    dim, nh, nkv, hd = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    rep = nh // nkv
    b, s, _ = x.shape
    q = nn.linear_no_bias(B, dim, nh * hd, params, p + ".q_proj", x)
    k = nn.linear_no_bias(B, dim, nkv * hd, params, p + ".k_proj", x)
    v = nn.linear_no_bias(B, dim, nkv * hd, params, p + ".v_proj", x)
    q = B.transpose(B.reshape(q, (b, s, nh, hd)), 1, 2)
    k = B.transpose(B.reshape(k, (b, s, nkv, hd)), 1, 2)
    v = B.transpose(B.reshape(v, (b, s, nkv, hd)), 1, 2)
    q = B.reshape(q, (b * s * nh, hd))
    k = B.reshape(k, (b * s * nkv, hd))
    q = rmsnorm(B, cfg.rms_norm_eps, params, p + ".q_norm", q)
    k = rmsnorm(B, cfg.rms_norm_eps, params, p + ".k_norm", k)
    q = B.reshape(q, (b, nh, s, hd))
    k = B.reshape(k, (b, nkv, s, hd))
    k = H.repeat_kv(B, rep, k)
    v = H.repeat_kv(B, rep, v)
    cos, sin = cache
    q = H.apply_rope_embedding(B, pos, hd, cos, sin, q)
    k = H.apply_rope_embedding(B, pos, hd, cos, sin, k)
    attn = B.matmul(q, B.transpose(k, 2, 3))
    sh = attn.shape
    attn = B.div(attn, nn.constant(B, float(np.sqrt(np.float32(hd), dtype=np.float32)), sh))
    attn = B.add(attn, B.broadcast(H.causal_mask(B, s), sh))
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.reshape(B.transpose(attn, 1, 2), (b, s, nh * hd))
    return nn.linear_no_bias(B, nh * hd, dim, params, p + ".o_proj", attn)


def mlp(B, cfg, params, p, x):
    """qwen3.rs dense FFN (same as llama.rs:12-35)"""
    gate = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".gate_proj", x)
    up = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".up_proj", x)
    return nn.linear_no_bias(B, cfg.intermediate_size, cfg.hidden_size, params, p + ".down_proj", B.mul(nn.silu(B, gate), up))


def forward(B, cfg, params, tokens, max_sequence_length, want_logits=False, expert_ids=None):
    """`Qwen3Model::def` (qwen3.rs:264-358).  `expert_ids`, when a list, receives the top-k
    expert ids of every sparse layer."""
    cache = H.rope_tables(B, cfg.rope_theta, max_sequence_length, cfg.head_dim)
    x = H.embeddings(B, params, "model.embed_tokens", tokens)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        res = x
        x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".input_layernorm", x)
        x = attention(B, cfg, params, cache, 0, p + ".self_attn", x)
        x = B.add(res, x)
        res = x
        x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_attention_layernorm", x)
        if cfg.num_local_experts > 1 and (i + 1) % cfg.decoder_sparse_step == 0:  # qwen3.rs:297-298
            x, ids = moe(B, cfg, params, p + ".mlp", x)
            if expert_ids is not None:
                expert_ids.append(ids)
        else:
            x = mlp(B, cfg, params, p + ".mlp", x)
        x = B.add(x, res)
    x = rmsnorm(B, cfg.rms_norm_eps, params, "model.norm", x)
    head = "model.embed_tokens" if cfg.tie_word_embeddings else "lm_head"
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, head, x)
    out = B.argmax(logits)
    return (out, logits) if want_logits else out
