"""catgrad-llm/src/models/granite.rs as backend calls: the Llama graph with four scalar
multipliers (embedding, attention scores instead of 1/sqrt(d), both residual branches) and,
when `num_experts_per_tok > 0`, the Granite-MoE block (top-k on the raw router outputs, softmax
over the k chosen values, gate and up stacked in one `input_linear` matrix per expert)."""
from __future__ import annotations

from . import helpers as H
from . import llama
from . import nn


def moe(B, cfg, params, p, x):
    """granite.rs:38-89"""
    _, seq_len, _ = x.shape
    moe_input = params[p + ".input_linear.weight"]    # [E, 2 F, H]
    moe_output = params[p + ".output_linear.weight"]  # [E, H, F]
    routed = nn.linear_no_bias(B, cfg.hidden_size, cfg.num_local_experts, params, p + ".router.layer", x)
    values, indices = B.topk(routed, cfg.num_experts_per_tok)
    sh = (seq_len, cfg.num_experts_per_tok)
    indices = B.reshape(indices, sh)
    values = B.reshape(values, sh)
    values = nn.softmax(B, values)
    fullx = B.transpose(x, 0, 1)
    sumk = nn.constant(B, 0.0, fullx.shape)
    for i in range(cfg.num_experts_per_tok):
        idx = B.slice(indices, 1, i, 1)
        val = B.slice(values, 1, i, 1)
        gate_up = B.index(moe_input, 0, idx)
        out = B.index(moe_output, 0, idx)
        g, u = H.chunk(B, 1, 2, cfg.intermediate_size, gate_up)
        gate = B.matmul(fullx, B.transpose(g, 1, 2))
        up = B.matmul(fullx, B.transpose(u, 1, 2))
        y = B.matmul(B.mul(nn.silu(B, gate), up), B.transpose(out, 1, 2))
        v = B.broadcast(H.unsqueeze(B, 2, val), y.shape)
        sumk = B.add(sumk, B.mul(y, v))
    return B.transpose(sumk, 0, 1), indices


def attention(B, cfg, params, cache, pos, p, x):
    """granite.rs:91-173: rope before repeat_kv, scores scaled by `attention_multiplier`"""
    dim, nh, nkv = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads
    hd = dim // nh
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
    cos, sin = cache
    q = H.apply_rope_embedding(B, pos, hd, cos, sin, q)
    k = H.apply_rope_embedding(B, pos, hd, cos, sin, k)
    k = H.repeat_kv(B, rep, k)
    v = H.repeat_kv(B, rep, v)
    attn = B.matmul(q, B.transpose(k, 2, 3))
    sh = attn.shape
    attn = B.mul(attn, nn.constant(B, cfg.attention_multiplier, sh))
    attn = B.add(attn, B.broadcast(H.causal_mask(B, s), sh))
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.reshape(B.transpose(attn, 1, 2), (b, s, dim))
    return nn.linear_no_bias(B, dim, dim, params, p + ".o_proj", attn)


def layer(B, cfg, params, cache, pos, p, x, expert_ids=None):
    """granite.rs:175-213"""
    res = x
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".input_layernorm", x)
    x = attention(B, cfg, params, cache, pos, p + ".self_attn", x)
    mul = nn.constant(B, cfg.residual_multiplier, x.shape)
    x = B.add(res, B.mul(x, mul))
    res = x
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_attention_layernorm", x)
    if cfg.num_experts_per_tok == 0:
        x = llama.mlp(B, cfg, params, p + ".mlp", x)
    else:
        x, ids = moe(B, cfg, params, p + ".block_sparse_moe", x)
        if expert_ids is not None:
            expert_ids.append(ids)
    return B.add(B.mul(x, mul), res)


def forward(B, cfg, params, tokens, max_sequence_length, want_logits=False, expert_ids=None):
    """`GraniteModel::def` (granite.rs:216-271): tied head"""
    cache = H.rope_tables(B, cfg.rope_theta, max_sequence_length, cfg.hidden_size // cfg.num_attention_heads)
    emb = H.embeddings(B, params, "model.embed_tokens", tokens)
    x = B.mul(nn.constant(B, cfg.embedding_multiplier, emb.shape), emb)
    for i in range(cfg.num_hidden_layers):
        x = layer(B, cfg, params, cache, 0, f"model.layers.{i}", x, expert_ids)
    x = H.rmsnorm(B, cfg.rms_norm_eps, params, "model.norm", x)
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, "model.embed_tokens", x)
    out = B.argmax(logits)
    return (out, logits) if want_logits else out


def param_shapes(cfg) -> dict:
    H_, F, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    d = H_ // nh
    s = {"model.embed_tokens.weight": (V, H_), "model.norm.weight": (H_,)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (H_,)
        s[p + "post_attention_layernorm.weight"] = (H_,)
        s[p + "self_attn.q_proj.weight"] = (nh * d, H_)
        s[p + "self_attn.k_proj.weight"] = (nkv * d, H_)
        s[p + "self_attn.v_proj.weight"] = (nkv * d, H_)
        s[p + "self_attn.o_proj.weight"] = (H_, nh * d)
        if cfg.num_experts_per_tok == 0:
            s[p + "mlp.gate_proj.weight"] = (F, H_)
            s[p + "mlp.up_proj.weight"] = (F, H_)
            s[p + "mlp.down_proj.weight"] = (H_, F)
        else:
            E = cfg.num_local_experts
            s[p + "block_sparse_moe.router.layer.weight"] = (E, H_)
            s[p + "block_sparse_moe.input_linear.weight"] = (E, 2 * F, H_)
            s[p + "block_sparse_moe.output_linear.weight"] = (E, H_, F)
    return s
