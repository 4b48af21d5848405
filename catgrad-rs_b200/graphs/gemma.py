"""catgrad-llm/src/models/gemma3.rs as backend calls, with the three Gemma-2 features the
reference tree lacks (attention logit soft-cap, final logit soft-cap, sliding-window mask)
composed from reference ops: cap * tanh(x / cap) with the stdlib's tanh
(catgrad/src/stdlib/nn/mod.rs:138-144) and a second `lt` on the arange grids of
`causal_mask` (catgrad-llm/src/helpers.rs:239-257).  With qk_norm=False, one rope base and the
soft-caps/window set, this is the Gemma-2-shaped benchmark configuration; with qk_norm=True, no
caps and sliding_window_pattern / rope_local_base_freq set it is the reference's Gemma3 graph,
whose local layers rotate with their own rope base (gemma3.rs:154-159)."""
from __future__ import annotations

import numpy as np

from . import helpers as H
from . import nn

F32 = 0


def rmsnorm(B, eps, params, path, x):
    """gemma3.rs:41-68: lr * (1 + gamma)"""
    gamma = params[path + ".weight"]
    lr = H.rmsnorm_raw(B, eps, x)
    gamma = B.broadcast(gamma, lr.shape)
    one = nn.constant(B, 1.0, gamma.shape)
    return B.mul(lr, B.add(one, gamma))


def softcap(B, cap, x):
    sh = x.shape
    c = nn.constant(B, cap, sh)
    return B.mul(c, nn.tanh(B, B.div(x, c)))


def window_mask(B, size, window):
    """f32::MIN where the key is more than window-1 positions behind the query."""
    i = B.broadcast(B.arange(size), (size, size))                      # key index (columns)
    j = B.broadcast(B.reshape(B.arange(size), (size, 1)), (size, size))  # query index (rows)
    w = B.broadcast(B.ndarray_from_vec_u32([window - 1], ()), (size, size))
    far = B.cast(B.lt(B.add(i, w), j), F32)
    return B.mul(far, nn.constant(B, H.F32_MIN, (size, size)))


def mlp(B, cfg, params, p, x):
    """gemma3.rs:13-36: GeGLU"""
    gate = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".gate_proj", x)
    up = nn.linear_no_bias(B, cfg.hidden_size, cfg.intermediate_size, params, p + ".up_proj", x)
    return nn.linear_no_bias(B, cfg.intermediate_size, cfg.hidden_size, params, p + ".down_proj", B.mul(nn.gelu(B, gate), up))


def attention(B, cfg, params, layer_id, pos, p, x):
    """gemma3.rs:70-190"""
    dim, nh, nkv, hd = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    rep = nh // nkv
    b, s, _ = x.shape
    q = nn.linear_no_bias(B, dim, nh * hd, params, p + ".q_proj", x)
    k = nn.linear_no_bias(B, dim, nkv * hd, params, p + ".k_proj", x)
    v = nn.linear_no_bias(B, dim, nkv * hd, params, p + ".v_proj", x)
    q = B.transpose(B.reshape(q, (b, s, nh, hd)), 1, 2)
    k = B.transpose(B.reshape(k, (b, s, nkv, hd)), 1, 2)
    v = B.transpose(B.reshape(v, (b, s, nkv, hd)), 1, 2)
    if cfg.qk_norm:
        q = B.reshape(q, (b * s * nh, hd))
        k = B.reshape(k, (b * s * nkv, hd))
        q = rmsnorm(B, cfg.rms_norm_eps, params, p + ".q_norm", q)
        k = rmsnorm(B, cfg.rms_norm_eps, params, p + ".k_norm", k)
        q = B.reshape(q, (b, nh, s, hd))
        k = B.reshape(k, (b, nkv, s, hd))
    # every sliding_window_pattern-th layer is global, the others local, with different rope
    # frequencies (gemma3.rs:154-159); tables rebuilt per call (gemma3.rs:160-161)
    theta = cfg.rope_theta
    if cfg.sliding_window_pattern > 0 and (layer_id + 1) % cfg.sliding_window_pattern != 0:
        theta = cfg.rope_local_base_freq
    q = H.rope(B, theta, pos, s, hd, q)
    k = H.rope(B, theta, pos, s, hd, k)
    k = H.repeat_kv(B, rep, k)
    v = H.repeat_kv(B, rep, v)
    attn = B.matmul(q, B.transpose(k, 2, 3))
    sh = attn.shape
    attn = B.div(attn, nn.constant(B, float(np.sqrt(np.float32(hd), dtype=np.float32)), sh))
    if cfg.attn_logit_softcap > 0:
        attn = softcap(B, cfg.attn_logit_softcap, attn)
    mask = H.causal_mask(B, s)
    if cfg.sliding_window > 0 and layer_id % 2 == 0:  # even layers are local
        mask = B.add(mask, window_mask(B, s, cfg.sliding_window))
    attn = B.add(attn, B.broadcast(mask, sh))
    attn = nn.softmax(B, attn)
    attn = B.matmul(attn, v)
    attn = B.reshape(B.transpose(attn, 1, 2), (b, s, nh * hd))
    return nn.linear_no_bias(B, nh * hd, dim, params, p + ".o_proj", attn)


def layer(B, cfg, params, layer_id, pos, p, x):
    """gemma3.rs:192-238: four norms per layer"""
    res = x
    x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".input_layernorm", x)
    x = attention(B, cfg, params, layer_id, pos, p + ".self_attn", x)
    x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_attention_layernorm", x)
    x = B.add(res, x)
    res = x
    x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".pre_feedforward_layernorm", x)
    x = mlp(B, cfg, params, p + ".mlp", x)
    x = rmsnorm(B, cfg.rms_norm_eps, params, p + ".post_feedforward_layernorm", x)
    return B.add(x, res)


def forward(B, cfg, params, tokens, max_sequence_length, want_logits=False):
    """`Gemma3Model::def` (gemma3.rs:245-290): embeddings * sqrt(H), tied head."""
    x = H.embeddings(B, params, "model.embed_tokens", tokens)
    x = B.mul(x, nn.constant(B, float(np.sqrt(np.float32(cfg.hidden_size), dtype=np.float32)), x.shape))
    for i in range(cfg.num_hidden_layers):
        x = layer(B, cfg, params, i, 0, f"model.layers.{i}", x)
    x = rmsnorm(B, cfg.rms_norm_eps, params, "model.norm", x)
    logits = nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, params, "model.embed_tokens", x)
    if cfg.final_logit_softcap > 0:
        logits = softcap(B, cfg.final_logit_softcap, logits)
    out = B.argmax(logits)
    return (out, logits) if want_logits else out
