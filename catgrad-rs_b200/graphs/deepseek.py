"""The mixture-of-experts block of catgrad-llm/src/models/deepseek.rs as backend calls:
sigmoid router with a per-expert score-correction bias, group-limited top-k (experts are split
into `n_group` groups, groups are ranked by the sum of their two best scores, only the best
`topk_group` groups stay eligible -- built from `arange`, `eq`, `sum` and `cast`, there is no
scatter in the op set), renormalisation with a routed scaling factor, the per-slot expert
application shared with Qwen3-MoE, and the always-on shared experts.

The multi-head latent attention of the same file (deepseek.rs:166-330) is not emitted: it adds
no backend method beyond those exercised here and by the other graphs."""
from __future__ import annotations

from . import helpers as H
from . import nn

F32 = 0


def mlp(B, cfg, params, p, x, width):
    """deepseek.rs:14-37"""
    gate = nn.linear_no_bias(B, cfg.hidden_size, width, params, p + ".gate_proj", x)
    up = nn.linear_no_bias(B, cfg.hidden_size, width, params, p + ".up_proj", x)
    return nn.linear_no_bias(B, width, cfg.hidden_size, params, p + ".down_proj", B.mul(nn.silu(B, gate), up))


def moe_topk_router(B, cfg, params, p, x):
    """deepseek.rs:39-110 -> (values [S, k], indices [S, k])"""
    _, seq_len, _ = x.shape
    E, n_groups = cfg.num_local_experts, cfg.n_group
    routed = nn.linear_no_bias(B, cfg.hidden_size, E, params, p, x)
    routed = nn.sigmoid(B, routed)
    bias = params[p + ".e_score_correction_bias"]
    routed_sh = routed.shape
    scores_for_choice = B.add(routed, B.broadcast(bias, routed_sh))
    per_group = E // n_groups
    group_scores = B.reshape(scores_for_choice, (seq_len, n_groups, per_group))
    group_scores = B.topk(group_scores, 2)[0]
    group_scores = B.sum(group_scores)
    group_scores = B.reshape(group_scores, (seq_len, n_groups))
    group_idx = B.topk(group_scores, cfg.topk_group)[1]
    # the reference reshapes the [S, topk_group] indices to [S, experts_per_group, 1]: the two
    # extents coincide in the checkpoints it targets (deepseek.rs:66-67)
    group_idx = B.reshape(group_idx, (seq_len, per_group, 1))
    # group_mask.scatter_(1, group_idx, 1) without a scatter: compare against every group id
    sh = (seq_len, per_group, n_groups)
    cols = B.broadcast(B.arange(n_groups), sh)
    group_idx = B.broadcast(group_idx, sh)
    matches = B.transpose(B.eq(cols, group_idx), 1, 2)
    mask = B.sum(matches)                                   # [S, n_groups, 1], u32
    mask = B.broadcast(mask, (seq_len, n_groups, per_group))
    mask = B.cast(B.reshape(mask, routed_sh), F32)
    scores_for_choice = B.mul(mask, scores_for_choice)
    values, indices = B.topk(scores_for_choice, cfg.num_experts_per_tok)
    sh = (seq_len, cfg.num_experts_per_tok)
    indices = B.reshape(indices, sh)
    values = B.reshape(values, sh)
    if cfg.norm_topk_prob:
        sv = B.sum(values)
        sv = B.add(sv, nn.constant(B, 1e-20, sv.shape))
        values = B.div(values, B.broadcast(sv, sh))
        values = B.mul(values, nn.constant(B, cfg.routed_scaling_factor, values.shape))
    return values, indices


def moe(B, cfg, params, p, x, expert_ids=None):
    """deepseek.rs:112-164"""
    res = x
    values, indices = moe_topk_router(B, cfg, params, p + ".gate", x)
    if expert_ids is not None:
        expert_ids.append(indices)
    gate_all = params[p + ".experts.gate_proj.weight"]
    up_all = params[p + ".experts.up_proj.weight"]
    down_all = params[p + ".experts.down_proj.weight"]
    fullx = B.transpose(x, 0, 1)
    sumk = nn.constant(B, 0.0, fullx.shape)
    for i in range(cfg.num_experts_per_tok):
        idx = B.slice(indices, 1, i, 1)
        val = B.slice(values, 1, i, 1)
        gate = B.transpose(B.index(gate_all, 0, idx), 1, 2)
        up = B.transpose(B.index(up_all, 0, idx), 1, 2)
        down = B.transpose(B.index(down_all, 0, idx), 1, 2)
        y = B.matmul(B.mul(nn.silu(B, B.matmul(fullx, gate)), B.matmul(fullx, up)), down)
        v = B.broadcast(H.unsqueeze(B, 2, val), y.shape)
        sumk = B.add(sumk, B.mul(y, v))
    sumk = B.transpose(sumk, 0, 1)
    shared = mlp(B, cfg, params, p + ".shared_experts", res, cfg.moe_intermediate_size * cfg.n_shared_experts)
    return B.add(sumk, shared)
