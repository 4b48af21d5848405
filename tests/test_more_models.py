"""The remaining catgrad-llm model graphs on the trait path: GPT-2 (LayerNorm with bias, learned
positions, biased linear layers with pre-transposed weights, `chunk`), Granite (dense and
mixture-of-experts, four scalar multipliers, top-k before softmax) and the DeepSeek
mixture-of-experts block (sigmoid router, group-limited top-k built from `eq` / `sum` masks,
shared experts).  Each graph is the reference's op stream (catgrad-llm/src/models/gpt2.rs,
granite.rs, deepseek.rs:13-164) replayed on the CUDA backend and on the CPU checker in f32:
logits within 1e-4 of the logit scale, arg-max tokens and expert ids bit-exact.
"""
from types import SimpleNamespace

import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
graphs, synth = cg.graphs, cg.synth


def random_params(shapes, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name in sorted(shapes):
        shp = shapes[name]
        if len(shp) == 1:
            base = 0.0 if name.endswith(".bias") else 1.0
            out[name] = (base + rng.standard_normal(shp, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
        else:
            out[name] = rng.standard_normal(shp, dtype=np.float32) * np.float32(0.05)
    return out


def both(oracle, cuda, fn):
    res = []
    for B in (oracle, cuda):
        res.append(fn(B))
    return res


GPT2 = SimpleNamespace(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=512,
                       max_position_embeddings=64, layer_norm_epsilon=1e-5)


def test_gpt2_op_stream_parity(oracle, cuda):
    host = random_params(graphs.gpt2.param_shapes(GPT2), 1)
    ids = np.random.Generator(np.random.PCG64(2)).integers(0, GPT2.vocab_size, size=(1, 19)).astype(np.uint32)

    def run(B):
        params = {n: B.from_numpy(w) for n, w in host.items()}
        y, lg = graphs.gpt2.forward(B, GPT2, params, B.from_numpy(ids), 19, want_logits=True)
        return B.to_vec(y), B.to_numpy(lg)

    (yo, lo), (yc, lc) = both(oracle, cuda, run)
    assert np.abs(lc - lo).max() <= 1e-4 * np.abs(lo).max()
    np.testing.assert_array_equal(yo, yc)


GRANITE = SimpleNamespace(hidden_size=128, intermediate_size=192, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, vocab_size=512, rms_norm_eps=1e-5, rope_theta=10000.0,
                          attention_multiplier=0.0078125, residual_multiplier=0.22, embedding_multiplier=12.0,
                          num_experts_per_tok=0, num_local_experts=0)
GRANITE_MOE = SimpleNamespace(**{**GRANITE.__dict__, "num_experts_per_tok": 2, "num_local_experts": 8, "intermediate_size": 64})


@pytest.mark.parametrize("cfg", [GRANITE, GRANITE_MOE], ids=["dense", "moe"])
def test_granite_op_stream_parity(oracle, cuda, cfg):
    host = random_params(graphs.granite.param_shapes(cfg), 3)
    ids = np.random.Generator(np.random.PCG64(4)).integers(0, cfg.vocab_size, size=(1, 17)).astype(np.uint32)

    def run(B):
        params = {n: B.from_numpy(w) for n, w in host.items()}
        eids = []
        y, lg = graphs.granite.forward(B, cfg, params, B.from_numpy(ids), 17, want_logits=True, expert_ids=eids)
        return B.to_vec(y), B.to_numpy(lg), [B.to_numpy(e) for e in eids]

    (yo, lo, eo), (yc, lc, ec) = both(oracle, cuda, run)
    assert np.abs(lc - lo).max() <= 1e-4 * np.abs(lo).max()
    np.testing.assert_array_equal(yo, yc)
    assert len(eo) == len(ec) == (cfg.num_hidden_layers if cfg.num_experts_per_tok else 0)
    for a, b in zip(eo, ec):
        np.testing.assert_array_equal(a, b)


DEEPSEEK = SimpleNamespace(hidden_size=96, num_local_experts=16, n_group=8, topk_group=2, num_experts_per_tok=4,
                           norm_topk_prob=True, routed_scaling_factor=2.5, moe_intermediate_size=48, n_shared_experts=2)


def test_deepseek_router_and_expert_block_parity(oracle, cuda):
    cfg = DEEPSEEK
    H, E, Fe = cfg.hidden_size, cfg.num_local_experts, cfg.moe_intermediate_size
    shapes = {"mlp.gate.weight": (E, H), "mlp.gate.e_score_correction_bias": (E,),
              "mlp.experts.gate_proj.weight": (E, Fe, H), "mlp.experts.up_proj.weight": (E, Fe, H),
              "mlp.experts.down_proj.weight": (E, H, Fe),
              "mlp.shared_experts.gate_proj.weight": (Fe * cfg.n_shared_experts, H),
              "mlp.shared_experts.up_proj.weight": (Fe * cfg.n_shared_experts, H),
              "mlp.shared_experts.down_proj.weight": (H, Fe * cfg.n_shared_experts)}
    host = random_params(shapes, 5)
    host["mlp.gate.e_score_correction_bias"] = (host["mlp.gate.e_score_correction_bias"] - 1.0).astype(np.float32)
    x = np.random.Generator(np.random.PCG64(6)).standard_normal((1, 13, H), dtype=np.float32)

    def run(B):
        params = {n: B.from_numpy(w) for n, w in host.items()}
        vals, idx = graphs.deepseek.moe_topk_router(B, cfg, params, "mlp.gate", B.from_numpy(x))
        y = graphs.deepseek.moe(B, cfg, params, "mlp", B.from_numpy(x))
        return B.to_numpy(vals), B.to_numpy(idx), B.to_numpy(y)

    (vo, io, yo), (vc, ic, yc) = both(oracle, cuda, run)
    np.testing.assert_array_equal(io, ic)                      # expert ids: bit-exact
    np.testing.assert_allclose(vc, vo, rtol=2e-6, atol=0)
    # the mask leaves exactly topk_group groups eligible: chosen experts come from at most that many groups
    per_group = cfg.num_local_experts // cfg.n_group
    assert all(len(set(row // per_group)) <= cfg.topk_group for row in io)
    assert np.abs(yc - yo).max() <= 1e-4 * np.abs(yo).max()
