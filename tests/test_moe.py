"""Mixture-of-experts block (catgrad-llm/src/models/qwen3.rs:64-133) on the fused path.

The checker replays the reference's op stream (softmax -> topk -> renorm, then per slot a
gathered expert matrix per token and batched matmuls); the CUDA path groups the (token, slot)
pairs by expert and runs grouped tensor-core GEMMs.  Expert ids must be identical; outputs
agree to bf16-operand accuracy (inputs are made bf16-representable, so only the rounding of the
intermediate act(gate) * up to bf16 and the f32 summation order differ).
"""
import dataclasses

import numpy as np
import pytest

from conftest import cg

synth, graphs = cg.synth, cg.graphs


def moe_case(seed, S, H, E, Fe):
    rng = np.random.Generator(np.random.PCG64(seed))
    r = lambda *sh, s=1.0: synth.bf16_round((rng.standard_normal(sh, dtype=np.float32) * np.float32(s)).astype(np.float32))
    return {
        "x": r(1, S, H),
        "m.gate.weight": r(E, H, s=0.3),
        "m.experts.gate_proj.weight": r(E, Fe, H, s=0.1),
        "m.experts.up_proj.weight": r(E, Fe, H, s=0.1),
        "m.experts.down_proj.weight": r(E, H, Fe, s=0.1),
    }


# (tokens, hidden, experts, expert width, top-k, renormalise): the token counts walk through
# every tile width of the grouped GEMM (16, 32, 64, 128 tokens) and ragged group sizes
CASES = [
    (1, 64, 8, 32, 2, True),
    (5, 128, 16, 96, 4, True),
    (37, 128, 16, 96, 4, False),
    (40, 128, 4, 64, 2, True),
    (70, 128, 4, 64, 2, True),
    (300, 128, 4, 256, 2, True),
    (33, 256, 128, 64, 8, True),
]


@pytest.mark.gpu
@pytest.mark.parametrize("S,H,E,Fe,k,renorm", CASES)
def test_fused_moe_matches_op_stream(oracle, cuda_bf16, S, H, E, Fe, k, renorm):
    C = cuda_bf16
    w = moe_case(S * 7 + E, S, H, E, Fe)
    cfg = synth.ModelConfig("moe-unit", H, 2 * H, 1, 2, 2, 64, head_dim=64, arch="qwen3", num_local_experts=E,
                            num_experts_per_tok=k, moe_intermediate_size=Fe, norm_topk_prob=renorm)
    po = {n: oracle.from_numpy(a) for n, a in w.items() if n != "x"}
    want, want_ids = graphs.qwen3.moe(oracle, cfg, po, "m", oracle.from_numpy(w["x"]))
    want = oracle.to_numpy(want).reshape(S, H)
    want_ids = oracle.to_numpy(want_ids).reshape(S, k)
    up = lambda n: C.from_numpy(w[n])
    got, ids = C.fused_moe(C.from_numpy(w["x"].reshape(S, H)), up("m.gate.weight"), up("m.experts.gate_proj.weight"),
                           up("m.experts.up_proj.weight"), up("m.experts.down_proj.weight"), k, renorm, 0)
    assert (C.to_numpy(ids) == want_ids).all()
    got = C.to_numpy(got)
    scale = float(np.abs(want).max())
    assert np.abs(got - want).max() <= 1e-2 * scale + 1e-6, float(np.abs(got - want).max() / scale)


@pytest.mark.gpu
@pytest.mark.parametrize("S,H,E,Fe,k,renorm", [CASES[1], CASES[5]])
def test_fused_moe_f32_router(oracle, cuda, S, H, E, Fe, k, renorm):
    """On an f32-precision context the router matrix stays f32 and the per-token f32 router
    kernel runs instead of the split-precision tensor-core router."""
    C = cuda
    w = moe_case(S * 11 + E, S, H, E, Fe)
    cfg = synth.ModelConfig("moe-unit", H, 2 * H, 1, 2, 2, 64, head_dim=64, arch="qwen3", num_local_experts=E,
                            num_experts_per_tok=k, moe_intermediate_size=Fe, norm_topk_prob=renorm)
    po = {n: oracle.from_numpy(a) for n, a in w.items() if n != "x"}
    want, want_ids = graphs.qwen3.moe(oracle, cfg, po, "m", oracle.from_numpy(w["x"]))
    up = lambda n: C.from_numpy(w[n])
    got, ids = C.fused_moe(C.from_numpy(w["x"].reshape(S, H)), up("m.gate.weight"), up("m.experts.gate_proj.weight"),
                           up("m.experts.up_proj.weight"), up("m.experts.down_proj.weight"), k, renorm, 0)
    assert (C.to_numpy(ids) == oracle.to_numpy(want_ids).reshape(S, k)).all()
    want = oracle.to_numpy(want).reshape(S, H)
    assert np.abs(C.to_numpy(got) - want).max() <= 1e-2 * float(np.abs(want).max()) + 1e-6


@pytest.mark.gpu
def test_fused_moe_ties_and_errors(cuda_bf16):
    C = cuda_bf16
    S, H, E, Fe = 3, 64, 8, 32
    w = moe_case(1, S, H, E, Fe)
    w["m.gate.weight"][:] = 0  # every expert has the same probability: the k lowest ids win
    up = lambda n: C.from_numpy(w[n])
    args = [up("m.gate.weight"), up("m.experts.gate_proj.weight"), up("m.experts.up_proj.weight"), up("m.experts.down_proj.weight")]
    _, ids = C.fused_moe(C.from_numpy(w["x"].reshape(S, H)), *args, 3, True, 0)
    assert (C.to_numpy(ids) == np.tile(np.uint32([0, 1, 2]), (S, 1))).all()
    with pytest.raises(cg.BackendPanic):
        C.fused_moe(C.from_numpy(w["x"].reshape(S, H)[:, :32].copy()), *args, 2, True, 0)  # hidden size mismatch
    with pytest.raises(cg.BackendPanic):
        C.fused_moe(C.from_numpy(w["x"].reshape(S, H)), *args, 9, True, 0)  # more slots than experts
    out, ids = C.fused_moe(C.from_numpy(np.zeros((0, H), np.float32)), *args, 2, True, 0)  # no tokens
    assert out.shape == (0, H) and ids.shape == (0, 2)
