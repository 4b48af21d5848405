"""Committed fixtures (tests/golden/model_fixtures.json, made by tests/golden/make_golden.py).

They are outputs of the CPU restatement, not of the reference (which cannot be built here):
CPU test -- the restatement still reproduces them (guards the checker itself against drift);
GPU tests -- the CUDA trait path reproduces the greedy tokens and expert ids exactly and the
logits within 1e-4 of the logit scale.
"""
import json
import os

import numpy as np
import pytest

from conftest import ROOT, cg

synth, graphs = cg.synth, cg.graphs
FIX = json.load(open(os.path.join(ROOT, "tests", "golden", "model_fixtures.json")))


def tiny_tokens(B):
    cfg = synth.TINY_LLAMA
    f = FIX["tiny_llama_f32"]
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, f["weights_seed"])}
    prompt = synth.make_tokens(cfg, 1, 32, seed=f["prompt_seed"])[0]
    assert [int(t) for t in prompt] == f["prompt"]  # the generator itself is part of the fixture
    toks = graphs.llama.generate(B, cfg, params, prompt, 17)
    ids = np.asarray(prompt, dtype=np.uint32).reshape(1, -1)
    _, lg = graphs.llama.forward(B, cfg, params, B.from_numpy(ids), 32, want_logits=True)
    return [int(t) for t in toks], B.to_numpy(lg)[0, -1]


def check_tiny(B, tol):
    f = FIX["tiny_llama_f32"]
    toks, last = tiny_tokens(B)
    assert toks == f["greedy_tokens"]
    top = f["prefill_last_logits_top8"]
    scale = float(np.abs(last).max())
    assert np.abs(last[top["index"]] - np.float32(top["value"])).max() <= tol * scale
    assert abs(float(np.abs(last).sum(dtype=np.float64)) - f["prefill_last_logits_abs_sum"]) <= tol * scale * last.size


def moe_ids(B):
    f = FIX["qwen3_moe_small_f32"]
    cfg = synth.ModelConfig(**f["config"])
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, f["weights_seed"])}
    prompt = synth.make_tokens(cfg, 1, 24, seed=f["prompt_seed"])
    ids = []
    _, lg = graphs.qwen3.forward(B, cfg, params, B.from_numpy(prompt), 24, want_logits=True, expert_ids=ids)
    return [B.to_numpy(t).reshape(24, -1).astype(int).tolist() for t in ids], B.to_numpy(lg)[0, -1]


def test_checker_reproduces_fixtures(oracle):
    check_tiny(oracle, 1e-6)
    ids, last = moe_ids(oracle)
    assert ids == FIX["qwen3_moe_small_f32"]["expert_ids"]


@pytest.mark.gpu
def test_cuda_trait_path_reproduces_fixtures(cuda):
    check_tiny(cuda, 1e-4)
    ids, last = moe_ids(cuda)
    f = FIX["qwen3_moe_small_f32"]
    assert ids == f["expert_ids"]  # top-k expert ids: exact
    top = f["last_logits_top8"]
    assert np.abs(last[top["index"]] - np.float32(top["value"])).max() <= 1e-4 * float(np.abs(last).max())
