"""Regenerates tests/golden/model_fixtures.json.

The reference is a Rust workspace that cannot be built in this environment, so these fixtures do
NOT come from the reference: they are outputs of the CPU restatement (oracle/) running the
reference's own op streams (catgrad-rs_b200/graphs/) on seeded synthetic checkpoints.  They pin
regressions of the restatement and give the GPU tests fixed numbers to hit; for whole models the
parity claim stays "unpinned" (no reference test holds logits or tokens).  The vectors that DO come
from the reference's tests are in tests/test_oracle_golden.py, each with its file:line.

    python tests/golden/make_golden.py        # rewrites the JSON next to this script
"""
import ctypes
import importlib
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
cg = importlib.import_module("catgrad-rs_b200")
synth, graphs = cg.synth, cg.graphs

QWEN_MOE = dict(name="qwen3-moe-small", hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, vocab_size=512, head_dim=64, arch="qwen3", rope_theta=1e6, num_local_experts=16,
                num_experts_per_tok=4, moe_intermediate_size=96, norm_topk_prob=True)


def oracle_backend():
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = ctypes.CDLL(path)
    lib.cgo_ctx_create.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]
    ctx = ctypes.c_void_p()
    assert lib.cgo_ctx_create(0, ctypes.byref(ctx)) == 0
    return cg.TraitBackend(lib, "cgo_", ctx)


def top(logits, n=8):
    idx = np.argsort(-logits, kind="stable")[:n]
    return {"index": [int(i) for i in idx], "value": [float(logits[i]) for i in idx]}


def tiny_llama(B):
    """The CPU-runnable benchmark configuration: prefill of 32 seeded ids, then 16 greedy decode steps."""
    cfg = synth.TINY_LLAMA
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, 0)}
    prompt = synth.make_tokens(cfg, 1, 32, seed=1)[0]
    tokens = graphs.llama.generate(B, cfg, params, prompt, 17)
    ids = np.asarray(prompt, dtype=np.uint32).reshape(1, -1)
    _, lg = graphs.llama.forward(B, cfg, params, B.from_numpy(ids), ids.shape[1], want_logits=True)
    last = B.to_numpy(lg)[0, -1]
    return {"config": cfg.name, "weights_seed": 0, "prompt_seed": 1, "prompt": [int(t) for t in prompt],
            "greedy_tokens": [int(t) for t in tokens], "prefill_last_logits_top8": top(last),
            "prefill_last_logits_abs_sum": float(np.abs(last).sum(dtype=np.float64))}


def qwen_moe(B):
    """Top-k expert ids of every sparse layer for a 24-token prompt (ids must be exact)."""
    cfg = synth.ModelConfig(**QWEN_MOE)
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, 0)}
    prompt = synth.make_tokens(cfg, 1, 24, seed=3)
    ids = []
    _, lg = graphs.qwen3.forward(B, cfg, params, B.from_numpy(prompt), 24, want_logits=True, expert_ids=ids)
    last = B.to_numpy(lg)[0, -1]
    return {"config": QWEN_MOE, "weights_seed": 0, "prompt_seed": 3,
            "expert_ids": [B.to_numpy(t).reshape(24, -1).astype(int).tolist() for t in ids],
            "last_logits_top8": top(last)}


def main():
    B = oracle_backend()
    out = {"generator": "oracle/ (CPU restatement) through catgrad-rs_b200/graphs; numpy " + np.__version__,
           "tiny_llama_f32": tiny_llama(B), "qwen3_moe_small_f32": qwen_moe(B)}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "model_fixtures.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
