"""Parity of the fused bf16 decoder at the benchmark configurations' own widths.

The other decoder tests run two-layer models a few hundred wide.  Here the checker (the CPU
restatement running the reference's op stream in f32 on the same bf16-rounded weights) and the
decoder meet at the real shapes: the whole Llama-3.2-1B-shaped model (16 layers, hidden 2048,
vocab 128 256), and slices of the first layers of the Gemma-2-2B, Qwen3-30B-A3B and Llama-3-8B
shapes (full width, full vocabulary, all 128 experts).  One prompt row is prefilled, then a few
decode steps are teacher-forced with the checker's tokens so both sides stay on one sequence.

What is asserted: the last-position logits agree within the stated bound at every step, and the
decoder's greedy token equals the checker's wherever the checker's top-1 / top-2 margin exceeds
twice the observed logit error.  The bound is relative to the logit scale (the largest |logit|
of the checker's row): 2.5e-2 of it.  The two-layer models of the other tests meet 2e-2 absolute
at a logit scale near 1; at these widths and depths the logits reach 4 and the rounding of every
activation to bf16 (2^-9 relative, once per GEMM input, through up to 16 layers of a random
network whose residual stream carries perturbations at unit gain) accumulates to 1.5-2 % of the
scale -- measured 7e-2 absolute on the 16-layer model -- while every greedy token still equals
the f32 run's.  What is reported (printed, and appended as a JSON line to the
file named by the environment variable CG_PARITY_REPORT when it is set): the largest logit
difference, the checker's margin at every step, and the number of steps at which the two greedy
tokens differ -- nothing is hidden behind an agreement threshold.
"""
import dataclasses
import json
import os
import time

import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
synth, graphs = cg.synth, cg.graphs


def forward_of(cfg):
    return {"llama": graphs.llama.forward, "qwen3": graphs.qwen3.forward, "gemma": graphs.gemma.forward}[cfg.arch]


def run_case(oracle, C, cfg, prompt_len, steps, tol):
    t_start = time.perf_counter()
    fwd = forward_of(cfg)
    dec = cg.Decoder(C, cfg, max_seq=prompt_len + steps + 2, max_batch=1)
    po = {}
    for name, w in synth.make_weights(cfg, 0):     # one pass: the same host array feeds both sides
        po[name] = oracle.from_numpy(w)
        dec.set_param(name, C.from_numpy(w))
    dec.finalize()
    row = list(synth.make_tokens(cfg, 1, prompt_len, seed=1)[0])
    lg = C.to_numpy(dec.prefill(C.from_numpy(np.uint32(row).reshape(1, -1)), want_logits=True))[0]
    report = {"config": cfg.name, "layers": cfg.num_hidden_layers, "prompt": prompt_len, "steps": [],
              "bound_relative_to_logit_scale": tol}
    for step in range(steps + 1):
        ids = np.asarray(row, dtype=np.uint32).reshape(1, -1)
        _, ref = fwd(oracle, cfg, po, oracle.from_numpy(ids), ids.shape[1], want_logits=True)
        want = oracle.to_numpy(ref)[0, -1]
        err = float(np.abs(lg - want).max())
        top2 = np.sort(want)[-2:]
        margin = float(top2[1] - top2[0])
        pick = len(want) - 1 - int(np.argmax(want[::-1]))   # last index on ties, like the reference
        mine = len(lg) - 1 - int(np.argmax(lg[::-1]))
        report["steps"].append({"position": len(row), "max_abs_err": err, "logit_scale": float(np.abs(want).max()),
                                "top1_top2_margin": margin, "checker_token": pick, "decoder_token": mine})
        row.append(pick)
        if step < steps:
            lg = C.to_numpy(dec.step_with(C.from_numpy(np.uint32([pick])), want_logits=True))[0]
    dec.close()
    report["max_abs_err"] = max(s["max_abs_err"] for s in report["steps"])
    report["token_disagreements"] = sum(s["checker_token"] != s["decoder_token"] for s in report["steps"])
    report["seconds"] = time.perf_counter() - t_start
    print("\nparity report:", json.dumps(report))
    path = os.environ.get("CG_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(report) + "\n")
    for s in report["steps"]:
        assert s["max_abs_err"] <= tol * max(1.0, s["logit_scale"]), s
        if s["top1_top2_margin"] > 2 * s["max_abs_err"]:
            assert s["checker_token"] == s["decoder_token"], s
    return report


def test_llama_1b_shape_whole_model(oracle, cuda_bf16):
    """Every layer of the configuration the benchmark is quoted on; 512-token prompt as there.
    bf16 logits within 2.5e-2 of the logit scale of the f32 run, identical greedy tokens."""
    run_case(oracle, cuda_bf16, synth.LLAMA_32_1B, prompt_len=512, steps=4, tol=2.5e-2)


def test_gemma2_2b_shape_four_layers(oracle, cuda_bf16):
    """Head size 256, GeGLU, (1 + gamma) norms, four norms per layer, both soft-caps, 256 000-entry
    tied vocabulary.  The window (4096) is longer than the prompt here; the windowed kernels are
    covered at a small window by the model-family tests."""
    cfg = dataclasses.replace(synth.GEMMA_2_2B, name="gemma-2-2b-shape-4layer", num_hidden_layers=4)
    run_case(oracle, cuda_bf16, cfg, prompt_len=256, steps=3, tol=2.5e-2)


def test_qwen3_moe_shape_two_layers(oracle, cuda_bf16):
    """All 128 experts at their real width with top-8 routing, per-head q/k norms, head size 128."""
    cfg = dataclasses.replace(synth.QWEN3_30B_A3B, name="qwen3-30b-a3b-shape-2layer", num_hidden_layers=2)
    run_case(oracle, cuda_bf16, cfg, prompt_len=48, steps=3, tol=2.5e-2)


def test_llama_8b_shape_four_layers(oracle, cuda_bf16):
    """Hidden 4096, FFN 14336, head size 128, untied 128 256-entry head."""
    cfg = dataclasses.replace(synth.LLAMA_3_8B, name="llama-3-8b-shape-4layer", num_hidden_layers=4)
    run_case(oracle, cuda_bf16, cfg, prompt_len=256, steps=3, tol=2.5e-2)
