"""Host-side logic of bench.py that needs no GPU: how a fixed job is spread over several GPUs."""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from conftest import cg

bench = importlib.import_module("bench")
synth = cg.synth


def test_parallelism_rule():
    small, big, moe = synth.LLAMA_32_1B, synth.LLAMA_3_8B, synth.QWEN3_30B_A3B
    # one GPU: nothing to choose
    assert bench.choose_parallelism("auto", small, 8, 1) == "tp"
    # a model whose decode step is bound by dependent latency keeps whole copies and splits the rows ...
    for world in (2, 4, 8):
        assert bench.choose_parallelism("auto", small, 8, world) == "dp"
    # ... unless the rows do not divide
    assert bench.choose_parallelism("auto", small, 8, 3) == "tp"
    # a model whose weight stream dominates is split
    for world in (2, 4, 8):
        assert bench.choose_parallelism("auto", big, 32, world) == "tp"
    # mixture-of-experts: experts and rows split when both divide
    assert bench.choose_parallelism("auto", moe, 8, 8) == "ep"
    assert bench.choose_parallelism("auto", moe, 8, 3) == "tp"
    # an explicit choice is kept
    for asked in ("tp", "dp", "ep"):
        assert bench.choose_parallelism(asked, small, 8, 2) == asked


def test_workloads_name_known_configurations():
    for name, (cfg_name, batch, prompt, decode) in bench.WORKLOADS.items():
        cfg = getattr(synth, cfg_name)
        assert batch >= 1 and prompt >= 1 and decode >= 1
        assert cfg.num_hidden_layers >= 1 and cfg.vocab_size > 0
        assert bench.dense_params_per_step(cfg) > 0
