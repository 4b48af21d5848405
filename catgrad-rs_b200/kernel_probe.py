"""Achieved HBM bandwidth of the memory-bound kernels, one at a time.

    python catgrad-rs_b200/kernel_probe.py [--iters N] [--once] [--decoder]

Each kernel runs on inputs larger than the L2 cache (126 MB on B200), so every iteration streams
from HBM; the time is taken with CUDA events on the library's stream and the figure printed is
algorithmic bytes (what the operation must read and write once) divided by that time, next to
the measured copy bandwidth it is compared with.  `--once` runs every kernel a single time after
one warm-up (the mode a profiler capture uses).  `--decoder` also runs a prefill and a few decode
steps of a 4-layer model of the benchmark's widths, which launches the kernels that only the
fused decoder uses (embedding gather, rope + cache append, partial arg-max, decode attention).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--decoder", action="store_true")
    args = ap.parse_args()
    iters = 1 if args.once else args.iters
    import torch
    cg = importlib.import_module("catgrad-rs_b200")
    if not torch.cuda.is_available():
        raise SystemExit("kernel_probe.py needs a CUDA device")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    C = cg.CudaBackend(0, cg.PREC_F32, stream=stream.cuda_stream)
    peak = 6650.0
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = float(json.load(open(p))["hbm_gbs"])

    def timed(fn):
        fn()
        C.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        C.sync()
        return e0.elapsed_time(e1) / iters

    rows, results = 32768, []
    H = 4096

    def report(name, kernel, nbytes, ms):
        gbs = nbytes / (ms * 1e-3) / 1e9
        results.append({"op": name, "kernel": kernel, "algorithmic_MB": nbytes / 1e6, "ms": ms, "GB_s": gbs, "frac_of_copy_peak": gbs / peak})
        print(f"{name:34s} {kernel:22s} {nbytes / 1e6:9.1f} MB {ms:8.4f} ms {gbs:8.1f} GB/s  {gbs / peak:5.2f} of {peak:.0f}", flush=True)

    x = C.randn((rows, H), 1)                      # 537 MB f32
    g = C.randn((H,), 2)
    report("rmsnorm f32 [32768, 4096]", "k_rmsnorm<0>", 2 * rows * H * 4, timed(lambda: C.fused_rmsnorm(x, g, 1e-5)))
    report("softmax f32 [32768, 4096]", "k_softmax", 2 * rows * H * 4, timed(lambda: C.fused_softmax(x)))
    y = C.randn((rows, H), 3)
    report("silu(gate) * up f32 [32768, 4096]", "k_act_mul_f32", 3 * rows * H * 4, timed(lambda: C.fused_act_mul(x, y, 0)))
    report("add f32 [32768, 4096] (eager op)", "k_binary", 3 * rows * H * 4, timed(lambda: C.add(x, y)))
    del y
    x4 = C.reshape(x, (8, 32, 4096, 128))          # [b, heads, s, d]
    report("rope f32 [8, 32, 4096, 128]", "k_rope_apply", 2 * rows * H * 4, timed(lambda: C.fused_rope(x4, 500000.0)))
    report("argmax f32 [32768, 4096] (eager op)", "k_reduce", rows * H * 4, timed(lambda: C.argmax(x)))
    report("sum f32 [32768, 4096] (eager op)", "k_reduce", rows * H * 4, timed(lambda: C.sum(x)))
    ids = C.from_numpy(np.random.Generator(np.random.PCG64(4)).integers(0, rows, size=(rows,)).astype(np.uint32))
    report("index rows f32 [32768 of 32768, 4096]", "k_index", 2 * rows * H * 4, timed(lambda: C.index(x, 0, ids)))
    del x, x4
    if args.decoder:
        import dataclasses
        synth = cg.synth
        Cb = cg.CudaBackend(0, cg.PREC_BF16, stream=stream.cuda_stream)
        for name, base, B, S in (("llama-1b-4layer", synth.LLAMA_32_1B, 8, 512), ("qwen3moe-4layer", synth.QWEN3_30B_A3B, 8, 256)):
            cfg = dataclasses.replace(base, name=name, num_hidden_layers=4)
            dec = cg.Decoder(Cb, cfg, max_seq=S + 8, max_batch=B)
            dec.load_random(cfg, 0)
            prompt = Cb.from_numpy(synth.make_tokens(cfg, B, S, seed=1))
            ms = timed(lambda: (dec.prefill(prompt), dec.decode(4)))
            print(f"{name}: prefill {B}x{S} + 4 decode steps {ms:.3f} ms", flush=True)
            dec.close()
    print(json.dumps({"peak_GB_s": peak, "results": results}))


if __name__ == "__main__":
    main()
