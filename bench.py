"""Benchmark of the hot path: greedy generation on a Llama-3.2-1B-shaped decoder.

One "step" is one whole job on synthetic data: prefill of B x PROMPT token ids followed by
DECODE greedy steps, for all B rows.  The metric is tokens per second over prompt and
generated tokens.  `value` is timed on the device with the token ids already resident in
HBM; `e2e` is the same job through the host-buffer entry point (ids copied host->device, all
steps enqueued back to back, the token history [B, 1 + DECODE] read back device->host in one
strided copy at the end).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by torchrun, one rank per GPU.  `--parallelism` says how the fixed job is spread:
tp = the model is tensor-parallel over the N ranks (decode steps exchange the partial products of
the two row-split projections of every layer through mapped peer memory, plain stores and flags,
no collective call; prefill uses an NCCL all-reduce with a bf16 payload); dp = whole model per
GPU, batch rows split, no collective; ep = experts and rows split, all-gather + reduce-scatter on
every expert layer.  The default picks by model size (choose_parallelism).

`--impl reference` times the CPU restatement of the reference's ndarray backend running the
reference's own op stream (one full forward per generated token, no KV cache) on the host
cores, on a bounded sample of the same job.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode+prefill tok/s, Llama-3.2-1B shape"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples every 200 ms while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                c = [x.strip() for x in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1]))
                    mx.append(float(c[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


# name -> (model shape in synth, batch, prompt, decode steps)
WORKLOADS = {
    "llama1b": ("LLAMA_32_1B", 8, 512, 128),
    "llama1b-b1": ("LLAMA_32_1B", 1, 512, 128),
    "gemma2": ("GEMMA_2_2B", 4, 2048, 128),
    "qwen3moe": ("QWEN3_30B_A3B", 8, 1024, 64),
    "llama8b": ("LLAMA_3_8B", 32, 4096, 256),
}


def dense_params_per_step(cfg) -> int:
    """Weights every decode step streams whatever the routing: all dense linear layers and the LM
    head (expert matrices are excluded: how many a step touches depends on the router)."""
    H, F, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    total = cfg.vocab_size * H
    for i in range(cfg.num_hidden_layers):
        total += H * (nh * d) + 2 * H * (nkv * d) + (nh * d) * H
        sparse = cfg.num_local_experts > 1 and (i + 1) % cfg.decoder_sparse_step == 0
        total += cfg.num_local_experts * H if sparse else 3 * H * F
    return total


def reference_job_seconds(t_forward: float, prompt: int, decode: int, batch: int) -> float:
    """Cost of the whole job on the reference's driver from one measured forward of `prompt`
    tokens: every generated token is a full forward over all tokens so far
    (catgrad-llm/examples/llama/main.rs:118-127), rows one at a time (the graphs are batch-1).
    Forward cost is taken as linear in the length (the linear layers dominate)."""
    lengths = [prompt + t for t in range(decode + 1)]
    return batch * sum(t_forward * n / prompt for n in lengths)


def run_reference_sample(cg, cfg, prompt_len: int, threads: int = 0):
    """One full forward of one row through the reference op stream on the CPU checker."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = ctypes.CDLL(path)
    lib.cgo_ctx_create.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]
    lib.cgo_ctx_threads.argtypes = [ctypes.c_void_p]
    ctx = ctypes.c_void_p()
    assert lib.cgo_ctx_create(threads, ctypes.byref(ctx)) == 0
    O = cg.TraitBackend(lib, "cgo_", ctx)
    cores = int(lib.cgo_ctx_threads(ctx))
    params = {n: O.from_numpy(w) for n, w in cg.synth.make_weights(cfg, 0)}
    ids = cg.synth.make_tokens(cfg, 1, prompt_len, seed=1)

    def forward():
        t0 = time.perf_counter()
        y = cg.graphs.llama.forward(O, cfg, params, O.from_numpy(ids), prompt_len)
        O.to_vec(y)
        return time.perf_counter() - t0

    return forward, cores


def torch_cpu_kv_baseline(cg, cfg, prompt_len: int, decode_steps: int, batch: int, sample_steps: int = 6):
    """A second CPU baseline, with the optimisation the reference's interpreter path lacks: a KV
    cache.  The same model (f32 weights, all host cores, torch CPU matmuls) runs one row's prompt
    in one forward and then `sample_steps` single-token steps against the cache; the job is
    estimated as batch x (prefill + decode_steps x mean step).  Not the reference's algorithm
    (which recomputes the whole sequence per token) -- it shows what a well-built CPU runner of the
    same model would do on this host."""
    import torch
    torch.manual_seed(0)
    H, F, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    nh, nkv, d, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size
    g = torch.Generator().manual_seed(0)
    W = lambda o, i: torch.randn(o, i, generator=g) * 0.02
    layers = [dict(q=W(nh * d, H), k=W(nkv * d, H), v=W(nkv * d, H), o=W(H, nh * d), gate=W(F, H), up=W(F, H), down=W(H, F))
              for _ in range(L)]
    emb = W(V, H)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2).float() / d))

    def rope(x, pos0):
        t = torch.arange(pos0, pos0 + x.shape[2]).float()[:, None] * inv[None, :]
        cos, sin = torch.cat([t.cos(), t.cos()], -1), torch.cat([t.sin(), t.sin()], -1)
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return x * cos + torch.cat([-x2, x1], -1) * sin

    def norm(x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)

    def forward(ids, cache, pos0):
        x = emb[ids][None]
        S = x.shape[1]
        for li, Lw in enumerate(layers):
            h = norm(x)
            q = (h @ Lw["q"].T).view(1, S, nh, d).transpose(1, 2)
            k = (h @ Lw["k"].T).view(1, S, nkv, d).transpose(1, 2)
            v = (h @ Lw["v"].T).view(1, S, nkv, d).transpose(1, 2)
            q, k = rope(q, pos0), rope(k, pos0)
            if cache[li] is not None:
                k, v = torch.cat([cache[li][0], k], 2), torch.cat([cache[li][1], v], 2)
            cache[li] = (k, v)
            a = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(nh // nkv, 1), v.repeat_interleave(nh // nkv, 1),
                                                                 is_causal=S > 1)
            x = x + a.transpose(1, 2).reshape(1, S, nh * d) @ Lw["o"].T
            h = norm(x)
            x = x + (torch.nn.functional.silu(h @ Lw["gate"].T) * (h @ Lw["up"].T)) @ Lw["down"].T
        return int((norm(x[:, -1]) @ emb.T).argmax())

    with torch.no_grad():
        ids = torch.randint(0, V, (prompt_len,), generator=g)
        cache = [None] * L
        t0 = time.perf_counter()
        tok = forward(ids, cache, 0)
        t_prefill = time.perf_counter() - t0
        t0 = time.perf_counter()
        for i in range(sample_steps):
            tok = forward(torch.tensor([tok]), cache, prompt_len + i)
        t_step = (time.perf_counter() - t0) / sample_steps
    job = batch * (t_prefill + decode_steps * t_step)
    return {"value": batch * (prompt_len + decode_steps) / job, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "torch-cpu-f32-kv-cache",
            "sample": f"one row: prefill of {prompt_len} tokens in one forward ({t_prefill:.2f} s) and {sample_steps} cached single-token steps "
                      f"({t_step * 1e3:.0f} ms each); job = {batch} rows x (prefill + {decode_steps} steps), estimated from those"}


def choose_parallelism(asked: str, cfg, batch: int, world: int) -> str:
    """How a fixed job is spread over `world` GPUs.  A decode step costs (weight bytes this GPU
    streams) / (HBM bandwidth) plus a per-layer chain of small dependent kernels that sharding does
    not shorten and that tensor parallelism lengthens by two cross-GPU hand-overs per layer.  Where
    the first term dominates (dense weights of 8 GB and more per step: the 8B shape) the model is
    split (tp).  Where it does not (the 1B shape: 2.5 GB, 0.38 ms of a 0.9 ms step) every GPU keeps
    the whole model and takes its share of the batch rows (dp): nothing crosses NVLink on the data
    path, prefill divides by the number of GPUs and decode steps run on fewer rows.  Mixture-of-
    experts models split the experts and the rows (ep).  Measured on the 1B shape: one GPU 45.2 k
    tok/s; two GPUs dp 47.9 k, tp 32.8 k; four GPUs dp 51.1 k, tp 30.6 k."""
    if world == 1 or asked != "auto":
        return asked if asked != "auto" else "tp"
    rows_split = batch % world == 0
    if cfg.num_local_experts > 1:
        return "ep" if rows_split and cfg.num_local_experts % world == 0 else "tp"
    return "tp" if 2 * dense_params_per_step(cfg) >= 8e9 or not rows_split else "dp"


def check_tokens(cg, C, dec, cfg, prompt, job_tokens, T, rank, world, local, host_weights=True):
    """Compare the token history [B, 1 + T] the timed job produced with an independent run that
    is teacher-forced with those tokens (so one flipped near-tie does not cascade): at one GPU
    the same decoder stepping one kernel per operation, eagerly, one step at a time; under tensor
    parallelism a complete one-GPU decoder that rank 0 builds next to its shard.  Reports the
    fraction of equal tokens and where they differ."""
    if rank != 0 or job_tokens is None:
        return None
    B = prompt.shape[0]
    if world == 1:
        other, vs = dec, "the same decoder run eagerly, one kernel per operation, one step per call"
    else:
        other = cg.Decoder(C, cfg, max_seq=prompt.shape[1] + T + 1, max_batch=B, tp_rank=0, tp_world=1)
        if host_weights:
            other.load(cg.synth.make_weights(cfg, 0))
        else:
            other.load_random(cfg, 0)   # the same device-drawn checkpoint the job used
        vs = "a one-GPU (tp_world = 1) decoder built by rank 0 on its own GPU"
    try:
        other.reset()
        other.prefill(C.from_numpy(prompt))
        for i in range(T):
            other.step_with(C.from_numpy(np.ascontiguousarray(job_tokens[:, i])))
        mine = other.tokens()
    finally:
        if world > 1:
            other.close()
    eq = mine == job_tokens
    bad = np.argwhere(~eq)
    return {"tokens_equal_frac": float(eq.mean()), "vs": vs, "compared": int(eq.size), "disagreements": int((~eq).sum()),
            "first_disagreements_row_step": [[int(r), int(c)] for r, c in bad[:8]],
            "how": "teacher-forced with the job's tokens; every step's greedy pick compared"}


def trait_path(cg, C, cfg, args, B, S, workload):
    """Prefill through the trait methods alone: the model graph's op stream (one row at a time: the
    graphs are batch-1), on a bf16-precision context, eagerly and with the calls recorded and fused
    ("lazy").  Prints one JSON line; `value` is the recorded path's prompt tokens per second."""
    import torch
    synth, graphs = cg.synth, cg.graphs
    fwd = {"llama": graphs.llama.forward, "qwen3": graphs.qwen3.forward, "gemma": graphs.gemma.forward}[cfg.arch]
    params = {n: C.from_numpy(w) for n, w in synth.make_weights(cfg, 0)}
    prompt = synth.make_tokens(cfg, B, S, seed=1)
    rows = [C.from_numpy(prompt[b:b + 1]) for b in range(B)]

    def job():
        return [C.to_vec(fwd(C, cfg, params, r, S))[-1] for r in rows]

    out = {}
    for mode in ("eager", "recorded"):
        C.set_option("lazy", 1 if mode == "recorded" else 0)
        for _ in range(max(args.warmup, 1)):
            toks = job()
        C.sync()
        n0 = C.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            toks = job()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        out[mode] = {"ms_per_job": ms, "prefill_tok_s": B * S / (ms * 1e-3), "launches_per_row": (C.launch_count() - n0) / args.steps / B,
                     "next_tokens": [int(t) for t in toks]}
    # What the two modes disagree by (not timed): last-position logits of row 0.  On a bf16 context
    # every GEMM input is rounded to bf16, so the last-bit differences of the fused f32 kernels
    # flip roundings and reach the logits at the bf16 level; near-ties of a random-weight model
    # then pick another token, which `same_next_tokens` counts without judging.
    lg = {}
    for mode in ("eager", "recorded"):
        C.set_option("lazy", 1 if mode == "recorded" else 0)
        lg[mode] = np.asarray(C.to_vec(fwd(C, cfg, params, rows[0], S, want_logits=True)[1]), dtype=np.float32).reshape(S, -1)[-1]
    top2 = np.sort(lg["eager"])[-2:]
    logit_cmp = {"max_abs_diff": float(np.abs(lg["eager"] - lg["recorded"]).max()), "logit_scale": float(np.abs(lg["eager"]).max()),
                 "eager_top1_top2_margin": float(top2[1] - top2[0])}
    C.set_option("lazy", 0)
    # Generation through the trait methods: the reference's serving loop with an explicit KV cache
    # (catgrad-llm/src/run.rs:219-305) for ONE row -- the prompt in one call, then one token per
    # call, the cache tensors handed from call to call.
    gen = None
    if cfg.arch == "llama":
        T = min(args.decode, 32)
        gen = {}
        for mode in ("eager", "recorded"):
            C.set_option("lazy", 1 if mode == "recorded" else 0)
            res = None
            for it in range(2):  # first pass warms up
                runner = graphs.llama_kv.KVRunner(C, cfg, params, S + T + 8)
                stream = iter(runner.complete([int(t) for t in prompt[0]]))
                C.sync()
                e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                n0 = C.launch_count()
                e[0].record()
                toks = [next(stream)]
                e[1].record()
                n1 = C.launch_count()
                toks += [next(stream) for _ in range(T)]
                e[2].record()
                torch.cuda.synchronize()
                res = {"prefill_ms": e[0].elapsed_time(e[1]), "ms_per_token": e[1].elapsed_time(e[2]) / T,
                       "decode_tok_s": 1e3 * T / e[1].elapsed_time(e[2]), "launches_per_token": (C.launch_count() - n1) / T,
                       "launches_prefill": n1 - n0, "tokens": toks}
            gen[mode] = res
        C.set_option("lazy", 0)
        gen["same_tokens_frac"] = float(np.mean([a == b for a, b in zip(gen["eager"]["tokens"], gen["recorded"]["tokens"])]))
        gen["what"] = f"one row: {S}-token prompt in one call, then {T} single-token calls with the cache tensors passed along"
        for mode in ("eager", "recorded"):
            gen[mode]["tokens"] = gen[mode]["tokens"][:8]
    print(json.dumps({
        "generation": gen,
        "metric": "prefill tok/s through the trait methods, Llama-3.2-1B shape", "value": out["recorded"]["prefill_tok_s"], "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": out["recorded"]["ms_per_job"], "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "config": {"workload": workload + " (prefill only, rows one at a time)", "path": "trait"},
        "eager": out["eager"], "recorded": out["recorded"],
        "same_next_tokens": int(sum(a == b for a, b in zip(out["eager"]["next_tokens"], out["recorded"]["next_tokens"]))),
        "rows": B, "last_position_logits_row0": logit_cmp}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama1b", choices=sorted(WORKLOADS),
                    help="llama1b is the configuration the metric is quoted on; the others are the remaining "
                         "model shapes at their own batch / prompt / decode sizes")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=0)
    ap.add_argument("--decode", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "tp", "dp", "ep"],
                    help="with several GPUs: tp = the model is tensor-parallel over the ranks; dp = every rank holds the whole model and runs its share of the batch rows, no "
                         "collective on the data path (what pays for a model this small: its decode step is bound by dependent latency, not bytes); ep (mixture-of-experts "
                         "workloads) = data-parallel attention with the experts split over the ranks, rows all-gathered and expert "
                         "sums reduce-scattered on every expert layer; auto (default) = the fastest of these for the model and batch by "
                         "the rule in choose_parallelism(): tp where the weight stream dominates a decode step, rows split otherwise")
    ap.add_argument("--path", default="decoder", choices=["decoder", "trait"],
                    help="decoder (default): the fused KV-cached runner, the line the metric is quoted on; trait: the "
                         "reference's unchanged op stream through the 28 trait methods, prefill only, eager and recorded")
    ap.add_argument("--small", action="store_true", help="a 4-layer model of the same widths (profiling captures)")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE",
                    help="library switch (cg_set_option), e.g. fa=0; for experiments, not for the reported line")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours" and not args.small:
        args.warmup = 3

    cg = importlib.import_module("catgrad-rs_b200")
    synth = cg.synth
    import dataclasses
    cfg_name, B0, S0, T0 = WORKLOADS[args.workload]
    cfg = getattr(synth, cfg_name)
    args.batch, args.prompt, args.decode = args.batch or B0, args.prompt or S0, args.decode or T0
    headline = args.workload == "llama1b"
    if args.small:
        cfg = dataclasses.replace(cfg, name=cfg.name + "-4layer", num_hidden_layers=4)
    B, S, T = args.batch, args.prompt, args.decode
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    workload = f"{cfg.name} bf16, batch {B}, prompt {S}, {T} greedy decode steps"
    tokens_per_job = B * (S + T)

    if args.impl == "reference":
        if rank != 0:
            return
        forward, cores = run_reference_sample(cg, cfg, S)
        for _ in range(max(args.warmup, 0)):
            forward()
        ts = [forward() for _ in range(max(args.steps, 1))]
        t_fwd = float(np.mean(ts))
        job = reference_job_seconds(t_fwd, S, T, B)
        val = tokens_per_job / job
        sample = (f"one full forward of 1 of {B} rows at {S} tokens per step ({t_fwd:.2f} s); the job "
                  f"({B} rows x {T + 1} forwards of {S}..{S + T} tokens, no KV cache) is extrapolated linearly in length; "
                  f"the reference's own ndarray build is single-threaded, this port uses {cores} threads")
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": job * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "global_batch": B, "prompt": S, "decode": T, "parallelism": "cpu"},
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # a named stream shared with torch, so torch.cuda.Event brackets the library's work
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    C = cg.CudaBackend(local, cg.PREC_BF16, stream=tstream.cuda_stream)
    for kv in args.opt:
        name, _, val = kv.partition("=")
        C.set_option(name, int(val))
    par = choose_parallelism(args.parallelism, cfg, B, world)
    ep = world > 1 and par == "ep"
    dp = world > 1 and par in ("dp", "ep")   # rows are split over the ranks in both
    if dp and B % world:
        raise SystemExit(f"--parallelism dp needs the batch ({B}) to divide by the ranks ({world})")
    tpw, tpr = (1, 0) if dp else (world, rank)   # tensor-parallel degree and place of this rank's decoder
    Bl = B // world if dp else B                 # rows this rank runs
    if world > 1 and (ep or not dp):
        importlib.import_module("catgrad-rs_b200.tp").init_comm(C, rank, world)
        mapped, why = C.peer_exchange()
        collective = "decode: partial products pushed over mapped peer memory, no collective call; prefill: NCCL" if mapped \
            else "NCCL all-reduce / all-gather (peer mapping unavailable: " + why + ")"

    if args.path == "trait":
        return trait_path(cg, C, cfg, args, B, S, workload)

    dec = cg.Decoder(C, cfg, max_seq=S + T + 1, max_batch=Bl, tp_rank=tpr, tp_world=tpw,
                     ep_rank=rank if ep else 0, ep_world=world if ep else 1)
    if headline:
        dec.load(synth.make_weights(cfg, 0))
        generator = f"numpy {np.__version__} PCG64, weights seed 0 N(0,0.02) rounded to bf16, ids seed 1"
    else:
        dec.load_random(cfg, 0)  # tens of GB: drawn on the device instead of crossing the host link
        generator = "weights N(0,0.02) from the library's counter-based device generator (seed 0), ids numpy PCG64 seed 1"
    prompt = synth.make_tokens(cfg, B, S, seed=1)
    if dp:
        prompt = np.ascontiguousarray(prompt[rank * Bl:(rank + 1) * Bl])   # this rank's rows of the job
    prompt_dev = C.from_numpy(prompt)
    C.sync()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def job_device():
        dec.prefill(prompt_dev)
        dec.decode(T)

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(args.warmup):
        job_device()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = C.launch_count()
    ms_total = timed(job_device, args.steps)
    launches = C.launch_count() - launches0
    # the host-buffer path: same job through cg_decoder_generate
    out_tokens = None

    def job_host():
        nonlocal out_tokens
        out_tokens = dec.generate(prompt, T)

    job_host()
    ms_e2e = timed(job_host, args.steps)
    clocks = sampler.stop()

    # what was timed is checked: the job's greedy tokens against an independent run
    token_check = check_tokens(cg, C, dec, cfg, prompt, out_tokens, T, rank, world if ep else tpw, local, headline)
    if dist is not None:
        dist.barrier()

    # phase split and the kernel-level roofline, measured live
    ms_prefill = timed(lambda: dec.prefill(prompt_dev), args.steps) / args.steps
    dec.prefill(prompt_dev)
    dec.decode(1)
    ms_decode = timed(lambda: dec.decode(T - 1), 1) / max(T - 1, 1)
    gemm_ms, gemm_launches = dec.time_gemms(Bl, 20)
    peak, peak_kind = measured_peaks()
    weight_bytes = 2 * dense_params_per_step(cfg) / tpw
    kv_bytes = Bl * synth.kv_bytes_per_token(cfg) * (S + T / 2) / tpw
    expert_bytes = 0.0
    if cfg.num_local_experts > 1:
        # expected distinct experts a step of B tokens touches under uniform routing, per sparse layer
        E, k = cfg.num_local_experts, cfg.num_experts_per_tok
        distinct = E * (1.0 - (1.0 - 1.0 / E) ** (Bl * k))
        sparse_layers = sum(1 for i in range(cfg.num_hidden_layers) if (i + 1) % cfg.decoder_sparse_step == 0)
        expert_bytes = sparse_layers * distinct * 3 * cfg.moe_intermediate_size * cfg.hidden_size * 2 / (world if ep else tpw)
    achieved = weight_bytes / (gemm_ms * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath) and world == 1 and not args.small:
        traffic = json.load(open(tpath)).get("decode_gemm_sweep_dram_bytes")

    value = tokens_per_job * args.steps / (ms_total * 1e-3)
    e2e = tokens_per_job * args.steps / (ms_e2e * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "global_batch": B, "prompt": S, "decode": T, "parallelism": (f"ep{world}: dense weights whole and 1/{world} of the experts per GPU, {Bl} rows each, all-gather + "
                                   "reduce-scatter per expert layer" if ep else
                                   f"dp{world}: whole model per GPU, {Bl} rows each, no collective" if dp else f"tp{world}"),
                   **({"tp_collective": collective} if world > 1 and not dp else {}),
                   "l2": "inputs larger than L2: every decode step streams the full weight set "
                         f"({weight_bytes / 1e9:.2f} GB per GPU) plus the KV cache",
                   "generator": generator},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": int(prompt.nbytes) * (world if dp else 1),
                "d2h_bytes_per_step": int(B * (T + 1) * 4)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "k_gemm_dec (k_gemm_tc for the LM head): all dense weight-streaming GEMMs of one decode step",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                     "traffic": traffic,
                     "traffic_source": ("profiles/traffic.json: one ncu capture of the decode GEMMs (dram__bytes_read.sum + "
                                        "dram__bytes_write.sum), not measured in this run" if traffic else None),
                     "algorithmic_bytes_per_sweep": weight_bytes, "launches_per_sweep": gemm_launches,
                     "ms_per_sweep": gemm_ms},
        "phases": {"prefill_ms": ms_prefill, "prefill_tok_s": B * S / (ms_prefill * 1e-3),
                   "decode_ms_per_step": ms_decode, "decode_tok_s": B / (ms_decode * 1e-3),
                   "decode_step_hbm_floor_ms": (weight_bytes + kv_bytes + expert_bytes) / (peak * 1e9) * 1e3,
                   "decode_step_frac_of_hbm_roofline": (weight_bytes + kv_bytes + expert_bytes) / (peak * 1e9) * 1e3 / ms_decode,
                   "decode_step_bytes": {"dense_weights": weight_bytes, "kv_cache": kv_bytes,
                                         "experts_expected": expert_bytes}},
    }
    if token_check is not None:
        line["tokens_equal_frac"] = token_check["tokens_equal_frac"]
        line["token_check"] = token_check
    if rank == 0 and world == 1 and not args.no_cpu_baseline and headline:
        forward, cores = run_reference_sample(cg, dataclasses.replace(cfg, dtype="bf16"), S)
        t_fwd = forward()
        job = reference_job_seconds(t_fwd, S, T, B)
        line["cpu_baseline"] = {
            "value": tokens_per_job / job, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"one full forward of 1 of {B} rows at {S} tokens ({t_fwd:.2f} s) through the reference op stream on the "
                      f"CPU restatement; the job ({B} rows x {T + 1} full forwards, no KV cache) extrapolated linearly in length"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline and headline:
        try:
            line["cpu_baseline_kv_cache"] = torch_cpu_kv_baseline(cg, cfg, S, T, B)
        except Exception as e:  # the headline baseline is the one above; this one is extra
            line["cpu_baseline_kv_cache"] = {"unavailable": str(e)[:200]}
    if rank == 0:
        print(json.dumps(line))
    dec.close()
    if dist is not None:
        dist.destroy_process_group()
    if token_check is not None and token_check["tokens_equal_frac"] < 0.9:
        raise SystemExit(f"token check failed: only {token_check['tokens_equal_frac']:.3f} of the job's tokens equal the "
                         "independent run's")


if __name__ == "__main__":
    main()
