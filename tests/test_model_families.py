"""Qwen3 (dense and mixture-of-experts) and Gemma-shaped graphs.

Trait path: the reference's op stream (catgrad-llm/src/models/qwen3.rs, gemma3.rs) on the CUDA
backend against the same stream on the CPU checker, f32: logits within 1e-4 of the logit scale,
arg-max tokens and top-k expert ids bit-exact.  Decoder path (bf16): the switches of the fused
runner (q/k-norm, GeGLU, (1 + gamma) norms, post-norms, embedding scale, soft-caps, sliding
window) against the f32 checker within 2e-2, teacher-forced."""
import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
synth, graphs = cg.synth, cg.graphs

QWEN_DENSE = synth.ModelConfig("qwen3-dense-small", 256, 512, 2, 4, 2, 1024, head_dim=64, arch="qwen3",
                               rope_theta=1e6, tie_word_embeddings=False)
QWEN_MOE = synth.ModelConfig("qwen3-moe-small", 128, 256, 2, 4, 2, 512, head_dim=64, arch="qwen3", rope_theta=1e6,
                             num_local_experts=16, num_experts_per_tok=4, moe_intermediate_size=96,
                             norm_topk_prob=True)
GEMMA2 = synth.ModelConfig("gemma2-small", 256, 512, 2, 4, 2, 1024, head_dim=64, arch="gemma", rope_theta=10000.0,
                           tie_word_embeddings=True, attn_logit_softcap=50.0, final_logit_softcap=30.0,
                           sliding_window=8)
# three layers with pattern 2: local, global, local -- the local layers rotate with their own base
GEMMA3 = synth.ModelConfig("gemma3-small", 256, 512, 3, 4, 2, 1024, head_dim=64, arch="gemma", rope_theta=1e6,
                           tie_word_embeddings=True, qk_norm=True, sliding_window_pattern=2,
                           rope_local_base_freq=10000.0)


def fwd_of(cfg):
    return graphs.qwen3.forward if cfg.arch == "qwen3" else graphs.gemma.forward


def weights(cfg, seed=0):
    """Synthetic checkpoint with non-trivial norm gains so (1 + gamma) and q/k-norm are exercised."""
    rng = np.random.Generator(np.random.PCG64(100 + seed))
    for name, w in synth.make_weights(cfg, seed):
        if w.ndim == 1:
            w = (w + rng.standard_normal(w.shape, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
        yield name, w


@pytest.mark.parametrize("cfg", [QWEN_DENSE, QWEN_MOE, GEMMA2, GEMMA3], ids=lambda c: c.name)
def test_op_stream_parity_f32(oracle, cuda, cfg):
    ids = synth.make_tokens(cfg, 1, 21, seed=4)
    outs = []
    for B in (oracle, cuda):
        params = {n: B.from_numpy(w) for n, w in weights(cfg)}
        extra = {}
        if cfg.num_local_experts > 1:
            extra["expert_ids"] = []
        y, lg = fwd_of(cfg)(B, cfg, params, B.from_numpy(ids), 21, want_logits=True, **extra)
        outs.append((B.to_vec(y), B.to_numpy(lg), [B.to_numpy(e) for e in extra.get("expert_ids", [])]))
    (yo, lo, eo), (yc, lc, ec) = outs
    assert np.abs(lc - lo).max() <= 1e-4 * np.abs(lo).max()
    np.testing.assert_array_equal(yo, yc)
    assert len(eo) == len(ec)
    for a, b in zip(eo, ec):
        np.testing.assert_array_equal(a, b)   # top-k expert ids: bit-exact


@pytest.mark.parametrize("cfg", [QWEN_DENSE, QWEN_MOE, GEMMA2, GEMMA3], ids=lambda c: c.name)
def test_decoder_switches_match_checker(oracle, cuda_bf16, cfg):
    import dataclasses
    cfg = dataclasses.replace(cfg, dtype="bf16")
    C = cuda_bf16
    batch, seq, steps, tol = 2, 24, 5, 2e-2
    po = {n: oracle.from_numpy(w) for n, w in weights(cfg)}
    dec = cg.Decoder(C, cfg, max_seq=seq + steps + 1, max_batch=batch)
    dec.load(weights(cfg))
    prompt = synth.make_tokens(cfg, batch, seq, seed=1)
    lg = C.to_numpy(dec.prefill(C.from_numpy(prompt), want_logits=True))
    rows = [list(prompt[b]) for b in range(batch)]
    for step in range(steps + 1):
        forced = []
        for b in range(batch):
            ids = np.asarray(rows[b], dtype=np.uint32).reshape(1, -1)
            _, ref = fwd_of(cfg)(oracle, cfg, po, oracle.from_numpy(ids), ids.shape[1], want_logits=True)
            want = oracle.to_numpy(ref)[0, -1]
            assert np.abs(lg[b] - want).max() <= tol, (step, b, float(np.abs(lg[b] - want).max()))
            pick = len(want) - 1 - int(np.argmax(want[::-1]))
            top2 = np.sort(want)[-2:]
            if top2[1] - top2[0] > 2 * tol:
                assert int(np.argmax(lg[b])) == pick
            forced.append(pick)
            rows[b].append(pick)
        if step < steps:
            lg = C.to_numpy(dec.step_with(C.from_numpy(np.uint32(forced)), want_logits=True))
    dec.close()
