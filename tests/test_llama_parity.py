"""Whole-model parity.  No reference test pins logits or greedy tokens ("parity unpinned"),
so the checker is the CPU restatement running the reference's own op stream.

* tiny Llama, f32 (the CPU-runnable benchmark configuration): the same op stream on the CUDA backend — logits within
  1e-4 relative of the checker, identical greedy tokens over prefill + 16 decode steps.
* the fused, KV-cached decoder (bf16) on shrunken Llama shapes: logits within 2e-2 of the f32
  checker on the same bf16-rounded weights, tokens identical wherever the checker's own
  top-1/top-2 margin exceeds twice that bound; cached decode equals recomputation.
"""
import dataclasses

import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
llama, synth = cg.graphs.llama, cg.synth


def load(B, cfg, seed=0):
    return {name: B.from_numpy(w) for name, w in synth.make_weights(cfg, seed)}


def test_tiny_llama_f32_op_stream_parity(oracle, cuda):
    cfg = synth.TINY_LLAMA
    prompt = synth.make_tokens(cfg, 1, 32, seed=1)[0]
    steps = 17  # the prompt's next token + 16 decode steps
    po, pc = load(oracle, cfg), load(cuda, cfg)
    toks_o = llama.generate(oracle, cfg, po, prompt, steps)
    toks_c = llama.generate(cuda, cfg, pc, prompt, steps)
    assert toks_o == toks_c
    ids = np.concatenate([prompt, np.uint32(toks_o[:-1])]).reshape(1, -1)
    _, lo = llama.forward(oracle, cfg, po, oracle.from_numpy(ids), ids.shape[1], want_logits=True)
    _, lc = llama.forward(cuda, cfg, pc, cuda.from_numpy(ids), ids.shape[1], want_logits=True)
    lo, lc = oracle.to_numpy(lo), cuda.to_numpy(lc)
    scale = np.abs(lo).max()
    assert np.abs(lc - lo).max() <= 1e-4 * scale  # 1e-4 relative to the logit scale


SMALL = synth.ModelConfig("small-llama-bf16", 256, 512, 2, 4, 2, 1024, rms_norm_eps=1e-5, rope_theta=500000.0,
                          tie_word_embeddings=True, dtype="bf16")
SMALL_D128 = synth.ModelConfig("small-llama-d128", 512, 768, 2, 4, 2, 2048, head_dim=128, rms_norm_eps=1e-5,
                               rope_theta=500000.0, tie_word_embeddings=False, dtype="bf16")


def checker_logits(oracle, cfg, params, ids_row):
    ids = np.asarray(ids_row, dtype=np.uint32).reshape(1, -1)
    _, lg = llama.forward(oracle, cfg, params, oracle.from_numpy(ids), ids.shape[1], want_logits=True)
    return oracle.to_numpy(lg)[0]  # [S, V]


SMALL_D256 = synth.ModelConfig("small-llama-d256", 512, 768, 2, 2, 1, 1024, head_dim=256, rms_norm_eps=1e-5,
                               rope_theta=500000.0, tie_word_embeddings=True, dtype="bf16")


# the two long prompts exercise many key tiles per slice in the decode attention (8-slice clusters)
@pytest.mark.parametrize("cfg,batch,seq,steps", [(SMALL, 2, 24, 6), (SMALL_D128, 3, 70, 4), (SMALL, 1, 1, 5),
                                                 (SMALL_D128, 1, 2050, 2), (SMALL_D256, 2, 2050, 2)])
def test_decoder_matches_checker(oracle, cuda_bf16, cfg, batch, seq, steps):
    C = cuda_bf16
    po = load(oracle, cfg)
    dec = cg.Decoder(C, cfg, max_seq=seq + steps + 1, max_batch=batch)
    dec.load(synth.make_weights(cfg, 0))
    prompt = synth.make_tokens(cfg, batch, seq, seed=1)
    tol = 2e-2
    # prefill: last-position logits of every row
    lg = C.to_numpy(dec.prefill(C.from_numpy(prompt), want_logits=True))
    rows = [list(prompt[b]) for b in range(batch)]
    for step in range(steps + 1):
        forced = []
        for b in range(batch):
            want = checker_logits(oracle, cfg, po, rows[b])[-1]
            assert np.abs(lg[b] - want).max() <= tol, (step, b)
            top2 = np.sort(want)[-2:]
            pick = int(np.argmax(want[::-1]))  # last index on ties, like the reference
            pick = len(want) - 1 - pick
            if top2[1] - top2[0] > 2 * tol:
                assert int(np.argmax(lg[b])) == pick
            forced.append(pick)
            rows[b].append(pick)
        if step == steps:
            break
        # teacher-force the checker's token so both sides stay on the same sequence
        lg = C.to_numpy(dec.step_with(C.from_numpy(np.uint32(forced)), want_logits=True))
    dec.close()


WIDE = synth.ModelConfig("wide-llama-bf16", 2048, 4096, 1, 32, 8, 512, rms_norm_eps=1e-5, rope_theta=500000.0,
                         tie_word_embeddings=True, dtype="bf16")


def test_wide_prefill_matches_checker(oracle, cuda_bf16):
    """A prompt batch large enough (7104 tokens per chunk, 2048-wide projections) that the
    prefill GEMMs take their 256-row two-accumulator tiles, including the residual epilogue and
    the paired gate/up epilogue."""
    C, cfg, batch, seq = cuda_bf16, WIDE, 37, 256
    po = load(oracle, cfg)
    dec = cg.Decoder(C, cfg, max_seq=seq + 2, max_batch=batch)
    dec.load(synth.make_weights(cfg, 0))
    prompt = synth.make_tokens(cfg, batch, seq, seed=3)
    lg = C.to_numpy(dec.prefill(C.from_numpy(prompt), want_logits=True))
    for b in (0, 17, 36):
        want = checker_logits(oracle, cfg, po, prompt[b])[-1]
        # this model's logits are several times larger than the small models' (2048-wide tied
        # embedding): the bound is 1% of the logit scale rather than 2e-2 absolute
        scale = float(np.abs(want).max())
        assert np.abs(lg[b] - want).max() <= 1e-2 * max(scale, 2.0), (b, float(np.abs(lg[b] - want).max()), scale)
        assert int(np.argmax(lg[b])) == int(np.argmax(want)) or np.sort(want)[-1] - np.sort(want)[-2] < 2e-2 * scale
    dec.close()


def test_cached_decode_equals_recompute_and_graph_replay(cuda_bf16):
    """Size-independent property: prefill(n) + k cached steps == prefill(n + k) on the tokens
    the decoder itself generated; the captured-graph replay gives the eager step's tokens."""
    C = cuda_bf16
    cfg = SMALL
    batch, seq, steps = 4, 40, 12
    dec = cg.Decoder(C, cfg, max_seq=seq + steps + 2, max_batch=batch)
    dec.load(synth.make_weights(cfg, 0))
    prompt = synth.make_tokens(cfg, batch, seq, seed=3)
    dec.prefill(C.from_numpy(prompt))
    last = C.to_numpy(dec.decode(steps, want_logits=True))  # 1 eager step + graph replays
    toks = dec.tokens()
    assert toks.shape == (batch, steps + 1)
    # recompute: run the whole sequence as a prompt; its last logits are the last step's
    full = np.concatenate([prompt, toks[:, :-1]], axis=1)
    dec.reset()
    again = C.to_numpy(dec.prefill(C.from_numpy(full), want_logits=True))
    np.testing.assert_allclose(again, last, rtol=0, atol=3e-2)
    assert (np.argmax(again, 1) == np.argmax(last, 1)).mean() >= 0.75
    # eager single steps reproduce the graph's tokens bit for bit
    dec.reset()
    dec.prefill(C.from_numpy(prompt))
    for i in range(steps):
        dec.step_with(C.from_numpy(toks[:, i].copy()))
    np.testing.assert_array_equal(dec.tokens(), toks)
    # host-buffer entry point
    dec.reset()
    out = dec.generate(prompt, steps)
    np.testing.assert_array_equal(out, toks)
    dec.close()


def test_batch_rows_are_independent(cuda_bf16):
    """The reference graphs are batch-1; a batched run must equal each row run alone."""
    C = cuda_bf16
    cfg = SMALL
    prompt = synth.make_tokens(cfg, 3, 40, seed=5)  # 120 and 40 tokens: the same GEMM path and k order
    dec = cg.Decoder(C, cfg, max_seq=64, max_batch=3)
    dec.load(synth.make_weights(cfg, 0))
    batched = dec.generate(prompt, 8)
    for b in range(3):
        dec.reset()
        np.testing.assert_array_equal(dec.generate(prompt[b:b + 1], 8)[0], batched[b])
    dec.close()


@pytest.mark.parametrize("cfg", [SMALL, SMALL_D128], ids=lambda c: c.name)
def test_chunked_prefill_equals_one_chunk_and_kernel_variants_agree(cuda_bf16, cfg):
    """Size-independent properties of the prefill: processing the prompt in position chunks
    (later chunks attend to the cache with a position offset) gives the logits of one chunk, and
    the tcgen05 attention / persistent GEMM give the logits of the mma.sync / per-tile kernels,
    and so do the CTA-pair GEMMs."""
    C = cuda_bf16
    batch, seq = 2, 600
    dec = cg.Decoder(C, cfg, max_seq=seq + 2, max_batch=batch)
    dec.load(synth.make_weights(cfg, 0))
    prompt = C.from_numpy(synth.make_tokens(cfg, batch, seq, seed=5))
    ref = C.to_numpy(dec.prefill(prompt, want_logits=True))
    try:
        C.set_option("prefill_chunk", 256)  # 128 positions per chunk and row
        chunked = C.to_numpy(dec.prefill(prompt, want_logits=True))
        C.set_option("prefill_chunk", 8192)
        C.set_option("fa", 0)
        C.set_option("persistent", 0)
        legacy = C.to_numpy(dec.prefill(prompt, want_logits=True))
        C.set_option("fa", 1)
        C.set_option("persistent", 1)
        C.set_option("pair_cta", 2)  # every prefill GEMM, gate/up included, on CTA pairs
        paired = C.to_numpy(dec.prefill(prompt, want_logits=True))
    finally:
        C.set_option("prefill_chunk", 8192)
        C.set_option("fa", 1)
        C.set_option("persistent", 1)
        C.set_option("pair_cta", 1)
    np.testing.assert_allclose(chunked, ref, rtol=0, atol=2e-2)
    np.testing.assert_allclose(legacy, ref, rtol=0, atol=2e-2)
    np.testing.assert_allclose(paired, ref, rtol=0, atol=2e-2)
    dec.close()


@pytest.mark.parametrize("cfg,batch,seq,steps", [(SMALL, 2, 24, 6), (SMALL, 8, 300, 12), (SMALL_D128, 3, 70, 4),
                                                 (SMALL_D128, 20, 40, 6), (SMALL, 1, 1, 5)])
def test_resident_decode_kernel_agrees_with_per_operation_path(cuda_bf16, cfg, batch, seq, steps):
    """The "resident" option runs all decode steps of a call as one kernel (decode_resident.cu).
    Its sums run in another order (K split four ways inside a cluster instead of up to sixteen),
    so logits agree within bf16 rounding rather than bit for bit: teacher-forced with the default
    path's tokens, every step's logits within 2e-2, and the greedy pick equal wherever the default
    path's top-1 / top-2 margin exceeds twice that.  Batches above 16 take the 32-column tiles."""
    C = cuda_bf16
    dec = cg.Decoder(C, cfg, max_seq=seq + steps + 2, max_batch=batch)
    dec.load(synth.make_weights(cfg, 0))
    prompt = synth.make_tokens(cfg, batch, seq, seed=1)
    dec.prefill(C.from_numpy(prompt))
    dec.decode(steps)
    toks = dec.tokens()

    def forced(resident):
        C.set_option("resident", resident)
        dec.reset()
        dec.prefill(C.from_numpy(prompt))
        out = [C.to_numpy(dec.step_with(C.from_numpy(np.ascontiguousarray(toks[:, i])), want_logits=True))
               for i in range(steps)]
        return out, dec.tokens()

    try:
        l1, t1 = forced(1)
        # one call for all steps: the kernel loops over the steps itself
        dec.reset()
        dec.prefill(C.from_numpy(prompt))
        dec.decode(steps)
        t_free = dec.tokens()
        l0, t0 = forced(0)
    finally:
        C.set_option("resident", 0)
    for a, b in zip(l0, l1):
        assert np.abs(a - b).max() <= 2e-2
        top2 = np.sort(a, axis=1)[:, -2:]
        sure = top2[:, 1] - top2[:, 0] > 4e-2
        assert (np.argmax(a, 1)[sure] == np.argmax(b, 1)[sure]).all()
    assert (t0 == t1).mean() >= 0.9
    # the multi-step call follows the same sequence as long as no near-tie flips a token
    first_diff = np.argmax(np.concatenate([t_free != toks, np.ones((batch, 1), bool)], axis=1), axis=1)
    assert (first_diff >= 1).all()   # the prefill's token is common to both
    dec.close()
