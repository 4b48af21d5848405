"""The explicit-KV-cache graph and runner (catgrad-llm/src/run.rs:149-305,
legacy/models/utils.rs:210-228) on the trait path, and the serving interface over the fused
decoder.  Size-independent property: a cached run equals full recomputation -- identical greedy
tokens, logits within f32 rounding -- on the CPU checker alone (no GPU) and on the CUDA backend."""
import itertools

import numpy as np
import pytest

from conftest import cg

graphs, synth = cg.graphs, cg.synth
SMALL_F32 = synth.ModelConfig("small-llama-f32", 128, 256, 2, 4, 2, 512, rms_norm_eps=1e-5, rope_theta=10000.0,
                              tie_word_embeddings=False, dtype="f32")


def recompute_tokens(B, cfg, params, prompt, steps):
    return graphs.llama.generate(B, cfg, params, prompt, steps)


def run_both(B, cfg, steps=9, plen=13):
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, 0)}
    prompt = [int(t) for t in synth.make_tokens(cfg, 1, plen, seed=1)[0]]
    want = recompute_tokens(B, cfg, params, prompt, steps)
    runner = graphs.llama_kv.KVRunner(B, cfg, params, max_sequence_length=plen + steps + 8)
    got = list(itertools.islice(runner.complete(prompt), steps))
    return prompt, want, got, runner, params


def test_cached_run_equals_recomputation_on_the_checker(oracle):
    prompt, want, got, runner, params = run_both(oracle, SMALL_F32)
    assert got == want
    assert runner.total_tokens == len(prompt) + len(got) - 1
    # extending the context keeps the cache (only the new tokens are run); a changed context drops it
    more = prompt + got + [5, 6]
    runner.set_context(more)
    assert runner.tokens == got[-1:] + [5, 6]
    with pytest.raises(ValueError):          # more than one token on a non-empty cache: the reference's mask cannot broadcast
        next(runner)
    runner.set_context([1, 2, 3])
    assert runner.kv_cache is None and runner.tokens == [1, 2, 3]
    assert next(runner) == recompute_tokens(oracle, SMALL_F32, params, [1, 2, 3], 1)[0]


@pytest.mark.gpu
def test_cached_run_equals_recomputation_on_cuda_and_matches_the_checker(oracle, cuda):
    _, want_o, got_o, _, _ = run_both(oracle, SMALL_F32)
    _, want_c, got_c, runner, _ = run_both(cuda, SMALL_F32)
    assert got_c == want_c == got_o == want_o
    # the cache tensors are device tensors of the growing length
    k, v = runner.kv_cache[0]
    assert k.shape == (1, SMALL_F32.num_key_value_heads, runner.total_tokens, SMALL_F32.head_dim)


@pytest.mark.gpu
def test_decoder_lm_prefix_reuse(cuda_bf16):
    """`DecoderLM` (serve.rs's LM over the fused decoder): completing a context, then a context that
    shares a prefix, gives the tokens of fresh runs while only the differing suffix is recomputed."""
    C = cuda_bf16
    cfg = synth.ModelConfig("small-llama-bf16", 256, 512, 2, 4, 2, 1024, rms_norm_eps=1e-5, rope_theta=500000.0,
                            tie_word_embeddings=True, dtype="bf16")
    dec = cg.Decoder(C, cfg, max_seq=96, max_batch=1)
    dec.load(synth.make_weights(cfg, 0))
    prompt = [int(t) for t in synth.make_tokens(cfg, 1, 30, seed=1)[0]]

    def fresh(context, n):
        dec.reset()
        return [int(t) for t in dec.generate(np.uint32(context).reshape(1, -1), n - 1)[0]]

    want = fresh(prompt, 6)
    lm = cg.serve.DecoderLM(dec)
    dec.reset()
    got = list(itertools.islice(lm.complete(prompt), 6))
    assert got == want
    # a follow-up that keeps the first 20 tokens: 20 positions stay cached, the rest is re-run
    follow = prompt[:20] + [7, 8, 9, 10]
    want2 = fresh(follow, 4)
    dec.reset()
    lm = cg.serve.DecoderLM(dec)
    list(itertools.islice(lm.complete(prompt), 3))
    lm.set_context(follow)
    assert lm.cached == prompt[:20] and lm.pending == [7, 8, 9, 10]
    assert dec.position()[0] == 20
    got2 = list(itertools.islice(lm, 4))
    assert got2 == want2
    # end-of-sequence tokens end the iteration and are not emitted
    stop = next((i for i in range(1, len(want)) if want[i] not in want[:i]), 0)   # first token not seen before it
    lm = cg.serve.DecoderLM(dec, eos_token_ids=[want[stop]])
    dec.reset()
    assert list(lm.complete(prompt)) == want[:stop]
    dec.close()
