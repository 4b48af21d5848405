"""Deferred evaluation with pattern fusion behind the unchanged trait (the "lazy" option).

The same op streams as everywhere else -- the reference's model graphs replayed call by call,
nothing in them changed -- run on the CUDA backend twice, eagerly and recorded.  Recorded, the
chains of catgrad's stdlib (rmsnorm, softmax, silu * up, rope, the attention core with its mask and
repeat_kv) are replaced by fused kernels when results are needed.  Checked: integer results
(arg-max tokens, expert ids) identical, logits within 1e-4 of the logit scale of eager mode and of
the CPU checker, far fewer kernel launches, and the bookkeeping around handles (values the caller
keeps are materialised, dropped values are not computed, errors surface when a call is recorded).
"""
import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
graphs, synth = cg.graphs, cg.synth

LLAMA = synth.ModelConfig("lazy-llama", 256, 512, 3, 4, 2, 1024, rms_norm_eps=1e-5, rope_theta=10000.0,
                          tie_word_embeddings=False, dtype="f32")
LLAMA_D128 = synth.ModelConfig("lazy-llama-d128", 512, 768, 2, 4, 2, 1024, head_dim=128, rms_norm_eps=1e-5,
                               rope_theta=500000.0, tie_word_embeddings=True, dtype="f32")
QWEN = synth.ModelConfig("lazy-qwen3", 256, 512, 2, 4, 2, 1024, head_dim=64, arch="qwen3", rope_theta=1e6,
                         tie_word_embeddings=False)
QWEN_MOE = synth.ModelConfig("lazy-qwen3-moe", 128, 256, 2, 4, 2, 512, head_dim=64, arch="qwen3", rope_theta=1e6,
                             num_local_experts=16, num_experts_per_tok=4, moe_intermediate_size=96, norm_topk_prob=True)
GEMMA3 = synth.ModelConfig("lazy-gemma3", 256, 512, 3, 4, 2, 1024, head_dim=64, arch="gemma", rope_theta=1e6,
                           tie_word_embeddings=True, qk_norm=True, sliding_window_pattern=2, rope_local_base_freq=10000.0)


def forward_of(cfg):
    return {"llama": graphs.llama.forward, "qwen3": graphs.qwen3.forward, "gemma": graphs.gemma.forward}[cfg.arch]


def run(B, cfg, ids, seed=0):
    params = {n: B.from_numpy(w) for n, w in synth.make_weights(cfg, seed)}
    extra = {"expert_ids": []} if cfg.num_local_experts > 1 else {}
    before = B.launch_count() if hasattr(B, "launch_count") else 0
    y, lg = forward_of(cfg)(B, cfg, params, B.from_numpy(ids), ids.shape[1], want_logits=True, **extra)
    toks = B.to_vec(y)
    logits = B.to_numpy(lg)
    launches = (B.launch_count() - before) if hasattr(B, "launch_count") else 0
    return toks, logits, [B.to_numpy(e) for e in extra.get("expert_ids", [])], launches


@pytest.mark.parametrize("cfg", [LLAMA, LLAMA_D128, QWEN, QWEN_MOE, GEMMA3], ids=lambda c: c.name)
def test_recorded_stream_equals_eager_and_checker(oracle, cfg):
    C = cg.CudaBackend(0, cg.PREC_F32)
    ids = synth.make_tokens(cfg, 1, 45, seed=3)
    try:
        te, le, ee, n_eager = run(C, cfg, ids)
        C.set_option("lazy", 1)
        r0, f0, _ = C.lazy_stats()
        tl, ll, el, n_lazy = run(C, cfg, ids)
        r1, f1, pending = C.lazy_stats()
    finally:
        C.set_option("lazy", 0)
    to, lo, eo, _ = run(oracle, cfg, ids)
    np.testing.assert_array_equal(te, tl)                       # greedy tokens: identical
    np.testing.assert_array_equal(to, tl)
    scale = np.abs(lo).max()
    assert np.abs(ll - le).max() <= 1e-4 * scale
    assert np.abs(ll - lo).max() <= 1e-4 * scale
    for a, b, c in zip(ee, el, eo):
        np.testing.assert_array_equal(a, b)                     # expert ids: identical
        np.testing.assert_array_equal(c, b)
    assert pending == 0 and r1 - r0 > 100
    L = cfg.num_hidden_layers
    fused = f1 - f0
    # per layer: two rmsnorms, the rope of q, the attention core (which takes k's rope with it), and on
    # dense llama-style layers silu(gate) * up; q/k norms add two more on qwen3 / gemma3
    assert fused >= 4 * L, (fused, L)
    print(f"\n{cfg.name}: launches eager {n_eager} -> recorded {n_lazy}; {r1 - r0} calls recorded, {fused} chains fused")
    assert n_lazy < n_eager * (0.55 if cfg.num_local_experts <= 1 else 0.8)   # per-slot expert matmuls stay as they are
    C.close()


def test_launches_per_layer_of_the_llama_stream():
    """The dense Llama layer comes down to 15 launches: 2 rmsnorm, 7 linear layers, rope of q, rope of
    the un-repeated k + the attention core, silu * up, 2 residual adds."""
    C = cg.CudaBackend(0, cg.PREC_F32)
    ids = synth.make_tokens(LLAMA, 1, 64, seed=3)
    import dataclasses
    try:
        C.set_option("lazy", 1)
        counts = []
        for layers in (2, 4):
            cfg = dataclasses.replace(LLAMA, num_hidden_layers=layers)
            counts.append(run(C, cfg, ids)[3])
    finally:
        C.set_option("lazy", 0)
    per_layer = (counts[1] - counts[0]) / 2
    print(f"\nlaunches with 2 and 4 layers: {counts}; per recorded llama layer: {per_layer}")
    assert per_layer <= 15
    C.close()


def test_handles_the_caller_keeps_are_materialised_and_dropped_ones_are_not_computed():
    C = cg.CudaBackend(0, cg.PREC_F32)
    rng = np.random.Generator(np.random.PCG64(1))
    x = rng.standard_normal((4, 6, 32), dtype=np.float32)
    try:
        C.set_option("lazy", 1)
        X = C.from_numpy(x)
        # a softmax whose intermediate `ex` the caller keeps: the chain must not swallow it
        sh = X.shape
        m = C.max(X)
        d = C.sub(X, C.broadcast(m, sh))
        ex = graphs.nn.exp(C, d)
        s = C.sum(ex)
        y = C.div(ex, C.broadcast(s, sh))
        f_before = C.lazy_stats()[1]
        got_y, got_ex = C.to_numpy(y), C.to_numpy(ex)
        assert C.lazy_stats()[1] == f_before                      # not fused: `ex` is visible outside
        want_ex = np.exp(x - x.max(-1, keepdims=True))
        np.testing.assert_allclose(got_ex, want_ex, rtol=2e-6)
        np.testing.assert_allclose(got_y, want_ex / want_ex.sum(-1, keepdims=True), rtol=2e-6)
        # the same with nothing kept: one fused kernel
        y2 = graphs.nn.softmax(C, X)
        n0 = C.launch_count()
        got = C.to_numpy(y2)
        assert C.lazy_stats()[1] == f_before + 1 and C.launch_count() - n0 == 1
        np.testing.assert_allclose(got, got_y, rtol=2e-6)
        # a value that is dropped before anyone needs it never runs
        n0 = C.launch_count()
        t = C.mul(X, X)
        t = C.add(t, t)
        del t
        C.sync()
        assert C.launch_count() == n0
        # shape errors surface at the call, as in eager mode
        with pytest.raises(cg.BackendPanic):
            C.add(X, C.from_numpy(x[:, :3]))
        with pytest.raises(cg.BackendPanic):
            C.matmul(X, X)
        # views of pending values, and a reshape that needs a copy
        z = C.transpose(C.add(X, X), 1, 2)
        w = C.reshape(z, (4, 32 * 6))
        np.testing.assert_array_equal(C.to_numpy(w), (x + x).transpose(0, 2, 1).reshape(4, -1))
        np.testing.assert_array_equal(C.to_numpy(C.slice(z, 1, 3, 5)), (x + x).transpose(0, 2, 1)[:, 3:8])
    finally:
        C.set_option("lazy", 0)
        C.close()
