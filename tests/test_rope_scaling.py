"""Rotary tables with the frequency rescaling of long-context checkpoints.

catgrad-llm/src/legacy/nn/rope.rs:32-201 builds "llama3" and "yarn" tables as expression trees of
f32 tensor ops.  The checker below evaluates those trees with numpy in float32, operation by
operation in the reference's order; the library computes the same expressions in one kernel with
un-fused f32 arithmetic, so the per-frequency factors agree to the last bit or two and the tables
to a few 1e-6 at the positions checked (the angle pos * inv_freq magnifies one ulp of inv_freq by
the position).  A decoder configured with a scaling is also checked end to end against the
checker's op stream run with the scaled tables."""
import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
synth, graphs = cg.synth, cg.graphs
f32 = np.float32

LLAMA3 = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
YARN = {"rope_type": "yarn", "factor": 40.0, "beta_fast": 32.0, "beta_slow": 1.0, "original_max_position_embeddings": 4096}


def reference_tables(theta, seq_len, head_dim, rs):
    """rope.rs:8-30 / :32-98 / :139-201 in numpy float32 -> cos, sin [T, d/2] (before the concat)."""
    half = head_dim // 2
    f = np.arange(half, dtype=f32) * f32(2.0 / head_dim)
    freq = np.power(np.float64(f32(theta)), f.astype(np.float64)).astype(f32)   # the backends' pow goes through f64
    inv = (f32(1.0) / freq).astype(f32)
    scale = f32(1.0)
    kind = (rs or {}).get("rope_type")
    if kind == "llama3":
        old = f32(rs["original_max_position_embeddings"])
        low_wl, high_wl = old / f32(rs["low_freq_factor"]), old / f32(rs["high_freq_factor"])
        factor, lff, hff = f32(rs["factor"]), f32(rs["low_freq_factor"]), f32(rs["high_freq_factor"])
        wavelen = (f32(2.0 * np.pi) / inv).astype(f32)
        low = wavelen > low_wl
        inv = np.where(low, (inv / factor).astype(f32), inv)
        high = wavelen < high_wl
        smooth = ((old / wavelen - lff) / (hff - lff)).astype(f32)
        smoothed = ((smooth * inv).astype(f32) + (((f32(1.0) - smooth) * inv).astype(f32) / factor).astype(f32)).astype(f32)
        inv = np.where(~high & ~low, smoothed, inv)
    elif kind == "yarn":
        two_pi = f32(2.0) * f32(np.pi)
        omp = f32(rs["original_max_position_embeddings"])

        def corr(rot):
            return f32(f32(head_dim) * np.log(omp / (f32(rot) * two_pi), dtype=f32)) / (f32(2.0) * np.log(f32(theta), dtype=f32))
        lo, hi = corr(rs["beta_fast"]), corr(rs["beta_slow"])
        ramp = np.clip(((np.arange(half, dtype=f32) - lo) / (hi - lo)).astype(f32), f32(0), f32(1))
        ext = (f32(1.0) - ramp).astype(f32)
        interp = (inv / f32(rs["factor"])).astype(f32)
        inv = ((interp * (f32(1.0) - ext)).astype(f32) + (inv * ext).astype(f32)).astype(f32)
        scale = f32(1.0) if rs["factor"] <= 1.0 else f32(0.1) * np.log(f32(rs["factor"]), dtype=f32) + f32(1.0)
    ang = (np.arange(seq_len, dtype=f32)[:, None] * inv[None, :]).astype(f32)
    cos = (np.cos(ang.astype(np.float64)).astype(f32) * scale).astype(f32)
    sin = (np.sin(ang.astype(np.float64)).astype(f32) * scale).astype(f32)
    return cos, sin


@pytest.mark.parametrize("rs", [None, LLAMA3, YARN], ids=["plain", "llama3", "yarn"])
@pytest.mark.parametrize("theta,d", [(500000.0, 64), (10000.0, 128)])
def test_tables_match_the_f32_expression_tree(cuda, rs, theta, d):
    T = 300
    c, s = cuda.rope_tables(theta, T, d, rs)
    c, s = cuda.to_numpy(c), cuda.to_numpy(s)
    wc, ws = reference_tables(theta, T, d, rs)
    # position 1 exposes the per-frequency factor itself: cos/sin of inv_freq
    np.testing.assert_allclose(c[1], wc[1], rtol=0, atol=2e-7)
    np.testing.assert_allclose(s[1], ws[1], rtol=0, atol=2e-7)
    np.testing.assert_allclose(c, wc, rtol=0, atol=2e-5)
    np.testing.assert_allclose(s, ws, rtol=0, atol=2e-5)
    if rs is not None:
        # the scaling changes some per-frequency factor by a large ratio (the test would be vacuous otherwise)
        _, ps = reference_tables(theta, T, d, None)
        assert np.abs(ws[1] / ps[1] - 1).max() > 0.5


@pytest.mark.parametrize("rs", [LLAMA3, YARN], ids=["llama3", "yarn"])
def test_decoder_with_scaled_rope_matches_checker(oracle, cuda_bf16, rs):
    import dataclasses
    C = cuda_bf16
    # a context long enough (original_max_position_embeddings 64) that some frequencies are rescaled
    rs = dict(rs, original_max_position_embeddings=64)
    cfg = synth.ModelConfig("small-llama-scaled-rope", 256, 512, 2, 4, 2, 1024, rms_norm_eps=1e-5, rope_theta=10000.0,
                            tie_word_embeddings=True, dtype="bf16", rope_scaling=rs)
    weights = list(synth.make_weights(cfg, 0))
    po = {n: oracle.from_numpy(w) for n, w in weights}
    seq = 90
    wc, ws = reference_tables(cfg.rope_theta, seq + 8, cfg.head_dim, rs)
    cache = (oracle.from_numpy(np.concatenate([wc, wc], 1)), oracle.from_numpy(np.concatenate([ws, ws], 1)))

    def checker_forward(ids):
        # llama.rs:159-204 with the scaled tables in place of Cache::init's
        B = oracle
        x = graphs.helpers.embeddings(B, po, "model.embed_tokens", B.from_numpy(ids))
        for i in range(cfg.num_hidden_layers):
            x = graphs.llama.layer(B, cfg, po, cache, 0, f"model.layers.{i}", x)
        x = graphs.helpers.rmsnorm(B, cfg.rms_norm_eps, po, "model.norm", x)
        return B.to_numpy(graphs.nn.linear_no_bias(B, cfg.hidden_size, cfg.vocab_size, po, "model.embed_tokens", x))[0, -1]

    dec = cg.Decoder(C, cfg, max_seq=seq + 8, max_batch=1)
    dec.load(weights)
    row = list(synth.make_tokens(cfg, 1, seq, seed=1)[0])
    lg = C.to_numpy(dec.prefill(C.from_numpy(np.uint32(row).reshape(1, -1)), want_logits=True))[0]
    for step in range(3):
        want = checker_forward(np.uint32(row).reshape(1, -1))
        assert np.abs(lg - want).max() <= 2e-2, (step, float(np.abs(lg - want).max()))
        pick = len(want) - 1 - int(np.argmax(want[::-1]))
        row.append(pick)
        lg = C.to_numpy(dec.step_with(C.from_numpy(np.uint32([pick])), want_logits=True))[0]
    # the same model without the scaling gives different logits: the scaling reached the kernels
    plain = cg.Decoder(C, dataclasses.replace(cfg, rope_scaling=None), max_seq=seq + 8, max_batch=1)
    plain.load(weights)
    lp = C.to_numpy(plain.prefill(C.from_numpy(np.uint32(row[:seq]).reshape(1, -1)), want_logits=True))[0]
    dec.reset()
    ls = C.to_numpy(dec.prefill(C.from_numpy(np.uint32(row[:seq]).reshape(1, -1)), want_logits=True))[0]
    assert np.abs(lp - ls).max() > 1e-3
    dec.close()
    plain.close()
