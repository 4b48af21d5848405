"""The fused kernels and the tensor-core GEMM against the reference's op chains replayed on
the CPU checker.  Tolerances: f32 fused kernels 2e-5 relative (fast exp, different
summation order); anything that rounds operands to bf16 is compared against a checker run
on the same bf16-rounded inputs with 2e-2 absolute slack where products accumulate."""
import numpy as np
import pytest

from conftest import cg

pytestmark = pytest.mark.gpu
nn, H, synth = cg.graphs.nn, cg.graphs.helpers, cg.synth
RNG = np.random.Generator(np.random.PCG64(99))


def rnd(shape, scale=1.0):
    return (RNG.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


@pytest.mark.parametrize("shape", [(1, 3, 256), (2, 5, 2048), (1, 7, 100), (4, 64)])
@pytest.mark.parametrize("plus_one", [False, True])
def test_rmsnorm(oracle, cuda, shape, plus_one):
    x, g = rnd(shape), rnd((shape[-1],))
    got = cuda.to_numpy(cuda.fused_rmsnorm(cuda.from_numpy(x), cuda.from_numpy(g), 1e-5, plus_one))
    B = oracle
    lr = H.rmsnorm_raw(B, 1e-5, B.from_numpy(x))
    gam = B.broadcast(B.from_numpy(g), lr.shape)
    if plus_one:  # catgrad-llm/src/models/gemma3.rs:60-68
        gam = B.add(nn.constant(B, 1.0, lr.shape), gam)
    want = B.to_numpy(B.mul(lr, gam))
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("shape", [(3, 5), (2, 4, 512), (1, 2, 3, 4097)])
def test_softmax(oracle, cuda, shape):
    x = rnd(shape, 3.0)
    got = cuda.to_numpy(cuda.fused_softmax(cuda.from_numpy(x)))
    want = oracle.to_numpy(nn.softmax(oracle, oracle.from_numpy(x)))
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-7)
    # soft-capped: cap * tanh(x / cap) with the stdlib's tanh
    cap = 5.0
    B = oracle
    t = B.from_numpy(x)
    capped = B.mul(nn.constant(B, cap, shape), nn.tanh(B, B.div(t, nn.constant(B, cap, shape))))
    want = B.to_numpy(nn.softmax(B, capped))
    got = cuda.to_numpy(cuda.fused_softmax(cuda.from_numpy(x), cap))
    np.testing.assert_allclose(got, want, rtol=5e-5, atol=1e-7)


def test_softmax_with_reference_mask(oracle, cuda):
    # scores + causal mask as the Llama graph builds them: masked entries are f32::MIN
    s = 9
    x = rnd((1, 2, s, s))
    B = oracle
    m = B.broadcast(H.causal_mask(B, s), (1, 2, s, s))
    want = B.to_numpy(nn.softmax(B, B.add(B.from_numpy(x), m)))
    cm = cuda.broadcast(H.causal_mask(cuda, s), (1, 2, s, s))
    got = cuda.to_numpy(cuda.fused_softmax(cuda.add(cuda.from_numpy(x), cm)))
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("act", [0, 1])
def test_act_mul(oracle, cuda, act):
    g, u = rnd((2, 7, 300), 2.0), rnd((2, 7, 300))
    got = cuda.to_numpy(cuda.fused_act_mul(cuda.from_numpy(g), cuda.from_numpy(u), act))
    B = oracle
    f = nn.silu if act == 0 else nn.gelu
    want = B.to_numpy(B.mul(f(B, B.from_numpy(g)), B.from_numpy(u)))
    np.testing.assert_allclose(got, want, rtol=3e-5, atol=2e-6)


@pytest.mark.parametrize("d,theta,pos0", [(64, 10000.0, 0), (128, 500000.0, 5), (8, 1e6, 0)])
def test_rope(oracle, cuda, d, theta, pos0):
    x = rnd((2, 3, 11, d))
    got = cuda.to_numpy(cuda.fused_rope(cuda.from_numpy(x), theta, pos0))
    B = oracle
    cos, sin = H.rope_tables(B, theta, pos0 + 11, d)
    want = B.to_numpy(H.apply_rope_embedding(B, pos0, d, cos, sin, B.from_numpy(x)))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-5)


def test_eager_stream_matches_fused_on_device(cuda):
    # the same op chain the interpreter would send, run eagerly on the GPU, equals the fused kernel
    x, g = rnd((1, 5, 384)), rnd((384,))
    eager = cuda.to_numpy(H.rmsnorm(cuda, 1e-5, {"n.weight": cuda.from_numpy(g)}, "n", cuda.from_numpy(x)))
    fused = cuda.to_numpy(cuda.fused_rmsnorm(cuda.from_numpy(x), cuda.from_numpy(g), 1e-5))
    np.testing.assert_allclose(fused, eager, rtol=2e-5, atol=1e-6)


GEMM_SHAPES = [(1, 128, 64), (8, 256, 2048), (5, 3072, 2048), (16, 200, 72), (17, 136, 128), (33, 128, 4096),
               (100, 384, 512), (130, 256, 192), (300, 1024, 320), (512, 640, 1024),
               # enough tiles for the 256-row two-accumulator variant (token tiles of 256 and of 128), ragged edges
               (1024, 10240, 128), (1100, 7700, 128), (128, 38000, 64),
               # several tiles per SM: the persistent kernel with double-buffered accumulators
               (1024, 9600, 320), (1300, 7700, 264)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_tensor_core_linear(oracle, cuda_bf16, M, N, K):
    """cg_linear on a bf16 weight = tcgen05 pipeline; operands are bf16-exact so the only
    difference to the f32 checker is accumulation order."""
    x = synth.bf16_round(rnd((1, M, K)))
    w = synth.bf16_round(rnd((N, K), 0.05))
    C = cuda_bf16
    wt = C.from_numpy(w)
    assert C.storage_of(wt) == 2
    got = C.to_numpy(C.linear(C.from_numpy(x), wt))
    B = oracle
    want = B.to_numpy(nn.linear_b_param(B, K, N, B.from_numpy(w), None, B.from_numpy(x)))
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4 * np.sqrt(K))
    # and through the trait's own matmul on the transposed view (what the interpreter sends)
    got2 = C.to_numpy(nn.linear_b_param(C, K, N, wt, None, C.from_numpy(x)))
    np.testing.assert_array_equal(got2, got)
    # cross-check against the exact-f32 CUDA-core kernel on the device
    C.set_option("gemm", 1)
    try:
        simt = C.to_numpy(C.linear(C.from_numpy(x), wt))
    finally:
        C.set_option("gemm", 0)
    np.testing.assert_allclose(got, simt, rtol=1e-4, atol=1e-4 * np.sqrt(K))


# shapes above the kernel's own threshold (one and a half 256 x 256 tiles per SM pair), one of them
# ragged in every dimension, and small ones that only the forced mode sends there
PAIR_SHAPES = [(2048, 9728, 512, 1), (1300, 12800, 520, 1), (300, 700, 192, 2), (20, 256, 64, 2), (513, 130, 1032, 2)]


@pytest.mark.parametrize("M,N,K,mode", PAIR_SHAPES)
def test_pair_cta_linear(oracle, cuda_bf16, M, N, K, mode):
    """The CTA-pair GEMM (tcgen05 cta_group::2, option "pair_cta") against the f32 checker and
    against the one-CTA kernels on the same operands."""
    x = synth.bf16_round(rnd((M, K)))
    w = synth.bf16_round(rnd((N, K), 0.05))
    C = cuda_bf16
    wt, xt = C.from_numpy(w), C.from_numpy(x)
    try:
        C.set_option("pair_cta", 0)
        base = C.to_numpy(C.linear(xt, wt))
        C.set_option("pair_cta", mode)
        got = C.to_numpy(C.linear(xt, wt))
    finally:
        C.set_option("pair_cta", 1)
    B = oracle
    want = B.to_numpy(nn.linear_b_param(B, K, N, B.from_numpy(w), None, B.from_numpy(x.reshape(1, M, K)))).reshape(M, N)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4 * np.sqrt(K))
    np.testing.assert_allclose(got, base, rtol=1e-5, atol=1e-5 * np.sqrt(K))


def test_pair_cta_linear_exact_small_integers(cuda_bf16):
    # integers survive bf16 and f32 accumulation exactly: any slip in which CTA holds which
    # rows of W or which half of the tokens shows as a wrong integer
    C = cuda_bf16
    M, N, K = 700, 600, 192
    x = RNG.integers(-3, 4, size=(M, K)).astype(np.float32)
    w = RNG.integers(-3, 4, size=(N, K)).astype(np.float32)
    C.set_option("pair_cta", 2)
    try:
        got = C.to_numpy(C.linear(C.from_numpy(x), C.from_numpy(w)))
    finally:
        C.set_option("pair_cta", 1)
    np.testing.assert_array_equal(got, x @ w.T)


@pytest.mark.parametrize("M,F,K,act", [(1024, 2560, 256, 0), (1100, 3008, 264, 1), (70, 96, 64, 0), (2048, 9472, 512, 0), (300, 1000, 128, 0)])
@pytest.mark.parametrize("mode", [0, 2])
def test_linear_glu(oracle, cuda_bf16, M, F, K, act, mode):
    """cg_linear_glu: act(x Wg^T) * (x Wu^T) in one kernel (the one-CTA kernel with two
    accumulators, and the CTA-pair kernel with gate and up rows interleaved) against the op
    chain of the FFN (catgrad-llm/src/models/llama.rs:24-28) on the checker; the result is
    rounded once to bf16."""
    x = synth.bf16_round(rnd((M, K)))
    w = synth.bf16_round(rnd((2 * F, K), 0.05))
    C = cuda_bf16
    C.set_option("pair_cta", mode)
    try:
        y = C.linear_glu(C.from_numpy(x), C.from_numpy(w), act)
        assert C.storage_of(y) == 2
        got = C.to_numpy(y)
    finally:
        C.set_option("pair_cta", 1)
    B = oracle
    xb = B.from_numpy(x.reshape(1, M, K))
    g = nn.linear_b_param(B, K, F, B.from_numpy(np.ascontiguousarray(w[:F])), None, xb)
    u = nn.linear_b_param(B, K, F, B.from_numpy(np.ascontiguousarray(w[F:])), None, xb)
    want = B.to_numpy(B.mul(nn.silu(B, g) if act == 0 else nn.gelu(B, g), u)).reshape(M, F)
    np.testing.assert_allclose(got, want, rtol=2.0 ** -7, atol=1e-4)


def test_bf16_operand_is_rounded_once_for_all_its_readers(cuda_bf16):
    """q, k and v (or gate and up) read the same activations: the bf16 copy a tensor-core GEMM
    makes of them is kept with the tensor and serves the later GEMMs, through `linear` and
    through the trait's matmul on a transposed weight alike; results are unchanged."""
    C = cuda_bf16
    M, K, N = 96, 256, 384
    x = rnd((1, M, K))
    w1, w2 = synth.bf16_round(rnd((N, K), 0.05)), synth.bf16_round(rnd((N, K), 0.05))
    t1, t2 = C.from_numpy(w1), C.from_numpy(w2)
    x0 = C.from_numpy(x)
    xt = C.add(x0, x0)  # a computed tensor is stored f32 (an upload of rank >= 2 would be bf16 already)
    assert C.storage_of(xt) == 0
    n0 = C.launch_count()
    a = C.to_numpy(C.linear(xt, t1))
    n1 = C.launch_count()
    b = C.to_numpy(nn.linear_b_param(C, K, N, t2, None, xt))
    n2 = C.launch_count()
    fresh = C.to_numpy(C.linear(C.add(x0, x0), t2))
    np.testing.assert_array_equal(b, fresh)
    assert (n1 - n0) - (n2 - n1) == 1  # the first GEMM rounds the activations, the second does not
    xb = 2 * synth.bf16_round(x)
    np.testing.assert_allclose(a, (xb.reshape(M, K) @ w1.T).reshape(1, M, N), rtol=1e-4, atol=1e-3)


def test_tensor_core_linear_exact_small_integers(cuda_bf16):
    # integers survive bf16 and f32 accumulation exactly: any layout or descriptor slip shows
    C = cuda_bf16
    M, N, K = 20, 256, 192
    x = RNG.integers(-3, 4, size=(M, K)).astype(np.float32)
    w = RNG.integers(-3, 4, size=(N, K)).astype(np.float32)
    got = C.to_numpy(C.linear(C.from_numpy(x), C.from_numpy(w)))
    np.testing.assert_array_equal(got, x @ w.T)


@pytest.mark.parametrize("b,nh,nkv,s,d", [(1, 4, 2, 32, 64), (2, 8, 2, 70, 64), (1, 4, 4, 130, 128), (1, 2, 1, 65, 256)])
@pytest.mark.parametrize("window,cap", [(0, 0.0), (16, 0.0), (0, 20.0)])
def test_fused_attention(oracle, cuda, b, nh, nkv, s, d, window, cap):
    q = synth.bf16_round(rnd((b, nh, s, d)))
    k = synth.bf16_round(rnd((b, nkv, s, d)))
    v = synth.bf16_round(rnd((b, nkv, s, d)))
    got = cuda.to_numpy(cuda.fused_attention(cuda.from_numpy(q), cuda.from_numpy(k), cuda.from_numpy(v), window, cap))
    B = oracle
    rep = nh // nkv
    want = np.empty_like(q)
    for bi in range(b):  # the reference graph is batch-1
        qq = B.from_numpy(q[bi:bi + 1])
        kk = H.repeat_kv(B, rep, B.from_numpy(k[bi:bi + 1]))
        vv = H.repeat_kv(B, rep, B.from_numpy(v[bi:bi + 1]))
        attn = B.matmul(qq, B.transpose(kk, 2, 3))
        sh = attn.shape
        attn = B.div(attn, nn.constant(B, float(np.sqrt(np.float32(d))), sh))
        if cap > 0:
            attn = B.mul(nn.constant(B, cap, sh), nn.tanh(B, B.div(attn, nn.constant(B, cap, sh))))
        mask = H.causal_mask(B, s)
        if window > 0:  # a second lt: keys more than window-1 behind the query
            i = B.broadcast(B.arange(s), (s, s))
            j = B.broadcast(B.reshape(B.arange(s), (s, 1)), (s, s))
            far = B.lt(B.add(i, B.broadcast(B.ndarray_from_vec_u32([window - 1], ()), (s, s))), j)
            mask = B.add(mask, B.mul(B.cast(far, cg.F32), nn.constant(B, H.F32_MIN, (s, s))))
        attn = B.add(attn, B.broadcast(mask, sh))
        attn = nn.softmax(B, attn)
        want[bi] = B.to_numpy(B.matmul(attn, vv))[0]
    # probabilities are rounded to bf16 before the second product and the result is stored bf16
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-2)
    assert np.abs(got - want).mean() < 3e-3


@pytest.mark.gpu
def test_randn_is_a_function_of_seed_and_index(cuda, cuda_bf16):
    """cg_randn: counter-based normals -- same seed, same tensor; moments as asked; storage follows
    the context's upload rule (bf16 for matrices on a bf16-precision context)."""
    a = cuda.to_numpy(cuda.randn((257, 1001), 42, std=0.02))
    b = cuda.to_numpy(cuda.randn((257, 1001), 42, std=0.02))
    c = cuda.to_numpy(cuda.randn((257, 1001), 43, std=0.02))
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    assert abs(float(((a / 0.02) ** 4).mean()) - 3.0) < 0.1  # kurtosis of a normal
    g = cuda.to_numpy(cuda.randn((64,), 0, std=0.0, mean=1.0))
    assert (g == 1.0).all()
    t = cuda_bf16.randn((64, 64), 7, std=0.02)
    assert cuda_bf16.storage_of(t) == 2 and cuda_bf16.to_numpy(t).shape == (64, 64)
    assert cuda.to_numpy(cuda.randn((0, 5), 1)).shape == (0, 5)


@pytest.mark.gpu
@pytest.mark.parametrize("b,nh,nkv,s,d", [(1, 4, 2, 128, 128), (2, 8, 2, 200, 64), (1, 4, 4, 385, 128), (1, 2, 1, 1000, 128),
                                          (3, 4, 1, 64, 64)])
@pytest.mark.parametrize("variant", [1, 2], ids=["keys128", "keys64"])
def test_fused_attention_tcgen05(cuda, b, nh, nkv, s, d, variant):
    """The TMEM / tcgen05 prefill attention against the mma.sync kernel (itself checked against
    the reference op stream above) and against a float64 numpy evaluation."""
    q = synth.bf16_round(rnd((b, nh, s, d)))
    k = synth.bf16_round(rnd((b, nkv, s, d)))
    v = synth.bf16_round(rnd((b, nkv, s, d)))
    args = [cuda.from_numpy(q), cuda.from_numpy(k), cuda.from_numpy(v)]
    cuda.set_option("fa", 0)
    base = cuda.to_numpy(cuda.fused_attention(*args))
    cuda.set_option("fa", variant)
    try:
        got = cuda.to_numpy(cuda.fused_attention(*args))
    finally:
        cuda.set_option("fa", 1)
    rep = nh // nkv
    kk, vv = np.repeat(k, rep, axis=1).astype(np.float64), np.repeat(v, rep, axis=1).astype(np.float64)
    sc = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), kk) / np.sqrt(d)
    sc = np.where(np.tril(np.ones((s, s), bool)), sc, -np.inf)
    pr = np.exp(sc - sc.max(-1, keepdims=True))
    want = np.einsum("bhqk,bhkd->bhqd", pr / pr.sum(-1, keepdims=True), vv)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-2)
    assert np.abs(got - want).mean() < 3e-3
    np.testing.assert_allclose(got, base, rtol=0, atol=2e-2)
