"""The CPU oracle against the reference's own golden vectors (gpt-pico-csa*), and the
decode restatement against the reference's CPU twin compiled from its source."""
import numpy as np
import pytest

import oracle
from helpers import PICO_BLOCK_CASES, PICO_CASES, csa_backward, csa_forward, csa_qkv, rel_err


@pytest.mark.parametrize("case", list(PICO_CASES))
def test_pico_forward(pico, case):
    H = PICO_CASES[case]
    g = lambda n: pico[f"{case}/{n}"]
    x = g("x")
    T = x.shape[1]
    q, k, v = csa_qkv(x, g("attn_weight"), g("attn_bias"), H)
    np.testing.assert_allclose(q, g("qt"), atol=2e-7)
    mask = oracle.causal_mask(T)
    has_npy = f"{case}/var_att" in pico.files  # csaB ships the text dumps only
    if has_npy:
        np.testing.assert_allclose(v, g("var_vt"), atol=2e-7)
    for f64 in (False, True):
        y, p = oracle.sdpa_forward(q, k, v, mask, 1, f64=f64, want_probs=True)
        if has_npy:
            np.testing.assert_allclose(p, g("var_att"), atol=2e-7)
            np.testing.assert_allclose(y, g("var_y"), atol=2e-7)
    full = csa_forward(x, g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), g("attn_proj_bias"), H,
                       lambda q, k, v: oracle.sdpa_forward(q, k, v, mask, 1))
    np.testing.assert_allclose(full, g("y"), atol=2e-7)


@pytest.mark.parametrize("case", list(PICO_CASES))
def test_pico_backward(pico, case):
    H = PICO_CASES[case]
    g = lambda n: pico[f"{case}/{n}"]
    x = g("x")
    T = x.shape[1]
    q, k, v = csa_qkv(x, g("attn_weight"), g("attn_bias"), H)
    mask = oracle.causal_mask(T)
    dy = g("grad_y_pre_transpose")
    for f64 in (False, True):
        dq, dk, dv = oracle.sdpa_backward(q, k, v, dy, mask, 1, f64=f64)
        np.testing.assert_allclose(dq, g("grad_qt"), atol=2e-8)
        np.testing.assert_allclose(dk, g("grad_kt"), atol=2e-8)
        np.testing.assert_allclose(dv, g("grad_vt"), atol=2e-8)


@pytest.mark.parametrize("case", ["ln", "ln3", "ln3B", "ln-blk"])
def test_pico_layernorm(pico_ln, case):
    """The LayerNorm restatement (layernorm.cu:291-384) against the reference's gpt-pico-ln* vectors: y, and the
    gradient at x from the gradient at y.  The vectors were generated with epsilon 1e-10, the layer's default
    (LayerNormParameter.cs), and no affine part."""
    g = lambda n: pico_ln[f"{case}/{n}"]
    y, stdev = oracle.layernorm_forward(g("x"), 1e-10)
    np.testing.assert_allclose(y, g("y"), atol=3e-7)
    if case == "ln-blk":
        np.testing.assert_allclose(stdev.reshape(g("std").shape), g("std"), rtol=1e-6)
    for y_in in (g("y"), y):
        dx = oracle.layernorm_backward(y_in, g("grad_1a_y"), stdev, 1e-10)
        assert rel_err(dx, g("grad_9_x")) < 1e-6      # fp32 round-off of a gradient with heavy cancellation


@pytest.mark.parametrize("case", list(PICO_BLOCK_CASES))
def test_pico_block_layernorm_then_attention(pico_ln, case):
    """Inside the reference's transformer-block vectors: 1_x -> LayerNorm -> 2_x_ln11 -> attention layer -> 3_x_attn,
    and back: grad_8_x_attn -> grad_9_ln1 -> (LayerNorm backward + the residual branch grad_8_x) -> grad_10_x."""
    H = PICO_BLOCK_CASES[case]
    g = lambda n: pico_ln[f"{case}/{n}"]
    ln1, stdev = oracle.layernorm_forward(g("1_x"), 1e-10)
    np.testing.assert_allclose(ln1, g("2_x_ln11"), atol=3e-7)
    mask = oracle.causal_mask(ln1.shape[1])
    attn = csa_forward(g("2_x_ln11"), g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), g("attn_proj_bias"), H,
                       lambda q, k, v: oracle.sdpa_forward(q, k, v, mask, 1))
    np.testing.assert_allclose(attn, g("3_x_attn"), atol=1e-7)
    d_ln1 = csa_backward(g("2_x_ln11"), g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), H, g("grad_8_x_attn"),
                         lambda q, k, v, dy: oracle.sdpa_backward(q, k, v, dy, mask, 1))
    assert rel_err(d_ln1, g("grad_9_ln1")) < 2e-7
    dx = oracle.layernorm_backward(ln1, g("grad_9_ln1"), stdev, 1e-10) + g("grad_8_x")
    assert rel_err(dx, g("grad_10_x")) < 2e-7


def test_masked_row_is_uniform():
    """Masked logits are -1e29, not -inf: a fully masked row is a uniform distribution
    (math.cu:2994-3002), and a batch key-mask hides keys per batch row (attn.cu:302-311)."""
    rng = np.random.default_rng(0)
    B, H, T, D = 2, 2, 5, 4
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    mask = np.ones((B, T), np.float32)
    mask[1, :] = 0
    mask[0, 3:] = 0
    y, p = oracle.sdpa_forward(q, k, v, mask, 2, want_probs=True)
    np.testing.assert_allclose(p[1], 1.0 / T, atol=1e-7)
    assert np.all(p[0, :, :, 3:] == 0)
    np.testing.assert_allclose(y[1], np.broadcast_to(v[1].mean(axis=1, keepdims=True), v[1].shape), atol=1e-6)


def test_backward_matches_finite_differences():
    rng = np.random.default_rng(1)
    B, H, T, D = 1, 2, 6, 4
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    mask = oracle.causal_mask(T)
    dq, dk, dv = oracle.sdpa_backward(q, k, v, dy, mask, 1, f64=True)

    def loss(q_, k_, v_):
        return float((oracle.sdpa_forward(q_, k_, v_, mask, 1, f64=True) * dy).sum())

    eps = 1e-3
    for arr, grad in ((q, dq), (k, dk), (v, dv)):
        for idx in [(0, 0, 0, 0), (0, 1, 3, 2), (0, 1, 5, 3)]:
            a = arr.copy(); a[idx] += eps
            b = arr.copy(); b[idx] -= eps
            args_p = [a if arr is x else x for x in (q, k, v)]
            args_m = [b if arr is x else x for x in (q, k, v)]
            num = (loss(*args_p) - loss(*args_m)) / (2 * eps)
            assert abs(num - grad[idx]) < 2e-3 * max(1.0, abs(num))


def test_rope_matches_complex_rotation():
    rng = np.random.default_rng(2)
    B, T, H, D = 2, 7, 3, 8
    x = rng.standard_normal((B, T, H, D)).astype(np.float32)
    cos_t, sin_t = oracle.rope_tables(T, D, 10000.0)
    y = oracle.rope_apply(x, T, H, D, cos_t, sin_t)
    freq = 1.0 / (10000.0 ** (np.arange(0, D, 2) / D))
    ang = np.arange(T)[:, None] * freq[None, :]
    xc = x[..., 0::2] + 1j * x[..., 1::2]
    yc = xc * np.exp(1j * ang)[None, :, None, :]
    np.testing.assert_allclose(y[..., 0::2], yc.real, atol=2e-6)
    np.testing.assert_allclose(y[..., 1::2], yc.imag, atol=2e-6)
    back = oracle.rope_apply(y, T, H, D, cos_t, sin_t, backward=True)
    np.testing.assert_allclose(back, x, atol=2e-6)
    # the llama2 table (llama2_cpu.cpp:388-414) is the same table
    fr, fi = oracle.llama_freqs(D, T)
    np.testing.assert_array_equal(fr, cos_t)
    np.testing.assert_array_equal(fi, sin_t)


def test_tft_matches_per_head_sdpa():
    rng = np.random.default_rng(3)
    B, H, Nh, Nf, d = 3, 4, 8, 4, 16
    Nk = Nh + Nf
    q = rng.standard_normal((B, H, Nf, d)).astype(np.float32)
    k = rng.standard_normal((B, H, Nk, d)).astype(np.float32)
    v = rng.standard_normal((B, Nk, d)).astype(np.float32)
    mask = oracle.tft_mask(Nh, Nf)
    assert mask.shape == (Nf, Nk) and mask[0, Nh + 1] == 1 and mask[0, Nh] == 0 and mask[Nf - 1].sum() == 0
    out, attn = oracle.tft_forward(q, k, v, mask, f64=True)
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(d)
    s = np.where(mask[None, None] == 1, -1e29, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    np.testing.assert_allclose(attn, p.mean(1), atol=1e-12)
    np.testing.assert_allclose(out, np.einsum("bij,bjd->bid", p.mean(1), v.astype(np.float64)), atol=1e-12)
    # backward against finite differences of the forward
    d_out = rng.standard_normal(out.shape).astype(np.float32)
    d_attn = rng.standard_normal(attn.shape).astype(np.float32)
    dq, dk, dv = oracle.tft_backward(q, k, v, mask, d_out, d_attn, f64=True)

    def loss(q_, k_, v_):
        o, a = oracle.tft_forward(q_, k_, v_, mask, f64=True)
        return float((o * d_out).sum() + (a * d_attn).sum())

    eps = 1e-3
    for arr, grad, idx in ((q, dq, (1, 2, 3, 5)), (k, dk, (2, 0, 9, 1)), (v, dv, (0, 7, 4))):
        a = arr.copy(); a[idx] += eps
        b = arr.copy(); b[idx] -= eps
        num = (loss(*[a if arr is x else x for x in (q, k, v)]) -
               loss(*[b if arr is x else x for x in (q, k, v)])) / (2 * eps)
        assert abs(num - grad[idx]) < 2e-3 * max(1.0, abs(num))


def _tiny_llama(tmp_path, dim=64, n_heads=4, n_kv_heads=4, seq_len=24, seed=0):
    rng = np.random.default_rng(seed)
    hidden, vocab, hs = 8, 16, dim // n_heads
    kv_dim = n_kv_heads * hs
    w = {
        "rms_att_weight": 1 + 0.02 * rng.standard_normal((1, dim)),
        "rms_ffn_weight": np.ones((1, dim)),
        "rms_final_weight": np.ones(dim),
        "token_embedding_table": rng.standard_normal((vocab, dim)),
        "wq": 0.1 * rng.standard_normal((1, dim, dim)),
        "wk": 0.1 * rng.standard_normal((1, kv_dim, dim)),
        "wv": 0.1 * rng.standard_normal((1, kv_dim, dim)),
        "wo": np.eye(dim)[None],
        "w1": np.zeros((1, hidden, dim)), "w2": np.zeros((1, dim, hidden)), "w3": np.zeros((1, hidden, dim)),
    }
    w = {k: v.astype(np.float32) for k, v in w.items()}
    path = tmp_path / "tiny.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, 1, n_heads, n_kv_heads, vocab, seq_len, w)
    return path, w, vocab


@pytest.mark.skipif(oracle.ref_lib() is None, reason="compiled reference twin not built")
def test_decode_restatement_matches_compiled_reference(tmp_path):
    """Drive the reference's TransformerCpu::forward (llama2_cpu.cpp:264-386) on a synthetic
    one-layer checkpoint with wo = I, so m_state.xb2 is the attention output, and compare
    the restated decode step bit-for-bit."""
    dim, n_heads, seq_len = 64, 4, 24
    path, w, vocab = _tiny_llama(tmp_path, dim, n_heads, n_heads, seq_len)
    ref = oracle.RefLlama(path)
    assert (ref.dim, ref.n_heads, ref.seq_len) == (dim, n_heads, seq_len)
    kc = np.zeros((1, seq_len, dim), np.float32)
    vc = np.zeros((1, seq_len, dim), np.float32)
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        x = w["token_embedding_table"][tokens[pos]]
        ref.forward(int(tokens[pos]), pos)
        xb = oracle.rmsnorm(x, w["rms_att_weight"][0])
        q = oracle.gemv(w["wq"][0], xb)
        k = oracle.gemv(w["wk"][0], xb)
        v = oracle.gemv(w["wv"][0], xb)
        out, q_rot, k_rot, att = oracle.llama_decode(q[None], k[None], v[None], kc, vc, [pos], n_heads, n_heads,
                                                     want_att=True)
        np.testing.assert_array_equal(q_rot[0], ref.state("q"))
        np.testing.assert_array_equal(k_rot[0], ref.state("k"))
        np.testing.assert_array_equal(kc[0].ravel(), ref.state("key_cache"))
        np.testing.assert_array_equal(vc[0].ravel(), ref.state("value_cache"))
        ref_att = ref.state("att").reshape(n_heads, seq_len)[:, :pos + 1]
        np.testing.assert_array_equal(att[0, :, :pos + 1], ref_att)
        np.testing.assert_array_equal(out[0], ref.state("xb2"))
    ref.close()


def test_decode_gqa_matches_expanded_heads():
    """n_kv_heads < n_heads (kv_mul, llama2_cpu.cpp:272,315): same result as repeating kv heads."""
    rng = np.random.default_rng(7)
    B, n_heads, n_kv, hs, seq_len = 3, 8, 2, 16, 40
    dim, kv_dim = n_heads * hs, n_kv * hs
    pos = np.array([5, 39, 17], np.int32)
    kc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    q = rng.standard_normal((B, dim)).astype(np.float32)
    k = rng.standard_normal((B, kv_dim)).astype(np.float32)
    v = rng.standard_normal((B, kv_dim)).astype(np.float32)
    rep = lambda a: np.ascontiguousarray(np.repeat(a.reshape(*a.shape[:-1], n_kv, hs), n_heads // n_kv, axis=-2)
                                         .reshape(*a.shape[:-1], dim))
    out = oracle.llama_decode(q, k, v, kc.copy(), vc.copy(), pos, n_heads, n_kv)
    out_full = oracle.llama_decode(q, rep(k), rep(v), rep(kc), rep(vc), pos, n_heads, n_heads)
    np.testing.assert_array_equal(out, out_full)


@pytest.mark.skipif(oracle.ref_lib() is None, reason="compiled reference twin not built")
def test_whole_step_restatement_matches_compiled_reference(tmp_path):
    """oracle.llama_forward (attention + feed-forward + classifier over several layers) against the
    logits of the reference's TransformerCpu::forward (llama2_cpu.cpp:264-386), token by token."""
    dim, hidden, n_layers, n_heads, vocab, seq_len = 64, 88, 3, 4, 32, 12
    rng = np.random.default_rng(3)
    g = lambda *s: (0.15 * rng.standard_normal(s)).astype(np.float32)
    w = {"rms_att_weight": 1 + g(n_layers, dim), "rms_ffn_weight": 1 + g(n_layers, dim), "rms_final_weight": 1 + g(dim),
         "token_embedding_table": rng.standard_normal((vocab, dim)).astype(np.float32),
         "wq": g(n_layers, dim, dim), "wk": g(n_layers, dim, dim), "wv": g(n_layers, dim, dim), "wo": g(n_layers, dim, dim),
         "w1": g(n_layers, hidden, dim), "w2": g(n_layers, dim, hidden), "w3": g(n_layers, hidden, dim)}
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_heads, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    cfg = dict(dim=dim, hidden_dim=hidden, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_heads, vocab_size=vocab,
               seq_len=seq_len)
    kc = np.zeros((n_layers, 1, seq_len, dim), np.float32)
    vc = np.zeros((n_layers, 1, seq_len, dim), np.float32)
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        logits = oracle.llama_forward(cfg, w, kc, vc, [tokens[pos]], [pos])
        # same operations in the same order; the SwiGLU exp may differ in the last bit between numpy and libm
        np.testing.assert_allclose(logits[0], ref.state("logits"), rtol=0, atol=2e-6 * np.abs(ref.state("logits")).max())
    np.testing.assert_allclose(kc.ravel(), ref.state("key_cache"), rtol=0, atol=5e-6)
    ref.close()


def test_layernorm_restatement_against_closed_form():
    """The op-by-op LayerNorm (layernorm.cu:291-384) against the textbook formulas in float64."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 5, 48)).astype(np.float32) * 2 + 0.5
    dy = rng.standard_normal(x.shape).astype(np.float32)
    eps = 1e-5
    y, sd = oracle.layernorm_forward(x, eps)
    x64 = x.astype(np.float64)
    mu = x64.mean(-1, keepdims=True)
    sd64 = np.sqrt(((x64 - mu) ** 2).mean(-1, keepdims=True) + eps)
    np.testing.assert_allclose(y, (x64 - mu) / sd64, atol=2e-6)
    np.testing.assert_allclose(sd, sd64.ravel(), rtol=1e-6)
    dx = oracle.layernorm_backward(y, dy, sd, eps)
    y64, dy64 = y.astype(np.float64), dy.astype(np.float64)
    ref = (dy64 - (y64 * (y64 * dy64).mean(-1, keepdims=True) + dy64.mean(-1, keepdims=True))) / sd64
    # the reference divides the first rows (= 15) elements of the flat tensor by stdev + eps
    np.testing.assert_allclose(dx, ref, atol=3e-5)
    flat, rows = dx.ravel(), 15
    np.testing.assert_allclose(flat[rows:], ref.ravel()[rows:], atol=3e-6)


def test_rmsnorm_layer_restatement_against_autograd_formula():
    """The op-by-op RMSNorm layer (RMSNormLayer.cs:156-231) against d/dx of w * x / sqrt(mean(x^2)+eps)
    in float64, by central differences on a scalar loss."""
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 6, 40)).astype(np.float32)
    w = (1 + 0.2 * rng.standard_normal(40)).astype(np.float32)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    eps = 1e-5
    f = lambda xx, ww: ww * xx / np.sqrt((xx ** 2).mean(-1, keepdims=True) + eps)
    y, inv = oracle.rmsnorm_layer_forward(x, w, eps)
    np.testing.assert_allclose(y, f(x.astype(np.float64), w.astype(np.float64)), atol=2e-6)
    np.testing.assert_allclose(inv, 1 / np.sqrt((x.astype(np.float64) ** 2).mean(-1) + eps).ravel(), rtol=1e-6)
    dx, dw = oracle.rmsnorm_layer_backward(x, w, dy, eps)
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    loss = lambda xx, ww: (f(xx, ww) * dy64).sum()
    num_dx = np.zeros_like(x64)
    h = 1e-6
    for idx in np.ndindex(*x.shape):
        xp, xm = x64.copy(), x64.copy()
        xp[idx] += h; xm[idx] -= h
        num_dx[idx] = (loss(xp, w64) - loss(xm, w64)) / (2 * h)
    np.testing.assert_allclose(dx, num_dx, atol=5e-6)
    num_dw = np.array([(loss(x64, w64 + h * np.eye(40)[j]) - loss(x64, w64 - h * np.eye(40)[j])) / (2 * h) for j in range(40)])
    np.testing.assert_allclose(dw, num_dw, atol=1e-5)
    # without weights
    y2, _ = oracle.rmsnorm_layer_forward(x, None, eps)
    np.testing.assert_allclose(y2, f(x64, 1.0), atol=2e-6)
    dx2, dw2 = oracle.rmsnorm_layer_backward(x, None, dy, eps)
    assert dw2 is None
