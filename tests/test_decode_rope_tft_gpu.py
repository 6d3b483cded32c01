"""Parity of the decode, RoPE and TFT kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle
from gpu_util import bf16_round
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


class Decoder:
    def __init__(self, cuda, B, n_heads, n_kv, hs, seq_len, bf16, theta=10000.0):
        self.cuda, self.B, self.nh, self.nkv, self.hs, self.seq_len, self.bf16 = cuda, B, n_heads, n_kv, hs, seq_len, bf16
        self.h = cuda.CreateDecode(B, n_heads, n_kv, hs, seq_len, bf16, theta)
        alloc = cuda.AllocMemoryBf16 if bf16 else cuda.AllocMemory
        kv_dim = n_kv * hs
        self.hKc, self.hVc = alloc(B * seq_len * kv_dim), alloc(B * seq_len * kv_dim)
        self.hQ, self.hK, self.hV = cuda.AllocMemory(B * n_heads * hs), cuda.AllocMemory(B * kv_dim), cuda.AllocMemory(B * kv_dim)
        self.hPos, self.hOut = cuda.AllocMemory(B), cuda.AllocMemory(B * n_heads * hs)

    def set_cache(self, kc, vc):
        self.cuda.SetMemory(self.hKc, kc)
        self.cuda.SetMemory(self.hVc, vc)

    def step(self, q, k, v, pos, max_len=None):
        c = self.cuda
        c.SetMemory(self.hQ, q); c.SetMemory(self.hK, k); c.SetMemory(self.hV, v)
        c.SetMemoryInt32(self.hPos, pos)
        c.DecodeStep(self.h, self.hQ, self.hK, self.hV, self.hKc, self.hVc, self.hPos, max_len or int(max(pos)) + 1,
                     self.hOut)
        return c.GetMemory(self.hOut, q.size).reshape(q.shape)

    def caches(self):
        n = self.B * self.seq_len * self.nkv * self.hs
        shape = (self.B, self.seq_len, self.nkv * self.hs)
        return self.cuda.GetMemory(self.hKc, n).reshape(shape), self.cuda.GetMemory(self.hVc, n).reshape(shape)

    def close(self):
        for h in (self.hKc, self.hVc, self.hQ, self.hK, self.hV, self.hPos, self.hOut):
            self.cuda.FreeMemory(h)
        self.cuda.FreeDecode(self.h)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("B,n_heads,n_kv,hs,seq_len", [
    (1, 4, 4, 64, 300), (5, 8, 8, 128, 1500), (3, 8, 2, 128, 700), (2, 16, 2, 64, 520), (4, 32, 32, 128, 4096)])
def test_decode_step_matches_oracle(cuda, B, n_heads, n_kv, hs, seq_len, bf16):
    """One new token for B sequences of ragged length (llama2_cpu.cpp:290-342): RoPE on q/k, cache
    append at pos, attention over 0..pos."""
    rng = np.random.default_rng(B * 1000 + n_heads + seq_len)
    dim, kv_dim = n_heads * hs, n_kv * hs
    pos = rng.integers(0, seq_len, B).astype(np.int32)
    pos[0] = seq_len - 1
    if B > 1:
        pos[1] = 0
    kc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    if bf16:
        kc, vc = bf16_round(kc), bf16_round(vc)
    q = rng.standard_normal((B, dim)).astype(np.float32)
    k = rng.standard_normal((B, kv_dim)).astype(np.float32)
    v = rng.standard_normal((B, kv_dim)).astype(np.float32)
    d = Decoder(cuda, B, n_heads, n_kv, hs, seq_len, bf16)
    d.set_cache(kc, vc)
    out = d.step(q, k, v, pos)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    ref = oracle.llama_decode(q, k, v, kc_ref, vc_ref, pos, n_heads, n_kv)
    if bf16:
        # the kernel attends to the bf16-rounded new row, as a later step would read it back
        for b in range(B):
            kc_ref[b, pos[b]] = bf16_round(kc_ref[b, pos[b]])
            vc_ref[b, pos[b]] = bf16_round(vc_ref[b, pos[b]])
        ref = oracle.llama_decode(q, k, v, kc_ref.copy(), vc_ref.copy(), pos, n_heads, n_kv)
    assert rel_err(out, ref) < (2e-2 if bf16 else 1e-4)
    if not bf16:
        assert rel_err(out, ref) < 2e-5
    kc_got, vc_got = d.caches()
    for b in range(B):  # the appended rows, and nothing else, changed
        np.testing.assert_allclose(kc_got[b, pos[b]], kc_ref[b, pos[b]], atol=2e-6 if not bf16 else 2e-2)
        np.testing.assert_allclose(vc_got[b, pos[b]], vc_ref[b, pos[b]], atol=0 if not bf16 else 2e-2)
        keep = np.arange(seq_len) != pos[b]
        np.testing.assert_array_equal(kc_got[b, keep], kc[b, keep])
        np.testing.assert_array_equal(vc_got[b, keep], vc[b, keep])
    d.close()


def test_decode_generation_loop_matches_reference_twin(cuda, tmp_path):
    """Token-by-token decode from an empty cache, against the reference's own TransformerCpu
    (compiled from its source) on a synthetic one-layer checkpoint with wo = I."""
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference twin not available")
    dim, n_heads, hs, seq_len = 256, 4, 64, 40
    rng = np.random.default_rng(0)
    hidden, vocab = 8, 16
    w = {"rms_att_weight": 1 + 0.02 * rng.standard_normal((1, dim)), "rms_ffn_weight": np.ones((1, dim)),
         "rms_final_weight": np.ones(dim), "token_embedding_table": rng.standard_normal((vocab, dim)),
         "wq": 0.1 * rng.standard_normal((1, dim, dim)), "wk": 0.1 * rng.standard_normal((1, dim, dim)),
         "wv": 0.1 * rng.standard_normal((1, dim, dim)), "wo": np.eye(dim)[None],
         "w1": np.zeros((1, hidden, dim)), "w2": np.zeros((1, dim, hidden)), "w3": np.zeros((1, hidden, dim))}
    w = {k_: v_.astype(np.float32) for k_, v_ in w.items()}
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, 1, n_heads, n_heads, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    d = Decoder(cuda, 1, n_heads, n_heads, hs, seq_len, False)
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        xb = oracle.rmsnorm(w["token_embedding_table"][tokens[pos]], w["rms_att_weight"][0])
        q, k, v = (oracle.gemv(w[n][0], xb)[None] for n in ("wq", "wk", "wv"))
        out = d.step(q, k, v, np.array([pos], np.int32))
        assert rel_err(out[0], ref.state("xb2")) < 2e-5
    kc, vc = d.caches()
    np.testing.assert_allclose(kc[0].ravel(), ref.state("key_cache"), atol=2e-6)
    np.testing.assert_array_equal(vc[0].ravel(), ref.state("value_cache"))
    d.close()
    ref.close()


@pytest.mark.parametrize("B,T,H,D", [(2, 7, 3, 8), (1, 128, 12, 64), (3, 33, 4, 128)])
def test_rope_forward_backward(cuda, B, T, H, D):
    """ROPE_FWD / ROPE_BWD on a (B,T,H,D) tensor (rope.cu:784-864)."""
    rng = np.random.default_rng(T)
    x = rng.standard_normal((B, T, H, D)).astype(np.float32)
    cos_t, sin_t = oracle.rope_tables(T, D)
    h = cuda.CreateRope(0, 0, x.size, B, T, H, D, 10000.0)
    hX, hY = cuda.AllocMemory(x), cuda.AllocMemory(x.size)
    cuda.RopeForward(h, x.size, hX, hY)
    y = cuda.GetMemory(hY, x.size).reshape(x.shape)
    np.testing.assert_allclose(y, oracle.rope_apply(x, T, H, D, cos_t, sin_t), atol=1e-6)
    cuda.RopeBackward(h, x.size, hX, hY, hX)  # hYdiff -> hXdiff
    back = cuda.GetMemory(hX, x.size).reshape(x.shape)
    np.testing.assert_allclose(back, x, atol=2e-6)
    # decode form: one position, table shifted by pos * D/2 (MultiheadAttentionLayer.cs:676-684)
    one = x[:, 3:4].copy()
    hO, hO2 = cuda.AllocMemory(one), cuda.AllocMemory(one.size)
    cuda.RopeForward(h, one.size, hO, hO2, 3 * D // 2)
    got = cuda.GetMemory(hO2, one.size).reshape(one.shape)
    np.testing.assert_allclose(got, oracle.rope_apply(one, T, H, D, cos_t, sin_t, freq_offset=3 * D // 2), atol=1e-6)
    # the first H*D/2 pairs sit at table position 0 + offset, i.e. position 3 (the reference's B = 1 use)
    np.testing.assert_allclose(got[0], y[0, 3:4], atol=1e-6)
    for m in (hX, hY, hO, hO2):
        cuda.FreeMemory(m)
    # a shared index returns the same handle (memory.h:2182-2226)
    s1 = cuda.CreateRope(7, 0, x.size, B, T, H, D, 10000.0)
    s2 = cuda.CreateRope(7, 0, x.size, B, T, H, D, 10000.0)
    assert s1 == s2
    cuda.FreeRope(s1); cuda.FreeRope(s2); cuda.FreeRope(h)


@pytest.mark.parametrize("B,H,Nh,Nf,d,self_attn", [(4, 4, 8, 4, 16, True), (256, 4, 168, 24, 64, True),
                                                    (16, 4, 168, 24, 64, False), (3, 2, 90, 30, 32, True),
                                                    (2, 3, 23, 7, 32, False), (2, 2, 200, 20, 16, True)])
def test_tft_interpretable_attention(cuda, B, H, Nh, Nf, d, self_attn):
    """BASELINE config 4: shared V, per-head Q/K, head-means of P and of P V
    (MultiHeadAttentionInterpLayer.cs:728-759); Nq = num_future (one bottom) or Nq = Nk (four bottoms)."""
    rng = np.random.default_rng(B + Nh)
    Nk = Nh + Nf
    Nq = Nf if self_attn else Nk
    q = rng.standard_normal((B, H, Nq, d)).astype(np.float32)
    k = rng.standard_normal((B, H, Nk, d)).astype(np.float32)
    v = rng.standard_normal((B, Nk, d)).astype(np.float32)
    mask = oracle.tft_mask(Nh, Nf) if self_attn else (np.triu(np.ones((Nk, Nk), np.float32), 1))
    hs = [cuda.AllocMemory(a) for a in (q, k, v, mask)]
    hOut, hAttn = cuda.AllocMemory(B * Nq * d), cuda.AllocMemory(B * Nq * Nk)
    cuda.TftAttnForward(hs[0], hs[1], hs[2], hs[3], B, H, Nq, Nk, d, hOut, hAttn)
    out = cuda.GetMemory(hOut, B * Nq * d).reshape(B, Nq, d)
    attn = cuda.GetMemory(hAttn, B * Nq * Nk).reshape(B, Nq, Nk)
    ref_out, ref_attn = oracle.tft_forward(q, k, v, mask, f64=True)
    assert rel_err(out, ref_out) < 2e-5
    assert rel_err(attn, ref_attn) < 2e-5
    np.testing.assert_allclose(attn.sum(-1), 1.0, atol=1e-5)
    for h in hs + [hOut, hAttn]:
        cuda.FreeMemory(h)


@pytest.mark.parametrize("B,H,Nh,Nf,d,self_attn,with_attn_grad", [
    (3, 4, 8, 4, 16, True, True), (64, 4, 168, 24, 64, True, True), (8, 4, 168, 24, 64, False, False),
    (5, 3, 21, 7, 32, True, False),
    # ragged shapes of the tiled kernel: Nk not a multiple of four, a last row tile of 6 and of 23 rows
    (2, 3, 23, 7, 32, False, True), (2, 4, 150, 41, 64, False, True), (3, 2, 150, 41, 16, True, False),
    # beyond the tiled kernel (Nk > 192, head size 24): the generic kernel
    (2, 2, 200, 20, 16, True, True), (2, 2, 30, 10, 24, False, True)])
def test_tft_interpretable_attention_backward(cuda, B, H, Nh, Nf, d, self_attn, with_attn_grad):
    """Gradients of the TFT attention block w.r.t. Q, K and the shared V, from the gradients of both
    outputs (MultiHeadAttentionInterpLayer.cs:780-859), against the fp64 oracle."""
    rng = np.random.default_rng(B * 7 + Nh)
    Nk = Nh + Nf
    Nq = Nf if self_attn else Nk
    q = rng.standard_normal((B, H, Nq, d)).astype(np.float32)
    k = rng.standard_normal((B, H, Nk, d)).astype(np.float32)
    v = rng.standard_normal((B, Nk, d)).astype(np.float32)
    mask = oracle.tft_mask(Nh, Nf) if self_attn else np.triu(np.ones((Nk, Nk), np.float32), 1)
    d_out = rng.standard_normal((B, Nq, d)).astype(np.float32)
    d_attn = rng.standard_normal((B, Nq, Nk)).astype(np.float32) if with_attn_grad else None
    hs = [cuda.AllocMemory(a) for a in (q, k, v, mask, d_out)]
    hdA = cuda.AllocMemory(d_attn) if with_attn_grad else 0
    hdQ, hdK, hdV = cuda.AllocMemory(q.size), cuda.AllocMemory(k.size), cuda.AllocMemory(v.size)
    cuda.TftAttnBackward(hs[0], hs[1], hs[2], hs[3], hs[4], hdA, B, H, Nq, Nk, d, hdQ, hdK, hdV)
    ref = oracle.tft_backward(q, k, v, mask, d_out, d_attn, f64=True)
    for h, r_, a in zip((hdQ, hdK, hdV), ref, (q, k, v)):
        assert rel_err(cuda.GetMemory(h, a.size).reshape(a.shape), r_) < 2e-5
    for h in hs + [hdQ, hdK, hdV] + ([hdA] if hdA else []):
        cuda.FreeMemory(h)


@pytest.mark.parametrize("bf16_weights", [False, True])
def test_decode_block_projections_match_reference_twin(cuda, tmp_path, bf16_weights):
    """The whole attention block of one decode step (llama2_gpu.cpp:56-81): fused RMSNorm + q,k,v
    projections, RoPE + cache append + attention, Wo projection + residual, against the reference's own
    TransformerCpu on a synthetic one-layer checkpoint."""
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference twin not available")
    dim, n_heads, hs, seq_len = 512, 8, 64, 24
    rng = np.random.default_rng(3)
    hidden, vocab = 8, 16
    mk = lambda *s: (0.05 * rng.standard_normal(s)).astype(np.float32)
    w = {"rms_att_weight": (1 + 0.1 * rng.standard_normal((1, dim))).astype(np.float32),
         "rms_ffn_weight": np.ones((1, dim), np.float32), "rms_final_weight": np.ones(dim, np.float32),
         "token_embedding_table": rng.standard_normal((vocab, dim)).astype(np.float32),
         "wq": mk(1, dim, dim), "wk": mk(1, dim, dim), "wv": mk(1, dim, dim), "wo": mk(1, dim, dim),
         "w1": np.zeros((1, hidden, dim), np.float32), "w2": np.zeros((1, dim, hidden), np.float32),
         "w3": np.zeros((1, hidden, dim), np.float32)}
    if bf16_weights:  # the reference then runs on the same (bf16-representable) weights in fp32
        for n_ in ("wq", "wk", "wv", "wo"):
            w[n_] = bf16_round(w[n_])
    path = tmp_path / "blk.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, 1, n_heads, n_heads, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    alloc_w = cuda.AllocMemoryBf16 if bf16_weights else cuda.AllocMemory
    hW = {n_: alloc_w(w[n_][0]) for n_ in ("wq", "wk", "wv", "wo")}
    hRms = cuda.AllocMemory(w["rms_att_weight"][0])
    d = Decoder(cuda, 1, n_heads, n_heads, hs, seq_len, False)
    hX, hAttn = cuda.AllocMemory(dim), cuda.AllocMemory(dim)
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        x0 = w["token_embedding_table"][tokens[pos]]
        ref.forward(int(tokens[pos]), pos)
        cuda.SetMemory(hX, x0)
        cuda.DecodeQkv(hX, hRms, hW["wq"], hW["wk"], hW["wv"], 1, dim, dim, d.hQ, d.hK, d.hV, 1e-5)
        v_got = cuda.GetMemory(d.hV, dim)
        assert rel_err(v_got, ref.state("v")) < 2e-5
        cuda.SetMemoryInt32(d.hPos, np.array([pos], np.int32))
        cuda.DecodeStep(d.h, d.hQ, d.hK, d.hV, d.hKc, d.hVc, d.hPos, pos + 1, hAttn)
        cuda.DecodeOut(hAttn, hW["wo"], 1, dim, hX)
        x1 = cuda.GetMemory(hX, dim)
        assert rel_err(x1 - x0, ref.state("xb2")) < 5e-5   # the residual update equals Wo . attention output
    kc, _ = d.caches()
    assert rel_err(kc[0].ravel(), ref.state("key_cache")) < 2e-5
    d.close()
    ref.close()


@pytest.mark.parametrize("B", [1, 3, 8, 13])
def test_fused_rmsnorm_qkv_batched(cuda, B):
    """Several sequences share one pass over the weights; GQA-shaped (kv_dim < dim) projections."""
    rng = np.random.default_rng(B)
    dim, kv_dim = 1024, 256
    x = rng.standard_normal((B, dim)).astype(np.float32)
    rw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    wq, wk, wv = ((0.05 * rng.standard_normal(s)).astype(np.float32) for s in ((dim, dim), (kv_dim, dim), (kv_dim, dim)))
    hs = [cuda.AllocMemory(a) for a in (x, rw, wq, wk, wv)]
    hQ, hK, hV = cuda.AllocMemory(B * dim), cuda.AllocMemory(B * kv_dim), cuda.AllocMemory(B * kv_dim)
    cuda.DecodeQkv(hs[0], hs[1], hs[2], hs[3], hs[4], B, dim, kv_dim, hQ, hK, hV, 1e-5)
    for b in range(B):
        xn = oracle.rmsnorm(x[b], rw)
        for h, wmat, n in ((hQ, wq, dim), (hK, wk, kv_dim), (hV, wv, kv_dim)):
            got = cuda.GetMemory(h, B * n).reshape(B, n)[b]
            assert rel_err(got, oracle.gemv(wmat, xn)) < 2e-5
    for h in hs + [hQ, hK, hV]:
        cuda.FreeMemory(h)


def test_kv_cache_decode_without_rope_matches_causal_sdpa(cuda):
    """theta <= 0: the KV-cache generation step of MultiheadAttentionLayer (MultiheadAttentionLayer.cs:713-777:
    append k, v at nPos, scores over 0..nPos, softmax, times V), here for two sequences at once.  Token t of the
    loop must equal row t of the causal SDPA over the whole sequence, and the caches must hold k, v verbatim."""
    rng = np.random.default_rng(11)
    B, H, D, T = 2, 4, 64, 40
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    ref = oracle.sdpa_forward(q, k, v, oracle.causal_mask(T), 1, f64=True)          # (B,H,T,D)
    d = Decoder(cuda, B, H, H, D, T, False, theta=0.0)
    for t in range(T):
        tok = lambda a: np.ascontiguousarray(a[:, :, t, :]).reshape(B, H * D)
        out = d.step(tok(q), tok(k), tok(v), np.full(B, t, np.int32))
        assert rel_err(out, tok(ref)) < 2e-5, t
    kc, vc = d.caches()
    np.testing.assert_array_equal(kc.reshape(B, T, H, D), k.transpose(0, 2, 1, 3))
    np.testing.assert_array_equal(vc.reshape(B, T, H, D), v.transpose(0, 2, 1, 3))
    d.close()
