"""Parity of the whole-transformer decode step (token -> logits) and of its feed-forward and
classifier kernels, through the C ABI, against the reference's own TransformerCpu compiled from its
source (llama2_cpu.cpp:264-386) and against the numpy restatement."""
import ctypes as C

import numpy as np
import pytest

import oracle
from gpu_util import bf16_round
from helpers import rel_err

pytestmark = pytest.mark.gpu


def synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab, scale=0.08):
    hs = dim // n_heads
    kv_dim = n_kv * hs
    g = lambda *s: (scale * rng.standard_normal(s)).astype(np.float32)
    return {"rms_att_weight": (1 + 0.05 * rng.standard_normal((n_layers, dim))).astype(np.float32),
            "rms_ffn_weight": (1 + 0.05 * rng.standard_normal((n_layers, dim))).astype(np.float32),
            "rms_final_weight": (1 + 0.05 * rng.standard_normal(dim)).astype(np.float32),
            "token_embedding_table": rng.standard_normal((vocab, dim)).astype(np.float32),
            "wq": g(n_layers, dim, dim), "wk": g(n_layers, kv_dim, dim), "wv": g(n_layers, kv_dim, dim),
            "wo": g(n_layers, dim, dim), "w1": g(n_layers, hidden, dim), "w2": g(n_layers, dim, hidden),
            "w3": g(n_layers, hidden, dim)}


def need_ref():
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference twin not available")


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("dim,hidden,n_layers,n_heads,n_kv", [(256, 344, 3, 4, 4), (512, 1376, 2, 4, 4), (1024, 96, 1, 8, 8)])
def test_generation_matches_reference_transformer(tmp_path, dim, hidden, n_layers, n_heads, n_kv, use_graph):
    """Token by token from an empty cache: logits of every step and the caches at the end equal
    TransformerCpu::forward's on the same checkpoint file."""
    need_ref()
    from mycaffe_b200.llama2 import TransformerGpu
    vocab, seq_len = 96, 36
    rng = np.random.default_rng(dim + n_layers)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    t = TransformerGpu(0, use_graph=use_graph)
    t.build(str(path))
    assert t.config == dict(dim=dim, hidden_dim=hidden, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv,
                            vocab_size=vocab, seq_len=seq_len)
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        got = t.forward(int(tokens[pos]), pos)
        assert rel_err(got, ref.state("logits")) < 1e-4, pos
    kv_dim = n_kv * (dim // n_heads)
    kc = t.key_cache.cpu().numpy().reshape(n_layers, seq_len, kv_dim)
    vc = t.value_cache.cpu().numpy().reshape(n_layers, seq_len, kv_dim)
    assert rel_err(kc.ravel(), ref.state("key_cache")) < 1e-5
    assert rel_err(vc.ravel(), ref.state("value_cache")) < 1e-5
    ref.close()


@pytest.mark.parametrize("dim,hidden,n_layers,n_heads,n_kv,B", [(512, 1376, 2, 4, 2, 1), (1024, 96, 2, 8, 1, 3)])
def test_grouped_query_generation_matches_restated_step(dim, hidden, n_layers, n_heads, n_kv, B):
    """n_kv_heads < n_heads.  The compiled reference cannot run this (its rope overruns the kv_dim-long
    k vector, llama2_cpu.cpp:243-246), so the checker is the restated step, which the CPU tests pin to
    the compiled reference where n_kv_heads == n_heads."""
    from mycaffe_b200.llama2 import TransformerGpu
    vocab, seq_len = 80, 20
    rng = np.random.default_rng(dim + B)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    w["wcls"] = w["token_embedding_table"]
    cfg = dict(dim=dim, hidden_dim=hidden, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv, vocab_size=vocab,
               seq_len=seq_len)
    t = TransformerGpu(0, batch=B)
    t.load_weights(cfg, w)
    kv_dim = n_kv * (dim // n_heads)
    kc = np.zeros((n_layers, B, seq_len, kv_dim), np.float32)
    vc = np.zeros((n_layers, B, seq_len, kv_dim), np.float32)
    tokens = rng.integers(0, vocab, (seq_len, B))
    for pos in range(seq_len):
        ref = oracle.llama_forward(cfg, w, kc, vc, tokens[pos], [pos] * B)
        got = t.forward_batch(tokens[pos], [pos] * B)
        assert rel_err(got, ref) < 1e-4, pos
    assert rel_err(t.key_cache.cpu().numpy(), kc) < 1e-5


@pytest.mark.parametrize("B,use_graph", [(16, False), (40, True)])
def test_many_sequences_step_on_the_tensor_core_projections(B, use_graph):
    """Above eight sequences every projection of the step (q/k/v, Wo, W1/W3, W2, classifier) is the tensor-core kernel;
    the whole step against the restated reference step, ragged positions included, eager and from a CUDA graph."""
    from mycaffe_b200.llama2 import TransformerGpu
    dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len = 256, 344, 2, 4, 4, 200, 24
    rng = np.random.default_rng(B)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    w["wcls"] = w["token_embedding_table"]
    cfg = dict(dim=dim, hidden_dim=hidden, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv, vocab_size=vocab,
               seq_len=seq_len)
    t = TransformerGpu(0, batch=B, use_graph=use_graph)
    t.load_weights(cfg, w)
    kv_dim = n_kv * (dim // n_heads)
    kc = np.zeros((n_layers, B, seq_len, kv_dim), np.float32)
    vc = np.zeros((n_layers, B, seq_len, kv_dim), np.float32)
    tokens = rng.integers(0, vocab, (seq_len, B))
    for pos in range(10):
        ref = oracle.llama_forward(cfg, w, kc, vc, tokens[pos], [pos] * B)
        got = t.forward_batch(tokens[pos], [pos] * B)
        assert rel_err(got, ref) < 1e-4, pos
    ragged = rng.integers(0, 11, B)                    # every sequence goes on from (or back to) its own position
    ref = oracle.llama_forward(cfg, w, kc, vc, tokens[10], ragged)
    got = t.forward_batch(tokens[10], ragged)
    assert rel_err(got, ref) < 1e-4
    assert rel_err(t.key_cache.cpu().numpy(), kc) < 1e-5


def test_batched_ragged_positions_match_independent_references(tmp_path):
    """B sequences with their own tokens step together; then each steps at its own position.  The
    reference runs one TransformerCpu per sequence."""
    need_ref()
    from mycaffe_b200.llama2 import TransformerGpu
    dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len, B = 256, 344, 2, 4, 4, 64, 40, 5
    rng = np.random.default_rng(11)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len, w)
    refs = [oracle.RefLlama(path) for _ in range(B)]
    t = TransformerGpu(0, batch=B)
    t.build(str(path))
    tokens = rng.integers(0, vocab, (seq_len, B))
    for pos in range(30):
        got = t.forward_batch(tokens[pos], [pos] * B)
        for b in range(B):
            refs[b].forward(int(tokens[pos, b]), pos)
            assert rel_err(got[b], refs[b].state("logits")) < 1e-4, (pos, b)
    # ragged: sequence b goes on from (or back to) its own position
    ragged = np.array([30, 3, 17, 29, 0], np.int32)
    tk = rng.integers(0, vocab, B)
    got = t.forward_batch(tk, ragged)
    for b in range(B):
        refs[b].forward(int(tk[b]), int(ragged[b]))
        assert rel_err(got[b], refs[b].state("logits")) < 1e-4, b
    for r in refs:
        r.close()


def test_bf16_weights_and_cache_within_tolerance(tmp_path):
    """Weights and caches held as bf16: against the reference run on the bf16-rounded weights,
    the difference left is the rounding of the cached rows."""
    need_ref()
    from mycaffe_b200.llama2 import TransformerGpu
    dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len = 256, 344, 2, 4, 4, 64, 24
    rng = np.random.default_rng(5)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    for n in ("wq", "wk", "wv", "wo", "w1", "w2", "w3"):
        w[n] = bf16_round(w[n])
    w["token_embedding_table"] = bf16_round(w["token_embedding_table"])  # shared with the bf16 classifier
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    t = TransformerGpu(0, weights_bf16=True, cache_bf16=True)
    t.build(str(path))
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        got = t.forward(int(tokens[pos]), pos)
        assert rel_err(got, ref.state("logits")) < 2e-2, pos
    ref.close()


def test_step_replays_from_a_cuda_graph(tmp_path):
    """The step only enqueues work and reads tokens and positions from device memory, so one
    captured graph serves every token."""
    need_ref()
    import torch
    from mycaffe_b200.llama2 import TransformerGpu
    dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len = 256, 344, 2, 4, 4, 64, 20
    rng = np.random.default_rng(9)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_kv, vocab)
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_kv, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    t = TransformerGpu(0)
    t.build(str(path))
    tokens = rng.integers(0, vocab, seq_len)
    ref.forward(int(tokens[0]), 0)
    t.forward(int(tokens[0]), 0)             # also the warm-up that sets the kernels' attributes
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph.capture_begin()
        t.enqueue(seq_len, stream=side)      # planned for the longest sequence the cache holds
        graph.capture_end()
    torch.cuda.current_stream().wait_stream(side)
    for pos in range(1, seq_len):
        ref.forward(int(tokens[pos]), pos)
        t._tokens.fill_(int(tokens[pos]))
        t._pos.fill_(pos)
        graph.replay()
        torch.cuda.synchronize()
        assert rel_err(t.logits.cpu().numpy()[0], ref.state("logits")) < 1e-4, pos
    ref.close()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("B,dim,hidden", [(1, 4096, 11008), (3, 4096, 11008), (8, 1024, 2816), (13, 264, 720)])
def test_feed_forward_kernels(B, dim, hidden, bf16):
    """x += W2 (silu(W1 xn) * W3 xn), xn = rmsnorm(x) (llama2_cpu.cpp:352-376)."""
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(B + dim)
    x = rng.standard_normal((B, dim)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    w1, w3 = (0.03 * rng.standard_normal((hidden, dim))).astype(np.float32), (0.03 * rng.standard_normal((hidden, dim))).astype(np.float32)
    w2 = (0.03 * rng.standard_normal((dim, hidden))).astype(np.float32)
    if bf16:
        w1, w2, w3 = bf16_round(w1), bf16_round(w2), bf16_round(w3)
    dev = torch.device("cuda", 0)
    wdt = torch.bfloat16 if bf16 else torch.float32
    up = lambda a, dt=torch.float32: torch.from_numpy(a).to(dev).to(dt).contiguous()
    xd, gd, w1d, w2d, w3d = up(x), up(g), up(w1, wdt), up(w2, wdt), up(w3, wdt)
    hd = torch.empty(B, hidden, device=dev)
    rc = lib.mca_decode_ffn(gd.data_ptr(), 1e-5, w1d.data_ptr(), w2d.data_ptr(), w3d.data_ptr(), int(bf16), B, dim, hidden,
                            hd.data_ptr(), xd.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = np.empty_like(x)
    hid = np.empty((B, hidden), np.float32)
    for b in range(B):
        xn = oracle.rmsnorm(x[b], g)
        a, c = oracle.gemv(w1, xn), oracle.gemv(w3, xn)
        hid[b] = a * (1.0 / (1.0 + np.exp(-a))) * c
        ref[b] = x[b] + oracle.gemv(w2, hid[b])
    assert rel_err(hd.cpu().numpy(), hid) < 1e-4
    assert rel_err(xd.cpu().numpy(), ref) < 1e-4


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("B,dim,vocab", [(1, 4096, 32000), (5, 512, 1001), (9, 264, 97)])
def test_classifier_kernel(B, dim, vocab, bf16):
    """logits = Wcls . rmsnorm(x) (llama2_cpu.cpp:379-383); x itself is left as it was."""
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(vocab)
    x = rng.standard_normal((B, dim)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    wc = (0.05 * rng.standard_normal((vocab, dim))).astype(np.float32)
    if bf16:
        wc = bf16_round(wc)
    dev = torch.device("cuda", 0)
    xd, gd = torch.from_numpy(x).to(dev), torch.from_numpy(g).to(dev)
    wd = torch.from_numpy(wc).to(dev).to(torch.bfloat16 if bf16 else torch.float32)
    out = torch.empty(B, vocab, device=dev)
    rc = lib.mca_decode_logits(xd.data_ptr(), gd.data_ptr(), 1e-5, wd.data_ptr(), int(bf16), B, dim, vocab, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = np.stack([oracle.gemv(wc, oracle.rmsnorm(x[b], g)) for b in range(B)])
    assert rel_err(out.cpu().numpy(), ref) < 1e-4
    np.testing.assert_array_equal(xd.cpu().numpy(), x)


def test_step_rejects_bad_arguments():
    from mycaffe_b200 import _lib, function_ids as ids
    from mycaffe_b200.llama2 import McaLlamaConfig
    lib = _lib.load()
    good = McaLlamaConfig(256, 344, 2, 4, 2, 64, 40)
    assert lib.mca_llama_workspace_floats(C.byref(good), 3, 40) > 0
    assert lib.mca_llama_workspace_floats(C.byref(good), 3, 41) == -1          # longer than the cache
    assert lib.mca_llama_workspace_floats(C.byref(McaLlamaConfig(256, 344, 2, 4, 3, 64, 40)), 1, 8) == -1
    assert lib.mca_llama_forward(C.byref(good), None, None, None, None, 1, 8, None, None) == ids.ERROR_PARAM_NULL


@pytest.mark.parametrize("bf16", [False, True])
def test_feed_forward_and_classifier_function_ids(bf16):
    """The handle-based route (ids 2015 / 2016) a host that owns its tensors through ALLOCMEM takes."""
    from mycaffe_b200 import CudaDnn
    cuda = CudaDnn(0)
    B, dim, hidden, vocab = 3, 512, 1376, 333
    rng = np.random.default_rng(21)
    x = rng.standard_normal((B, dim)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    w1, w3 = (0.05 * rng.standard_normal((hidden, dim))).astype(np.float32), (0.05 * rng.standard_normal((hidden, dim))).astype(np.float32)
    w2, wc = (0.05 * rng.standard_normal((dim, hidden))).astype(np.float32), (0.05 * rng.standard_normal((vocab, dim))).astype(np.float32)
    if bf16:
        w1, w2, w3, wc = (bf16_round(a) for a in (w1, w2, w3, wc))
    alloc_w = cuda.AllocMemoryBf16 if bf16 else cuda.AllocMemory
    hX, hG, hH, hL = cuda.AllocMemory(x), cuda.AllocMemory(g), cuda.AllocMemory(B * hidden), cuda.AllocMemory(B * vocab)
    hW1, hW2, hW3, hWc = alloc_w(w1), alloc_w(w2), alloc_w(w3), alloc_w(wc)
    cuda.DecodeFfn(hX, hG, hW1, hW2, hW3, B, dim, hidden, hH)
    got_x = cuda.GetMemory(hX, x.size).reshape(x.shape)
    cuda.DecodeLogits(hX, hG, hWc, B, dim, vocab, hL)
    got_l = cuda.GetMemory(hL, B * vocab).reshape(B, vocab)
    ref_x = np.empty_like(x)
    for b in range(B):
        xn = oracle.rmsnorm(x[b], g)
        a, c = oracle.gemv(w1, xn), oracle.gemv(w3, xn)
        ref_x[b] = x[b] + oracle.gemv(w2, a * (1.0 / (1.0 + np.exp(-a))) * c)
    ref_l = np.stack([oracle.gemv(wc, oracle.rmsnorm(ref_x[b], g)) for b in range(B)])
    assert rel_err(got_x, ref_x) < 1e-4
    assert rel_err(got_l, ref_l) < 1e-4
    for h in (hX, hG, hH, hL, hW1, hW2, hW3, hWc):
        cuda.FreeMemory(h)
    cuda.Dispose()
