"""The rest of the drop-in boundary on a GPU: the llama2 extension ABI, the query-string exports, the per-call
counters, and the robustness paths of the dispatch layer (mask handles that change under the handle, positions
outside the cache, a bounded device-side wait that runs out)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from gpu_util import Sdpa
from helpers import rel_err
from test_llama_step_gpu import synthetic_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


# ------------------------------------------------------------------------------------------ extension ABI

def test_llama2_extension_matches_reference_transformer(cuda, tmp_path):
    """CreateExtension -> CREATE -> LOAD -> QUERYSTATUS -> FORWARD x n -> DESTROY through the parent's
    CUDA_FN_EXTENSION_RUN packing (CudaDnn.cs:3703-3798), logits against the reference's own
    TransformerCpu::forward on the same checkpoint file."""
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference twin not available")
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    dim, hidden, n_layers, n_heads, vocab, seq_len = 256, 344, 2, 4, 96, 24
    rng = np.random.default_rng(11)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_heads, vocab)
    path = tmp_path / "m.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_heads, vocab, seq_len, w)
    ref = oracle.RefLlama(path)

    hExt = cuda.CreateExtension("")
    hLlm = int(cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_CREATE, [0.0, 0.9, 1.0])[0])
    st = cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_QUERYSTATUS, [hLlm])
    assert list(st) == [0.0, 0.0]                                   # not loaded yet (llm.cpp:161-177)
    with pytest.raises(CudaDnnError) as e:                          # missing model file: ERROR_LLM_LOAD_MODEL_MISSING_MODEL_FILE
        cuda.RunExtensionEx(hExt, ids.LLM_CUDA_EXTENSION_LOAD, [hLlm], str(tmp_path / "absent.bin") + ";tok.bin")
    assert e.value.code == 10002
    cuda.RunExtensionEx(hExt, ids.LLM_CUDA_EXTENSION_LOAD, [hLlm], f"{path};{tmp_path / 'tokenizer.bin'}")
    assert list(cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_QUERYSTATUS, [hLlm])) == [1.0, 1.0]
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        got = cuda.RunExtension(hExt, ids.MCA_LLM_EXTENSION_FORWARD, [hLlm, int(tokens[pos]), pos])
        assert got.shape == (vocab,)
        assert rel_err(got, ref.state("logits")) < 1e-4, pos
    with pytest.raises(CudaDnnError) as e:                          # position beyond the cache
        cuda.RunExtension(hExt, ids.MCA_LLM_EXTENSION_FORWARD, [hLlm, 1, seq_len])
    assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE
    with pytest.raises(CudaDnnError) as e:                          # text generation is not part of this library
        cuda.RunExtensionEx(hExt, ids.LLM_CUDA_EXTENSION_GENERATE, [hLlm], "hello")
    assert e.value.code == 50 and "not provided" in e.value.native_message
    with pytest.raises(CudaDnnError) as e:                          # an id the extension does not know
        cuda.RunExtension(hExt, 42, [hLlm])
    assert e.value.code == 50 and "not supported" in e.value.native_message
    with pytest.raises(CudaDnnError) as e:
        cuda.QueryExtensionStrings(hExt, ids.LLM_CUDA_EXTENSION_QUERYRESPONSE, [hLlm])
    assert e.value.code == 50
    cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_ABORT, [hLlm])
    cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_DESTROY, [hLlm])
    with pytest.raises(CudaDnnError):                               # destroyed handle
        cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_QUERYSTATUS, [hLlm])
    cuda.FreeExtension(hExt)
    with pytest.raises(CudaDnnError):
        cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_CREATE, [])
    ref.close()


def test_extension_loaded_by_path_binds_the_same_exports(cuda):
    """A parent that LoadLibrary's the extension by file name (extension.cu:33-83) finds the three entry points."""
    from mycaffe_b200 import _lib, function_ids as ids
    hExt = cuda.CreateExtension(str(_lib.LIB_PATH))
    hLlm = int(cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_CREATE, [])[0])
    assert hLlm > 0
    cuda.RunExtension(hExt, ids.LLM_CUDA_EXTENSION_DESTROY, [hLlm])
    cuda.FreeExtension(hExt)


def test_query_strings_and_counters(cuda):
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    name = cuda.GetDeviceName(0)
    assert "compute 10." in name and "GB" in name                   # "<name> (<GB> GB - P2P ...; compute M.m)", device.cu:550
    assert cuda.QueryString(ids.MCA_FN_QUERY_VERSION).endswith("sm_100a")
    with pytest.raises(CudaDnnError) as e:
        cuda.QueryString(1001, [0])                                 # CUDA_FN_GET_P2P_INFO: not on this path
    assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE
    cuda.SetTiming(True)
    h = cuda.AllocMemory(np.ones(1 << 20, np.float32))
    hL = cuda.CreateLayerNorm(0, 1 << 20, 1, 1024, 1024, 1e-5)
    hY = cuda.AllocMemory(1 << 20)
    for _ in range(3):
        cuda.LayerNormForward(hL, h, hY)
    cuda.SetTiming(False)
    c = cuda.QueryCounters()[ids.CUDA_FN_LAYERNORM_FWD]
    assert c["calls"] >= 3 and c["errors"] == 0 and 0 < c["gpu_ms_last"] < 50 and c["gpu_ms_total"] >= c["gpu_ms_last"]
    cuda.FreeLayerNorm(hL)
    cuda.FreeMemory(h); cuda.FreeMemory(hY)


# ------------------------------------------------------------------------------------------ mask handles

@pytest.mark.parametrize("dtype", ["f32", "tf32"])
def test_mask_rewritten_in_place_is_seen(cuda, dtype):
    """A (T,T) mask handle overwritten with SETMEM between two Forward calls: the second call must use the
    new contents (attn.cu:571-583 reads the mask every call), not a classification remembered from the first."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(5)
    B, H, T, D = 2, 3, 96, 64
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_TF32 if dtype == "tf32" else None)
    tol = 5e-3 if dtype == "tf32" else 1e-4
    tril = oracle.causal_mask(T)
    y1 = a.forward(q, k, v, tril)
    assert rel_err(y1, oracle.sdpa_forward(q, k, v, tril, 1, f64=True)) < tol
    band = np.triu(tril, -7).astype(np.float32)                     # a band: lower-triangular but not tril(ones)
    band[5, :] = 0.0                                                # and one fully masked row (uniform, -1e29 semantics)
    cuda.SetMemory(a.hMask, band)
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, a.hMask, a.hY, False)
    y2 = cuda.GetMemory(a.hY, q.size).reshape(q.shape)
    assert rel_err(y2, oracle.sdpa_forward(q, k, v, band, 1, f64=True)) < 1e-4   # a general mask runs the exact kernel
    cuda.SetMemory(a.hMask, tril)                                   # and back
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, a.hMask, a.hY, False)
    y3 = cuda.GetMemory(a.hY, q.size).reshape(q.shape)
    np.testing.assert_array_equal(y3, y1)
    a.close()


def test_backward_after_the_mask_was_freed_or_rewritten(cuda):
    """The reference's Backward reads neither hMask nor anything but what its Forward left in the handle
    (attn.cu:622-634).  The default handle does the same: its Forward packed the mask into keep-bits it owns, so the
    mask handle may be freed before Backward.  The exact-fp32 handle recomputes the probabilities from the mask itself
    and looks it up by handle: a freed one is an error, never a dangling pointer."""
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    rng = np.random.default_rng(6)
    B, H, T, D = 1, 2, 40, 32
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    mask = (rng.random((T, T)) < 0.7).astype(np.float32)
    mask[np.arange(T), np.arange(T)] = 1
    ref = oracle.sdpa_backward(q, k, v, dy, mask, 1, f64=True)
    for flags, freed_is_error in ((None, False), (ids.MCA_FLAG_EXACT_FP32, True)):
        a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_F32 if flags else None, flags=flags)
        a.forward(q, k, v, mask)
        for g_, r_ in zip(a.backward(dy), ref):
            assert rel_err(g_, r_) < 1e-4
        # the same address can come back from the allocator with other contents: free the mask
        cuda.FreeMemory(a.hMask)
        a._mem.remove(a.hMask)
        if freed_is_error:
            with pytest.raises(CudaDnnError) as e:
                a.backward(dy)
            assert e.value.code == ids.ERROR_MEMORY_NOT_FOUND
        else:
            for g_, r_ in zip(a.backward(dy), ref):
                assert rel_err(g_, r_) < 1e-4
        a.close()


# ------------------------------------------------------------------------------------------ decode positions

@pytest.mark.parametrize("bf16", [False, True])
def test_decode_position_outside_the_cache_is_refused(cuda, bf16):
    """pos[b] is device data: a value outside [0, maxLen) must neither read nor write outside that sequence's
    cache.  The sequence's output is zero, every cache is untouched, the other sequences are right, and the
    synchronous call reports ERROR_PARAM_OUT_OF_RANGE naming the sequence."""
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    from test_decode_rope_tft_gpu import Decoder
    from gpu_util import bf16_round
    B, nh, hs, S = 4, 4, 64, 300
    rng = np.random.default_rng(8)
    kc = rng.standard_normal((B, S, nh * hs)).astype(np.float32)
    vc = rng.standard_normal((B, S, nh * hs)).astype(np.float32)
    if bf16:
        kc, vc = bf16_round(kc), bf16_round(vc)
    q, k, v = (rng.standard_normal((B, nh * hs)).astype(np.float32) for _ in range(3))
    for bad in (S + 5, 1 << 20, -3):
        pos = np.array([17, bad, S - 1, 0], np.int32)
        d = Decoder(cuda, B, nh, nh, hs, S, bf16)
        d.set_cache(kc, vc)
        with pytest.raises(CudaDnnError) as e:
            d.step(q, k, v, pos, max_len=S)
        assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE and "sequence 1" in e.value.native_message
        out = cuda.GetMemory(d.hOut, q.size).reshape(q.shape)
        good = [0, 2, 3]
        kr, vr = kc.copy(), vc.copy()
        ref = oracle.llama_decode(q[good], k[good], v[good], kr[good].copy(), vr[good].copy(), pos[good], nh, nh)
        assert rel_err(out[good], ref) < (2e-2 if bf16 else 1e-4)
        assert not out[1].any()
        kg, vg = d.caches()
        np.testing.assert_array_equal(kg[1], kc[1])
        np.testing.assert_array_equal(vg[1], vc[1])
        # the next call with valid positions is clean again
        pos_ok = np.array([17, 3, S - 1, 0], np.int32)
        d.set_cache(kc, vc)
        out = d.step(q, k, v, pos_ok, max_len=S)
        ref = oracle.llama_decode(q, k, v, kc.copy(), vc.copy(), pos_ok, nh, nh)
        assert rel_err(out, ref) < (2e-2 if bf16 else 1e-4)
        d.close()


def test_decode_rejects_misaligned_caches():
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    B, nh, hs, S = 1, 2, 64, 128
    dev = torch.device("cuda", 0)
    buf = torch.zeros(2 * S * nh * hs + 64, device=dev)
    q = torch.zeros(nh * hs, device=dev)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    call = lambda kc, stride: lib.mca_decode_attention(q.data_ptr(), None, None, kc, kc, 0, stride, pos.data_ptr(), B, nh, nh, hs, S,
                                                       S, None, None, None, 0, q.data_ptr(), None)
    assert call(buf.data_ptr(), S * nh * hs) == 0
    assert call(buf.data_ptr() + 4, S * nh * hs) == ids.ERROR_PARAM_OUT_OF_RANGE      # base not 16-byte aligned
    assert call(buf.data_ptr(), S * nh * hs + 2) == ids.ERROR_PARAM_OUT_OF_RANGE      # stride not a whole vector
    torch.cuda.synchronize()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("n_heads,n_kv,hs", [(6, 6, 48), (4, 2, 32), (8, 2, 96), (5, 5, 32)])
def test_decode_other_head_sizes(cuda, n_heads, n_kv, hs, bf16):
    """Head sizes beyond 64 / 128 (the reference kernel takes any, primitives.cu:158-202; llama2.c's 15M model has 48)."""
    from test_decode_rope_tft_gpu import Decoder
    from gpu_util import bf16_round
    B, S = 3, 777
    rng = np.random.default_rng(hs + n_heads)
    kv_dim = n_kv * hs
    kc = rng.standard_normal((B, S, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((B, S, kv_dim)).astype(np.float32)
    if bf16:
        kc, vc = bf16_round(kc), bf16_round(vc)
    q = rng.standard_normal((B, n_heads * hs)).astype(np.float32)
    k, v = (rng.standard_normal((B, kv_dim)).astype(np.float32) for _ in range(2))
    pos = np.array([S - 1, 0, 391], np.int32)
    d = Decoder(cuda, B, n_heads, n_kv, hs, S, bf16)
    d.set_cache(kc, vc)
    out = d.step(q, k, v, pos)
    kr, vr = kc.copy(), vc.copy()
    ref = oracle.llama_decode(q, k, v, kr, vr, pos, n_heads, n_kv)
    if bf16:
        for b in range(B):
            kr[b, pos[b]] = bf16_round(kr[b, pos[b]]); vr[b, pos[b]] = bf16_round(vr[b, pos[b]])
        ref = oracle.llama_decode(q, k, v, kr.copy(), vr.copy(), pos, n_heads, n_kv)
    assert rel_err(out, ref) < (2e-2 if bf16 else 2e-5)
    kg, vg = d.caches()
    for b in range(B):
        np.testing.assert_allclose(kg[b, pos[b]], kr[b, pos[b]], atol=2e-2 if bf16 else 2e-6)
        keep = np.arange(S) != pos[b]
        np.testing.assert_array_equal(kg[b, keep], kc[b, keep])
        np.testing.assert_array_equal(vg[b, keep], vc[b, keep])
    d.close()


def test_llama_step_head_size_48(tmp_path):
    """llama2.c's 15M geometry cut down (dim 288, 6 heads of 48) against the reference twin."""
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference twin not available")
    from mycaffe_b200.llama2 import TransformerGpu
    dim, hidden, n_layers, n_heads, vocab, seq_len = 288, 768, 2, 6, 64, 20
    rng = np.random.default_rng(48)
    w = synthetic_weights(rng, dim, hidden, n_layers, n_heads, n_heads, vocab)
    path = tmp_path / "m15.bin"
    oracle.write_llama_checkpoint(path, dim, hidden, n_layers, n_heads, n_heads, vocab, seq_len, w)
    ref = oracle.RefLlama(path)
    t = TransformerGpu(0)
    t.build(str(path))
    tokens = rng.integers(0, vocab, seq_len)
    for pos in range(seq_len):
        ref.forward(int(tokens[pos]), pos)
        assert rel_err(t.forward(int(tokens[pos]), pos), ref.state("logits")) < 1e-4, pos
    ref.close()


# ------------------------------------------------------------------------------------------ bounded waits

def test_bounded_wait_runs_out_and_is_reported(cuda):
    """A device-side wait that nothing will ever satisfy gives up after its limit, the kernel returns, the status
    words turn into ERROR_ATTN_KERNEL_TIMEOUT with the place in the message, and the handle works again after."""
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    rng = np.random.default_rng(9)
    B, H, T, D = 1, 2, 256, 64
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    y0 = a.forward(q, k, v)
    g = lambda h: cuda.GetMemory(h, q.size).reshape(q.shape)
    ref = oracle.sdpa_forward(g(a.hQ), g(a.hK), g(a.hV), None, 3, f64=True)
    assert rel_err(y0, ref) < 2e-2
    with pytest.raises(CudaDnnError) as e:
        cuda._invoke(ids.MCA_FN_WAIT_PROBE, None, [a.hAttn, 1000])            # 1 ms
    assert e.value.code == ids.ERROR_ATTN_KERNEL_TIMEOUT and "stage 99" in e.value.native_message
    # the words were cleared by the report: the next launch runs and is right
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, 0, a.hY, False)
    np.testing.assert_array_equal(g(a.hY), y0)

    # asynchronous mode: the give-up is reported by the next synchronising call; a launch in between finds the
    # status set, leaves y alone, and nothing is lost
    cuda.SetAsync(True)
    cuda.SetMemory(a.hY, np.full(q.size, 7.0, np.float32))
    cuda._invoke(ids.MCA_FN_WAIT_PROBE, None, [a.hAttn, 1000])
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, 0, a.hY, False)
    with pytest.raises(CudaDnnError) as e:
        cuda.SynchronizeDevice()
    assert e.value.code == ids.ERROR_ATTN_KERNEL_TIMEOUT
    assert np.all(g(a.hY) == 7.0)
    cuda.SynchronizeDevice()                                                   # clean now
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, 0, a.hY, False)
    cuda.SynchronizeDevice()
    cuda.SetAsync(False)
    np.testing.assert_array_equal(g(a.hY), y0)
    a.close()


def test_preset_status_aborts_the_raw_launch():
    """mca_sdpa_forward_tc with status[0] already set: every CTA leaves at once and y is untouched."""
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, H, T, D = 1, 2, 256, 128
    q, k, v = (torch.randn(B, H, T, D, device=dev).bfloat16() for _ in range(3))
    y = torch.full_like(q, 3.0)
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    st[0] = 1
    rc = lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D, y.data_ptr(), None,
                                 st.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0 and bool((y == 3.0).all()) and st[:4].tolist() == [1, 0, 0, 0]
    st.zero_()
    rc = lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D, y.data_ptr(), None,
                                 st.data_ptr(), None)
    torch.cuda.synchronize()
    ref = oracle.sdpa_forward(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), None, 3, f64=True)
    assert rc == 0 and st[0].item() == 0 and rel_err(y.float().cpu().numpy(), ref) < 2e-2


# ------------------------------------------------------------------------------------------ decode exchange

def _exchange(lib, src, bufs, flags, counter, status, rank, n, B, dl, gen, limit_ms=2000):
    dst = (C.c_void_p * n)(*[b.data_ptr() for b in bufs])
    fl = (C.c_void_p * n)(*[f.data_ptr() for f in flags])
    return lib.mca_decode_exchange(src.data_ptr(), dst, fl, flags[rank].data_ptr(), counter.data_ptr(), status.data_ptr(), n, rank, B, dl,
                                   n * dl, rank * dl, gen, limit_ms, None)


def test_decode_exchange_kernel_two_ranks_on_one_gpu():
    """The exchange that replaces the per-layer all-gather, with both "ranks" played one after the other on one GPU
    (two kernels that wait on each other must not share a GPU, so rank 1's arrival is written before rank 0 runs): each
    rank's slice lands at its columns of both buffers, and the flags carry the generation."""
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, dl, n = 5, 256, 2
    for gen in (1, 2, 3):
        src = [torch.randn(B, dl, device=dev) for _ in range(n)]
        if gen == 1:
            bufs = [torch.zeros(B, n * dl, device=dev) for _ in range(n)]
            flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(n)]
            counters = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(n)]
            status = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(n)]
        flags[0][1] = gen                               # rank 1 "has arrived" as far as rank 0 can see
        assert _exchange(lib, src[0], bufs, flags, counters[0], status[0], 0, n, B, dl, gen) == 0
        assert _exchange(lib, src[1], bufs, flags, counters[1], status[1], 1, n, B, dl, gen) == 0
        torch.cuda.synchronize()
        want = torch.cat(src, dim=1)
        for r in range(n):
            assert torch.equal(bufs[r], want)
            assert flags[r][:2].tolist() == [gen, gen] and status[r].tolist() == [0, 0, 0, 0] and counters[r].item() == 0


def test_decode_exchange_wait_is_bounded():
    """A peer that never arrives: the wait runs out after its limit, the kernel returns and says whom it waited for."""
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, dl, n = 3, 64, 2
    src = torch.randn(B, dl, device=dev)
    bufs = [torch.zeros(B, n * dl, device=dev) for _ in range(n)]
    flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(n)]
    counter, status = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(4, dtype=torch.int32, device=dev)
    assert _exchange(lib, src, bufs, flags, counter, status, 0, n, B, dl, 7, limit_ms=5) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [3, 1, 0, 7]              # gave up waiting for rank 1, whose flag was still 0
    assert torch.equal(bufs[1][:, :dl], src)            # its own stores were made all the same
    assert _exchange(lib, src, bufs, flags, counter, status, 0, n, B, 6, 8) == ids.ERROR_PARAM_OUT_OF_RANGE   # slice not a multiple of 4
