"""The benchmarked configurations at their full sizes against the CPU oracle: config 5 at T = 32768, config 2 at
B = 8, config 3 at batch 16 and 64.  The oracle checks a strided subset (rows, (batch, head) pairs, sequences) that
it finishes in seconds; size-independent properties cover the rest."""
import ctypes as C

import numpy as np
import pytest

import oracle
from gpu_util import Sdpa, bf16_round
from helpers import rel_err

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


def test_config5_T32768_matches_oracle_rows(cuda):
    """Config 5 at its longest sequence (16 heads x 128, bf16, causal, T = 32768, B = 1) through ATTN_FWD: 128
    strided query rows of every head against the oracle, and the two closed-form properties over all rows."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(32768)
    B, H, T, D = 1, 16, 32768, 128
    q, k, v = (bf16_round((rng.standard_normal((B, H, T, D)) / np.sqrt(D)).astype(np.float32)) for _ in range(3))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    y = a.forward(q, k, v, None)
    ref = oracle.sdpa_forward_rows(q, k, v, None, 3, 11, 257)
    assert ref.shape[2] >= 127
    assert rel_err(y[:, :, 11::257], ref) < BF16_TOL
    # the last rows see every key tile of the launch
    tail = oracle.sdpa_forward_rows(q, k, v, None, 3, T - 3, 1)
    assert rel_err(y[:, :, T - 3:], tail) < BF16_TOL
    cuda.SetMemory(a.hV, np.ones(v.size, np.float32))
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, 0, a.hY, False)
    y1 = cuda.GetMemory(a.hY, q.size)
    assert np.abs(y1 - 1).max() < 1e-2                       # V = 1: every output element is 1
    cuda.SetMemory(a.hV, v)
    cuda.SetMemory(a.hQ, np.zeros(q.size, np.float32))
    cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, a.hQ, a.hK, a.hV, 0, a.hY, False)
    y0 = cuda.GetMemory(a.hY, q.size).reshape(q.shape)
    cm = np.cumsum(v.astype(np.float64), axis=2) / np.arange(1, T + 1)[None, None, :, None]
    assert rel_err(y0, cm) < BF16_TOL                        # Q = 0: row i is the mean of V[0..i]
    a.close()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_config2_B8_forward_backward(cuda, dtype):
    """Config 2's attention core at its full batch (B = 8, 12 heads x 64, T = 1024), forward and backward through
    ATTN_FWD / ATTN_BWD; the oracle checks every 13th (batch, head) pair -- pairs are independent problems."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(1024)
    B, H, T, D = 8, 12, 1024, 64
    bf16 = dtype == "bf16"
    mk = lambda s: (s * rng.standard_normal((B, H, T, D))).astype(np.float32)
    q, k, v, dy = mk(0.5), mk(0.5), mk(0.5), mk(1.0)
    if bf16:
        q, k, v, dy = (bf16_round(a) for a in (q, k, v, dy))
    a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16 if bf16 else None)
    mask = oracle.causal_mask(T)
    y = a.forward(q, k, v, mask)
    dq, dk, dv = a.backward(dy)
    tol = BF16_TOL if bf16 else FP32_TOL
    pairs = list(range(0, B * H, 13))
    assert len(pairs) >= 8
    for p in pairs:
        b, h = divmod(p, H)
        sl = (slice(b, b + 1), slice(h, h + 1))
        assert rel_err(y[sl], oracle.sdpa_forward(q[sl], k[sl], v[sl], mask, 1, f64=True)) < tol, (b, h)
        ref = oracle.sdpa_backward(q[sl], k[sl], v[sl], dy[sl], mask, 1, f64=True)
        for name, g_, r_ in zip("qkv", (dq[sl], dk[sl], dv[sl]), ref):
            assert rel_err(g_, r_) < tol, (b, h, name)
    a.close()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("batch", [16, 64])
def test_config3_decode_full_batch(batch, bf16):
    """Config 3 at batch 16 and 64 (32 heads x 128, cache lengths uniform in [512, 4096], fp32 and bf16 caches)
    through mca_decode_attention on device tensors; six sequences, among them the shortest and the longest, are
    taken to the host and compared with the oracle, output and appended cache rows."""
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    nh, hs, S = 32, 128, 4096
    dim = nh * hs
    rng = np.random.default_rng(batch)
    lengths = rng.integers(512, S + 1, batch)
    lengths[0], lengths[1] = 512, S
    pos_h = (lengths - 1).astype(np.int32)
    g = torch.Generator(device=dev).manual_seed(batch)
    cdt = torch.bfloat16 if bf16 else torch.float32
    kc = torch.randn(batch, S, dim, device=dev, generator=g).to(cdt)
    vc = torch.randn(batch, S, dim, device=dev, generator=g).to(cdt)
    q, kn, vn = (torch.randn(batch, dim, device=dev, generator=g) for _ in range(3))
    pos = torch.from_numpy(pos_h).to(dev)
    out = torch.empty(batch, dim, device=dev)
    check = sorted({0, 1, 2, batch // 2, batch - 2, batch - 1})
    before = {b: (kc[b].float().cpu().numpy(), vc[b].float().cpu().numpy()) for b in check}
    sl, ns, need = C.c_int(), C.c_int(), C.c_int64()
    assert lib.mca_decode_plan(batch, nh, nh, hs, int(lengths.max()), C.byref(sl), C.byref(ns), C.byref(need)) == 0
    scratch = torch.empty(max(1, need.value), device=dev)
    fr, fi = oracle.llama_freqs(hs, S)
    frd, fid = torch.from_numpy(fr).to(dev), torch.from_numpy(fi).to(dev)
    rc = lib.mca_decode_attention(q.data_ptr(), kn.data_ptr(), vn.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(bf16), S * dim,
                                  pos.data_ptr(), batch, nh, nh, hs, S, int(lengths.max()), frd.data_ptr(), fid.data_ptr(),
                                  scratch.data_ptr(), scratch.numel(), out.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0
    st = (C.c_int * 3)()
    assert lib.mca_decode_status(st) == 0 and st[0] == 0
    out_h, qh, kh, vh = out.cpu().numpy(), q.cpu().numpy(), kn.cpu().numpy(), vn.cpu().numpy()
    for b in check:
        kb, vb = before[b][0][None].copy(), before[b][1][None].copy()
        ref = oracle.llama_decode(qh[b:b + 1], kh[b:b + 1], vh[b:b + 1], kb, vb, pos_h[b:b + 1], nh, nh)
        if bf16:  # the kernel attends to the bf16-rounded new row, as a later step reads it back
            kb[0, pos_h[b]], vb[0, pos_h[b]] = bf16_round(kb[0, pos_h[b]]), bf16_round(vb[0, pos_h[b]])
            ref = oracle.llama_decode(qh[b:b + 1], kh[b:b + 1], vh[b:b + 1], kb.copy(), vb.copy(), pos_h[b:b + 1], nh, nh)
        assert rel_err(out_h[b], ref[0]) < (BF16_TOL if bf16 else 2e-5), b
        k_row, v_row = kc[b, pos_h[b]].float().cpu().numpy(), vc[b, pos_h[b]].float().cpu().numpy()
        np.testing.assert_allclose(k_row, kb[0, pos_h[b]], atol=2e-2 if bf16 else 2e-6)
        np.testing.assert_allclose(v_row, vb[0, pos_h[b]], atol=2e-2 if bf16 else 0)
