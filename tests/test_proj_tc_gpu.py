"""Decode projections for 9 to 64 sequences: the tensor-core kernel against fp64 products and against the streaming
kernel it stands in for (the reference decodes one sequence per cublasSgemv call,
CudaExtension.llm32.llama2/Files/primitives.cu:322-340; the arithmetic is the CPU twin's, llama2_cpu.cpp:189-237)."""
import ctypes as C

import numpy as np
import pytest

from helpers import rel_err
from gpu_util import bf16_round

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5      # fp16 hi/lo halves of both operands, fp32 accumulation on the tensor core
TOL_BF16 = 5e-5     # bf16 weights are exact operands; the activations carry two bf16 pieces (16 mantissa bits)


def _rms(x, g, eps=1e-5):
    x = x.astype(np.float64)
    return g.astype(np.float64) * (x / np.sqrt((x * x).mean(-1, keepdims=True) + eps))


def _setup(bf16):
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    wdt = torch.bfloat16 if bf16 else torch.float32
    up = lambda a, dt=torch.float32: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dt).contiguous()
    return torch, lib, dev, wdt, up


def _status(lib):
    st = (C.c_int * 4)()
    assert lib.mca_proj_tc_status(st) == 0
    return list(st)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("B,dim,kv_dim", [(9, 264, 88), (16, 1024, 1024), (40, 512, 128), (64, 2048, 512)])
def test_qkv_and_out_projection(B, dim, kv_dim, bf16):
    torch, lib, dev, wdt, up = _setup(bf16)
    rng = np.random.default_rng(B + dim)
    x = rng.standard_normal((B, dim)).astype(np.float32)
    x[0, 3] = 300.0                                        # an outlier: the per-sequence scale must absorb it
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    mk = lambda r, c: (0.03 * rng.standard_normal((r, c))).astype(np.float32)
    wq, wk, wv, wo = mk(dim, dim), mk(kv_dim, dim), mk(kv_dim, dim), mk(dim, dim)
    if bf16:
        wq, wk, wv, wo = (bf16_round(w) for w in (wq, wk, wv, wo))
    xd, gd = up(x), up(g)
    wd = [up(w, wdt) for w in (wq, wk, wv, wo)]
    outs = {}
    for on in (1, 0):
        lib.mca_proj_tc_enable(on)
        q, k, v = torch.empty(B, dim, device=dev), torch.empty(B, kv_dim, device=dev), torch.empty(B, kv_dim, device=dev)
        rc = lib.mca_decode_qkv_rmsnorm(xd.data_ptr(), gd.data_ptr(), 1e-5, wd[0].data_ptr(), wd[1].data_ptr(), wd[2].data_ptr(),
                                        int(bf16), B, dim, kv_dim, q.data_ptr(), k.data_ptr(), v.data_ptr(), None)
        assert rc == 0
        res = up(x)                                        # residual stream, updated in place
        rc = lib.mca_decode_out_proj(q.data_ptr(), wd[3].data_ptr(), int(bf16), B, dim, res.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        outs[on] = [t.cpu().numpy() for t in (q, k, v, res)]
    lib.mca_proj_tc_enable(1)
    assert _status(lib)[0] == 0
    xn = _rms(x, g)
    ref_q = xn @ wq.astype(np.float64).T
    refs = [ref_q, xn @ wk.astype(np.float64).T, xn @ wv.astype(np.float64).T]
    tol = TOL_BF16 if bf16 else TOL_F32
    for got, ref in zip(outs[1][:3], refs):
        assert rel_err(got, ref) < tol
    ref_res = x.astype(np.float64) + outs[1][0].astype(np.float64) @ wo.astype(np.float64).T
    assert rel_err(outs[1][3], ref_res) < tol
    for a, b in zip(outs[1], outs[0]):                     # and the streaming kernel agrees
        assert rel_err(a, b) < 5e-5


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("B,dim,hidden", [(16, 1024, 2816), (33, 512, 1376), (64, 4096, 11008)])
def test_feed_forward_and_classifier(B, dim, hidden, bf16):
    torch, lib, dev, wdt, up = _setup(bf16)
    rng = np.random.default_rng(B * 3 + hidden)
    x = rng.standard_normal((B, dim)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    mk = lambda r, c: (0.03 * rng.standard_normal((r, c))).astype(np.float32)
    w1, w3, w2 = mk(hidden, dim), mk(hidden, dim), mk(dim, hidden)
    vocab = 1001
    wc = mk(vocab, dim)
    if bf16:
        w1, w2, w3, wc = (bf16_round(w) for w in (w1, w2, w3, wc))
    gd = up(g)
    w1d, w2d, w3d, wcd = (up(w, wdt) for w in (w1, w2, w3, wc))
    got = {}
    for on in (1, 0):
        lib.mca_proj_tc_enable(on)
        xd = up(x)
        hd = torch.empty(B, hidden, device=dev)
        rc = lib.mca_decode_ffn(gd.data_ptr(), 1e-5, w1d.data_ptr(), w2d.data_ptr(), w3d.data_ptr(), int(bf16), B, dim, hidden,
                                hd.data_ptr(), xd.data_ptr(), None)
        assert rc == 0
        logits = torch.empty(B, vocab, device=dev)
        rc = lib.mca_decode_logits(xd.data_ptr(), gd.data_ptr(), 1e-5, wcd.data_ptr(), int(bf16), B, dim, vocab, logits.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        got[on] = [t.cpu().numpy() for t in (hd, xd, logits)]
    lib.mca_proj_tc_enable(1)
    assert _status(lib)[0] == 0
    xn = _rms(x, g)
    a, c = xn @ w1.astype(np.float64).T, xn @ w3.astype(np.float64).T
    hid = a / (1.0 + np.exp(-a)) * c
    tol = TOL_BF16 if bf16 else TOL_F32
    assert rel_err(got[1][0], hid) < tol
    res = x.astype(np.float64) + got[1][0].astype(np.float64) @ w2.astype(np.float64).T
    assert rel_err(got[1][1], res) < tol
    assert rel_err(got[1][2], _rms(got[1][1], g) @ wc.astype(np.float64).T) < tol
    for u, v in zip(got[1], got[0]):
        assert rel_err(u, v) < 5e-5
    # a second run gives the same bits: the K slices are added in a fixed order
    xd = up(x)
    hd = torch.empty(B, hidden, device=dev)
    lib.mca_decode_ffn(gd.data_ptr(), 1e-5, w1d.data_ptr(), w2d.data_ptr(), w3d.data_ptr(), int(bf16), B, dim, hidden,
                       hd.data_ptr(), xd.data_ptr(), None)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(xd.cpu().numpy(), got[1][1])
