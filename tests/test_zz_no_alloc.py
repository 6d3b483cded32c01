"""The decode entry point that allocates nothing (mca_decode_attention_static).

A host that is only handed its inputs and outputs -- and may not call cudaMalloc where it decodes --
uses this variant: the split-KV partials go to a fixed 8 MiB array inside the library instead of a
caller-provided scratch buffer.  It must give exactly what mca_decode_attention gives, call after
call (the array keeps the previous call's contents), and refuse problems that do not fit.

Collected last on purpose, so that a run that stops at the first failure has already run
everything else; it passes alone in a fresh process as well."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(cuda, lib, rng, B, n_heads, n_kv, hs, seq_len, lengths, static):
    dim, kv_dim = n_heads * hs, n_kv * hs
    kc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    vc = rng.standard_normal((B, seq_len, kv_dim)).astype(np.float32)
    q, k, v = (rng.standard_normal((B, d)).astype(np.float32) for d in (dim, kv_dim, kv_dim))
    fr = np.empty((seq_len, hs // 2), np.float32)
    fi = np.empty_like(fr)
    fp = C.POINTER(C.c_float)
    lib.mca_rope_tables_host(seq_len, hs, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
    pos = (np.asarray(lengths) - 1).astype(np.int32)
    h = {n: cuda.AllocMemory(a) for n, a in dict(kc=kc, vc=vc, q=q, k=k, v=v, fr=fr, fi=fi).items()}
    h["pos"], h["out"] = cuda.AllocMemory(B), cuda.AllocMemory(B * dim)
    cuda.SetMemoryInt32(h["pos"], pos)
    ptr = {n: cuda.GetPointer(x) for n, x in h.items()}
    max_len = int(max(lengths))
    if static:
        rc = lib.mca_decode_attention_static(ptr["q"], ptr["k"], ptr["v"], ptr["kc"], ptr["vc"], 0, seq_len * kv_dim,
                                             ptr["pos"], B, n_heads, n_kv, hs, seq_len, max_len, ptr["fr"], ptr["fi"],
                                             ptr["out"], None)
    else:
        sl, ns, need = C.c_int(), C.c_int(), C.c_int64()
        assert lib.mca_decode_plan(B, n_heads, n_kv, hs, max_len, C.byref(sl), C.byref(ns), C.byref(need)) == 0
        h["scratch"] = cuda.AllocMemory(max(1, need.value))
        rc = lib.mca_decode_attention(ptr["q"], ptr["k"], ptr["v"], ptr["kc"], ptr["vc"], 0, seq_len * kv_dim,
                                      ptr["pos"], B, n_heads, n_kv, hs, seq_len, max_len, ptr["fr"], ptr["fi"],
                                      cuda.GetPointer(h["scratch"]), need.value, ptr["out"], None)
    cuda.SynchronizeDevice()
    out = cuda.GetMemory(h["out"], B * dim).reshape(B, dim) if rc == 0 else None
    for x in h.values():
        cuda.FreeMemory(x)
    return rc, out


def test_static_scratch_decode_matches_regular_entry_point_twice():
    from mycaffe_b200 import CudaDnn, _lib
    lib = _lib.load()
    cuda = CudaDnn(0)
    try:
        assert lib.mca_decode_static_scratch_floats() == 2 * 1024 * 1024
        # two different problems back to back: the second call finds the first call's partials in the array
        for seed, (B, n_heads, n_kv, hs, seq_len) in enumerate([(6, 32, 32, 128, 4096), (3, 16, 4, 64, 1500)]):
            lengths = np.random.default_rng(100 + seed).integers(seq_len // 4, seq_len + 1, B)
            lengths[0] = seq_len
            rc_s, out_s = _run(cuda, lib, np.random.default_rng(seed), B, n_heads, n_kv, hs, seq_len, lengths, True)
            rc_r, out_r = _run(cuda, lib, np.random.default_rng(seed), B, n_heads, n_kv, hs, seq_len, lengths, False)
            assert rc_s == 0 and rc_r == 0
            assert np.isfinite(out_s).all()
            # same kernels, same inputs: identical up to nothing (tolerance of the decode tests: 2e-5 of scale)
            assert np.max(np.abs(out_s - out_r)) <= 2e-5 * np.max(np.abs(out_r))
        # a problem whose partials exceed the built-in array (128 x 64 heads x 2 splits x 130 floats)
        # is refused before anything is launched, not truncated; the buffers are never touched
        h = cuda.AllocMemory(16)
        d = cuda.GetPointer(h)
        rc = lib.mca_decode_attention_static(d, d, d, d, d, 0, 2048 * 1024, d, 128, 64, 8, 128, 2048, 2048, d, d, d, None)
        assert rc == 90906
        cuda.FreeMemory(h)
    finally:
        cuda.Dispose()
