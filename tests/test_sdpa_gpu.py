"""Parity of the CUDA attention path against the CPU oracle, through the C ABI
(function ids ATTN_CREATE/SET/FWD/BWD as CudaDnn.cs:5611-5701 packs them).

Tolerances: max-abs error relative to the output scale <= 1e-4 for fp32, <= 2e-2 for bf16
(the targets stated for this path); most fp32 cases are held to 2e-5."""
import numpy as np
import pytest

import oracle
from gpu_util import Sdpa, bf16_round
from helpers import PICO_CASES, csa_forward, csa_qkv, rel_err

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
FP32_TIGHT = 2e-5
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


def rand_qkv(rng, B, H, T, D, scale=1.0):
    return tuple((scale * rng.standard_normal((B, H, T, D))).astype(np.float32) for _ in range(3))


@pytest.mark.parametrize("case", list(PICO_CASES))
def test_pico_golden_forward_backward(cuda, pico, case):
    """The reference's own golden vectors (gpt-pico-csa*) through ATTN_FWD / ATTN_BWD."""
    H = PICO_CASES[case]
    g = lambda n: pico[f"{case}/{n}"]
    x = g("x")
    B, T, C = x.shape
    q, k, v = csa_qkv(x, g("attn_weight"), g("attn_bias"), H)
    a = Sdpa(cuda, B, T, H, C // H, training=True)
    y = a.forward(q, k, v, oracle.causal_mask(T))
    if f"{case}/var_y" in pico.files:
        np.testing.assert_allclose(y, g("var_y"), atol=3e-7)
    full = csa_forward(x, g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), g("attn_proj_bias"), H,
                       lambda *_: y)
    np.testing.assert_allclose(full, g("y"), atol=3e-7)
    dq, dk, dv = a.backward(g("grad_y_pre_transpose"))
    np.testing.assert_allclose(dq, g("grad_qt"), atol=3e-8)
    np.testing.assert_allclose(dk, g("grad_kt"), atol=3e-8)
    np.testing.assert_allclose(dv, g("grad_vt"), atol=3e-8)
    a.close()


def test_config1_causal_block(cuda):
    """BASELINE config 1: one CausalSelfAttention block forward, fp32, B=1, T=128, 4 heads x 16."""
    import torch
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(1, 128, 64, generator=gen).numpy()
    w_attn = (0.02 * torch.randn(192, 64, generator=gen)).numpy()
    w_proj = (0.02 * torch.randn(64, 64, generator=gen)).numpy()
    zeros = np.zeros
    mask = oracle.causal_mask(128)
    a = Sdpa(cuda, 1, 128, 4, 16)
    got = csa_forward(x, w_attn, zeros(192, np.float32), w_proj, zeros(64, np.float32), 4,
                      lambda q, k, v: a.forward(q, k, v, mask))
    ref = csa_forward(x, w_attn, zeros(192, np.float32), w_proj, zeros(64, np.float32), 4,
                      lambda q, k, v: oracle.sdpa_forward(q, k, v, mask, 1, f64=True))
    assert rel_err(got, ref) < FP32_TIGHT
    a.close()


def test_reference_self_consistency_recipe(cuda):
    """TestCudaAttentionForward/Backward (TestGPT_MultiheadAttentionLayer.cs:945-1036): random
    (3,8,200,64), all-ones batch mask, composed route vs the direct route."""
    rng = np.random.default_rng(0)
    B, H, T, D = 3, 8, 200, 64
    q, k, v = rand_qkv(rng, B, H, T, D)
    mask = np.ones((B, T), np.float32)
    a = Sdpa(cuda, B, T, H, D, training=True)
    y = a.forward(q, k, v, mask, batch_mask=True)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, 2, f64=True)) < FP32_TIGHT
    dy = rng.standard_normal(q.shape).astype(np.float32)
    got = a.backward(dy)
    ref = oracle.sdpa_backward(q, k, v, dy, mask, 2, f64=True)
    for g_, r_ in zip(got, ref):
        assert rel_err(g_, r_) < FP32_TIGHT
    a.close()


@pytest.mark.parametrize("T", [1, 2, 3, 5, 17, 64, 127, 129, 200])
@pytest.mark.parametrize("D", [1, 3, 16, 32, 64, 128])
def test_forward_backward_ragged_shapes_causal(cuda, T, D):
    rng = np.random.default_rng(T * 131 + D)
    B, H = 2, 3
    q, k, v = rand_qkv(rng, B, H, T, D)
    mask = oracle.causal_mask(T)
    a = Sdpa(cuda, B, T, H, D, training=True)
    y = a.forward(q, k, v, mask)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, 1, f64=True)) < FP32_TIGHT
    dy = rng.standard_normal(q.shape).astype(np.float32)
    got = a.backward(dy)
    ref = oracle.sdpa_backward(q, k, v, dy, mask, 1, f64=True)
    for g_, r_ in zip(got, ref):
        assert rel_err(g_, r_) < FP32_TIGHT
    a.close()


@pytest.mark.parametrize("mode", ["none", "random_tt", "batch_with_dead_row"])
def test_mask_forms(cuda, mode):
    """No mask (hMask = 0), an arbitrary (T,T) mask, and a (B,T) key mask with one batch row fully
    masked: masked logits are -1e29, so that row becomes a uniform distribution (math.cu:2994-3002)."""
    rng = np.random.default_rng(11)
    B, H, T, D = 3, 2, 150, 32
    q, k, v = rand_qkv(rng, B, H, T, D)
    dy = rng.standard_normal(q.shape).astype(np.float32)
    if mode == "none":
        mask, omode, batch = None, 0, False
    elif mode == "random_tt":
        mask = (rng.random((T, T)) > 0.3).astype(np.float32)
        mask[7, :] = 0  # one fully masked query row
        omode, batch = 1, False
    else:
        mask = (rng.random((B, T)) > 0.2).astype(np.float32)
        mask[1, :] = 0
        omode, batch = 2, True
    a = Sdpa(cuda, B, T, H, D, training=True)
    y = a.forward(q, k, v, mask, batch_mask=batch)
    ref = oracle.sdpa_forward(q, k, v, mask, omode, f64=True)
    assert rel_err(y, ref) < FP32_TIGHT
    if mode == "batch_with_dead_row":
        np.testing.assert_allclose(y[1], np.broadcast_to(v[1].mean(axis=1, keepdims=True), v[1].shape), atol=2e-6)
    got = a.backward(dy)
    for g_, r_ in zip(got, oracle.sdpa_backward(q, k, v, dy, mask, omode, f64=True)):
        assert rel_err(g_, r_) < FP32_TIGHT
    a.close()


def test_forward_shorter_than_block(cuda):
    """Forward accepts nBlockSize <= the configured block size (attn.cu:530-531)."""
    rng = np.random.default_rng(5)
    B, H, T, D = 2, 4, 40, 16
    q, k, v = rand_qkv(rng, B, H, T, D)
    a = Sdpa(cuda, B, 64, H, D)
    y = a.forward(q, k, v, oracle.causal_mask(T), T=T)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, oracle.causal_mask(T), 1, f64=True)) < FP32_TIGHT
    a.close()


def test_gpt2_small_shape_layer(cuda):
    """BASELINE config 2 shape (12 heads x 64, T=1024), one layer's attention core, B reduced to 2
    so that the CPU oracle finishes in seconds."""
    rng = np.random.default_rng(2)
    B, H, T, D = 2, 12, 1024, 64
    q, k, v = rand_qkv(rng, B, H, T, D, 0.5)
    mask = oracle.causal_mask(T)
    a = Sdpa(cuda, B, T, H, D, training=True)
    y = a.forward(q, k, v, mask)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, 1)) < FP32_TOL
    dy = rng.standard_normal(q.shape).astype(np.float32)
    got = a.backward(dy)
    for g_, r_ in zip(got, oracle.sdpa_backward(q, k, v, dy, mask, 1)):
        assert rel_err(g_, r_) < FP32_TOL
    a.close()


def test_error_paths(cuda):
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    rng = np.random.default_rng(3)
    q, k, v = rand_qkv(rng, 1, 2, 8, 16)
    a = Sdpa(cuda, 1, 8, 2, 16, training=True)
    with pytest.raises(CudaDnnError) as e:  # T above the configured block size
        a.forward(q, k, v, None, T=9)
    assert e.value.code == ids.ERROR_ATTN_INVALID_BLOCK_SIZE
    with pytest.raises(CudaDnnError) as e:  # backward before any forward on this handle
        a.hQ = a.hK = a.hV = a.hY = a._alloc(q)
        a.backward(q)
    assert e.value.code == ids.ERROR_ATTN_BACKWARD_WITHOUT_FORWARD
    with pytest.raises(CudaDnnError) as e:  # unknown memory handle
        cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, 8, 99999, a.hK, a.hV, 0, a.hY, False)
    assert e.value.code == ids.ERROR_MEMORY_NOT_FOUND
    with pytest.raises(CudaDnnError) as e:  # tensor smaller than B*H*T*D
        small = a._alloc(4)
        cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, 8, small, a.hK, a.hV, 0, a.hY, False)
    assert e.value.code == ids.ERROR_MEMORY_TOO_SMALL
    with pytest.raises(CudaDnnError) as e:  # wrong number of longs (device.h:2492 wants exactly 9)
        cuda._invoke(ids.CUDNN_FN_ATTN_FWD, None, [1, 2, 3])
    assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE
    with pytest.raises(CudaDnnError) as e:  # forward on a handle that was never Set
        h = cuda.CreateAttn()
        cuda.AttnScaledDotProductForward(a.hCudnn, h, 8, a.hQ, a.hK, a.hV, 0, a.hY, False)
    assert e.value.code == ids.ERROR_ATTN_NOT_INITIALIZED
    a.close()
    # attention dropout in training: the reference's guard always errors on this route (attn.cu:265)
    d = Sdpa(cuda, 1, 8, 2, 16, training=True, dropout=0.1)
    with pytest.raises(CudaDnnError) as e:
        d.forward(q, k, v, None)
    assert e.value.code == ids.ERROR_ATTN_MISSING_DESCRIPTOR
    d.close()
    with pytest.raises(CudaDnnError) as e:  # head size beyond the kernels
        Sdpa(cuda, 1, 8, 2, 256)
    assert e.value.code == ids.ERROR_ATTN_UNSUPPORTED_SHAPE


def test_memory_roundtrip_and_pinned_result(cuda):
    rng = np.random.default_rng(4)
    data = rng.standard_normal(1000).astype(np.float32)
    h = cuda.AllocMemory(data)
    np.testing.assert_array_equal(cuda.GetMemory(h, 1000), data)
    np.testing.assert_array_equal(cuda.GetMemory(h), data)      # count -1: library-owned pinned buffer
    cuda.SetMemory(h, data[::-1].copy())
    np.testing.assert_array_equal(cuda.GetMemory(h, 10), data[::-1][:10])
    hb = cuda.AllocMemoryBf16(data)
    np.testing.assert_array_equal(cuda.GetMemory(hb, 1000), bf16_round(data))
    assert cuda.GetPointer(h) % 256 == 0
    cuda.FreeMemory(h)
    cuda.FreeMemory(hb)


# --------------------------------------------------------------------------- tensor-core path

@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [128, 256, 200, 384, 1000, 2048])
@pytest.mark.parametrize("causal", [True, False])
def test_bf16_tensor_core_forward(cuda, T, D, causal):
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(T + D)
    B, H = 1, 3
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, H, T, D))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16,
             flags=ids.MCA_FLAG_CAUSAL_IMPLICIT if causal else 0)
    y = a.forward(q, k, v, None)
    mask = oracle.causal_mask(T) if causal else None
    ref = oracle.sdpa_forward(q, k, v, mask, 1 if causal else 0, f64=True)
    assert rel_err(y, ref) < BF16_TOL
    a.close()


def test_bf16_tensor_core_accepts_causal_mask_handle(cuda):
    """A (T,T) tril mask passed the reference's way is recognised as causal and runs the tensor-core kernel; any other
    mask (general (T,T), batch) runs the exact fp32 kernels on fp32 copies, forward and backward, with the reference's
    mask semantics (a fully masked row is uniform)."""
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    rng = np.random.default_rng(9)
    B, H, T, D = 2, 2, 256, 64
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, H, T, D))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16)
    y = a.forward(q, k, v, oracle.causal_mask(T))
    assert rel_err(y, oracle.sdpa_forward(q, k, v, oracle.causal_mask(T), 1, f64=True)) < BF16_TOL
    a.close()
    dy = bf16_round(rng.standard_normal(q.shape).astype(np.float32))
    general = np.ones((T, T), np.float32) - np.eye(T, dtype=np.float32)
    general[5] = 0.0                                          # one fully masked row
    keys = (rng.random((B, T)) > 0.3).astype(np.float32)      # batch mask: keys kept per batch item
    # on the tensor cores (keep-bits), and with MCA_FLAG_EXACT_FP32 through the exact fp32 kernels on fp32 copies
    for flags in (None, ids.MCA_FLAG_EXACT_FP32):
        for mask, mode, batch in ((general, 1, False), (keys, 2, True)):
            b = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16, flags=flags)
            y = b.forward(q, k, v, mask, batch_mask=batch)
            assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, mode, f64=True)) < BF16_TOL
            got = b.backward(dy)
            for g_, r_ in zip(got, oracle.sdpa_backward(q, k, v, dy, mask, mode, f64=True)):
                assert rel_err(g_, r_) < BF16_TOL
            b.close()
    b = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16)      # inference handle: forward only
    y = b.forward(q, k, v, general)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, general, 1, f64=True)) < BF16_TOL
    np.testing.assert_allclose(y[:, :, 5], v.mean(axis=2), atol=2e-2)     # the fully masked row is uniform
    b.close()


def test_long_context_shape_properties(cuda):
    """BASELINE config 5 shape (16 heads x 128, bf16, causal) at T = 8192: the CPU oracle checks a
    strided subset of query rows, and a size-independent property checks the rest: with V = 1 every
    output element is 1, and with Q = 0 row i is the mean of V[0..i]."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(8)
    B, H, T, D = 1, 16, 8192, 128
    q, k, v = (bf16_round(a / np.sqrt(np.float32(D))) for a in rand_qkv(rng, B, H, T, D))
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    y = a.forward(q, k, v, None)
    ref = oracle.sdpa_forward_rows(q, k, v, None, 3, 5, 257)
    assert rel_err(y[:, :, 5::257], ref) < BF16_TOL
    ones = np.ones_like(v)
    y1 = a.forward(q, k, ones, None)
    assert np.abs(y1 - 1).max() < 1e-2
    y0 = a.forward(np.zeros_like(q), k, v, None)
    cm = np.cumsum(v.astype(np.float64), axis=2) / np.arange(1, T + 1)[None, None, :, None]
    assert rel_err(y0, cm) < BF16_TOL
    a.close()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [128, 256, 200, 640, 1024])
@pytest.mark.parametrize("causal", [True, False])
def test_bf16_tensor_core_backward(cuda, T, D, causal):
    """ATTN_BWD with bf16 handles: tcgen05 dQ and dK/dV kernels against the fp64 oracle."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(7 * T + D)
    B, H = 2, 2
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, H, T, D))
    dy = bf16_round(rng.standard_normal(q.shape).astype(np.float32))
    a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16,
             flags=ids.MCA_FLAG_CAUSAL_IMPLICIT if causal else 0)
    y = a.forward(q, k, v, None)
    mode = 3 if causal else 0
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, mode, f64=True)) < BF16_TOL
    got = a.backward(dy)
    ref = oracle.sdpa_backward(q, k, v, dy, None, mode, f64=True)
    for name, g_, r_ in zip("qkv", got, ref):
        assert rel_err(g_, r_) < BF16_TOL, name
    a.close()


TF32_TOL = 5e-3  # tf32 products keep 10 mantissa bits; this variant sits behind a flag for that reason


@pytest.mark.parametrize("T", [128, 200, 1024])
@pytest.mark.parametrize("causal", [True, False])
def test_tf32_tensor_core_forward(cuda, T, causal):
    """dtype = MCA_DTYPE_TF32 on fp32 handles: tcgen05 kind::tf32 for 64-wide heads (inference)."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(T)
    B, H, D = 2, 3, 64
    q, k, v = rand_qkv(rng, B, H, T, D)
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_TF32, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT if causal else 0)
    y = a.forward(q, k, v, None)
    err = rel_err(y, oracle.sdpa_forward(q, k, v, None, 3 if causal else 0, f64=True))
    assert 1e-6 < err < TF32_TOL   # not the exact-fp32 kernel, and within the tf32 budget
    a.close()


def test_tf32_falls_back_to_exact_fp32_when_training_or_wide(cuda):
    """What single-pass tf32 does not cover goes the way of an fp32 handle: training at head size 64 runs the
    split-operand tensor-core kernels (fp32 accuracy, forward and backward), 128-wide heads the exact kernel, other head
    sizes and other masks whichever of the two applies."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(1)
    B, H, T, D = 1, 2, 256, 64
    q, k, v = rand_qkv(rng, B, H, T, D)
    dy = rng.standard_normal(q.shape).astype(np.float32)
    a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_TF32, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    y = a.forward(q, k, v, None)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, 3, f64=True)) < FP32_TIGHT
    for g_, r_ in zip(a.backward(dy), oracle.sdpa_backward(q, k, v, dy, None, 3, f64=True)):
        assert rel_err(g_, r_) < FP32_TIGHT
    a.close()
    q, k, v = rand_qkv(rng, 1, 2, 256, 128)
    b = Sdpa(cuda, 1, 256, 2, 128, dtype=ids.MCA_DTYPE_TF32)
    assert rel_err(b.forward(q, k, v, oracle.causal_mask(256)), oracle.sdpa_forward(q, k, v, None, 3, f64=True)) < FP32_TIGHT
    b.close()
    # head size 32, and head size 64 with a key mask (inference): fp32 accuracy as well
    q, k, v = rand_qkv(rng, 2, 2, 200, 32)
    c = Sdpa(cuda, 2, 200, 2, 32, dtype=ids.MCA_DTYPE_TF32, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    assert rel_err(c.forward(q, k, v, None), oracle.sdpa_forward(q, k, v, None, 3, f64=True)) < FP32_TIGHT
    c.close()
    q, k, v = rand_qkv(rng, 2, 2, 200, 64)
    keys = (rng.random((2, 200)) > 0.3).astype(np.float32)
    d = Sdpa(cuda, 2, 200, 2, 64, dtype=ids.MCA_DTYPE_TF32)
    assert rel_err(d.forward(q, k, v, keys, batch_mask=True), oracle.sdpa_forward(q, k, v, keys, 2, f64=True)) < FP32_TIGHT
    d.close()


def test_gpt2_small_shape_layer_bf16(cuda):
    """BASELINE config 2 shape in bf16 (12 heads x 64, T = 1024), forward + backward, B reduced to 2."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(12)
    B, H, T, D = 2, 12, 1024, 64
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, H, T, D, 0.5))
    dy = bf16_round(rng.standard_normal(q.shape).astype(np.float32))
    a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16)
    y = a.forward(q, k, v, oracle.causal_mask(T))   # the mask handle the C# layer passes
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, 3)) < BF16_TOL
    got = a.backward(dy)
    for g_, r_ in zip(got, oracle.sdpa_backward(q, k, v, dy, None, 3)):
        assert rel_err(g_, r_) < BF16_TOL
    a.close()


def _to_bf16_bits(a):
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def _from_bf16_bits(u):
    return (u.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("host", ["f32", "bf16"])
@pytest.mark.parametrize("B,H,T,D,chunk", [(1, 1, 128, 64, 0), (2, 3, 200, 128, 0), (2, 5, 384, 64, 3),
                                           (1, 7, 1000, 128, 2), (3, 4, 256, 128, 1)])
def test_forward_from_host_tensors_pipelined(cuda, host, B, H, T, D, chunk):
    """Chunked three-stream pipeline over host tensors (id 2003): same result as the oracle whatever the
    chunking (including a ragged last chunk), for fp32 and bf16 host tensors, and identical to the
    handle-based bf16 path."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(B * 1000 + T + D)
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, H, T, D))
    ref = oracle.sdpa_forward(q, k, v, oracle.causal_mask(T), 1, f64=True)
    if host == "f32":
        y = np.zeros_like(q)
        cuda.AttnForwardHost(q, k, v, y, True, chunk)
    else:
        yb = np.zeros(q.shape, np.uint16)
        cuda.AttnForwardHost(_to_bf16_bits(q), _to_bf16_bits(k), _to_bf16_bits(v), yb, True, chunk)
        y = _from_bf16_bits(yb)
    assert rel_err(y, ref) < BF16_TOL
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16, flags=ids.MCA_FLAG_CAUSAL_IMPLICIT)
    y2 = a.forward(q, k, v, None)
    a.close()
    np.testing.assert_array_equal(y, y2)


def test_forward_from_host_rejects_bad_arguments(cuda):
    from mycaffe_b200 import CudaDnnError
    q = np.zeros((1, 1, 128, 32), np.float32)
    with pytest.raises(CudaDnnError) as ei:
        cuda.AttnForwardHost(q, q, q, q.copy(), True)
    assert ei.value.code == 90901      # no tensor-core kernel for this head size


def _split_packed(qkv, H):
    """(B,T,3C) c_attn output -> q, k, v as (B,H,T,D): the split + head transpose of
    CausalSelfAttentionLayer.cs:537-557 restated in numpy."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    return tuple(np.ascontiguousarray(qkv[:, :, i * C:(i + 1) * C].reshape(B, T, H, C // H).transpose(0, 2, 1, 3))
                 for i in range(3))


def _merge_heads(y):
    B, H, T, D = y.shape
    return np.ascontiguousarray(y.transpose(0, 2, 1, 3).reshape(B, T, H * D))


@pytest.mark.parametrize("dtype,B,H,T,D,mask_kind", [
    ("f32", 2, 3, 70, 16, "causal_handle"), ("f32", 1, 4, 128, 16, "none"), ("f32", 2, 2, 200, 64, "batch"),
    ("f32", 2, 2, 200, 128, "causal_handle"), ("f32", 1, 2, 300, 128, "batch"),
    ("bf16", 2, 3, 200, 64, "causal"), ("bf16", 1, 2, 384, 128, "causal"), ("bf16", 2, 2, 256, 128, "none")])
def test_packed_qkv_layout_forward_backward(cuda, dtype, B, H, T, D, mask_kind):
    """Ids 2004/2005: q, k, v read in place from the (B,T,3C) projection output, y written as (B,T,C), and the
    backward producing the (B,T,3C) gradient from a (B,T,C) one -- against the oracle on the split tensors."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(B * 100 + T + D)
    C = H * D
    bf16 = dtype == "bf16"
    tol = BF16_TOL if bf16 else FP32_TIGHT
    rnd = bf16_round if bf16 else (lambda a: a)
    qkv = rnd(rng.standard_normal((B, T, 3 * C)).astype(np.float32))
    dy = rnd(rng.standard_normal((B, T, C)).astype(np.float32))
    q, k, v = _split_packed(qkv, H)
    mask, mode, hmask_data, batch = None, 0, None, False
    if mask_kind in ("causal", "causal_handle"):
        mask, mode = oracle.causal_mask(T), 1
        if mask_kind == "causal_handle":
            hmask_data = mask
    elif mask_kind == "batch":
        mask = (rng.random((B, T)) > 0.3).astype(np.float32)
        mask[:, 0] = 1
        mode, hmask_data, batch = 2, mask, True
    alloc = cuda.AllocMemoryBf16 if bf16 else cuda.AllocMemory
    hC, hA = cuda.CreateCuDNN(), cuda.CreateAttn()
    cuda.SetAttn(hC, hA, 0, True, B, T, H, D, 0.0, 0, ids.MCA_DTYPE_BF16 if bf16 else ids.MCA_DTYPE_F32,
                 ids.MCA_FLAG_CAUSAL_IMPLICIT if mask_kind == "causal" else 0)
    hQKV, hdQKV, hY, hdY = alloc(qkv), alloc(qkv.size), alloc(B * T * C), alloc(dy)
    hMask = cuda.AllocMemory(hmask_data) if hmask_data is not None else 0
    cuda.AttnScaledDotProductForwardPacked(hC, hA, T, hQKV, hMask, hY, batch)
    y = cuda.GetMemory(hY, B * T * C).reshape(B, T, C)
    y_ref = oracle.sdpa_forward(q, k, v, mask, mode, f64=True)
    assert rel_err(y, _merge_heads(y_ref)) < tol
    cuda.AttnScaledDotProductBackwardPacked(hC, hA, hQKV, hdQKV, 0, hY, hdY)
    dqkv = cuda.GetMemory(hdQKV, qkv.size).reshape(B, T, 3 * C)
    dy_h = np.ascontiguousarray(dy.reshape(B, T, H, D).transpose(0, 2, 1, 3))
    ref = oracle.sdpa_backward(q, k, v, dy_h, mask, mode, f64=True)
    for i, name in enumerate("qkv"):
        assert rel_err(dqkv[:, :, i * C:(i + 1) * C], _merge_heads(ref[i])) < (tol if bf16 else FP32_TOL), name
    # a backward in the other layout does not match this forward
    from mycaffe_b200 import CudaDnnError
    if not bf16:
        n = B * H * T * D
        hs = [cuda.AllocMemory(n) for _ in range(7)]
        with pytest.raises(CudaDnnError) as ei:
            cuda.AttnScaledDotProductBackward(hC, hA, hs[0], hs[1], hs[2], hs[3], hs[4], hs[5], 0, hY, hs[6])
        assert ei.value.code == 90903
        for h in hs:
            cuda.FreeMemory(h)
    for h in (hQKV, hdQKV, hY, hdY) + ((hMask,) if hMask else ()):
        cuda.FreeMemory(h)
    cuda.FreeAttn(hA)
    cuda.FreeCuDNN(hC)


def test_scatter_epilogue_writes_every_destination(cuda):
    """mca_sdpa_forward_tc_scatter: the heads of one rank land, at their offset, in every destination buffer
    of the full (B, H_total, T, D) output (two local buffers stand in for this GPU's and a peer's)."""
    import ctypes as C
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    rng = np.random.default_rng(5)
    B, Hl, Htot, h_lo, T, D = 2, 2, 6, 3, 200, 128
    q, k, v = (bf16_round(a) for a in rand_qkv(rng, B, Hl, T, D))
    hq, hk, hv = (cuda.AllocMemoryBf16(a) for a in (q, k, v))
    n_full = B * Htot * T * D
    dst = [cuda.AllocMemoryBf16(np.full(n_full, 7.0, np.float32)) for _ in range(2)]
    hst = cuda.AllocMemory(np.zeros(8, np.float32))
    ptrs = (C.c_void_p * 2)(*[cuda.GetPointer(h) + h_lo * T * D * 2 for h in dst])
    rc = lib.mca_sdpa_forward_tc_scatter(cuda.GetPointer(hq), cuda.GetPointer(hk), cuda.GetPointer(hv), ids.MCA_DTYPE_BF16, 1,
                                         B, Hl, T, D, ptrs, 2, Htot * T * D, T * D, D, None, cuda.GetPointer(hst), None)
    assert rc == 0
    cuda.SynchronizeDevice()
    ref = oracle.sdpa_forward(q, k, v, None, 3, f64=True)
    outs = [cuda.GetMemory(h, n_full).reshape(B, Htot, T, D) for h in dst]
    np.testing.assert_array_equal(outs[0], outs[1])
    assert rel_err(outs[0][:, h_lo:h_lo + Hl], ref) < BF16_TOL
    untouched = np.ones(Htot, bool)
    untouched[h_lo:h_lo + Hl] = False
    assert np.all(outs[0][:, untouched] == 7.0)          # other ranks' heads are not written
    assert np.all(cuda.GetMemory(hst, 8).view(np.int32)[:4] == 0)
    for h in [hq, hk, hv, hst] + dst:
        cuda.FreeMemory(h)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [200, 640])
def test_bf16_tensor_core_general_and_batch_masks(cuda, T, D):
    """bf16 handles with the reference's other mask forms over several key tiles: random (T,T) mask with a fully masked
    row, (B,T) key mask with a batch item that masks everything; forward and backward on the tensor cores."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(T + D)
    B, H = 2, 2
    q, k, v, dy = (bf16_round(a) for a in (*rand_qkv(rng, B, H, T, D), rng.standard_normal((B, H, T, D)).astype(np.float32)))
    general = (rng.random((T, T)) > 0.5).astype(np.float32)
    general[T // 4] = 0.0
    keys = (rng.random((B, T)) > 0.3).astype(np.float32)
    keys[B - 1] = 0.0
    for mask, mode, batch in ((general, 1, False), (keys, 2, True)):
        a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16)
        y = a.forward(q, k, v, mask, batch_mask=batch)
        assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, mode, f64=True)) < BF16_TOL
        for g_, r_ in zip(a.backward(dy), oracle.sdpa_backward(q, k, v, dy, mask, mode, f64=True)):
            assert rel_err(g_, r_) < BF16_TOL
        a.close()


@pytest.mark.parametrize("dtype_name,D", [("bf16", 64), ("bf16", 128), ("fp32", 16), ("fp32", 32), ("fp32", 64)])
@pytest.mark.parametrize("T", [130, 640, 1300])
def test_one_tile_and_two_tile_ctas_agree(cuda, dtype_name, D, T):
    """Short sequences run the forward as CTAs of one query tile, two to an SM; long ones as CTAs of two tiles.  The
    arithmetic per query tile is the same, so the two shapes agree bit for bit: causal, no mask, general and batch
    masks; each is also held to the oracle."""
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    rng = np.random.default_rng(T + D)
    B, H = 2, 3
    bf16 = dtype_name == "bf16"
    q, k, v = rand_qkv(rng, B, H, T, D)
    if bf16:
        q, k, v = (bf16_round(a) for a in (q, k, v))
    general = (rng.random((T, T)) > 0.4).astype(np.float32)
    general[T // 3] = 0.0
    keys = (rng.random((B, T)) > 0.3).astype(np.float32)
    before = lib.mca_tc_narrow_len(-1)
    try:
        for mask, mode, batch in ((oracle.causal_mask(T), 1, False), (None, 0, False), (general, 1, False), (keys, 2, True)):
            out = []
            for limit in (0, 1 << 30):
                lib.mca_tc_narrow_len(limit)
                a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16 if bf16 else None)
                out.append(a.forward(q, k, v, mask, batch_mask=batch))
                a.close()
            np.testing.assert_array_equal(out[0], out[1])
            ref = oracle.sdpa_forward(q, k, v, mask, mode, f64=True)
            assert rel_err(out[0], ref) < (BF16_TOL if bf16 else FP32_TIGHT)
    finally:
        lib.mca_tc_narrow_len(before)
    assert lib.mca_tc_narrow_len(-1) == before


def test_backward_refuses_gradients_that_alias_inputs(cuda):
    """The dQ kernel and the dK/dV kernel run side by side, both reading q, k, v and dY: a gradient handle naming an
    input's memory is refused (a blob's diff and data never share memory)."""
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    rng = np.random.default_rng(4)
    q, k, v = rand_qkv(rng, 1, 2, 64, 32)
    a = Sdpa(cuda, 1, 64, 2, 32, training=True)
    a.forward(q, k, v, oracle.causal_mask(64))
    hdY, hd = a._alloc(q), a._alloc(q.size)
    for args in ((a.hQ, a.hQ, a.hK, hd, a.hV, hd), (a.hQ, hd, a.hK, hdY, a.hV, hd), (a.hQ, hd, a.hK, hd, a.hV, a.hK)):
        with pytest.raises(CudaDnnError) as e:
            cuda.AttnScaledDotProductBackward(a.hCudnn, a.hAttn, *args, 0, a.hY, hdY)
        assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE
    g = a.backward(q)          # distinct handles: fine
    assert all(np.isfinite(x).all() for x in g)
    a.close()


@pytest.mark.parametrize("dtype_name", ["fp32", "bf16"])
def test_mask_class_is_verified_on_every_forward(cuda, dtype_name):
    """A (T,T) mask handle is classified on every Forward; in synchronous mode the kernels are chosen on the class the
    last verified call found and the class is checked with the status read that ends the call.  Rewriting the mask in
    place between calls -- lower triangle, then a band, then the lower triangle again -- must give the right result
    every time (the call whose guess was wrong runs again before it returns)."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(9)
    B, H, T, D = 2, 3, 256, 64
    bf16 = dtype_name == "bf16"
    q, k, v = rand_qkv(rng, B, H, T, D)
    if bf16:
        q, k, v = (bf16_round(a) for a in (q, k, v))
    tol = BF16_TOL if bf16 else FP32_TIGHT
    tril = oracle.causal_mask(T)
    band = np.triu(tril, -7).astype(np.float32)
    a = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_BF16 if bf16 else None)
    alloc = cuda.AllocMemoryBf16 if bf16 else cuda.AllocMemory
    hq, hk, hv, hy = alloc(q), alloc(k), alloc(v), alloc(q.size)
    hm = cuda.AllocMemory(tril)
    for m in (tril, tril, band, band, tril, band, tril):
        cuda.SetMemory(hm, m)
        cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, hq, hk, hv, hm, hy, False)
        y = cuda.GetMemory(hy, q.size).reshape(q.shape)
        assert rel_err(y, oracle.sdpa_forward(q, k, v, m, 1, f64=True)) < tol
    for h in (hq, hk, hv, hy, hm):
        cuda.FreeMemory(h)
    a.close()
