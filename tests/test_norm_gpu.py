"""Parity of the one-pass LayerNorm and RMSNorm-layer kernels against the op-by-op restatement of
the reference (layernorm.cu:291-384, RMSNormLayer.cs:156-231), through the function ids a C# layer
would call and through the raw entry points."""
import numpy as np
import pytest

import oracle
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


# (outer, channels, inner): GPT-2 block input, llama width, TFT width, ragged and unaligned rows
SHAPES = [(8, 128, 768), (2, 33, 4096), (4, 192, 64), (3, 7, 1000), (2, 5, 250), (1, 3, 8192), (2, 3, 1539), (1, 2, 16384)]


@pytest.mark.parametrize("outer,channels,inner", SHAPES)
def test_layernorm_ids_match_reference_math(cuda, outer, channels, inner):
    """CREATE_LAYERNORM / LAYERNORM_FWD / LAYERNORM_BWD (ids 970, 975, 976) with the reference's packing."""
    rng = np.random.default_rng(inner)
    x = (rng.standard_normal((outer, channels, inner)) * 1.5 + 0.3).astype(np.float32)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    eps = 1e-5
    h = cuda.CreateLayerNorm(0, x.size, outer, channels, inner, eps)
    hX, hY, hdY, hdX = cuda.AllocMemory(x), cuda.AllocMemory(x.size), cuda.AllocMemory(dy), cuda.AllocMemory(x.size)
    cuda.LayerNormForward(h, hX, hY)
    y = cuda.GetMemory(hY, x.size).reshape(x.shape)
    y_ref, sd = oracle.layernorm_forward(x, eps)
    assert rel_err(y, y_ref) < 1e-5
    cuda.LayerNormBackward(h, hY, hdY, hdX)
    dx = cuda.GetMemory(hdX, x.size).reshape(x.shape)
    dx_ref = oracle.layernorm_backward(y_ref, dy, sd, eps)
    assert rel_err(dx, dx_ref) < 1e-5
    for m in (hX, hY, hdY, hdX):
        cuda.FreeMemory(m)
    cuda.FreeLayerNorm(h)


def test_layernorm_handle_errors(cuda):
    from mycaffe_b200 import CudaDnnError, function_ids as ids
    with pytest.raises(CudaDnnError) as e:
        cuda.CreateLayerNorm(0, 100, 2, 5, 11, 1e-5)   # count != outer * channels * inner
    assert e.value.code == ids.ERROR_PARAM_OUT_OF_RANGE
    with pytest.raises(CudaDnnError) as e:
        cuda.LayerNormForward(12345, 1, 1)
    assert e.value.code == ids.ERROR_LAYERNORM_NOT_INITIALIZED
    h = cuda.CreateLayerNorm(0, 64, 1, 2, 32, 1e-5)
    hA = cuda.AllocMemory(64)
    with pytest.raises(CudaDnnError) as e:
        cuda.LayerNormBackward(h, hA, hA, hA)           # no forward yet: no stdev to divide by
    assert e.value.code == ids.ERROR_LAYERNORM_NOT_INITIALIZED
    cuda.FreeMemory(hA)
    cuda.FreeLayerNorm(h)


@pytest.mark.parametrize("weights", [True, False])
@pytest.mark.parametrize("outer,channels,inner", SHAPES)
def test_rmsnorm_layer_ids_match_reference_math(cuda, outer, channels, inner, weights):
    rng = np.random.default_rng(inner + 1)
    x = rng.standard_normal((outer, channels, inner)).astype(np.float32)
    w = (1 + 0.2 * rng.standard_normal(inner)).astype(np.float32) if weights else None
    dy = rng.standard_normal(x.shape).astype(np.float32)
    eps, rows = 1e-5, outer * channels
    hX, hY, hdY, hdX = cuda.AllocMemory(x), cuda.AllocMemory(x.size), cuda.AllocMemory(dy), cuda.AllocMemory(x.size)
    hInv = cuda.AllocMemory(rows)
    hW = cuda.AllocMemory(w) if weights else 0
    hdW = cuda.AllocMemory(inner) if weights else 0
    cuda.RmsNormForward(hX, hW, hY, hInv, rows, inner, eps)
    y = cuda.GetMemory(hY, x.size).reshape(x.shape)
    y_ref, inv_ref = oracle.rmsnorm_layer_forward(x, w, eps)
    assert rel_err(y, y_ref) < 1e-5
    assert rel_err(cuda.GetMemory(hInv, rows), inv_ref) < 1e-5
    cuda.RmsNormBackward(hX, hW, hdY, hInv, hdX, hdW, rows, inner)
    dx = cuda.GetMemory(hdX, x.size).reshape(x.shape)
    dx_ref, dw_ref = oracle.rmsnorm_layer_backward(x, w, dy, eps)
    assert rel_err(dx, dx_ref) < 1e-5
    if weights:
        assert rel_err(cuda.GetMemory(hdW, inner), dw_ref) < 1e-5
    for m in (hX, hY, hdY, hdX, hInv, hW, hdW):
        if m:
            cuda.FreeMemory(m)


def test_rmsnorm_backward_is_deterministic_and_many_rows(cuda):
    """More rows than CTAs: the weight gradient goes through per-CTA partials added in a fixed order."""
    rng = np.random.default_rng(3)
    rows, inner = 20000, 768
    x = rng.standard_normal((rows, inner)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(inner)).astype(np.float32)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    hX, hW, hdY, hdX = cuda.AllocMemory(x), cuda.AllocMemory(w), cuda.AllocMemory(dy), cuda.AllocMemory(x.size)
    hY, hInv, hdW = cuda.AllocMemory(x.size), cuda.AllocMemory(rows), cuda.AllocMemory(inner)
    cuda.RmsNormForward(hX, hW, hY, hInv, rows, inner, 1e-5)
    cuda.RmsNormBackward(hX, hW, hdY, hInv, hdX, hdW, rows, inner)
    dw1 = cuda.GetMemory(hdW, inner)
    cuda.RmsNormBackward(hX, hW, hdY, hInv, hdX, hdW, rows, inner)
    dw2 = cuda.GetMemory(hdW, inner)
    np.testing.assert_array_equal(dw1, dw2)
    _, dw_ref = oracle.rmsnorm_layer_backward(x, w, dy, 1e-5)
    assert rel_err(dw1, dw_ref) < 1e-5
    for m in (hX, hW, hdY, hdX, hY, hInv, hdW):
        cuda.FreeMemory(m)


def test_raw_entry_points_reject_bad_arguments():
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    assert lib.mca_layernorm_forward_f32(None, None, None, 4, 8, 1e-5, None) == ids.ERROR_PARAM_NULL
    assert lib.mca_rmsnorm_forward_f32(None, None, None, None, 4, 8, 1e-5, None) == ids.ERROR_PARAM_NULL
    assert lib.mca_rmsnorm_backward_scratch_floats(768) >= 768


@pytest.mark.parametrize("case", ["ln", "ln3", "ln3B", "ln-blk"])
def test_layernorm_ids_match_the_reference_vectors(cuda, pico_ln, case):
    """ids 970 / 975 / 976 on the reference's own LayerNorm vectors (gpt-pico-ln*, epsilon 1e-10): y from x, and the
    gradient at x from the gradient at y."""
    g = lambda n: pico_ln[f"{case}/{n}"]
    x = g("x")
    outer, channels, inner = x.shape
    h = cuda.CreateLayerNorm(0, x.size, outer, channels, inner, 1e-10)
    hX, hY, hdY, hdX = cuda.AllocMemory(x), cuda.AllocMemory(x.size), cuda.AllocMemory(g("grad_1a_y")), cuda.AllocMemory(x.size)
    cuda.LayerNormForward(h, hX, hY)
    np.testing.assert_allclose(cuda.GetMemory(hY, x.size).reshape(x.shape), g("y"), atol=5e-7)
    cuda.LayerNormBackward(h, hY, hdY, hdX)
    assert rel_err(cuda.GetMemory(hdX, x.size).reshape(x.shape), g("grad_9_x")) < 1e-5
    for m in (hX, hY, hdY, hdX):
        cuda.FreeMemory(m)
    cuda.FreeLayerNorm(h)


@pytest.mark.parametrize("case", ["blk", "blk3", "blk3B"])
def test_block_layernorm_then_attention_matches_the_reference_vectors(cuda, pico_ln, case):
    """The reference's transformer-block vectors through the library: 1_x -> LAYERNORM_FWD -> 2_x_ln11 -> the
    attention layer with ATTN_FWD at its core -> 3_x_attn; back: grad_8_x_attn -> ATTN_BWD -> grad_9_ln1 ->
    LAYERNORM_BWD (+ the residual branch) -> grad_10_x.  The InnerProduct glue either side of the attention core is
    the C# layer's and is restated in numpy."""
    from gpu_util import Sdpa
    from helpers import PICO_BLOCK_CASES, csa_backward, csa_forward
    H = PICO_BLOCK_CASES[case]
    g = lambda n: pico_ln[f"{case}/{n}"]
    x = g("1_x")
    B, T, Cn = x.shape
    hL = cuda.CreateLayerNorm(0, x.size, B, T, Cn, 1e-10)
    hX, hY = cuda.AllocMemory(x), cuda.AllocMemory(x.size)
    cuda.LayerNormForward(hL, hX, hY)
    ln1 = cuda.GetMemory(hY, x.size).reshape(x.shape)
    np.testing.assert_allclose(ln1, g("2_x_ln11"), atol=5e-7)

    a = Sdpa(cuda, B, T, H, Cn // H, training=True)
    mask = oracle.causal_mask(T)
    attn = csa_forward(ln1, g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), g("attn_proj_bias"), H,
                       lambda q, k, v: a.forward(q, k, v, mask))
    np.testing.assert_allclose(attn, g("3_x_attn"), atol=3e-7)
    d_ln1 = csa_backward(ln1, g("attn_weight"), g("attn_bias"), g("attn_proj_weight"), H, g("grad_8_x_attn"),
                         lambda q, k, v, dy: a.backward(dy))
    assert rel_err(d_ln1, g("grad_9_ln1")) < 1e-5
    hdY, hdX = cuda.AllocMemory(g("grad_9_ln1")), cuda.AllocMemory(x.size)
    cuda.LayerNormBackward(hL, hY, hdY, hdX)
    dx = cuda.GetMemory(hdX, x.size).reshape(x.shape) + g("grad_8_x")
    assert rel_err(dx, g("grad_10_x")) < 1e-5
    a.close()
    for m in (hX, hY, hdY, hdX):
        cuda.FreeMemory(m)
    cuda.FreeLayerNorm(hL)
