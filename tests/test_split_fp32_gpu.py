"""The split-operand tensor-core forward for fp32 callers (every operand carried as two fp16 halves, three products
per contraction): parity with the fp64 oracle at fp32 accuracy, through the raw entry point and through ATTN_FWD on a
default (fp32) handle."""
import numpy as np
import pytest

import oracle
from gpu_util import Sdpa
from helpers import rel_err

pytestmark = pytest.mark.gpu

SPLIT_TOL = 2e-5   # the tolerance the exact CUDA-core kernel is held to; measured 1e-7 .. 7e-6 (long unmasked rows are the worst)


@pytest.fixture(scope="module")
def cuda():
    from mycaffe_b200 import CudaDnn
    c = CudaDnn(0)
    yield c
    c.Dispose()


def run_raw(q, k, v, causal, want_stats=False, layout=0, dy=None):
    import torch
    from mycaffe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, H, T, D = q.shape
    if layout == 1:   # (B,T,3C) projection output, y as (B,T,C)
        C_ = H * D
        qkv = np.concatenate([a.transpose(0, 2, 1, 3).reshape(B, T, C_) for a in (q, k, v)], axis=-1)
        t = torch.from_numpy(np.ascontiguousarray(qkv)).to(dev)
        qd, kd, vd = t, t, t
        ptrs = (t.data_ptr(), t.data_ptr() + C_ * 4, t.data_ptr() + 2 * C_ * 4)
    else:
        qd, kd, vd = (torch.from_numpy(a).to(dev) for a in (q, k, v))
        ptrs = (qd.data_ptr(), kd.data_ptr(), vd.data_ptr())
    y = torch.empty(B * H * T * D, device=dev)
    rm, rs = torch.empty(B * H * T, device=dev), torch.empty(B * H * T, device=dev)
    yc = torch.empty(B * H * T * D, device=dev)
    nbytes = lib.mca_sdpa_forward_f32_tc_workspace_bytes_d(B, H, T, D)
    if D <= 64:
        assert nbytes == lib.mca_sdpa_forward_f32_tc_workspace_bytes(B, H, T)
    ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
    wp = (ws.data_ptr() + 1023) // 1024 * 1024
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    lse = torch.empty(B * H * T, device=dev)
    stats = want_stats or dy is not None
    rc = lib.mca_sdpa_forward_f32_tc(*ptrs, int(causal), B, H, T, D, y.data_ptr(), rm.data_ptr() if want_stats else None,
                                     rs.data_ptr() if want_stats else None, yc.data_ptr() if stats else None,
                                     lse.data_ptr() if stats else None, wp, nbytes, st.data_ptr(), layout, None)
    torch.cuda.synchronize()
    assert rc == 0 and st[0].item() == 0, (rc, st[:4].tolist())
    yh = y.cpu().numpy()
    yh = yh.reshape(B, T, H, D).transpose(0, 2, 1, 3) if layout == 1 else yh.reshape(B, H, T, D)
    if dy is not None:
        # backward from what the forward left in the workspace; gradients in the layout of the inputs
        to_bt = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3).reshape(B, T, H * D))
        dyd = torch.from_numpy(to_bt(dy) if layout == 1 else dy).to(dev)
        delta = torch.empty(B * H * T, device=dev)
        if layout == 1:
            g = torch.zeros(B, T, 3 * H * D, device=dev)
            gp = (g.data_ptr(), g.data_ptr() + H * D * 4, g.data_ptr() + 2 * H * D * 4)
        else:
            gq, gk, gv = (torch.zeros(B, H, T, D, device=dev) for _ in range(3))
            gp = (gq.data_ptr(), gk.data_ptr(), gv.data_ptr())
        rc = lib.mca_sdpa_backward_f32_tc(dyd.data_ptr(), yc.data_ptr(), lse.data_ptr(), delta.data_ptr(), int(causal), B, H, T, D,
                                          *gp, wp, nbytes, st.data_ptr(), layout, None)
        torch.cuda.synchronize()
        assert rc == 0 and st[0].item() == 0, (rc, st[:4].tolist())
        if layout == 1:
            gh = g.cpu().numpy().reshape(B, T, 3, H, D).transpose(2, 0, 3, 1, 4)
            return yh, gh[0], gh[1], gh[2]
        return yh, gq.cpu().numpy(), gk.cpu().numpy(), gv.cpu().numpy()
    if want_stats:
        return yh, rm.cpu().numpy().reshape(B, H, T), rs.cpu().numpy().reshape(B, H, T), yc.cpu().numpy().reshape(B, H, T, D)
    return yh


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [16, 32, 64, 128])
@pytest.mark.parametrize("T", [1, 17, 128, 200, 257, 1024])
def test_split_forward_matches_fp64(T, D, causal):
    rng = np.random.default_rng(31 * T + D)
    B, H = 2, 3
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    y = run_raw(q, k, v, causal)
    ref = oracle.sdpa_forward(q, k, v, None, 3 if causal else 0, f64=True)
    assert rel_err(y, ref) < SPLIT_TOL


@pytest.mark.parametrize("scale", [1e-4, 0.02, 300.0, 1e6])
def test_split_forward_is_scale_free(scale):
    """Each tensor is scaled by a power of two before it is split, so tiny and huge tensors keep fp32 accuracy
    (unscaled, their low halves would leave the fp16 range)."""
    rng = np.random.default_rng(7)
    B, H, T, D = 1, 2, 300, 64
    q = (scale * rng.standard_normal((B, H, T, D))).astype(np.float32)
    k = (rng.standard_normal((B, H, T, D)) / scale).astype(np.float32)     # logits stay O(1)
    v = (scale * rng.standard_normal((B, H, T, D))).astype(np.float32)
    y = run_raw(q, k, v, True)
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, 3, f64=True)) < SPLIT_TOL
    z = np.zeros_like(q)                                                    # an all-zero tensor has no scale
    y0 = run_raw(z, k, v, True)
    cm = np.cumsum(v.astype(np.float64), axis=2) / np.arange(1, T + 1)[None, None, :, None]
    assert rel_err(y0, cm) < SPLIT_TOL


def test_split_forward_statistics_and_packed_layout():
    rng = np.random.default_rng(11)
    B, H, T, D = 2, 4, 160, 32
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    ref, p = oracle.sdpa_forward(q, k, v, None, 3, f64=True, want_probs=True)
    y, rm, rs, yc = run_raw(q, k, v, True, want_stats=True)
    assert rel_err(y, ref) < SPLIT_TOL
    np.testing.assert_array_equal(yc, y)
    # exp(s - row_max) / row_sum must be the probabilities (row_max need not be the true maximum)
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(D)
    got = np.exp(s - rm[..., None]) / rs[..., None]
    got = np.where(np.tril(np.ones((T, T), bool)), got, 0.0)
    assert np.abs(got - p).max() < 1e-5
    yp = run_raw(q, k, v, True, layout=1)
    np.testing.assert_array_equal(yp, y)


def test_default_fp32_handle_uses_it_and_the_flag_switches_it_off(cuda):
    """ATTN_FWD / ATTN_BWD on a default handle (what an unmodified C# layer creates): forward and backward on the
    tensor cores with split operands; with MCA_FLAG_EXACT_FP32 both in exact fp32 on CUDA cores."""
    from mycaffe_b200 import function_ids as ids
    rng = np.random.default_rng(12)
    B, H, T, D = 2, 4, 384, 64
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    mask = oracle.causal_mask(T)
    ref = oracle.sdpa_forward(q, k, v, mask, 1, f64=True)
    gref = oracle.sdpa_backward(q, k, v, dy, mask, 1, f64=True)
    outs = {}
    for name, flags in (("default", None), ("exact", ids.MCA_FLAG_EXACT_FP32)):
        a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_F32 if flags else None, flags=flags)
        outs[name] = a.forward(q, k, v, mask)
        assert rel_err(outs[name], ref) < 2e-5
        for g_, r_ in zip(a.backward(dy), gref):
            assert rel_err(g_, r_) < 2e-5
        a.close()
    assert rel_err(outs["default"], ref) < SPLIT_TOL
    assert not np.array_equal(outs["default"], outs["exact"])     # two different kernels ran
    # a general (non-causal) mask is packed into keep-bits and applied by the same tensor-core kernel
    band = np.triu(mask, -5).astype(np.float32)
    a = Sdpa(cuda, B, T, H, D)
    assert rel_err(a.forward(q, k, v, band), oracle.sdpa_forward(q, k, v, band, 1, f64=True)) < 2e-5
    a.close()


def test_gpt2_layer_shape_split(cuda):
    """Config 2's layer shape (12 heads x 64, T = 1024) on the default handle, B = 2, every (batch, head)."""
    rng = np.random.default_rng(2)
    B, H, T, D = 2, 12, 1024, 64
    q, k, v = ((0.5 * rng.standard_normal((B, H, T, D))).astype(np.float32) for _ in range(3))
    a = Sdpa(cuda, B, T, H, D)
    y = a.forward(q, k, v, oracle.causal_mask(T))
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, 3, f64=True)) < SPLIT_TOL
    a.close()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [16, 32, 64])
@pytest.mark.parametrize("T", [1, 17, 128, 200, 257, 1024])
def test_split_backward_matches_fp64(T, D, causal):
    """dQ, dK, dV of the split-operand backward kernels (three fp16 products per contraction, P^T / dS split) against
    the fp64 oracle, at the tolerance of the exact fp32 kernels."""
    rng = np.random.default_rng(17 * T + D)
    B, H = 2, 2
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    y, dq, dk, dv = run_raw(q, k, v, causal, dy=dy)
    mode = 3 if causal else 0
    assert rel_err(y, oracle.sdpa_forward(q, k, v, None, mode, f64=True)) < SPLIT_TOL
    for name, g_, r_ in zip("qkv", (dq, dk, dv), oracle.sdpa_backward(q, k, v, dy, None, mode, f64=True)):
        assert rel_err(g_, r_) < SPLIT_TOL, name


@pytest.mark.parametrize("dy_scale", [1e-6, 1.0, 3e4])
def test_split_backward_gradient_scales_and_packed_layout(dy_scale):
    """Tiny (loss-scaled) and large output gradients keep their accuracy: dY is scaled by a power of two before it is
    split.  Packed layout: dy (B,T,C), gradients the thirds of a (B,T,3C) tensor."""
    rng = np.random.default_rng(23)
    B, H, T, D = 2, 3, 320, 64
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    dy = (dy_scale * rng.standard_normal((B, H, T, D))).astype(np.float32)
    ref = oracle.sdpa_backward(q, k, v, dy, None, 3, f64=True)
    got = run_raw(q, k, v, True, dy=dy)[1:]
    for name, g_, r_ in zip("qkv", got, ref):
        assert rel_err(g_, r_) < SPLIT_TOL, name
    got_p = run_raw(q, k, v, True, dy=dy, layout=1)[1:]
    for a_, b_ in zip(got, got_p):
        np.testing.assert_array_equal(a_, b_)


@pytest.mark.parametrize("T", [130, 640])
def test_head_size_128_handle(cuda, T):
    """128-wide heads: the forward is the split-operand tensor-core kernel (one query tile per CTA), with every mask
    form for inference; training keeps the exact fp32 backward, fed by the row statistics that forward leaves (causal /
    no mask) or by the exact forward (general and batch masks)."""
    rng = np.random.default_rng(128 + T)
    B, H, D = 2, 3, 128
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    from mycaffe_b200 import _lib
    lib = _lib.load()
    assert lib.mca_sdpa_forward_f32_tc_supported(D) == 1 and lib.mca_sdpa_backward_f32_tc_supported(D) == 0
    masks = [(oracle.causal_mask(T), 1, False), (None, 0, False)] + list(_masks(rng, B, T))
    for mask, mode, batch in masks:
        ref = oracle.sdpa_forward(q, k, v, mask, mode, f64=True)
        a = Sdpa(cuda, B, T, H, D)
        assert rel_err(a.forward(q, k, v, mask, batch_mask=batch), ref) < SPLIT_TOL, mode
        a.close()
        a = Sdpa(cuda, B, T, H, D, training=True)
        assert rel_err(a.forward(q, k, v, mask, batch_mask=batch), ref) < SPLIT_TOL, mode
        for name, g_, r_ in zip("qkv", a.backward(dy), oracle.sdpa_backward(q, k, v, dy, mask, mode, f64=True)):
            assert rel_err(g_, r_) < SPLIT_TOL, (name, mode)
        a.close()


def _masks(rng, B, T):
    """A general (T,T) mask with ragged rows, one fully masked row and one fully kept row; a (B,T) key mask whose last
    batch item masks every key."""
    general = (rng.random((T, T)) > 0.4).astype(np.float32)
    general[T // 3] = 0.0
    general[T // 2] = 1.0
    keys = (rng.random((B, T)) > 0.3).astype(np.float32)
    keys[B - 1] = 0.0
    return ((general, 1, False), (keys, 2, True))


@pytest.mark.parametrize("D", [16, 32, 64])
@pytest.mark.parametrize("T", [8, 200, 384, 1000])
def test_default_fp32_handle_with_general_and_batch_masks(cuda, T, D):
    """The reference's other mask forms (apply_mask / apply_mask_batch, attn.cu:302-311) on the split-operand
    tensor-core kernels: forward and backward against the fp64 oracle, including rows whose every key is masked (the
    reference's -1e29 makes them uniform) and, with the batch mask, a batch item without a single visible key."""
    rng = np.random.default_rng(5 * T + D)
    B, H = 3, 2
    q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
    for mask, mode, batch in _masks(rng, B, T):
        a = Sdpa(cuda, B, T, H, D, training=True)
        y = a.forward(q, k, v, mask, batch_mask=batch)
        assert rel_err(y, oracle.sdpa_forward(q, k, v, mask, mode, f64=True)) < SPLIT_TOL
        for name, g_, r_ in zip("qkv", a.backward(dy), oracle.sdpa_backward(q, k, v, dy, mask, mode, f64=True)):
            assert rel_err(g_, r_) < SPLIT_TOL, (name, mode)
        a.close()
    # the fully masked row is the mean of V
    general = _masks(np.random.default_rng(5 * T + D), B, T)[0][0]
    a = Sdpa(cuda, B, T, H, D)
    y = a.forward(q, k, v, general)
    np.testing.assert_allclose(y[:, :, T // 3], v.mean(axis=2), atol=2e-5)
    a.close()


def test_masked_entry_points_are_what_the_handle_runs(cuda):
    """mca_mask_pack + mca_sdpa_forward_f32_tc_masked called directly give bit for bit what ATTN_FWD on a default handle
    returns for the same mask: the handle runs the tensor-core kernel, not the CUDA-core one."""
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(77)
    B, H, T, D = 2, 3, 300, 64
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    keys = (rng.random((B, T)) > 0.3).astype(np.float32)
    qd, kd, vd, md = (torch.from_numpy(a).to(dev) for a in (q, k, v, keys))
    wpr = lib.mca_mask_bits_row_words(T)
    assert wpr == 4 * ((T + 127) // 128)
    bits = torch.zeros(B * wpr, dtype=torch.int32, device=dev)
    assert lib.mca_mask_pack(md.data_ptr(), 2, B, T, bits.data_ptr(), None, None) == 0
    torch.cuda.synchronize()
    packed = bits.cpu().numpy().view(np.uint32).reshape(B, wpr)
    for b in range(B):
        for j in (0, 31, 32, T - 1):
            assert (packed[b, j // 32] >> (j % 32)) & 1 == int(keys[b, j] != 0)
    assert packed[:, (T + 31) // 32:].sum() == 0                      # nothing beyond T
    y = torch.empty(B * H * T * D, device=dev)
    nbytes = lib.mca_sdpa_forward_f32_tc_workspace_bytes_d(B, H, T, D)
    if D <= 64:
        assert nbytes == lib.mca_sdpa_forward_f32_tc_workspace_bytes(B, H, T)
    ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
    wp = (ws.data_ptr() + 1023) // 1024 * 1024
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = lib.mca_sdpa_forward_f32_tc_masked(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 0, B, H, T, D, y.data_ptr(), None, None, None,
                                            None, wp, nbytes, st.data_ptr(), 0, bits.data_ptr(), 2, None)
    torch.cuda.synchronize()
    assert rc == 0 and st[0].item() == 0
    a = Sdpa(cuda, B, T, H, D)
    via_handle = a.forward(q, k, v, keys, batch_mask=True)
    a.close()
    np.testing.assert_array_equal(y.cpu().numpy().reshape(B, H, T, D), via_handle)
    e = Sdpa(cuda, B, T, H, D, dtype=ids.MCA_DTYPE_F32, flags=ids.MCA_FLAG_EXACT_FP32)
    exact = e.forward(q, k, v, keys, batch_mask=True)
    e.close()
    assert not np.array_equal(exact, via_handle) and rel_err(exact, via_handle) < 2e-5
    # a mask mode without its bits, or bits with a causal call, are refused
    assert lib.mca_sdpa_forward_f32_tc_masked(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 0, B, H, T, D, y.data_ptr(), None, None, None,
                                              None, wp, nbytes, st.data_ptr(), 0, None, 2, None) == ids.ERROR_PARAM_NULL
    assert lib.mca_sdpa_forward_f32_tc_masked(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 1, B, H, T, D, y.data_ptr(), None, None, None,
                                              None, wp, nbytes, st.data_ptr(), 0, bits.data_ptr(), 2, None) == ids.ERROR_ATTN_UNSUPPORTED_SHAPE
