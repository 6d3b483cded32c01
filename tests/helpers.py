"""Shared helpers for the parity tests: the CausalSelfAttention layer glue in numpy
(CausalSelfAttentionLayer.cs:526-628) around a pluggable SDPA, and error metrics."""
import numpy as np

PICO_CASES = {"csa": 1, "csa3": 3, "csaB": 1, "csa3B": 3}  # case -> heads


def rel_err(a, ref):
    """max-abs error relative to the output scale (max-abs of the reference).  A reference that is
    identically zero (e.g. dQ, dK at T = 1, where the softmax is constant) has no scale of its own;
    the error is then taken against 1, the scale of the unit-variance test inputs."""
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    scale = np.max(np.abs(ref))
    return float(np.max(np.abs(a - ref)) / (scale if scale > 0 else 1.0))


def split_heads(x, H):
    B, T, C = x.shape
    return np.ascontiguousarray(x.reshape(B, T, H, C // H).transpose(0, 2, 1, 3))


def merge_heads(y):
    B, H, T, D = y.shape
    return np.ascontiguousarray(y.transpose(0, 2, 1, 3).reshape(B, T, H * D))


def csa_qkv(x, w_attn, b_attn, H):
    """c_attn InnerProduct (weights (3C,C) row-major = (out,in)), split, head transpose."""
    ca = x @ w_attn.T + b_attn
    C = x.shape[-1]
    q, k, v = ca[..., :C], ca[..., C:2 * C], ca[..., 2 * C:]
    return split_heads(q, H), split_heads(k, H), split_heads(v, H)


def csa_forward(x, w_attn, b_attn, w_proj, b_proj, H, sdpa):
    """Full layer forward; ``sdpa(q,k,v)`` -> (B,H,T,D)."""
    q, k, v = csa_qkv(x, w_attn, b_attn, H)
    y = merge_heads(np.asarray(sdpa(q, k, v), np.float32))
    return y @ w_proj.T + b_proj


PICO_BLOCK_CASES = {"blk": 1, "blk3": 3, "blk3B": 3}  # case -> heads


def csa_backward(x, w_attn, b_attn, w_proj, H, d_out, sdpa_bwd):
    """Gradient of the layer output w.r.t. the layer input (CausalSelfAttentionLayer.cs:641-744):
    c_proj backward, head split, ``sdpa_bwd(q,k,v,dy)`` -> (dq,dk,dv), head merge, c_attn backward."""
    q, k, v = csa_qkv(x, w_attn, b_attn, H)
    dy = split_heads(d_out @ w_proj, H)
    dq, dk, dv = (np.asarray(g, np.float32) for g in sdpa_bwd(q, k, v, dy))
    d_ca = np.concatenate([merge_heads(dq), merge_heads(dk), merge_heads(dv)], axis=-1)
    return d_ca @ w_attn
