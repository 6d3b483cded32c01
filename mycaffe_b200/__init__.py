"""B200-native (sm_100a) replacement for the attention hot path of MyCaffe: the scaled-dot-product
core behind CausalSelfAttentionLayer / MultiheadAttentionLayer, the TFT interpretable attention and
the llama2 KV-cache decode.  The product is the C-ABI library ``lib/libmycaffe_attn.so`` (CUDA
sources in ``csrc/``); this package is the host-side mirror of the reference's ``CudaDnn<T>``
interface for that path."""
from .cudadnn import CudaDnn, CudaDnnError  # noqa: F401
from . import function_ids  # noqa: F401

__all__ = ["CudaDnn", "CudaDnnError", "function_ids"]
