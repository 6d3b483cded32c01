"""Helpers for the GPU parity tests: drive the library the way the C# layers do, through the
CudaDnn mirror (handles + function ids), with host arrays in and out."""
import numpy as np

from mycaffe_b200 import CudaDnn, function_ids as ids


class Sdpa:
    """One attn handle configured like CausalSelfAttentionLayer.LayerSetUp does."""

    def __init__(self, cuda: CudaDnn, B, block, H, D, training=False, dropout=0.0, dtype=None, flags=None):
        self.cuda, self.B, self.block, self.H, self.D = cuda, B, block, H, D
        self.bf16 = dtype == ids.MCA_DTYPE_BF16
        self.hCudnn = cuda.CreateCuDNN()
        self.hAttn = cuda.CreateAttn()
        cuda.SetAttn(self.hCudnn, self.hAttn, 0, training, B, block, H, D, dropout, 0, dtype, flags)
        self._mem = []

    def _alloc(self, data_or_count):
        h = (self.cuda.AllocMemoryBf16 if self.bf16 else self.cuda.AllocMemory)(data_or_count)
        self._mem.append(h)
        return h

    def forward(self, q, k, v, mask=None, batch_mask=False, T=None):
        T = T or q.shape[2]
        self.hQ, self.hK, self.hV = self._alloc(q), self._alloc(k), self._alloc(v)
        self.hY = self._alloc(q.size)
        self.hMask = 0
        if mask is not None:
            self.hMask = self.cuda.AllocMemory(mask)
            self._mem.append(self.hMask)
        self.cuda.AttnScaledDotProductForward(self.hCudnn, self.hAttn, T, self.hQ, self.hK, self.hV, self.hMask, self.hY,
                                              batch_mask)
        return self.cuda.GetMemory(self.hY, q.size).reshape(q.shape)

    def backward(self, dy):
        n = dy.size
        hdY = self._alloc(dy)
        hdQ, hdK, hdV = self._alloc(n), self._alloc(n), self._alloc(n)
        # the C# layers pass 0 for the mask in Backward (CausalSelfAttentionLayer.cs:672)
        self.cuda.AttnScaledDotProductBackward(self.hCudnn, self.hAttn, self.hQ, hdQ, self.hK, hdK, self.hV, hdV, 0,
                                               self.hY, hdY)
        g = lambda h: self.cuda.GetMemory(h, n).reshape(dy.shape)
        return g(hdQ), g(hdK), g(hdV)

    def close(self):
        for h in self._mem:
            self.cuda.FreeMemory(h)
        self._mem = []
        self.cuda.FreeAttn(self.hAttn)
        self.cuda.FreeCuDNN(self.hCudnn)


def bf16_round(a):
    """Round-to-nearest-even float32 -> bfloat16 -> float32 (what the device conversion does)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))
