"""Helper of test_launch_chain_gpu.py: forward + backward of a few shapes through the C ABI, printing one digest of
every output.  Run as a script so that the environment (MCA_NO_PDL) can differ between two runs."""
import hashlib
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    from gpu_util import Sdpa, bf16_round
    from mycaffe_b200 import CudaDnn, function_ids as ids
    import oracle
    cuda = CudaDnn(0)
    cuda.SetAsync(True)     # no synchronisation between calls: a call's first kernel follows the previous call's last
    h = hashlib.sha256()
    for (B, H, T, D, dtype) in ((8, 12, 1024, 64, "f32"), (8, 12, 1024, 64, "bf16"), (2, 4, 640, 128, "bf16"), (3, 5, 300, 32, "f32")):
        rng = np.random.default_rng(T + D)
        q, k, v, dy = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4))
        if dtype == "bf16":
            q, k, v, dy = (bf16_round(a) for a in (q, k, v, dy))
        a = Sdpa(cuda, B, T, H, D, training=True, dtype=ids.MCA_DTYPE_BF16 if dtype == "bf16" else None)
        hq, hk, hv, hdy = (a._alloc(x) for x in (q, k, v, dy))
        hy, hdq, hdk, hdv = (a._alloc(q.size) for _ in range(4))
        hm = cuda.AllocMemory(oracle.causal_mask(T))
        for rep in range(3):   # back-to-back calls: every kernel has a predecessor to overlap with
            cuda.AttnScaledDotProductForward(a.hCudnn, a.hAttn, T, hq, hk, hv, hm, hy, False)
            cuda.AttnScaledDotProductBackward(a.hCudnn, a.hAttn, hq, hdq, hk, hdk, hv, hdv, 0, hy, hdy)
        cuda.SynchronizeDevice()
        for hh in (hy, hdq, hdk, hdv):
            h.update(np.ascontiguousarray(cuda.GetMemory(hh, q.size)).tobytes())
        cuda.FreeMemory(hm)
        a.close()
    cuda.Dispose()
    print("DIGEST", h.hexdigest())


if __name__ == "__main__":
    main()
