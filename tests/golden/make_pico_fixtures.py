"""Pack the reference's in-tree CausalSelfAttention golden vectors into one small .npz.

Source: <reference>/MyCaffe.test/test_data/data/text/gpt/gpt-pico-csa{,3,B,3B}/ -- text dumps
("# (shape)" header, one value per line) and .npy files written by the reference's own
generator (test_data/projects/gpt-mini/chargpt/mingpt/model.py:168-304): layer input x, the
c_attn / c_proj weights, q after the head transpose, softmax probabilities, P.V, the layer
output y, and in iter_0/ the gradient of every intermediate.

Run here (the reference tree does not exist on the GPU box); the output
tests/golden/pico_csa.npz is committed and is what the tests read:

    python tests/golden/make_pico_fixtures.py [/root/reference]
"""
import ast
import sys
from pathlib import Path

import numpy as np


def read_txt(path):
    with open(path) as f:
        shape = ast.literal_eval(f.readline().lstrip("#").strip())
        data = np.array([float(v) for v in f.read().split()], dtype=np.float32)
    return data.reshape(shape)


def main():
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    base = ref / "MyCaffe.test" / "test_data" / "data" / "text" / "gpt"
    out = {}
    for case in ["gpt-pico-csa", "gpt-pico-csa3", "gpt-pico-csaB", "gpt-pico-csa3B"]:
        d = base / case
        tag = case.replace("gpt-pico-", "")
        for p in sorted(d.glob("*.txt")) + sorted((d / "iter_0").glob("*.txt")):
            out[f"{tag}/{p.stem}"] = read_txt(p)
        for p in sorted(d.glob("*.npy")):
            out[f"{tag}/{p.stem}"] = np.load(p).astype(np.float32)
    dst = Path(__file__).resolve().parent / "pico_csa.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} with {len(out)} arrays")


if __name__ == "__main__":
    main()
