"""Pack the reference's in-tree GPT golden vectors into two small .npz files.

Source: <reference>/MyCaffe.test/test_data/data/text/gpt/ -- text dumps ("# (shape)" header, one
value per line) and .npy files written by the reference's own generator
(test_data/projects/gpt-mini/chargpt/mingpt/model.py):

* gpt-pico-csa{,3,B,3B}/ (model.py:168-304): CausalSelfAttention layer input x, the c_attn / c_proj
  weights, q after the head transpose, softmax probabilities, P.V, the layer output y, and in
  iter_0/ the gradient of every intermediate                                  -> pico_csa.npz
* gpt-pico-ln{,3,3B}/ (model.py:309-430, LayerNormalization with epsilon 1e-10 and no affine
  part): x, y, the gradient arriving at y (grad_1a_y) and the gradient leaving at x (grad_9_x);
  gpt-pico-ln-blk/: the same with every intermediate (mean, xmu, var1, std)
* gpt-pico-blk{,3,3B}/: a whole transformer block -- 1_x, 2_x_ln11 (after the first LayerNorm),
  3_x_attn (after the attention layer), the attention weights, and in iter_0/ grad_8_x_attn,
  grad_9_ln1, grad_8_x, grad_10_x                                              -> pico_ln_blk.npz

Run where the reference tree is (it does not exist where the GPU tests run); the two outputs are
committed and are what the tests read:

    python tests/golden/make_pico_fixtures.py <reference root>
(default: $MYCAFFE_REFERENCE, else a directory named `reference` beside this repository)
"""
import ast
import os
import sys
from pathlib import Path

import numpy as np


def read_txt(path):
    with open(path) as f:
        shape = ast.literal_eval(f.readline().lstrip("#").strip())
        data = np.array([float(v) for v in f.read().split()], dtype=np.float32)
    return data.reshape(shape)


def pack(base, cases, dst):
    out = {}
    for case in cases:
        d = base / case
        tag = case.replace("gpt-pico-", "")
        for p in sorted(d.glob("*.txt")) + sorted((d / "iter_0").glob("*.txt")):
            out[f"{tag}/{p.stem}"] = read_txt(p)
        for p in sorted(d.glob("*.npy")):
            out[f"{tag}/{p.stem}"] = np.load(p).astype(np.float32)
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} with {len(out)} arrays")


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MYCAFFE_REFERENCE")
    if not root:
        root = Path(__file__).resolve().parents[3] / "reference"
    if not Path(root).is_dir():
        raise SystemExit(__doc__)
    base = Path(root) / "MyCaffe.test" / "test_data" / "data" / "text" / "gpt"
    here = Path(__file__).resolve().parent
    pack(base, ["gpt-pico-csa", "gpt-pico-csa3", "gpt-pico-csaB", "gpt-pico-csa3B"], here / "pico_csa.npz")
    pack(base, ["gpt-pico-ln", "gpt-pico-ln3", "gpt-pico-ln3B", "gpt-pico-ln-blk", "gpt-pico-blk", "gpt-pico-blk3", "gpt-pico-blk3B"],
         here / "pico_ln_blk.npz")


if __name__ == "__main__":
    main()
