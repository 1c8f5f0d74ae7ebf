"""Golden vectors for the checkpoint quantisers, produced by the reference's own tools/convert.py
(`quant_q4`, `quant_q8`) on seeded weights. Run where the reference checkout is present:

    python tests/golden/make_quant_golden.py <path to the drama-rs checkout>

Writes tests/golden/quant_seed7.npz: the float32 weights and the reference's packed int4 codes, (scale, min)
pairs, int8 codes and scales.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    spec = importlib.util.spec_from_file_location("refconvert", os.path.join(ref_root, "tools", "convert.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)
    g = torch.Generator().manual_seed(7)
    # expert-like weights: N(0, 0.02) with a few outliers per row, plus a constant group and an all-zero group
    w = torch.randn(3, 24, 512, generator=g) * 0.02
    w[:, :, 5] *= 6.0
    w[0, 0, :64] = 0.0123
    w[0, 1, :64] = 0.0
    packed, sm = conv.quant_q4(w)
    w8 = torch.randn(40, 384, generator=g) * 0.05
    w8[3, :128] = 0.0
    q8 = conv.quant_q8(w8)
    np.savez_compressed(os.path.join(HERE, "quant_seed7.npz"), w=w.numpy(), q4=packed.numpy(), sm=sm.numpy(), w8=w8.numpy(),
                        q8=q8["q8"].numpy(), s8=q8["s"].numpy())
    print("wrote quant_seed7.npz", packed.shape, sm.shape)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_quant_golden.py <path to the drama-rs checkout>")
    main(sys.argv[1])
