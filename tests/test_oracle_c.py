"""The plain-C oracle against the numpy oracle (which is pinned to the reference's outputs)."""

import os

import numpy as np

from drama_rs_b200 import synth
from oracle import c_oracle
from oracle import moe_oracle as orc


def test_c_decode_layer_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe_decode_seed0.npz"))
    layer = synth.make_layer(0)
    x = synth.make_x(0, 1, 2048)[0]
    y, idx, wts = c_oracle.moe_decode_layer(layer, x)
    assert np.array_equal(idx, g["idx"][0])
    assert np.abs(wts - g["wts"][0]).max() <= 2e-6
    ref = x.astype(np.float64) + g["out_hf64"][0]
    # Sequential fp32 sums over 2048 terms: a few 1e-6 of the output magnitude (~4e3 here), which is
    # already above the 1e-2 absolute bar the GPU kernels are held to.
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) <= 1e-5


def test_c_decode_small_expert_count():
    layer = synth.make_layer(3, synth.MoeShape(experts=16))
    x = synth.make_x(4, 1, 2048)[0]
    y, idx, wts = c_oracle.moe_decode_layer(layer, x)
    ref, ridx, rwts, _, _ = orc.moe_layer(layer, x[None], 8, 1e-6, np.float64)
    assert np.array_equal(idx, ridx[0])
    assert np.linalg.norm(y - ref[0]) / np.linalg.norm(ref[0]) <= 1e-5


def test_c_gemv_q8():
    q, s = synth.make_q8(9, 300, 4096)
    x = synth.make_x(9, 1, 4096)[0]
    res = synth.make_x(10, 1, 300)[0]
    y = c_oracle.gemv_q8(q, s, x, res=res)
    ref = orc.gemv_q8(q, s, x, res=res, dtype=np.float64)
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
