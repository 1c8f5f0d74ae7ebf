"""The CPU oracle against the fixtures produced by the reference's own PyTorch code."""

import os

import numpy as np
import pytest

from drama_rs_b200 import synth
from oracle import moe_oracle as orc


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_dequant_known_answers(golden_dir):
    g = load(golden_dir, "unpack_kat.npz")
    # Hand-checkable vectors in the style of the reference's own unpack test (src/apple.rs:189-224).
    assert np.array_equal(orc.dequant_q8(g["q8"], g["s8"]), g["w8"])
    assert np.array_equal(orc.dequant_q4(g["q4"], g["sm"]), g["w4"])
    # low nibble first, w = nib * scale + bias, written out independently of both implementations
    packed, sm = g["q4"].reshape(2, 64), g["sm"].reshape(2, 2, 2).astype(np.float32)
    for r in range(2):
        for i, b in enumerate(packed[r]):
            grp = i // 32
            for j, nib in enumerate((b & 15, b >> 4)):
                assert g["w4"][0, r, 2 * i + j] == nib * sm[r, grp, 0] + sm[r, grp, 1]
    assert np.array_equal(orc.dequant_q4(g["rq"], g["rsm"]), g["rw4"])
    assert np.array_equal(orc.dequant_q8(g["r8"], g["rs"]), g["rw8"])


@pytest.mark.parametrize("n,k,seed", [(4096, 2048, 100), (2048, 4096, 101), (8192, 2048, 102), (151936, 2048, 103)])
def test_gemv_q8_golden(golden_dir, n, k, seed):
    g = load(golden_dir, "gemv_q8.npz")
    q, s = synth.make_q8(seed, n, k)
    x = synth.make_x(seed, 1, k)[0]
    assert synth.checksum({"q": q, "s": s, "x": x}) == int(g[f"crc_{n}_{k}"])
    step = max(1, n // 4096)
    y = orc.gemv_q8(q, s, x)[::step]
    y64 = orc.gemv_q8(q, s, x, dtype=np.float64)[::step]
    assert np.allclose(y64, g[f"y64_{n}_{k}"], rtol=0, atol=1e-9)
    assert np.abs(y - g[f"y_{n}_{k}"]).max() <= 2e-4 * np.abs(y64).max()


@pytest.mark.parametrize(
    "name,experts",
    [("moe_decode_seed0", 256), ("moe_decode_seed1", 256), ("moe_e16_seed3", 16), ("moe_rows40_seed2", 256)],
)
def test_moe_block_golden(golden_dir, name, experts):
    g = load(golden_dir, name + ".npz")
    shape = synth.MoeShape(experts=experts)
    layer = synth.make_layer(int(g["seed"]), shape)
    x = synth.make_x(int(g["seed"]), int(g["rows"]), shape.hidden)
    assert synth.checksum(layer) == int(g["crc"]), "the synthetic generator no longer reproduces the fixture inputs"
    assert synth.checksum({"x": x}) == int(g["x_crc"])
    xh = orc.rmsnorm(x, layer["post_norm"], shape.eps)
    assert np.abs(xh - g["xh"]).max() <= 1e-5
    out, idx, wts, sgate, logits = orc.moe_block(layer, g["xh"], shape.topk)
    # routing: bit-exact expert selection in rank order
    assert np.array_equal(idx, g["idx"])
    assert np.abs(wts - g["wts"]).max() <= 1e-6
    assert np.abs(logits - g["logits"]).max() <= 1e-4
    ref64 = g["out_hf64"]
    scale = np.abs(ref64).max()
    # the oracle in fp32 sits inside the reference's own fp32 noise (its fp32 vs fp64 deviation)
    floor = np.abs(g["out_hf"] - ref64).max()
    assert np.abs(out - ref64).max() <= max(4 * floor, 1e-6 * scale)
    out64 = orc.moe_block(layer, g["xh"], shape.topk, dtype=np.float64)[0]
    assert np.abs(out64 - ref64).max() <= 1e-7 * scale
    rel = np.linalg.norm(out - g["out_ref"]) / np.linalg.norm(g["out_ref"])
    assert rel <= 1e-5


def test_route_ties_go_to_lower_index():
    logits = np.zeros((1, 9), dtype=np.float32)
    logits[0, [5, 2, 7]] = 1.0
    idx, wts, sgate = orc.route(logits, 8, 4)
    assert idx.tolist() == [[2, 5, 7, 0]]
    assert abs(float(wts.sum()) - 1.0) < 1e-6


def test_prefill_bookkeeping():
    rng = np.random.Generator(np.random.PCG64(5))
    idx = rng.integers(0, 16, size=(10, 4)).astype(np.int32)
    counts = orc.moe_count(idx, 16)
    off = orc.moe_offsets(counts)
    assert counts.sum() == 40 and off[0] == 0 and np.all(np.diff(off) == counts[:-1])


def test_e4m3_table_and_encoder_match_torch():
    """The oracle's E4M3 decode table and the generator's encoder against torch's float8_e4m3fn (an independent
    implementation of the format the reference's fp8 kernels convert with __nv_cvt_fp8x2_to_halfraw2)."""
    import torch

    t = orc.e4m3_table()
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(t), np.isnan(ref)) and np.array_equal(t[~np.isnan(t)], ref[~np.isnan(ref)])
    a = (np.random.default_rng(0).standard_normal(50000).astype(np.float32) * 112).clip(-448, 448)
    mine = synth.to_e4m3(a)
    th = torch.from_numpy(a).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    differ = mine != th  # only exact ties may round differently
    assert np.allclose(np.abs(t[mine[differ]] - a[differ]), np.abs(t[th[differ]] - a[differ]))


def test_dequant_fp8_blocks():
    rng = np.random.default_rng(1)
    w = rng.integers(0, 127, size=(256, 384), dtype=np.uint8)
    s = rng.random((2, 3), dtype=np.float32) + 0.5
    d = orc.dequant_fp8(w, s)
    t = orc.e4m3_table()
    for (r, c) in ((0, 0), (127, 127), (128, 128), (255, 383), (130, 5)):
        assert d[r, c] == np.float32(t[w[r, c]] * s[r // 128, c // 128])


def test_fp8_layer_oracle_runs_small():
    shape = synth.MoeShape(experts=16)
    host = synth.make_layer(5, shape)
    host.update(synth.make_fp8_experts(5, shape))
    x = synth.make_x(5, 2, 2048)
    y32 = orc.moe_layer(host, x, 8, 1e-6, np.float32)[0]
    y64 = orc.moe_layer(host, x.astype(np.float64), 8, 1e-6, np.float64)[0]
    assert np.isfinite(y64).all() and np.abs(y32 - y64).max() <= 1e-4 * np.abs(y64).max()
