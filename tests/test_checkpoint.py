"""The checkpoint boundary: a layer file written by the reference's own converter reads back as the reference's own
reader sees it; a layer written under the converter's tensor names by this package reads back bit for bit."""

import os

import numpy as np

from drama_rs_b200 import model, synth
from oracle import moe_oracle as orc

CKPT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ckpt_tiny")


def test_layer_safetensors_round_trip(tmp_path):
    t = synth.make_layer(4, synth.MoeShape(experts=4))
    path = str(tmp_path / "layer00.safetensors")
    model.save_layer_safetensors(t, path)
    back = model.load_layer_safetensors(path)
    assert sorted(back) == sorted(model.LAYER_TENSORS)
    for k in model.LAYER_TENSORS:
        assert back[k].dtype == t[k].dtype and np.array_equal(back[k], t[k]), k
    assert synth.checksum(back) == synth.checksum(t)


def test_converter_written_layer_loads_as_the_reference_reads_it():
    """tests/golden/ckpt_tiny/layer00.safetensors was written by the reference's tools/make_tiny.py + tools/convert.py
    (its quantisers, its tensor names, its safetensors writer; tests/golden/make_checkpoint_golden.py).
    reference_weights.npz is what the reference's tools/reference.py `Weights` makes of that file. The loader's tensors,
    dequantised by the oracle's restatement of the layouts, must be those values exactly."""
    t = model.load_layer_safetensors(os.path.join(CKPT, "layer00.safetensors"))
    ref = np.load(os.path.join(CKPT, "reference_weights.npz"))
    e, n2i, hh = t["moe.gate_up.q4"].shape
    h, i = hh * 2, n2i // 2
    assert (e, h, i) == (4, 256, 128)
    assert t["moe.router"].dtype == np.uint16 and t["moe.router"].shape == (e + 1, h)
    assert t["moe.shared_gate_up.q8"].dtype == np.int8 and t["moe.shared_gate_up.s"].shape == (2 * i, h // 128)
    assert t["moe.gate_up.sm"].shape == (e, 2 * i, h // 64, 2) and t["moe.down.sm"].shape == (e, h, i // 64, 2)
    assert np.array_equal(orc.bf16_bits_to_f32(t["moe.router"]), ref["router"])
    assert np.array_equal(t["post_norm"], ref["post_norm"])
    assert np.array_equal(orc.dequant_q8(t["moe.shared_gate_up.q8"], t["moe.shared_gate_up.s"]), ref["shared_gate_up"])
    assert np.array_equal(orc.dequant_q8(t["moe.shared_down.q8"], t["moe.shared_down.s"]), ref["shared_down"])
    for k in range(e):
        assert np.array_equal(orc.dequant_q4(t["moe.gate_up.q4"][k], t["moe.gate_up.sm"][k]), ref[f"gate_up_{k}"]), k
        assert np.array_equal(orc.dequant_q4(t["moe.down.q4"][k], t["moe.down.sm"][k]), ref[f"down_{k}"]), k
    # and the forward pass of the oracle runs on it (top-2 of 4 experts at these widths)
    x = synth.make_x(3, 2, h)
    y, idx, _, _, _ = orc.moe_layer(t, x, 2, 1e-6, np.float64)
    assert np.isfinite(y).all() and idx.shape == (2, 2)
