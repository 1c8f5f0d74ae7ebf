"""A layer written under the converter's tensor names reads back bit for bit."""

import numpy as np

from drama_rs_b200 import model, synth


def test_layer_safetensors_round_trip(tmp_path):
    t = synth.make_layer(4, synth.MoeShape(experts=4))
    path = str(tmp_path / "layer00.safetensors")
    model.save_layer_safetensors(t, path)
    back = model.load_layer_safetensors(path)
    assert sorted(back) == sorted(model.LAYER_TENSORS)
    for k in model.LAYER_TENSORS:
        assert back[k].dtype == t[k].dtype and np.array_equal(back[k], t[k]), k
    assert synth.checksum(back) == synth.checksum(t)
