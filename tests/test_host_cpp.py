"""The C++ host (drama_rs_b200/host): safetensors loader on CPU, decode through its MoeDecoder on the GPU.

The host mirrors the reference's Rust host (src/gpu.rs, src/model.rs, src/engine.rs record_step / step); the
GPU test reads like the reference's own decode check: load a checkpoint's layers, run a step eagerly and from a
captured graph, compare with the model's reference implementation.
"""

import os
import subprocess

import numpy as np
import pytest

from drama_rs_b200 import build, synth
from drama_rs_b200.model import LAYER_TENSORS, save_layer_safetensors
from helpers import assert_parity

SHAPE = synth.MoeShape(experts=16)


def _binary() -> str:
    return build.build_host()


def test_inspect_reads_safetensors_header(tmp_path):
    t = synth.make_layer(11, SHAPE)
    path = str(tmp_path / "layer00.safetensors")
    save_layer_safetensors(t, path)
    out = subprocess.run([_binary(), "--inspect", path], capture_output=True, text=True, check=True).stdout.splitlines()
    seen = {}
    for line in out:
        name, dtype, *rest = line.split()
        seen[name] = (dtype, [int(v) for v in rest[:-1]], int(rest[-1].split("=")[1]))
    names = {"uint8": "U8", "int8": "I8", "float16": "F16", "float32": "F32", "uint16": "BF16"}
    for k in LAYER_TENSORS:
        dtype, shape, nbytes = seen[k]
        assert dtype == names[t[k].dtype.name], k
        assert shape == list(t[k].shape), k
        assert nbytes == t[k].nbytes, k


def test_inspect_rejects_missing_tensor(tmp_path):
    import torch
    from safetensors.torch import save_file

    path = str(tmp_path / "bad.safetensors")
    save_file({"moe.router": torch.zeros(4, 4)}, path)
    r = subprocess.run([_binary(), "--inspect", path], capture_output=True, text=True)
    assert r.returncode == 1 and "missing tensor" in r.stderr


@pytest.mark.gpu
def test_cpp_decoder_matches_oracle(tmp_path):
    from oracle import moe_oracle as orc

    layers = [synth.make_layer(20 + k, SHAPE) for k in range(3)]
    files = []
    for k, t in enumerate(layers):
        files.append(str(tmp_path / f"layer{k:02d}.safetensors"))
        save_layer_safetensors(t, files[-1])
    x = synth.make_x(5, 1)[0]
    xp, ea, gr = (str(tmp_path / n) for n in ("x.f32", "eager.f32", "graph.f32"))
    x.tofile(xp)
    r = subprocess.run([_binary(), "--x", xp, "--out-eager", ea, "--out-graph", gr, "--steps", "1", *files], capture_output=True,
                       text=True)
    assert r.returncode == 0, r.stderr + r.stdout
    want = x.astype(np.float64)
    for t in layers:
        want = orc.moe_layer(t, want[None, :], SHAPE.topk, SHAPE.eps, np.float64)[0][0]
    eager, graph = np.fromfile(ea, np.float32), np.fromfile(gr, np.float32)
    # the hidden state grows layer over layer (no final norm): the absolute bar scales with it, as for the stack tests
    assert_parity(eager, want, "C++ host, eager", max_abs=max(1e-2, 4e-6 * np.abs(want).max()))
    assert np.array_equal(eager.view(np.uint32), graph.view(np.uint32)), "graph replay differs from the eager step"
    assert '"device_error": 0' in r.stdout
