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
    seen = _inspect(path)
    names = {"uint8": "U8", "int8": "I8", "float16": "F16", "float32": "F32", "uint16": "BF16"}
    for k in LAYER_TENSORS:
        dtype, shape, nbytes, _ = seen[k]
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


def _inspect(path):
    out = subprocess.run([_binary(), "--inspect", path], capture_output=True, text=True, check=True).stdout.splitlines()
    seen = {}
    for line in out:
        name, dtype, *rest = line.split()
        seen[name] = (dtype, [int(v) for v in rest[:-2]], int(rest[-2].split("=")[1]), int(rest[-1].split("=")[1]))
    return seen


def test_cpp_loader_reads_the_converter_written_layer():
    """The layer file written by the reference's own converter (tests/golden/ckpt_tiny): the C++ loader sees the same
    dtypes, shapes and bytes (CRC-32) as the Python loader."""
    import zlib

    from drama_rs_b200.model import load_layer_safetensors

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ckpt_tiny", "layer00.safetensors")
    seen = _inspect(path)
    t = load_layer_safetensors(path)
    names = {"uint8": "U8", "int8": "I8", "float16": "F16", "float32": "F32", "uint16": "BF16"}
    for k in LAYER_TENSORS:
        dtype, shape, nbytes, crc = seen[k]
        assert dtype == names[t[k].dtype.name] and shape == list(t[k].shape) and nbytes == t[k].nbytes, k
        assert crc == zlib.crc32(np.ascontiguousarray(t[k]).tobytes()), k


def test_cpp_loader_refuses_truncated_and_inconsistent_files(tmp_path):
    """A file cut short, a tensor whose byte range does not match its shape, offsets in the wrong order and a header
    that ends inside an array are all refused on the host with an error, before anything could reach the device."""
    import json
    import struct

    t = synth.make_layer(11, synth.MoeShape(experts=2))
    good = str(tmp_path / "good.safetensors")
    save_layer_safetensors(t, good)
    raw = open(good, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])

    def write(name, hdr, body):
        js = json.dumps(hdr, separators=(",", ":")).encode() if isinstance(hdr, dict) else hdr
        p = str(tmp_path / name)
        with open(p, "wb") as f:
            f.write(struct.pack("<Q", len(js)) + js + body)
        return p

    cases = {}
    cases["truncated"] = write("truncated.safetensors", header, raw[8 + n:-4096])
    h2 = json.loads(json.dumps(header))
    h2["moe.down.q4"]["shape"][0] += 1  # right offsets, wrong shape
    cases["size"] = write("size.safetensors", h2, raw[8 + n:])
    h3 = json.loads(json.dumps(header))
    b, e = h3["post_norm"]["data_offsets"]
    h3["post_norm"]["data_offsets"] = [e, b]
    cases["order"] = write("order.safetensors", h3, raw[8 + n:])
    js = json.dumps(header, separators=(",", ":")).encode()
    cut = js[: js.index(b'"shape":[') + 12]  # the header ends inside an array
    cases["header"] = write("header.safetensors", cut, raw[8 + n:])
    for what, p in cases.items():
        r = subprocess.run([_binary(), "--inspect", p], capture_output=True, text=True, timeout=20)
        assert r.returncode == 1 and "moe_decode_main:" in r.stderr, (what, r.stderr)
    assert subprocess.run([_binary(), "--inspect", good], capture_output=True, text=True).returncode == 0


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
