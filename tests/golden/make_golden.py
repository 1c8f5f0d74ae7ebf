#!/usr/bin/env python3
"""Generate tests/golden/*.npz by running the reference's own PyTorch code on seeded inputs.

Run once in a container that has the reference checkout (its path is the only argument);
the fixtures it writes are committed and are what the CPU and GPU tests read. Inputs are
not stored: they are regenerated from the seed by drama_rs_b200.synth, and each fixture
carries the CRC32 of the generated tensors so a drifting generator fails loudly.

Sources of truth used here:
  * tools/reference.py  dequant_q4, dequant_q8, rms, Drama3Ref.moe (fp32, CPU)
  * transformers' Qwen3_5MoeSparseMoeBlock (the upstream class the reference vendors
    under ref/hf_modeling_qwen3_5_moe.py), fp32, fed the identically dequantised weights
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from drama_rs_b200 import synth  # noqa: E402


def load_reference(ref_root: str):
    spec = importlib.util.spec_from_file_location("drama_reference", os.path.join(ref_root, "tools", "reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return t(bits.view(np.int16)).view(torch.bfloat16)


class MemWeights:
    """In-memory stand-in for reference.Weights: only raw() differs; dense()/expert()/f() are the reference's."""

    def __init__(self, ref, tensors: dict[str, torch.Tensor]):
        self._t = tensors
        self.dense = ref.Weights.dense.__get__(self)
        self.expert = ref.Weights.expert.__get__(self)
        self.f = ref.Weights.f.__get__(self)

    def raw(self, name: str) -> torch.Tensor:
        return self._t[name]


def reference_model(ref, layer: dict[str, np.ndarray], shape: synth.MoeShape):
    tensors = {}
    for k, v in layer.items():
        tensors["layer00." + k] = bf16_tensor(v) if k == "moe.router" else t(v)
    m = object.__new__(ref.Drama3Ref)
    m.w = MemWeights(ref, tensors)
    m.tc = {
        "num_experts": shape.experts,
        "num_experts_per_tok": shape.topk,
        "moe_intermediate_size": shape.inter,
        "shared_expert_intermediate_size": shape.inter,
    }
    return m


def hf_block(ref, layer: dict[str, np.ndarray], shape: synth.MoeShape):
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeSparseMoeBlock

    cfg = Qwen3_5MoeTextConfig(
        hidden_size=shape.hidden,
        num_experts=shape.experts,
        num_experts_per_tok=shape.topk,
        moe_intermediate_size=shape.inter,
        shared_expert_intermediate_size=shape.inter,
    )
    with torch.device("meta"):
        blk = Qwen3_5MoeSparseMoeBlock(cfg)
    blk = blk.to_empty(device="cpu").float()
    router = bf16_tensor(layer["moe.router"]).float()
    sgu = ref.dequant_q8(t(layer["moe.shared_gate_up.q8"]), t(layer["moe.shared_gate_up.s"]))
    with torch.no_grad():
        blk.gate.weight.copy_(router[: shape.experts])
        blk.shared_expert_gate.weight.copy_(router[shape.experts :])
        blk.experts.gate_up_proj.copy_(ref.dequant_q4(t(layer["moe.gate_up.q4"]), t(layer["moe.gate_up.sm"])))
        blk.experts.down_proj.copy_(ref.dequant_q4(t(layer["moe.down.q4"]), t(layer["moe.down.sm"])))
        blk.shared_expert.gate_proj.weight.copy_(sgu[: shape.inter])
        blk.shared_expert.up_proj.weight.copy_(sgu[shape.inter :])
        blk.shared_expert.down_proj.weight.copy_(ref.dequant_q8(t(layer["moe.shared_down.q8"]), t(layer["moe.shared_down.s"])))
    return blk.eval()


def golden_unpack(ref, out_dir: str) -> None:
    """Known-answer inputs in the style of src/apple.rs:189-224, run through the reference's dequantisers."""
    signed = ((np.arange(256) * 3) & 0xFF).astype(np.uint8).view(np.int8).reshape(2, 128)
    s8 = np.array([[0.125], [0.25]], dtype=np.float16)
    packed = np.arange(128, dtype=np.uint8).reshape(1, 2, 64)
    sm = np.array([0.25, -2.0, 0.5, -3.0, 0.125, 1.0, 0.375, -1.0], dtype=np.float16).reshape(1, 2, 2, 2)
    rng = np.random.Generator(np.random.PCG64(7))
    rq = rng.integers(0, 256, size=(3, 5, 96), dtype=np.uint8)
    rsm = (rng.standard_normal((3, 5, 3, 2)) * 0.1).astype(np.float16)
    r8 = rng.integers(-127, 128, size=(6, 384), dtype=np.int8)
    rs = np.abs(rng.standard_normal((6, 3)) * 0.01).astype(np.float16)
    np.savez(
        os.path.join(out_dir, "unpack_kat.npz"),
        q8=signed, s8=s8, w8=ref.dequant_q8(t(signed), t(s8)).numpy(),
        q4=packed, sm=sm, w4=ref.dequant_q4(t(packed), t(sm)).numpy(),
        rq=rq, rsm=rsm, rw4=ref.dequant_q4(t(rq), t(rsm)).numpy(),
        r8=r8, rs=rs, rw8=ref.dequant_q8(t(r8), t(rs)).numpy(),
    )


def golden_moe(ref, out_dir: str, seed: int, rows: int, shape: synth.MoeShape, name: str) -> None:
    layer = synth.make_layer(seed, shape)
    x = synth.make_x(seed, rows, shape.hidden)
    xh = ref.rms(t(x), t(layer["post_norm"]), shape.eps)
    with torch.no_grad():
        m = reference_model(ref, layer, shape)
        out_ref = m.moe(0, xh)
        logits = xh @ m.w.f("layer00.moe.router").T
        probs = logits[:, : shape.experts].softmax(-1)
        topv, topi = probs.topk(shape.topk, -1)
        topv = topv / topv.sum(-1, keepdim=True)
        blk = hf_block(ref, layer, shape)
        out_hf = blk(xh[None])[0]
        # fp64 run of the same reference math, to measure the fp32 noise floor.
        blk64 = blk.double()
        out_hf64 = blk64(xh.double()[None])[0]
    print(f"{name}: |ref - hf| max {float((out_ref - out_hf).abs().max()):.3e}; "
          f"|hf32 - hf64| max {float((out_hf.double() - out_hf64).abs().max()):.3e}; "
          f"|out| max {float(out_hf.abs().max()):.3e}")
    np.savez(
        os.path.join(out_dir, name + ".npz"),
        seed=seed, rows=rows, shape=np.array([shape.hidden, shape.inter, shape.experts, shape.topk]),
        crc=synth.checksum(layer), x_crc=synth.checksum({"x": x}),
        xh=xh.numpy(), logits=logits.numpy(), idx=topi.numpy().astype(np.int32), wts=topv.numpy(),
        out_ref=out_ref.numpy(), out_hf=out_hf.numpy(), out_hf64=out_hf64.numpy(),
    )


def golden_gemv(ref, out_dir: str) -> None:
    shapes = [(4096, 2048), (2048, 4096), (8192, 2048), (151936, 2048)]
    out = {}
    for j, (n, k) in enumerate(shapes):
        q, s = synth.make_q8(100 + j, n, k)
        x = synth.make_x(100 + j, 1, k)[0]
        y = ref.dequant_q8(t(q), t(s)) @ t(x)
        y64 = ref.dequant_q8(t(q), t(s)).double() @ t(x).double()
        out[f"y_{n}_{k}"] = y.numpy()[:: max(1, n // 4096)]
        out[f"y64_{n}_{k}"] = y64.numpy()[:: max(1, n // 4096)]
        out[f"crc_{n}_{k}"] = synth.checksum({"q": q, "s": s, "x": x})
    np.savez(os.path.join(out_dir, "gemv_q8.npz"), **out)


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DRAMA_REFERENCE", "")
    if not os.path.isdir(ref_root):
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    torch.manual_seed(0)
    torch.set_num_threads(os.cpu_count() or 1)
    ref = load_reference(ref_root)
    golden_unpack(ref, HERE)
    golden_gemv(ref, HERE)
    full = synth.MoeShape()
    golden_moe(ref, HERE, 0, 1, full, "moe_decode_seed0")
    golden_moe(ref, HERE, 1, 1, full, "moe_decode_seed1")
    golden_moe(ref, HERE, 2, 40, full, "moe_rows40_seed2")
    # A small expert count exercises the same code with cheap fixtures (E <= 256 is allowed by the ABI).
    golden_moe(ref, HERE, 3, 5, synth.MoeShape(experts=16), "moe_e16_seed3")


if __name__ == "__main__":
    main()
