#!/usr/bin/env python3
"""Writes tests/golden/ckpt_tiny/: one layer file produced by the REFERENCE's own tools, for the loader tests.

    python tests/golden/make_checkpoint_golden.py /path/to/reference-checkout

The reference's tools/make_tiny.py writes a small random checkpoint in the original layout (block-FP8 experts) from a
model config; tools/convert.py (its main(), --device cpu --only layer:0) converts it into a drama-rs-v1 layer file with
its own quantisers and its own safetensors writer. The real model's config.json is not part of the reference
checkout, so a config with the keys those two tools read, at small widths, is written here. Beside the layer file
(committed as the converter wrote it) this script stores what the reference's tools/reference.py `Weights` class
makes of that file: the dequantised MoE tensors, which the loader tests compare with.
"""

from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "ckpt_tiny")

CONFIG = {
    "eos_token_id": 1, "semantic_start_token_id": 8, "semantic_end_token_id": 15,
    "text_config": {
        "hidden_size": 256, "vocab_size": 64, "num_hidden_layers": 1, "layer_types": ["linear_attention"],
        "mlp_layer_types": ["sparse"], "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
        "shared_expert_intermediate_size": 128, "linear_num_key_heads": 2, "linear_num_value_heads": 2,
        "linear_key_head_dim": 64, "linear_value_head_dim": 64, "num_attention_heads": 2, "num_key_value_heads": 1,
        "head_dim": 64, "rms_norm_eps": 1e-6,
    },
    "audio_decoder_config": {
        "dim": 128, "vocab_size": 16, "num_codebooks": 2, "n_head": 2, "n_local_heads": 1, "head_dim": 64,
        "shared_enrichment_layers": 1, "intermediate_size": 128,
    },
}


def main() -> None:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DRAMA_REFERENCE")
    if not ref or not os.path.isdir(ref):
        raise SystemExit("usage: make_checkpoint_golden.py <reference checkout>")
    tools = os.path.join(ref, "tools")
    with tempfile.TemporaryDirectory() as tmp:
        cfg = os.path.join(tmp, "config.json")
        with open(cfg, "w") as f:
            json.dump(CONFIG, f)
        src, dst = os.path.join(tmp, "src"), os.path.join(tmp, "dst")
        subprocess.run([sys.executable, os.path.join(tools, "make_tiny.py"), cfg, src, "--layers", "1", "--experts", "4", "--seed", "5"], check=True)
        subprocess.run([sys.executable, os.path.join(tools, "convert.py"), src, dst, "--device", "cpu", "--only", "layer:0"], check=True)
        os.makedirs(OUT, exist_ok=True)
        shutil.copy(os.path.join(dst, "layer00.safetensors"), os.path.join(OUT, "layer00.safetensors"))
        sys.path.insert(0, tools)
        import reference  # noqa: E402  (the reference's own reader)

        w = reference.Weights(dst, device="cpu")
        out = {
            "router": w.f("layer00.moe.router").numpy(),
            "post_norm": w.f("layer00.post_norm").numpy(),
            "shared_gate_up": w.dense("layer00.moe.shared_gate_up").numpy(),
            "shared_down": w.dense("layer00.moe.shared_down").numpy(),
        }
        for e in range(CONFIG["text_config"]["num_experts"]):
            out[f"gate_up_{e}"] = w.expert("layer00", "gate_up", e).numpy()
            out[f"down_{e}"] = w.expert("layer00", "down", e).numpy()
        np.savez_compressed(os.path.join(OUT, "reference_weights.npz"), **out)
    print("wrote", OUT, {k: os.path.getsize(os.path.join(OUT, k)) for k in os.listdir(OUT)})


if __name__ == "__main__":
    main()
