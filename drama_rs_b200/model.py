"""Device-resident weights of the MoE path in the reference's layouts.

Mirrors the reference's src/model.rs: `Q8` with `rows(row0)` (model.rs:16-29), `Q4` with
`expert(e)` (model.rs:31-43), `Dense` (model.rs:45-58) and the per-layer MoE members of `Layer`
(model.rs:108-121). Tensors come in under the converter's names (see drama_rs_b200.synth).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from .gpu import DevBuf, Stream


@dataclass
class Q8:
    """int8 weight, one f16 scale per 128 inputs of a row."""

    q: DevBuf
    s: DevBuf
    n: int
    k: int

    def rows(self, row0: int) -> tuple[C.c_void_p, C.c_void_p]:
        return self.q.at(row0 * self.k), self.s.at(row0 * (self.k // 128) * 2)

    @property
    def nbytes(self) -> int:
        return self.n * self.k + self.n * (self.k // 128) * 2


@dataclass
class Q4:
    """Routed experts, int4 asymmetric with group 64: q [E, N, K/2], sm [E, N, K/64, 2]."""

    q: DevBuf
    sm: DevBuf
    e: int
    n: int
    k: int

    def expert(self, e: int) -> tuple[C.c_void_p, C.c_void_p]:
        return self.q.at(e * self.n * self.k // 2), self.sm.at(e * self.n * (self.k // 64) * 4)

    @property
    def q_bytes_per_expert(self) -> int:
        return self.n * self.k // 2

    @property
    def sm_bytes_per_expert(self) -> int:
        return self.n * (self.k // 64) * 4


@dataclass
class Fp8Experts:
    """Routed experts in the checkpoint's block-FP8 form (src/model.rs:99-106): E4M3 bytes w [E, N, K] with one
    f32 scale per 128 x 128 block, s [E, N/128, K/128]; gate rows then up rows in gate_up."""

    gu_w: DevBuf
    gu_s: DevBuf
    d_w: DevBuf
    d_s: DevBuf
    e: int
    hidden: int
    inter: int

    @classmethod
    def upload(cls, t: dict[str, np.ndarray], st: Stream) -> "Fp8Experts":
        e, n2, h = t["moe.gate_up.fp8"].shape
        up = lambda name: DevBuf.from_array(t[name], st)
        return cls(up("moe.gate_up.fp8"), up("moe.gate_up.fp8_s"), up("moe.down.fp8"), up("moe.down.fp8_s"), e, h, n2 // 2)

    @property
    def bytes_per_expert(self) -> int:
        h, i = self.hidden, self.inter
        return 3 * h * i + 4 * ((2 * i // 128) * (h // 128) + (h // 128) * (i // 128))


@dataclass
class MoeLayer:
    router: DevBuf  # bf16 [E + 1, H]
    post_norm: DevBuf  # f32 [H]
    shared_gate_up: Q8
    shared_down: Q8
    gate_up: Q4
    down: Q4
    experts: int
    hidden: int
    inter: int

    @classmethod
    def upload(cls, t: dict[str, np.ndarray], st: Stream) -> "MoeLayer":
        up = lambda name: DevBuf.from_array(t[name], st)
        e, n2, kh = t["moe.gate_up.q4"].shape
        hidden, inter = kh * 2, n2 // 2
        return cls(
            router=up("moe.router"),
            post_norm=up("post_norm"),
            shared_gate_up=Q8(up("moe.shared_gate_up.q8"), up("moe.shared_gate_up.s"), 2 * inter, hidden),
            shared_down=Q8(up("moe.shared_down.q8"), up("moe.shared_down.s"), hidden, inter),
            gate_up=Q4(up("moe.gate_up.q4"), up("moe.gate_up.sm"), e, 2 * inter, hidden),
            down=Q4(up("moe.down.q4"), up("moe.down.sm"), e, hidden, inter),
            experts=e,
            hidden=hidden,
            inter=inter,
        )

    def free(self) -> None:
        for b in (self.router, self.post_norm, self.shared_gate_up.q, self.shared_gate_up.s, self.shared_down.q,
                  self.shared_down.s, self.gate_up.q, self.gate_up.sm, self.down.q, self.down.sm):
            b.free()


LAYER_TENSORS = ("moe.router", "post_norm", "moe.shared_gate_up.q8", "moe.shared_gate_up.s", "moe.shared_down.q8",
                 "moe.shared_down.s", "moe.gate_up.q4", "moe.gate_up.sm", "moe.down.q4", "moe.down.sm")


def save_layer_safetensors(t: dict[str, np.ndarray], path: str) -> None:
    """Writes the MoE tensors of one layer under the converter's names (tools/convert.py:299-346 writes one
    `layerNN.safetensors` per layer with exactly these keys next to the mixer's)."""
    import torch
    from safetensors.torch import save_file

    out = {}
    for k in LAYER_TENSORS:
        a = np.ascontiguousarray(t[k])
        out[k] = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16) if k == "moe.router" else torch.from_numpy(a)
    save_file(out, path)


def load_layer_safetensors(path: str) -> dict[str, np.ndarray]:
    """Reads the MoE tensors of a drama-rs-v1 `layerNN.safetensors` (src/model.rs:217-227 reads the same keys);
    other tensors in the file (mixer, norms) are ignored. bf16 comes back as uint16 bit patterns."""
    import torch
    from safetensors import safe_open

    out = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        for k in LAYER_TENSORS:
            v = f.get_tensor(k)
            out[k] = v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()
    return out
