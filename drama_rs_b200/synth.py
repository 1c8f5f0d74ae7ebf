"""Seeded synthetic weights and inputs in the drama-rs-v1 tensor layout.

The tensor names and bit layouts are the ones the reference's converter writes
(tools/convert.py:33-41 `quant_q8`, tools/convert.py:92-101 `quant_q4`,
tools/convert.py:225-227 router + shared gate row) and its loader reads
(src/model.rs:16-43 `Q8`, `Q4`):

  moe.gate_up.q4   u8  [E, 2I, H/2]      low nibble = even k, nibble in 0..15
  moe.gate_up.sm   f16 [E, 2I, H/64, 2]  (scale, min); w = q*scale + min
  moe.down.q4      u8  [E, H, I/2]
  moe.down.sm      f16 [E, H, I/64, 2]
  moe.shared_gate_up.q8 i8 [2I, H], .s f16 [2I, H/128]
  moe.shared_down.q8    i8 [H, I],  .s f16 [H, I/128]
  moe.router       bf16 [E+1, H]         row E is the shared-expert gate
  post_norm        f32 [H]               RMSNorm weight with its "+1" folded in

The value distributions are those of the benchmark configurations: symmetric
int4 uniform in [-8, 7] with one f16 scale ~ |N(0, 0.01)| per 64-group, stored
as q_u = q_s + 8 and min = -8*scale (exact in f16); int8 uniform in [-127, 127]
with one f16 scale ~ |N(0, 0.005)| per output row, replicated over the K/128
groups; router ~ N(0, 0.02) in bf16; activations ~ N(0, 1) rounded to bf16.

bf16 tensors are carried as uint16 bit patterns in numpy.
"""

from __future__ import annotations

import zlib
from dataclasses import dataclass

import numpy as np

Q4_GROUP = 64
Q8_GROUP = 128


# ----------------------------------------------------------------------------- bf16 helpers


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ----------------------------------------------------------------------------- shapes


@dataclass(frozen=True)
class MoeShape:
    hidden: int = 2048
    inter: int = 512
    experts: int = 256
    topk: int = 8
    eps: float = 1e-6

    @property
    def expert_bytes(self) -> int:
        """Bytes of one routed expert (gate_up + down, q and sm) in the reference layout."""
        gu = 2 * self.inter * (self.hidden // 2) + 2 * self.inter * (self.hidden // Q4_GROUP) * 4
        dn = self.hidden * (self.inter // 2) + self.hidden * (self.inter // Q4_GROUP) * 4
        return gu + dn

    @property
    def shared_bytes(self) -> int:
        gu = 2 * self.inter * self.hidden + 2 * self.inter * (self.hidden // Q8_GROUP) * 2
        dn = self.hidden * self.inter + self.hidden * (self.inter // Q8_GROUP) * 2
        return gu + dn

    @property
    def router_bytes(self) -> int:
        return (self.experts + 1) * self.hidden * 2

    @property
    def decode_layer_bytes(self) -> int:
        """Weight bytes one batch-1 decode layer must read: router, top-k experts, shared expert."""
        return self.router_bytes + self.topk * self.expert_bytes + self.shared_bytes


# ----------------------------------------------------------------------------- generators


def _q4(rng: np.random.Generator, e: int, n: int, k: int) -> tuple[np.ndarray, np.ndarray]:
    q = rng.integers(0, 256, size=(e, n, k // 2), dtype=np.uint8)
    scale = np.abs(rng.standard_normal((e, n, k // Q4_GROUP), dtype=np.float32) * np.float32(0.01)).astype(np.float16)
    # Keep scales away from zero so that no group degenerates to a constant.
    scale = np.maximum(scale, np.float16(1e-4))
    sm = np.empty((e, n, k // Q4_GROUP, 2), dtype=np.float16)
    sm[..., 0] = scale
    sm[..., 1] = (scale.astype(np.float32) * np.float32(-8.0)).astype(np.float16)
    return q, sm


def _q8(rng: np.random.Generator, n: int, k: int, std: float) -> tuple[np.ndarray, np.ndarray]:
    q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    row = np.abs(rng.standard_normal((n, 1), dtype=np.float32) * np.float32(std)).astype(np.float16)
    row = np.maximum(row, np.float16(1e-4))
    s = np.ascontiguousarray(np.broadcast_to(row, (n, k // Q8_GROUP)))
    return q, s


def make_layer(seed: int, shape: MoeShape = MoeShape(), norm_jitter: float = 0.1) -> dict[str, np.ndarray]:
    """One MoE layer's tensors. Draw order is fixed; the same seed gives the same bytes."""
    rng = np.random.Generator(np.random.PCG64(seed))
    h, i, e = shape.hidden, shape.inter, shape.experts
    out: dict[str, np.ndarray] = {}
    out["moe.router"] = f32_to_bf16_bits(rng.standard_normal((e + 1, h), dtype=np.float32) * np.float32(0.02))
    pn = np.float32(1.0) + rng.standard_normal(h, dtype=np.float32) * np.float32(norm_jitter)
    out["post_norm"] = pn.astype(np.float32)
    out["moe.shared_gate_up.q8"], out["moe.shared_gate_up.s"] = _q8(rng, 2 * i, h, 0.005)
    out["moe.shared_down.q8"], out["moe.shared_down.s"] = _q8(rng, h, i, 0.005)
    out["moe.gate_up.q4"], out["moe.gate_up.sm"] = _q4(rng, e, 2 * i, h)
    out["moe.down.q4"], out["moe.down.sm"] = _q4(rng, e, h, i)
    return out


def e4m3_values() -> np.ndarray:
    """The 256 values of FP8 E4M3 (finite-only) as float32; 0x7f and 0xff (NaN) are given as +-inf so that a
    nearest-value search never picks them."""
    b = np.arange(256, dtype=np.int64)
    e, m = (b >> 3) & 15, b & 7
    mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    v = np.where(b & 128, -mag, mag).astype(np.float32)
    v[0x7F], v[0xFF] = np.inf, -np.inf
    return v


def to_e4m3(a: np.ndarray) -> np.ndarray:
    """Nearest E4M3 code of every element (|a| <= 448), as uint8."""
    pos = e4m3_values()[:0x7F]  # 0 .. 448 ascending
    mid = (pos[1:] + pos[:-1]) * np.float32(0.5)
    code = np.searchsorted(mid, np.abs(a).astype(np.float32), side="left").astype(np.uint8)
    return np.where(a < 0, code | np.uint8(0x80), code).astype(np.uint8)


def make_fp8_experts(seed: int, shape: MoeShape = MoeShape()) -> dict[str, np.ndarray]:
    """Routed experts in the checkpoint's block-FP8 form (src/model.rs:99-106): E4M3 codes with one f32
    `scale_inv` per 128 x 128 block; gate rows then up rows. Values are N(0, 1) * 112 rounded to E4M3 (a block's
    largest magnitude lands near the format's 448, as a block-scaled quantiser leaves it), scales ~ |N(0, 0.01)| / 112,
    so that the effective weights have the spread of the int4 configuration."""
    rng = np.random.Generator(np.random.PCG64(seed ^ 0xF8))
    h, i, e = shape.hidden, shape.inter, shape.experts
    out: dict[str, np.ndarray] = {}
    for name, n, k in (("moe.gate_up", 2 * i, h), ("moe.down", h, i)):
        w = np.empty((e, n, k), dtype=np.uint8)
        for ex in range(e):  # expert by expert: the float32 draws of all experts at once would need gigabytes
            w[ex] = to_e4m3(np.clip(rng.standard_normal((n, k), dtype=np.float32) * np.float32(112.0), -448.0, 448.0))
        out[name + ".fp8"] = w
        sc = np.abs(rng.standard_normal((e, n // 128, k // 128), dtype=np.float32)) * np.float32(0.01 / 112.0)
        out[name + ".fp8_s"] = np.maximum(sc, np.float32(1e-7)).astype(np.float32)
    return out


def make_x(seed: int, rows: int, hidden: int = 2048) -> np.ndarray:
    """Activations ~ N(0,1), rounded to bf16 and widened back to f32 (what crosses the decode ABI)."""
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x5EED))
    return bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((rows, hidden), dtype=np.float32)))


def make_q8(seed: int, n: int, k: int, std: float = 0.005) -> tuple[np.ndarray, np.ndarray]:
    """A dense int8 linear for the GEMV sweep."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return _q8(rng, n, k, std)


def zipf_router_bias(seed: int, experts: int, s: float = 1.1, strength: float = 0.4) -> np.ndarray:
    """Additive router-logit bias that makes expert popularity follow Zipf(s) over a random ranking.

    Returned as an f32 [experts] vector b_e = -s * ln(rank_e) * strength. strength 0.4 is calibrated against the
    synthetic router (logit spread ~0.9): 300 rows x top-8 then touch ~234 of 256 experts, median group 4.
    """
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x21BF))
    rank = rng.permutation(experts).astype(np.float64) + 1.0
    return (-s * np.log(rank) * strength).astype(np.float32)


def checksum(layer: dict[str, np.ndarray]) -> int:
    """CRC32 over every tensor's bytes in name order; pins the generator's byte stream."""
    c = 0
    for name in sorted(layer):
        c = zlib.crc32(np.ascontiguousarray(layer[name]).view(np.uint8).reshape(-1), c)
    return c
