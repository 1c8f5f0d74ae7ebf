"""CPU restatement of the reference's routed-expert MoE path. TEST INFRASTRUCTURE ONLY.

Nothing outside tests/, the smoke check and the bench's CPU-baseline leg may import
this module; the product path is the CUDA library and must never route through it.

Each function cites the reference code it follows (paths are within the reference
project). Parity is pinned: tests/golden/*.npz hold outputs of the reference's own
PyTorch implementation (tools/reference.py `dequant_q4`, `dequant_q8`,
`Drama3Ref.moe`) and of the upstream Qwen3.5-MoE sparse block, produced by
tests/golden/make_golden.py, and tests/test_oracle.py checks this module against
them.

All arithmetic is numpy; `dtype` selects float32 (the reference's precision) or
float64 (used to measure the float32 noise floor).
"""

from __future__ import annotations

import numpy as np

Q4_GROUP = 64
Q8_GROUP = 128


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def round_bf16(a: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(a))


# ----------------------------------------------------------------------------- storage formats


def dequant_q8(q: np.ndarray, s: np.ndarray, dtype=np.float32) -> np.ndarray:
    """int8 [N, K] with one f16 scale per 128 inputs of a row -> [N, K].

    tools/reference.py:24-26 (= tools/convert.py:113-115); kernels/drama.cu:1114-1128.
    """
    n, k = q.shape
    g = q.astype(dtype).reshape(n, k // Q8_GROUP, Q8_GROUP)
    return (g * s.astype(dtype)[..., None]).reshape(n, k)


def dequant_q4(packed: np.ndarray, sm: np.ndarray, dtype=np.float32) -> np.ndarray:
    """Packed nibbles [..., K/2] (low nibble = even k) and f16 (scale, min) [..., K/64, 2] -> [..., K].

    w = q * scale + min. tools/reference.py:29-35 (= tools/convert.py:104-110);
    kernels/drama.cu:1136-1146; the same unpack order is pinned by src/apple.rs:206-224.
    """
    lo = (packed & 0xF).astype(dtype)
    hi = (packed >> 4).astype(dtype)
    q = np.stack((lo, hi), axis=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    k = q.shape[-1]
    q = q.reshape(*q.shape[:-1], k // Q4_GROUP, Q4_GROUP)
    w = q * sm[..., 0:1].astype(dtype) + sm[..., 1:2].astype(dtype)
    return w.reshape(*w.shape[:-2], k)


# ----------------------------------------------------------------------------- elementwise


def e4m3_table() -> np.ndarray:
    """The 256 values of the FP8 E4M3 (finite-only, "fn") encoding as float32: sign, 4 exponent bits (bias 7),
    3 mantissa bits; exponent 0 is subnormal (m / 8 * 2^-6); 0x7f and 0xff are NaN.
    What `__nv_cvt_fp8x2_to_halfraw2(.., __NV_E4M3)` returns per byte in kernels/drama.cu:606-618 (`fp8x16`)."""
    b = np.arange(256, dtype=np.int64)
    e, m = (b >> 3) & 15, b & 7
    mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    v = np.where(b & 128, -mag, mag)
    v[[0x7F, 0xFF]] = np.nan
    return v.astype(np.float32)


_E4M3 = e4m3_table()


def dequant_fp8(w: np.ndarray, s: np.ndarray, dtype=np.float32) -> np.ndarray:
    """Block-FP8 weights: w u8 [..., N, K] E4M3 codes, s f32 [..., N/128, K/128] (the checkpoint's scale_inv);
    value = e4m3(w) * s[n / 128, k / 128]. kernels/drama.cu:602-604 (layout), 620-645 (`dot_fp8`); src/model.rs:99-106."""
    v = _E4M3[w].astype(dtype)
    sc = np.repeat(np.repeat(s.astype(dtype), 128, axis=-2), 128, axis=-1)
    return v * sc


def rmsnorm(x: np.ndarray, w: np.ndarray | None, eps: float, dtype=np.float32) -> np.ndarray:
    """x * rsqrt(mean(x^2) + eps) * w, the weight's "+1" already folded in.

    kernels/drama.cu:180-200 (`stage_x_norm`), 1183-1196 (`k_rmsnorm`); tools/reference.py `rms`.
    """
    x = x.astype(dtype)
    if w is None:
        return x
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True, dtype=dtype) + dtype(eps))
    return (x * inv * w.astype(dtype)).astype(dtype)


def silu(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):  # exp(-x) -> inf for very negative x gives the correct -0
        return x / (1.0 + np.exp(-x))


def sigmoid(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return 1.0 / (1.0 + np.exp(-x))


# ----------------------------------------------------------------------------- dense GEMVs


def gemv_q8(q, s, x, res=None, nw=None, eps=0.0, dtype=np.float32):
    """y = W . rmsnorm?(x) (+ res). kernels/drama.cu:222-240 (`k_gemv_q8`)."""
    xh = rmsnorm(x, nw, eps, dtype)
    y = dequant_q8(q, s, dtype) @ xh
    return y + res.astype(dtype) if res is not None else y


def gemv_q8_swiglu(q, s, x, inter, nw=None, eps=0.0, dtype=np.float32):
    """y[j] = silu(W[j] . x) * (W[I + j] . x). kernels/drama.cu:242-261 (`k_gemv_q8_swiglu`)."""
    xh = rmsnorm(x, nw, eps, dtype)
    h = dequant_q8(q, s, dtype) @ xh
    return silu(h[:inter]) * h[inter:]


def gemv_bf16(w_bits, x, nw=None, eps=0.0, dtype=np.float32):
    """y = W . rmsnorm?(x) for bf16 weights. kernels/drama.cu:263-279 (`k_gemv_bf16`)."""
    xh = rmsnorm(x, nw, eps, dtype)
    return bf16_bits_to_f32(w_bits).astype(dtype) @ xh


# ----------------------------------------------------------------------------- routing


def route(logits: np.ndarray, experts: int, topk: int, dtype=np.float32):
    """Softmax over the first `experts` logits, top-k by probability with ties to the lower
    index, weights renormalised to sum to one; column `experts` is the shared-expert gate logit.

    logits [rows, >= experts + 1]. Returns idx int32 [rows, topk] in descending-probability
    order, wts [rows, topk], sgate [rows].
    kernels/drama.cu:322-367 (`k_moe_topk`), 397-435 (tail of `k_router_topk`);
    tools/reference.py:335-339; src/mlx/engine.rs:250-258.
    """
    l = logits[:, :experts].astype(dtype)
    m = l.max(axis=-1, keepdims=True)
    ex = np.exp(l - m)
    p = ex / ex.sum(axis=-1, keepdims=True, dtype=dtype)
    # Stable sort on -p keeps the lower index first among equal probabilities.
    order = np.argsort(-p, axis=-1, kind="stable")[:, :topk]
    topv = np.take_along_axis(p, order, axis=-1)
    total = np.zeros(topv.shape[0], dtype=dtype)
    for k in range(topk):  # the kernels accumulate in rank order
        total = total + topv[:, k]
    wts = topv / total[:, None]
    return order.astype(np.int32), wts.astype(dtype), logits[:, experts].astype(dtype)


def route_margin(logits: np.ndarray, experts: int, topk: int) -> np.ndarray:
    """Gap between the topk-th and (topk+1)-th softmax probability per row (float64)."""
    l = logits[:, :experts].astype(np.float64)
    ex = np.exp(l - l.max(axis=-1, keepdims=True))
    p = np.sort(ex / ex.sum(axis=-1, keepdims=True), axis=-1)[:, ::-1]
    return p[:, topk - 1] - p[:, topk]


def router_logits(layer: dict, xh: np.ndarray, dtype=np.float32) -> np.ndarray:
    """[rows, E+1] = xh . router^T (bf16 weights widened). kernels/drama.cu:385-390; src/engine.rs:554."""
    return xh.astype(dtype) @ bf16_bits_to_f32(layer["moe.router"]).astype(dtype).T


# ----------------------------------------------------------------------------- the MoE block


def expert_forward(layer: dict, e: int, xh: np.ndarray, dtype=np.float32, act_round=None) -> np.ndarray:
    """One routed expert on rows xh [n, H]: down(silu(gate . x) * (up . x)).

    tools/reference.py:343-347; kernels/drama.cu:475-518 + 521-585 (decode),
    806-959 (prefill, which rounds the intermediate to bf16: pass act_round=round_bf16).
    """
    fp8 = "moe.gate_up.fp8" in layer  # block-FP8 experts: kernels/drama.cu:647-742 (decode), 971-1109 (prefill)
    if fp8:
        gu = dequant_fp8(layer["moe.gate_up.fp8"][e], layer["moe.gate_up.fp8_s"][e], dtype)
    else:
        gu = dequant_q4(layer["moe.gate_up.q4"][e], layer["moe.gate_up.sm"][e], dtype)
    inter = gu.shape[0] // 2
    h = xh.astype(dtype) @ gu.T
    act = silu(h[:, :inter]) * h[:, inter:]
    if act_round is not None:
        act = act_round(act.astype(np.float32)).astype(dtype)
    if fp8:
        dn = dequant_fp8(layer["moe.down.fp8"][e], layer["moe.down.fp8_s"][e], dtype)
    else:
        dn = dequant_q4(layer["moe.down.q4"][e], layer["moe.down.sm"][e], dtype)
    return act @ dn.T


def shared_forward(layer: dict, xh: np.ndarray, dtype=np.float32) -> np.ndarray:
    """The int8 shared expert, before its sigmoid gate. tools/reference.py:349-351; kernels/drama.cu:486-495, 581."""
    gu = dequant_q8(layer["moe.shared_gate_up.q8"], layer["moe.shared_gate_up.s"], dtype)
    inter = gu.shape[0] // 2
    h = xh.astype(dtype) @ gu.T
    act = silu(h[:, :inter]) * h[:, inter:]
    return act @ dequant_q8(layer["moe.shared_down.q8"], layer["moe.shared_down.s"], dtype).T


def moe_block(layer: dict, xh: np.ndarray, topk: int, dtype=np.float32, logit_bias=None, act_round=None):
    """The sparse MoE block on already-normalised rows xh [rows, H].

    Returns (out, idx, wts, sgate, logits): out = sum_k w_k expert_k(xh) + sigmoid(sgate) * shared(xh).
    tools/reference.py:331-351 (`Drama3Ref.moe`); ref/hf_modeling_qwen3_5_moe.py:814-909.
    """
    experts = layer["moe.router"].shape[0] - 1
    logits = router_logits(layer, xh, dtype)
    if logit_bias is not None:
        logits = logits.copy()
        logits[:, :experts] += logit_bias.astype(dtype)
    idx, wts, sgate = route(logits, experts, topk, dtype)
    out = np.zeros_like(xh, dtype=dtype)
    for e in np.unique(idx):
        rows, slot = np.nonzero(idx == e)
        y = expert_forward(layer, int(e), xh[rows], dtype, act_round)
        out[rows] += y * wts[rows, slot][:, None]
    out = out + sigmoid(sgate.astype(dtype))[:, None] * shared_forward(layer, xh, dtype)
    return out, idx, wts, sgate, logits


def moe_layer(layer: dict, x: np.ndarray, topk: int, eps: float, dtype=np.float32, logit_bias=None, act_round=None):
    """x + moe_block(rmsnorm(x, post_norm)): what `dr_router_topk` + `dr_moe_decode` compute with
    x == res == y (src/engine.rs:959-1042), and what the prefill sequence of
    src/engine.rs:499-500, 544-604 computes per row."""
    xh = rmsnorm(x, layer["post_norm"], eps, dtype)
    out, idx, wts, sgate, logits = moe_block(layer, xh, topk, dtype, logit_bias, act_round)
    return x.astype(dtype) + out, idx, wts, sgate, logits


# ----------------------------------------------------------------------------- prefill bookkeeping


def moe_count(idx: np.ndarray, experts: int) -> np.ndarray:
    """Rows per expert. kernels/drama.cu:745-748."""
    return np.bincount(idx.reshape(-1), minlength=experts).astype(np.int32)


def moe_offsets(counts: np.ndarray) -> np.ndarray:
    """Exclusive prefix sum done on the host by the reference. src/engine.rs:567-574."""
    return (np.cumsum(counts) - counts).astype(np.int32)


def moe_combine(x, yp, slot_of, wts, sgate, shared, dtype=np.float32):
    """x[r] += sigmoid(sgate[r]) * shared[r] + sum_k w[r,k] * Y[slot_of[r,k]], k ascending.

    kernels/drama.cu:780-791.
    """
    rows, topk = slot_of.shape
    acc = sigmoid(sgate.astype(dtype))[:, None] * shared.astype(dtype)
    for k in range(topk):
        acc = acc + wts[:, k : k + 1].astype(dtype) * yp[slot_of[:, k]].astype(dtype)
    return x.astype(dtype) + acc
