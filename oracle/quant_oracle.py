"""CPU restatement of the reference's checkpoint quantisers (test infrastructure: only tests may import this).

Follows tools/convert.py of the reference: `quant_q8` (33-41), `quant_q4_groups` (44-89), `quant_q4` (92-101).
All arithmetic in float32, as the reference's torch code runs it.
"""

from __future__ import annotations

import numpy as np

F = np.float32


def _half(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).astype(np.float32)


def quant_q8(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Symmetric int8, one f16 scale per 128 inputs of a row. tools/convert.py:33-41."""
    n, k = w.shape
    g = w.astype(F).reshape(n, k // 128, 128)
    amax = np.maximum(np.abs(g).max(-1, keepdims=True), F(1e-12))
    scale = np.maximum(_half(amax / F(127.0)), F(1e-12))
    q = np.clip(np.rint(g / scale), -127, 127).astype(np.int8)
    return q.reshape(n, k), scale[..., 0].astype(np.float16)


def quant_q4_groups(g: np.ndarray, steps: int = 24):
    """Asymmetric 4-bit over the last dim (64) with a clipping search and one least-squares refit.
    tools/convert.py:44-89. Returns (q uint8 [..., 64], scale f16 [...], min f16 [...])."""
    g = g.astype(F)
    gmin, gmax = g.min(-1, keepdims=True), g.max(-1, keepdims=True)
    center = (gmin + gmax) * F(0.5)
    best_err = best = None
    for i in range(steps):
        shrink = F(1.0 - 0.5 * i / steps)
        lo_c = center + (gmin - center) * shrink
        hi_c = center + (gmax - center) * shrink
        scale = np.maximum((hi_c - lo_c) / F(15.0), F(1e-10))
        scale_h = np.maximum(_half(scale), F(1e-10))
        lo_h = _half(lo_c)
        q = np.clip(np.rint((g - lo_h) / scale_h), 0, 15).astype(F)
        err = ((q * scale_h + lo_h - g) ** 2).sum(-1, keepdims=True, dtype=F)
        if best_err is None:
            best_err, best = err, (q, scale_h, lo_h)
        else:
            better = err < best_err
            best_err = np.where(better, err, best_err)
            best = tuple(np.where(better, new, old) for new, old in zip((q, scale_h, lo_h), best))
    q, scale_h, lo_h = best
    n = F(g.shape[-1])
    sq, sqq = q.sum(-1, keepdims=True, dtype=F), (q * q).sum(-1, keepdims=True, dtype=F)
    sw, sqw = g.sum(-1, keepdims=True, dtype=F), (q * g).sum(-1, keepdims=True, dtype=F)
    det = n * sqq - sq * sq
    ok = np.abs(det) > F(1e-6)
    ls_scale = np.where(ok, (n * sqw - sq * sw) / np.where(ok, det, F(1.0)), scale_h).astype(F)
    ls_min = np.where(ok, (sw - ls_scale * sq) / n, lo_h).astype(F)
    ls_scale_h, ls_min_h = _half(ls_scale), _half(ls_min)
    ls_err = ((q * ls_scale_h + ls_min_h - g) ** 2).sum(-1, keepdims=True, dtype=F)
    use = (ls_err < best_err) & ok & (ls_scale_h > 0)
    scale_h = np.where(use, ls_scale_h, scale_h)
    lo_h = np.where(use, ls_min_h, lo_h)
    return q.astype(np.uint8), scale_h[..., 0].astype(np.float16), lo_h[..., 0].astype(np.float16)


def quant_q4(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """w [E, N, K] -> packed u8 [E, N, K/2] (low nibble = even k), f16 [E, N, K/64, 2]. tools/convert.py:92-101."""
    e, n, k = w.shape
    q, scale, mn = quant_q4_groups(w.reshape(e, n, k // 64, 64))
    q = q.reshape(e, n, k)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)
    return packed, np.stack((scale, mn), axis=-1)


def dequant_q4(packed: np.ndarray, sm: np.ndarray) -> np.ndarray:
    lo, hi = (packed & 0xF).astype(F), (packed >> 4).astype(F)
    q = np.stack((lo, hi), axis=-1).reshape(*packed.shape[:-1], -1)
    k = q.shape[-1]
    qg = q.reshape(*q.shape[:-1], k // 64, 64)
    return (qg * sm[..., 0:1].astype(F) + sm[..., 1:2].astype(F)).reshape(q.shape)
