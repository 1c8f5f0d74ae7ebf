"""Shared helpers of the GPU parity tests."""

from __future__ import annotations

import ctypes as C

import numpy as np

# Tolerances of the layer outputs against the fp64 oracle: the bar is max-abs 1e-2 and relative
# L2 1e-3; bit-exact for routing indices.
MAX_ABS = 1e-2
REL_L2 = 1e-3

NULL = C.c_void_p(0)


def parity(y: np.ndarray, ref: np.ndarray) -> tuple[float, float]:
    y = y.astype(np.float64).reshape(-1)
    ref = ref.astype(np.float64).reshape(-1)
    return float(np.abs(y - ref).max()), float(np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30))


def assert_parity(y, ref, what="", max_abs=MAX_ABS, rel_l2=REL_L2):
    a, r = parity(y, ref)
    assert a <= max_abs and r <= rel_l2, f"{what}: max-abs {a:.3e} (<= {max_abs}), rel-L2 {r:.3e} (<= {rel_l2})"
    return a, r


def device_error_word() -> int:
    from drama_rs_b200 import ffi

    w = C.c_uint(0)
    assert ffi.lib().drb_device_error(C.byref(w)) == 0
    return int(w.value)
