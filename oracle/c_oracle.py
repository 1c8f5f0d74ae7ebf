"""ctypes access to the plain-C oracle (libmoe_oracle.so). Test and baseline infrastructure only."""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build


class OrcLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("router", "post_norm", "gu_q", "gu_sm", "d_q", "d_sm", "sgu_q", "sgu_s", "sd_q", "sd_s")] + [
        ("e", C.c_int), ("h", C.c_int), ("i", C.c_int), ("topk", C.c_int), ("eps", C.c_float)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.C_LIB if os.path.exists(_build.C_LIB) else _build.build_c()
        _lib = C.CDLL(path)
        _lib.orc_moe_decode_layer.restype = C.c_int
        _lib.orc_moe_decode_layer.argtypes = [C.POINTER(OrcLayer), C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.orc_gemv_q8.restype = C.c_int
        _lib.orc_gemv_q8.argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_int, C.c_void_p, C.c_float]
        _lib.orc_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def layer_struct(t: dict[str, np.ndarray], topk: int, eps: float) -> OrcLayer:
    """Borrowed pointers into the tensors of one layer (keep `t` alive while the struct is used)."""
    e, n2, kh = t["moe.gate_up.q4"].shape
    return OrcLayer(_p(t["moe.router"]), _p(t["post_norm"]), _p(t["moe.gate_up.q4"]), _p(t["moe.gate_up.sm"]),
                    _p(t["moe.down.q4"]), _p(t["moe.down.sm"]), _p(t["moe.shared_gate_up.q8"]),
                    _p(t["moe.shared_gate_up.s"]), _p(t["moe.shared_down.q8"]), _p(t["moe.shared_down.s"]),
                    e, kh * 2, n2 // 2, topk, eps)


def moe_decode_layer(t: dict[str, np.ndarray], x: np.ndarray, topk: int = 8, eps: float = 1e-6):
    """x + moe(rmsnorm(x)) for one row; returns (y, idx, wts)."""
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    idx = np.zeros(topk, np.int32)
    wts = np.zeros(topk, np.float32)
    L = layer_struct(t, topk, eps)
    rc = lib().orc_moe_decode_layer(C.byref(L), _p(y), _p(idx), _p(wts))
    assert rc == 0
    return y, idx, wts


def gemv_q8(q, s, x, res=None, nw=None, eps=0.0):
    n, k = q.shape
    y = np.empty(n, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    rc = lib().orc_gemv_q8(_p(q), _p(s), _p(x), _p(res) if res is not None else None, _p(y), n, k,
                           _p(nw) if nw is not None else None, eps)
    assert rc == 0
    return y
