"""Thin RAII wrappers over device memory, streams and graphs through the C ABI.

The host-side mirror of the reference's src/gpu.rs: `check` (gpu.rs:9-15), `launched`
(gpu.rs:18-26), `DevBuf` (gpu.rs:35-120), `Stream` (gpu.rs:122-136), `Graph` (gpu.rs:138-163).
Everything goes through dr_* calls; torch is not involved.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from . import ffi


def check(code: int, what: str) -> None:
    if code != 0:
        msg = ffi.lib().dr_error_string(code).decode()
        raise RuntimeError(f"{what}: CUDA error {code} ({msg})")


def launched(code: int, what: str, debug: bool = True) -> None:
    """Status of a kernel launcher: its own argument check, then (debug) the launch error."""
    if code != 0:
        raise RuntimeError(f"{what}: unsupported shape (launcher returned {code})")
    if debug:
        check(ffi.lib().dr_last_error(), what)


class Stream:
    def __init__(self) -> None:
        self.raw = C.c_void_p()
        check(ffi.lib().dr_stream_create(C.byref(self.raw)), "stream_create")

    def sync(self) -> None:
        check(ffi.lib().dr_stream_sync(self.raw), "stream_sync")

    def close(self) -> None:
        if self.raw:
            ffi.lib().dr_stream_destroy(self.raw)
            self.raw = C.c_void_p()


class DevBuf:
    """A device allocation; pointers handed to kernels stay valid for its lifetime."""

    def __init__(self, nbytes: int) -> None:
        self.nbytes = int(nbytes)
        self._p = C.c_void_p()
        check(ffi.lib().dr_malloc(C.byref(self._p), max(self.nbytes, 16)), "malloc")

    @classmethod
    def from_array(cls, a: np.ndarray, st: Stream) -> "DevBuf":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        if a.nbytes:
            check(ffi.lib().dr_h2d(b._p, a.ctypes.data_as(C.c_void_p), a.nbytes, st.raw), "h2d")
            st.sync()  # the host array may be a temporary
        return b

    @classmethod
    def zeros(cls, nbytes: int, st: Stream) -> "DevBuf":
        b = cls(nbytes)
        b.zero(st)
        return b

    @property
    def ptr(self) -> int:
        return self._p.value or 0

    def at(self, byte_offset: int) -> C.c_void_p:
        return C.c_void_p(self.ptr + int(byte_offset))

    def zero(self, st: Stream) -> None:
        check(ffi.lib().dr_memset(self._p, 0, self.nbytes, st.raw), "memset")

    def fill(self, byte: int, st: Stream) -> None:
        check(ffi.lib().dr_memset(self._p, byte, self.nbytes, st.raw), "memset")

    def upload(self, a: np.ndarray, st: Stream, byte_offset: int = 0) -> None:
        a = np.ascontiguousarray(a)
        assert byte_offset + a.nbytes <= self.nbytes
        check(ffi.lib().dr_h2d(self.at(byte_offset), a.ctypes.data_as(C.c_void_p), a.nbytes, st.raw), "h2d")
        st.sync()

    def download(self, dtype, count: int, st: Stream, byte_offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        assert byte_offset + out.nbytes <= self.nbytes
        check(ffi.lib().dr_d2h(out.ctypes.data_as(C.c_void_p), self.at(byte_offset), out.nbytes, st.raw), "d2h")
        st.sync()
        return out

    def free(self) -> None:
        if self._p:
            ffi.lib().dr_free(self._p)
            self._p = C.c_void_p()

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass


class Graph:
    """Capture `record()` (a callable that issues launches on `st`) once; replay with launch()."""

    def __init__(self, st: Stream, record) -> None:
        l = ffi.lib()
        check(l.dr_graph_begin(st.raw), "graph_begin")
        try:
            record()
        except Exception:
            tmp = C.c_void_p()
            l.dr_graph_end(st.raw, C.byref(tmp))
            raise
        self.exec = C.c_void_p()
        check(l.dr_graph_end(st.raw, C.byref(self.exec)), "graph_end")

    def launch(self, st: Stream) -> None:
        check(ffi.lib().dr_graph_launch(self.exec, st.raw), "graph_launch")

    def destroy(self) -> None:
        if self.exec:
            ffi.lib().dr_graph_destroy(self.exec)
            self.exec = C.c_void_p()


class ExtBuf:
    """Device memory owned by someone else (for example a torch tensor), seen through DevBuf's interface."""

    def __init__(self, ptr: int, nbytes: int, keep=None) -> None:
        self._ptr, self.nbytes, self._keep = int(ptr), int(nbytes), keep

    @property
    def ptr(self) -> int:
        return self._ptr

    def at(self, byte_offset: int) -> C.c_void_p:
        return C.c_void_p(self._ptr + int(byte_offset))

    def free(self) -> None:
        self._keep = None
