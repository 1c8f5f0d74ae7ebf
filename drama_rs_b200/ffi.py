"""ctypes bindings of libdramakernels.so, one per launcher, mirroring the reference's src/ffi.rs.

The argument lists are the reference's (src/ffi.rs:12-117); include/dramakernels.h is the C
statement of the same. Loading fails loudly when the library has not been built: there is no
fallback path.
"""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# DRAMA_KERNELS_LIB points at another build of the same library.
LIB_PATH = os.environ.get("DRAMA_KERNELS_LIB") or os.path.join(HERE, "libdramakernels.so")

P, I32, F32, SZ, U32 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint

# name -> (restype, argtypes); the order within each tuple is the ABI.
SIGNATURES: dict[str, tuple] = {
    "dr_error_string": (C.c_char_p, [I32]),
    "dr_last_error": (I32, []),
    "dr_malloc": (I32, [C.POINTER(P), SZ]),
    "dr_free": (I32, [P]),
    "dr_host_alloc": (I32, [C.POINTER(P), SZ]),
    "dr_host_free": (I32, [P]),
    "dr_h2d": (I32, [P, P, SZ, P]),
    "dr_d2h": (I32, [P, P, SZ, P]),
    "dr_d2d": (I32, [P, P, SZ, P]),
    "dr_memset": (I32, [P, I32, SZ, P]),
    "dr_stream_create": (I32, [C.POINTER(P)]),
    "dr_stream_destroy": (I32, [P]),
    "dr_stream_sync": (I32, [P]),
    "dr_device_sync": (I32, []),
    "dr_mem_info": (I32, [C.POINTER(SZ), C.POINTER(SZ)]),
    "dr_graph_begin": (I32, [P]),
    "dr_graph_end": (I32, [P, C.POINTER(P)]),
    "dr_graph_launch": (I32, [P, P]),
    "dr_graph_destroy": (I32, [P]),
    "dr_cublas_create": (I32, [C.POINTER(P), P]),
    "dr_cublas_destroy": (I32, [P]),
    "dr_sample_init": (I32, []),
    "dr_gemm": (I32, [P, P, P, P, I32, I32, I32, F32]),
    "dr_gemv_q8": (I32, [P, P, P, P, P, I32, I32, P, F32, P, SZ, P]),
    "dr_gemv_q8_swiglu": (I32, [P, P, P, P, I32, I32, P, F32, P, SZ, P]),
    "dr_gemv_bf16": (I32, [P, P, P, I32, I32, P, F32, P, SZ, P]),
    "dr_router_topk": (I32, [P, P, P, F32, P, I32, I32, I32, P, P, P, P, P, P, P, P, SZ, SZ, SZ, SZ, P]),
    "dr_moe_topk": (I32, [P, I32, I32, I32, I32, P, P, P, P]),
    "dr_moe_decode": (I32, [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I32, I32, I32, P, F32, P, SZ, P]),
    "dr_moe_decode_fp8": (I32, [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I32, I32, I32, P, F32, P, SZ, P]),
    "dr_moe_decode_static": (I32, [P, P, P, P, P, P, P, P, P, P, P, P, P, P, I32, I32, I32, P, F32, P, SZ, P]),
    "dr_moe_count": (I32, [P, I32, P, P]),
    "dr_moe_permute": (I32, [P, I32, I32, P, P, P, P, P, I32, P]),
    "dr_moe_prefill": (I32, [P, P, P, P, P, P, P, P, P, I32, I32, I32, P]),
    "dr_moe_prefill_fp8": (I32, [P, P, P, P, P, P, P, P, P, I32, I32, I32, P]),
    "dr_moe_combine": (I32, [P, P, P, P, P, P, I32, I32, I32, P]),
    "dr_dequant_q8": (I32, [P, P, P, I32, I32, P]),
    "dr_f32_to_bf16": (I32, [P, P, SZ, P]),
    "dr_swiglu_rows": (I32, [P, P, I32, I32, P]),
    "dr_rmsnorm": (I32, [P, P, P, P, I32, I32, F32, P]),
    "drb_moe_stack_workspace_bytes": (I32, []),
    "drb_moe_stack_decode": (I32, [P, I32, P, P, I32, I32, I32, I32, F32, P, P, P]),
    "drb_moe_offsets": (I32, [P, I32, P, P]),
    "drb_moe_group": (I32, [P, I32, I32, I32, I32, P, P, P, P, P]),
    "drb_moe_prefill_block": (I32, [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I32, I32, I32, I32, I32, P, P]),
    "drb_ep_block_rows": (I32, [I32, I32]),
    "drb_ep_pack": (I32, [P, P, I32, I32, I32, I32, I32, I32, P, P, P, P, P]),
    "drb_ep_group": (I32, [P, I32, I32, I32, I32, P, P, P, P, P, P]),
    "drb_ep_put": (I32, [P, P, I32, I32, SZ, P]),
    "drb_ep_pack_peers": (I32, [P, P, I32, I32, I32, I32, I32, I32, P, I32, P, P, P, P]),
    "drb_moe_prefill_block_peers": (I32, [P] * 16 + [I32, I32, I32, I32, P, P, I32, I32, P]),
    "drb_ep_signal": (I32, [P, I32, I32, P, P]),
    "drb_ep_wait": (I32, [P, I32, P, U32, P]),
    "drb_ep_sync": (I32, [P, P, I32, I32, P, U32, P]),
    "drb_rmsnorm_f16": (I32, [P, P, P, I32, I32, F32, P]),
    "drb_router_logits_f16": (I32, [P, P, P, I32, I32, I32, F32, P]),
    "drb_router_logits": (I32, [P, P, P, I32, I32, I32, F32, P]),
    "drb_quant_q4": (I32, [P, SZ, P, P, P]),
    "drb_quant_q8": (I32, [P, SZ, P, P, P]),
    "drb_init": (I32, []),
    "drb_device_error": (I32, [C.POINTER(U32)]),
    "drb_test_wait_runs_out": (I32, [I32, U32, P, P, P]),
    "drb_grid_blocks": (I32, []),
}

_lib = None


def bind(path: str) -> C.CDLL:
    """Loads another library that exports (a subset of) the same ABI, for example the reference's own kernels built
    as a checker, and applies the signatures of the symbols it has. Used by tests and benchmarks only."""
    l = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(l, name)
        except AttributeError:
            continue
        fn.restype, fn.argtypes = res, args
    return l


def lib() -> C.CDLL:
    """The loaded library with every signature applied. Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m drama_rs_b200.build` (there is no fallback path)"
            )
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib
