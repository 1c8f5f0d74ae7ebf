"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""

import os
import re

from drama_rs_b200 import build, ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions() -> list[str]:
    text = open(os.path.join(ROOT, "include", "dramakernels.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dr_[a-z0-9_]+|drb_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    lib = ffi.lib()
    names = header_functions()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/dramakernels.h but not exported"


def test_bindings_cover_the_header():
    assert sorted(ffi.SIGNATURES) == [n for n in header_functions() if n not in ("dr_stream", "dr_graph_exec", "dr_bf16", "dr_half")]


def test_reference_symbol_names_and_arity():
    # Argument counts of the launchers on the path, as the reference's src/ffi.rs binds them.
    arity = {"dr_gemv_q8": 12, "dr_gemv_q8_swiglu": 11, "dr_gemv_bf16": 10, "dr_router_topk": 21, "dr_moe_topk": 9,
             "dr_moe_decode": 23, "dr_moe_decode_fp8": 23, "dr_moe_count": 4, "dr_moe_permute": 10, "dr_moe_prefill": 13, "dr_moe_prefill_fp8": 13, "dr_moe_combine": 10,
             "dr_dequant_q8": 6, "dr_f32_to_bf16": 4, "dr_swiglu_rows": 5, "dr_rmsnorm": 8, "dr_gemm": 8}
    for name, n in arity.items():
        assert len(ffi.SIGNATURES[name][1]) == n, name
