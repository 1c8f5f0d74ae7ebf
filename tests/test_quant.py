"""The checkpoint quantisers: numpy oracle against the reference converter's own output (CPU), GPU kernels against
the same fixture."""

import os

import numpy as np
import pytest

from oracle import quant_oracle as qo

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_seed7.npz")


def test_oracle_matches_reference_converter():
    g = np.load(GOLDEN)
    p, sm = qo.quant_q4(g["w"])
    assert np.array_equal(p, g["q4"]) and np.array_equal(sm.view(np.uint16), g["sm"].view(np.uint16))
    q8, s8 = qo.quant_q8(g["w8"])
    assert np.array_equal(q8, g["q8"]) and np.array_equal(s8.view(np.uint16), g["s8"].view(np.uint16))
    # degenerate groups of the fixture: a constant group and an all-zero group dequantise exactly / to zero
    d = qo.dequant_q4(g["q4"], g["sm"])
    assert np.abs(d[0, 0, :64] - g["w"][0, 0, :64]).max() <= 2e-5 and np.abs(d[0, 1, :64]).max() == 0.0


@pytest.mark.gpu
def test_gpu_quantisers_match_reference_converter():
    import ctypes as C

    from drama_rs_b200 import ffi
    from drama_rs_b200.gpu import DevBuf, Stream, launched

    g = np.load(GOLDEN)
    l, st = ffi.lib(), Stream()
    w = np.ascontiguousarray(g["w"], dtype=np.float32)
    groups = w.size // 64
    dw, dq, dsm = DevBuf.from_array(w, st), DevBuf(groups * 32), DevBuf(groups * 4)
    launched(l.drb_quant_q4(dw.at(0), C.c_size_t(groups), dq.at(0), dsm.at(0), st.raw), "quant_q4")
    q = dq.download(np.uint8, groups * 32, st).reshape(g["q4"].shape)
    sm = dsm.download(np.float16, groups * 2, st).reshape(g["sm"].shape)
    # bit for bit the converter's output: codes, scales and mins of every group (the 64-term sums that pick between
    # clipping candidates run in the converter's order)
    assert np.array_equal(q, g["q4"])
    assert np.array_equal(sm.view(np.uint16), g["sm"].view(np.uint16))
    w8 = np.ascontiguousarray(g["w8"], dtype=np.float32)
    g8 = w8.size // 128
    dw8, dq8, ds8 = DevBuf.from_array(w8, st), DevBuf(w8.size), DevBuf(g8 * 2)
    launched(l.drb_quant_q8(dw8.at(0), C.c_size_t(g8), dq8.at(0), ds8.at(0), st.raw), "quant_q8")
    assert np.array_equal(dq8.download(np.int8, w8.size, st).reshape(w8.shape), g["q8"])
    assert np.array_equal(ds8.download(np.float16, g8, st).view(np.uint16).reshape(g["s8"].shape), g["s8"].view(np.uint16))
