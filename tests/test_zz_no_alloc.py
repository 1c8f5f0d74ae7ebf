"""dr_moe_decode_static: the MoE decode layer with its scratch inside the library.

Meant for hosts that cannot allocate device memory when they call (fixed memory budget, foreign allocator,
a capture in progress elsewhere). The test calls it through the C ABI next to dr_moe_decode on the same
inputs, twice in a row with different activations, and expects identical results: both entry points run the
same two kernels and differ only in where the 4608 scratch floats live. Each pass ends with the call form the
reference's engine uses, one buffer passed as x, res and y. Collected last on purpose.
"""

import numpy as np
import pytest

from drama_rs_b200 import ffi, synth
from drama_rs_b200.gpu import DevBuf, Stream, launched
from drama_rs_b200.model import MoeLayer
from tests.helpers import NULL, device_error_word

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_dr_moe_decode():
    l = ffi.lib()
    st = Stream()
    host = synth.make_layer(5, synth.MoeShape(experts=16))
    dev = MoeLayer.upload(host, st)
    gq, gs = dev.gate_up.expert(0)
    dq, ds = dev.down.expert(0)
    sgq, sgs = dev.shared_gate_up.rows(0)
    sdq, sds = dev.shared_down.rows(0)
    idx = np.array([3, 15, 0, 7, 9, 1, 12, 4], dtype=np.int32)
    wts = np.array([0.3, 0.2, 0.15, 0.1, 0.1, 0.05, 0.05, 0.05], dtype=np.float32)
    didx, dw = DevBuf.from_array(idx, st), DevBuf.from_array(wts, st)
    dsg = DevBuf.from_array(np.array([0.25], np.float32), st)
    dact = DevBuf(9 * 512 * 4)
    for call in range(2):  # the second call runs on whatever the first left in the built-in scratch
        x = synth.make_x(40 + call, 1, 2048)[0]
        dx = DevBuf.from_array(x, st)
        y_ref, y_new = DevBuf(2048 * 4), DevBuf(2048 * 4)
        y_ref.fill(0xFF, st)
        y_new.fill(0xFF, st)
        launched(
            l.dr_moe_decode(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dx.at(0), dact.at(0),
                            y_ref.at(0), 2048, 512, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw), "moe_decode")
        launched(
            l.dr_moe_decode_static(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dx.at(0),
                                   y_new.at(0), 2048, 512, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw), "moe_decode_static")
        a = y_ref.download(np.float32, 2048, st)
        b = y_new.download(np.float32, 2048, st)
        assert np.isfinite(a).all() and np.abs(a).max() > 1.0
        assert np.array_equal(a, b), f"call {call}: max difference {np.abs(a - b).max()}"
        # the way the reference's engine calls the layer: one buffer is input, residual and output at once
        launched(
            l.dr_moe_decode_static(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dx.at(0),
                                   dx.at(0), 2048, 512, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw), "moe_decode_static in place")
        c = dx.download(np.float32, 2048, st)
        assert np.array_equal(a, c), f"call {call}, x == res == y: max difference {np.abs(a - c).max()}"
    # a shape whose scratch would not fit the built-in array is refused, not truncated
    assert l.dr_moe_decode_static(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dx.at(0),
                                  y_new.at(0), 2048, 1024, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw) == -1
    assert l.dr_moe_decode_static(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dx.at(0),
                                  y_new.at(0), 2048, 512, 16, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw) == -1
    assert device_error_word() == 0
