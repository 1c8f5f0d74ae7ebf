"""What the host sees when a device-side wait gives up: an error code, a context that still works, and the code
cleared by the read. The wait is made to run out on purpose and harmlessly: one block waits on a barrier nothing
arrives at, or on a tagged word nothing writes, for at most a few thousand polls; no kernel is killed, nothing
faults, and the launch completes normally."""

import ctypes as C
import time

import numpy as np
import pytest

from drama_rs_b200 import ffi, synth
from drama_rs_b200.engine import MoeDecoder, MoeStackDecoder
from drama_rs_b200.gpu import DevBuf, Stream, check
from drama_rs_b200.model import MoeLayer
from tests.helpers import assert_parity, device_error_word
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

FULL_WAIT, GRID_WAIT = 1, 3  # DrbError in csrc/common.cuh


@pytest.mark.parametrize("which,code", [(1, FULL_WAIT), (2, FULL_WAIT), (3, GRID_WAIT)])
def test_wait_that_runs_out_is_reported_and_the_context_stays_usable(which, code):
    lib = ffi.lib()
    st = Stream()
    assert device_error_word() == 0
    word = DevBuf.zeros(512, st)
    clocks = DevBuf.zeros(4, st)
    t0 = time.perf_counter()
    check(lib.drb_test_wait_runs_out(which, 2000, word.at(0), clocks.at(0), st.raw), "launch")
    check(lib.dr_stream_sync(st.raw), "the launch completes normally")
    assert time.perf_counter() - t0 < 0.5, "a wait of 2000 polls ends within milliseconds"
    assert device_error_word() == code
    assert device_error_word() == 0, "reading the word clears it"
    if which == 3:
        # once the block has given up, its later polls return at once instead of spinning to their own limit
        assert int(clocks.download(np.uint32, 1, st)[0]) < 20000
    # the same context then runs the real kernels, and they are exact
    shape = synth.MoeShape(experts=16)
    host = synth.make_layer(7, shape)
    dev = MoeLayer.upload(host, st)
    x = synth.make_x(7, 1, shape.hidden)[0]
    ref, ridx, _, _, _ = orc.moe_layer(host, x[None], shape.topk, shape.eps, np.float64)
    dec = MoeDecoder([dev], st=st)
    dec.set_x(x)
    y = dec.step_eager()
    assert np.array_equal(dec.routing()[0], ridx[0])
    assert_parity(y, ref[0], "decode after a reported wait", max_abs=max(1e-2, 4e-6 * np.abs(ref).max()))
    stack = MoeStackDecoder([dev], st=st)
    stack.set_x(x)
    assert_parity(stack.step(), ref[0], "stack decode after a reported wait", max_abs=max(1e-2, 4e-6 * np.abs(ref).max()))
    assert device_error_word() == 0


def test_wait_hook_refuses_long_limits():
    lib = ffi.lib()
    st = Stream()
    word = DevBuf.zeros(512, st)
    assert lib.drb_test_wait_runs_out(3, 1 << 20, word.at(0), None, st.raw) == -1
    assert lib.drb_test_wait_runs_out(0, 100, word.at(0), None, st.raw) == -1
    assert lib.drb_test_wait_runs_out(3, 100, None, None, st.raw) == -1
    assert device_error_word() == 0


def test_exchange_entry_points_on_one_rank_and_a_wait_nobody_answers():
    """The peer-store exchange with this rank as its own only peer: put + signal + wait, then sync, move the blocks and
    advance the step words. Then a wait for a step nobody signals: it gives up after its poll limit, the error word
    reads DRB_ERR_GRID_WAIT once, and the exchange works again afterwards."""
    lib = ffi.lib()
    st = Stream()
    block = np.arange(4096, dtype=np.float32)
    send = DevBuf.from_array(block, st)
    recv = DevBuf.zeros(block.nbytes, st)
    flags = DevBuf.zeros(256, st)
    steps = DevBuf.zeros(16, st)  # signalled, awaited (first exchange); signalled, awaited (sync)
    peer_recv = DevBuf.from_array(np.array([recv.ptr], dtype=np.uint64), st)
    peer_flags = DevBuf.from_array(np.array([flags.ptr], dtype=np.uint64), st)
    check(lib.drb_ep_put(send.at(0), peer_recv.at(0), 1, 0, block.nbytes, st.raw), "put")
    check(lib.drb_ep_signal(peer_flags.at(0), 1, 0, steps.at(0), st.raw), "signal")
    check(lib.drb_ep_wait(flags.at(0), 1, steps.at(4), 4000, st.raw), "wait")
    assert np.array_equal(recv.download(np.float32, block.size, st), block)
    assert device_error_word() == 0
    # signal and wait in one launch: the step words move on together
    check(lib.drb_ep_sync(peer_flags.at(0), flags.at(0), 1, 0, steps.at(0), 4000, st.raw), "sync")
    check(lib.dr_stream_sync(st.raw), "sync completes")
    assert steps.download(np.uint32, 2, st).tolist() == [2, 2] and flags.download(np.uint32, 1, st)[0] == 2
    assert device_error_word() == 0
    # nobody signals step 3: the wait runs out, reports, and leaves the context usable
    t0 = time.perf_counter()
    check(lib.drb_ep_wait(flags.at(0), 1, steps.at(4), 4000, st.raw), "wait that runs out")
    check(lib.dr_stream_sync(st.raw), "the launch completes normally")
    assert time.perf_counter() - t0 < 0.5
    assert device_error_word() == GRID_WAIT and device_error_word() == 0
    check(lib.drb_ep_signal(peer_flags.at(0), 1, 0, steps.at(0), st.raw), "signal")  # step 3 arrives after all
    check(lib.drb_ep_sync(peer_flags.at(0), flags.at(0), 1, 0, steps.at(0), 4000, st.raw), "sync")  # step 4 both ways
    check(lib.dr_stream_sync(st.raw), "sync completes")
    assert device_error_word() == 0
    assert lib.drb_ep_put(send.at(0), peer_recv.at(0), 1, 0, 24, st.raw) == -1  # not a multiple of 16 bytes
    assert lib.drb_ep_sync(peer_flags.at(0), flags.at(0), 1, 1, steps.at(0), 4000, st.raw) == -1  # rank outside the world
