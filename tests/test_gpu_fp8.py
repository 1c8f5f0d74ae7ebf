"""Block-FP8 routed experts: dr_moe_decode_fp8 against the fp64 oracle and against the reference's own kernel.

The reference has no Python path for these experts (tools/reference.py covers int4 only), so parity is pinned two
ways: the oracle's E4M3 table equals torch's float8_e4m3fn (tests/test_oracle.py), and on the GPU the output is
compared with the reference's kernels/drama.cu `dr_moe_decode_fp8`, compiled unchanged into oracle/_ref (same
buffers, same routing)."""

import ctypes as C
import os

import numpy as np
import pytest

from drama_rs_b200 import ffi, synth
from drama_rs_b200.gpu import DevBuf, Stream, launched
from drama_rs_b200.model import Fp8Experts, MoeLayer
from oracle import moe_oracle as orc
from tests.helpers import NULL, assert_parity, device_error_word

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libdrama_ref.so")


@pytest.fixture(scope="module")
def st():
    return Stream()


def run_layer(lib, st, dev, f8, x, fp8_symbol):
    """dr_router_topk (this library) + <fp8_symbol> from `lib` on x; returns (y, idx)."""
    l = ffi.lib()
    dx, dy = DevBuf.from_array(x, st), DevBuf(2048 * 4)
    dlog, didx, dw, dsg = DevBuf((dev.experts + 1) * 4), DevBuf(32), DevBuf(32), DevBuf(4)
    dact, dcnt = DevBuf(9 * 512 * 4), DevBuf.zeros(16, st)
    launched(l.dr_router_topk(dev.router.at(0), dx.at(0), dev.post_norm.at(0), 1e-6, dlog.at(0), dev.experts, 8, 2048, didx.at(0),
                              dw.at(0), dsg.at(0), dcnt.at(0), NULL, NULL, NULL, NULL, 0, 0, 0, 0, st.raw), "router_topk")
    sgq, sgs = dev.shared_gate_up.rows(0)
    sdq, sds = dev.shared_down.rows(0)
    fn = getattr(lib, fp8_symbol)
    fn.restype = C.c_int
    rc = fn(f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0),
            dx.at(0), dact.at(0), dy.at(0), C.c_int(2048), C.c_int(512), C.c_int(8), dev.post_norm.at(0), C.c_float(1e-6), NULL,
            C.c_size_t(0), st.raw)
    assert rc == 0
    st.sync()
    return dy.download(np.float32, 2048, st), didx.download(np.int32, 8, st)


@pytest.mark.parametrize("experts,seed", [(16, 5), (256, 6)])
def test_moe_decode_fp8(st, experts, seed):
    shape = synth.MoeShape(experts=experts)
    host = synth.make_layer(seed, shape)
    host.update(synth.make_fp8_experts(seed, shape))
    dev = MoeLayer.upload(host, st)
    f8 = Fp8Experts.upload(host, st)
    x = synth.make_x(seed, 1, 2048)[0]
    y, idx = run_layer(ffi.lib(), st, dev, f8, x, "dr_moe_decode_fp8")
    assert device_error_word() == 0
    ref, ridx, _, _, _ = orc.moe_layer(host, x.astype(np.float64)[None], 8, 1e-6, np.float64)
    assert np.array_equal(idx, ridx[0])
    a, r = assert_parity(y, ref[0], f"fp8 decode, {experts} experts")
    # the reference's own kernel on the same buffers
    if os.path.exists(REF_LIB):
        y_ref, _ = run_layer(C.CDLL(REF_LIB), st, dev, f8, x, "dr_moe_decode_fp8")
        # two fp32 implementations with different summation orders: the absolute bar scales with the output
        # (|y| reaches 1e4 here), as for the multi-layer tests
        bar = max(1e-2, 4e-6 * float(np.abs(ref).max()))
        assert_parity(y, y_ref.astype(np.float64), "fp8 decode against the reference kernel", max_abs=bar)
        assert_parity(y_ref, ref[0], "reference kernel against the oracle", max_abs=bar)


def test_moe_decode_fp8_rejects_other_shapes(st):
    l = ffi.lib()
    assert l.dr_moe_decode_fp8(NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, 2048, 256, 8,
                               NULL, 1e-6, NULL, 0, st.raw) == -1


@pytest.mark.parametrize("route", ["e4m3", "fp16"])
def test_moe_prefill_fp8_grouped_kernel(st, route, monkeypatch):
    """Both routes of dr_moe_prefill_fp8 (E4M3 weights straight into the tensor cores; dequantised to fp16 first, the route
    for more than 256 experts) on hand-made groups (one expert with more tokens than one accumulator holds, empty experts,
    groups of 1, 16 and 17 tokens; scales spread over four orders of magnitude): every output row against the fp64
    expert on the same bf16 row, and against the reference's own kernel."""
    l = ffi.lib()
    monkeypatch.setenv("DRB_FP8_DEQUANT", "1" if route == "fp16" else "0")
    shape = synth.MoeShape(experts=16)
    host = synth.make_layer(9, shape)
    f8h = synth.make_fp8_experts(9, shape)
    rng = np.random.Generator(np.random.PCG64(78))
    for k in ("moe.gate_up.fp8_s", "moe.down.fp8_s"):  # block scales from 1e-6 to 1e-2
        f8h[k] = (f8h[k] * np.exp(rng.uniform(np.log(0.01), np.log(100.0), size=f8h[k].shape))).astype(np.float32)
    host.update(f8h)
    f8 = Fp8Experts.upload(host, st)
    counts = np.array([300, 0, 1, 17, 16, 5, 0, 33, 2, 0, 7, 64, 3, 1, 0, 9], dtype=np.int32)
    offsets = (np.cumsum(counts) - counts).astype(np.int32)
    n = int(counts.sum())
    xf = rng.standard_normal((n, 2048), dtype=np.float32)
    zero_row = int(offsets[7]) + 20  # an all-zero token row: its largest magnitude is no normaliser
    xf[zero_row] = 0.0
    xb = synth.f32_to_bf16_bits(xf)
    dxp, dcnt, doff = DevBuf.from_array(xb, st), DevBuf.from_array(counts, st), DevBuf.from_array(offsets, st)

    def run(lib):
        dact, dy = DevBuf(n * 512 * 2), DevBuf(n * 2048 * 4)
        dy.fill(0xFF, st)
        fn = lib.dr_moe_prefill_fp8
        fn.restype = C.c_int
        assert fn(f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), dxp.at(0), doff.at(0), dcnt.at(0), dact.at(0), dy.at(0),
                  C.c_int(16), C.c_int(2048), C.c_int(512), st.raw) == 0
        st.sync()
        return dy.download(np.float32, n * 2048, st).reshape(n, 2048)

    y = run(l)
    assert device_error_word() == 0
    assert np.isfinite(y).all()  # max() below would let a NaN row pass
    assert not y[zero_row].any()
    x = synth.bf16_bits_to_f32(xb).astype(np.float64)
    y_ref = run(C.CDLL(REF_LIB)) if os.path.exists(REF_LIB) else None
    worst = worst_ref = 0.0
    for e in range(16):
        if counts[e] == 0:
            continue
        rows = slice(offsets[e], offsets[e] + counts[e])
        ref = orc.expert_forward(host, e, x[rows], np.float64)
        nrm = np.linalg.norm(ref, axis=1)
        nrm[nrm == 0.0] = 1.0  # the all-zero row: absolute error
        worst = max(worst, float((np.linalg.norm(y[rows] - ref, axis=1) / nrm).max()))
        if y_ref is not None:
            worst_ref = max(worst_ref, float((np.linalg.norm(y_ref[rows] - ref, axis=1) / nrm).max()))
    # three-term E4M3 token operands (about twelve bits) and an fp16 intermediate here, bf16 intermediate in the reference
    # kernel: a few 1e-4 / 1e-3 per row
    print(f"dr_moe_prefill_fp8 ({route}) worst per-row rel-L2 {worst:.3e} (the reference's kernel {worst_ref:.3e})")
    # measured: 3.3e-4 (e4m3), 1.1e-3 (fp16: a weight times its scale is rounded to fp16, and under a row's largest scale
    # the small scales' products are fp16 subnormals), the reference's kernel 2.4e-3
    assert worst <= (8e-4 if route == "e4m3" else 2e-3), worst
    assert worst_ref <= 6e-3, worst_ref


def test_moe_prefill_fp8_256_experts(st):
    """The model's own expert count with Zipf-like group sizes (every expert hit, a few of them with several 16-token
    groups): seven experts' rows against the fp64 expert, every row finite."""
    l = ffi.lib()
    shape = synth.MoeShape(experts=256)
    host = synth.make_fp8_experts(12, shape)
    f8 = Fp8Experts.upload(host, st)
    rng = np.random.Generator(np.random.PCG64(80))
    counts = np.minimum(1 + (300.0 / np.arange(1, 257) ** 1.1).astype(np.int32), 300).astype(np.int32)[rng.permutation(256)]
    offsets = (np.cumsum(counts) - counts).astype(np.int32)
    n = int(counts.sum())
    xb = synth.f32_to_bf16_bits(rng.standard_normal((n, 2048), dtype=np.float32))
    dxp, dcnt, doff = DevBuf.from_array(xb, st), DevBuf.from_array(counts, st), DevBuf.from_array(offsets, st)
    dact, dy = DevBuf(n * 512 * 2), DevBuf(n * 2048 * 4)
    dy.fill(0xFF, st)
    launched(l.dr_moe_prefill_fp8(f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), dxp.at(0), doff.at(0), dcnt.at(0),
                                  dact.at(0), dy.at(0), 256, 2048, 512, st.raw), "moe_prefill_fp8")
    st.sync()
    assert device_error_word() == 0
    y = dy.download(np.float32, n * 2048, st).reshape(n, 2048)
    assert np.isfinite(y).all()
    x = synth.bf16_bits_to_f32(xb).astype(np.float64)
    order = np.argsort(counts)
    for e in (*order[-3:], *order[:2], 0, 255):  # the three largest groups, two of the smallest, the first and last expert
        rows = slice(offsets[e], offsets[e] + counts[e])
        ref = orc.expert_forward(host, int(e), x[rows], np.float64)
        rel = np.linalg.norm(y[rows] - ref, axis=1) / np.linalg.norm(ref, axis=1)
        assert np.isfinite(rel).all() and rel.max() <= 8e-4, (int(e), float(rel.max()))


def test_moe_prefill_fp8_back_to_back(st):
    """Two hundred calls queued without a synchronisation between them (a block of one launch starts on a multiprocessor
    the moment a block of the launch before has left it): same bits every time, error word clear."""
    l = ffi.lib()
    shape = synth.MoeShape(experts=16)
    host = synth.make_layer(9, shape)
    host.update(synth.make_fp8_experts(9, shape))
    f8 = Fp8Experts.upload(host, st)
    rng = np.random.Generator(np.random.PCG64(79))
    counts = np.array([40, 3, 0, 16, 17, 1, 90, 5, 0, 31, 32, 33, 2, 8, 64, 11], dtype=np.int32)
    offsets = (np.cumsum(counts) - counts).astype(np.int32)
    n = int(counts.sum())
    xb = synth.f32_to_bf16_bits(rng.standard_normal((n, 2048), dtype=np.float32))
    dxp, dcnt, doff = DevBuf.from_array(xb, st), DevBuf.from_array(counts, st), DevBuf.from_array(offsets, st)
    dact, dy = DevBuf(n * 512 * 2), DevBuf(n * 2048 * 4)

    def call():
        launched(l.dr_moe_prefill_fp8(f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), dxp.at(0), doff.at(0), dcnt.at(0),
                                      dact.at(0), dy.at(0), 16, 2048, 512, st.raw), "moe_prefill_fp8", debug=False)

    call()
    st.sync()
    first = dy.download(np.float32, n * 2048, st)
    assert np.isfinite(first).all()
    for _ in range(200):
        call()
    st.sync()
    assert device_error_word() == 0
    assert np.array_equal(dy.download(np.float32, n * 2048, st), first)


def test_fp8_stack_through_the_engine(st):
    """Three layers of block-FP8 experts through MoeDecoder (router + dr_moe_decode_fp8 per layer), eager and from a
    graph, against the fp64 oracle."""
    from drama_rs_b200.engine import MoeDecoder

    shape = synth.MoeShape(experts=16)
    hosts = []
    for seed in (11, 12, 13):
        h = synth.make_layer(seed, shape)
        h.update(synth.make_fp8_experts(seed, shape))
        hosts.append(h)
    devs = [MoeLayer.upload(h, st) for h in hosts]
    f8s = [Fp8Experts.upload(h, st) for h in hosts]
    x = synth.make_x(4, 1, 2048)[0]
    ref = x.astype(np.float64)[None]
    for h in hosts:
        ref = orc.moe_layer(h, ref, 8, 1e-6, np.float64)[0]
    dec = MoeDecoder(devs, st=st, fp8=f8s)
    dec.set_x(x)
    y = dec.step_eager()
    assert_parity(y, ref[0], "fp8 stack", max_abs=max(1e-2, 4e-6 * float(np.abs(ref).max())))
    dec.capture()
    dec.set_x(x)
    assert np.array_equal(dec.step(), y)
    assert device_error_word() == 0
