"""Router, MoE decode and MoE prefill through the C ABI against the oracle and the golden vectors."""

import os

import numpy as np
import pytest

from drama_rs_b200 import ffi, synth
from drama_rs_b200.engine import MoeDecoder, MoePrefill, MoeStackDecoder
from drama_rs_b200.gpu import DevBuf, Stream, launched
from drama_rs_b200.model import MoeLayer
from oracle import moe_oracle as orc
from tests.helpers import MAX_ABS, NULL, REL_L2, assert_parity, device_error_word, parity

pytestmark = pytest.mark.gpu

SHAPE = synth.MoeShape()
# the reference's own kernels/drama.cu built unchanged as a checker (oracle/build.py); absent when no checkout was at hand
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libdrama_ref.so")


@pytest.fixture(scope="module")
def st():
    return Stream()


@pytest.fixture(scope="module")
def layers(st):
    """Seeded config-0 layers, generated once and kept on the device for the module."""
    cache = {}

    def get(seed, experts=256):
        key = (seed, experts)
        if key not in cache:
            host = synth.make_layer(seed, synth.MoeShape(experts=experts))
            cache[key] = (host, MoeLayer.upload(host, st))
        return cache[key]

    return get


def test_moe_topk_rows_and_ties(st):
    l = ffi.lib()
    rng = np.random.Generator(np.random.PCG64(3))
    for e, topk in ((256, 8), (16, 4), (200, 32), (8, 8)):
        rows = 33
        logits = rng.standard_normal((rows, e + 1)).astype(np.float32)
        logits[1, :e] = 0.0  # all tied: lowest indices win, in order
        logits[2, [3, 9 % e, 5]] = 4.0  # three-way tie at the top
        d = DevBuf.from_array(logits, st)
        didx, dw, dsg = DevBuf(rows * topk * 4), DevBuf(rows * topk * 4), DevBuf(rows * 4)
        launched(l.dr_moe_topk(d.at(0), rows, e, topk, e + 1, didx.at(0), dw.at(0), dsg.at(0), st.raw), "moe_topk")
        idx = didx.download(np.int32, rows * topk, st).reshape(rows, topk)
        wts = dw.download(np.float32, rows * topk, st).reshape(rows, topk)
        sg = dsg.download(np.float32, rows, st)
        ridx, rwts, rsg = orc.route(logits, e, topk)
        assert np.array_equal(idx, ridx), (e, topk)
        assert idx[1].tolist() == list(range(topk))
        assert np.abs(wts - rwts).max() <= 2e-6
        assert np.array_equal(sg, rsg)
    assert l.dr_moe_topk(d.at(0), 1, 300, 8, 301, didx.at(0), dw.at(0), dsg.at(0), st.raw) == -1


@pytest.mark.parametrize("seed,experts,topk", [(0, 256, 8), (1, 256, 8), (3, 16, 8), (3, 16, 3)])
def test_router_topk(st, layers, golden_dir, seed, experts, topk):
    l = ffi.lib()
    host, dev = layers(seed, experts)
    x = synth.make_x(seed, 1, 2048)[0]
    dx = DevBuf.from_array(x, st)
    dlog, didx, dw, dsg = DevBuf((experts + 1) * 4), DevBuf(topk * 4), DevBuf(topk * 4), DevBuf(4)
    counter = DevBuf.zeros(16, st)
    for rep in range(3):  # the counter must come back to zero so that the call can be repeated
        launched(
            l.dr_router_topk(dev.router.at(0), dx.at(0), dev.post_norm.at(0), 1e-6, dlog.at(0), experts, topk, 2048,
                             didx.at(0), dw.at(0), dsg.at(0), counter.at(0), NULL, NULL, NULL, NULL, 0, 0, 0, 0, st.raw),
            "router_topk")
        st.sync()
        assert counter.download(np.uint32, 4, st).tolist() == [0, 0, 0, 0]
    logits = dlog.download(np.float32, experts + 1, st)
    idx, wts, sg = didx.download(np.int32, topk, st), dw.download(np.float32, topk, st), dsg.download(np.float32, 1, st)
    xh = orc.rmsnorm(x[None], host["post_norm"], 1e-6, np.float64)
    ref_logits = orc.router_logits(host, xh, np.float64)
    ridx, rwts, rsg = orc.route(ref_logits, experts, topk, np.float64)
    assert np.abs(logits - ref_logits[0]).max() <= 2e-5
    assert np.array_equal(idx, ridx[0])
    assert np.abs(wts - rwts[0]).max() <= 2e-5
    assert abs(float(sg[0]) - float(rsg[0])) <= 2e-5
    if experts == 256 and topk == 8 and seed in (0, 1):
        g = np.load(os.path.join(golden_dir, f"moe_decode_seed{seed}.npz"))
        assert np.array_equal(idx, g["idx"][0])  # the reference's own PyTorch routing
    assert device_error_word() == 0


@pytest.mark.parametrize("seed", [0, 1])
def test_moe_decode_layer_golden(st, layers, golden_dir, seed):
    """One config-0 layer, x == res == y, eager and as a replayed graph."""
    g = np.load(os.path.join(golden_dir, f"moe_decode_seed{seed}.npz"))
    host, dev = layers(seed)
    x = synth.make_x(seed, 1, 2048)[0]
    ref = x.astype(np.float64) + g["out_hf64"][0]
    dec = MoeDecoder([dev], st=st)
    dec.set_x(x)
    y = dec.step_eager()
    idx, wts, sg = dec.routing()
    assert np.array_equal(idx, g["idx"][0])
    assert np.abs(wts - g["wts"][0]).max() <= 2e-5
    a, r = assert_parity(y, ref, f"decode seed {seed} eager")
    # the reference's own fp32 result is not closer to fp64 than this by more than its own noise
    floor = np.abs(g["out_hf"][0].astype(np.float64) - g["out_hf64"][0]).max()
    print(f"seed {seed}: max-abs {a:.3e} rel-L2 {r:.3e}; reference fp32 noise floor {floor:.3e}")
    dec.capture()
    for _ in range(3):
        dec.set_x(x)
        y2 = dec.step()
        assert np.array_equal(y2, y), "graph replay differs from the eager launch"
    assert device_error_word() == 0


def test_moe_decode_routed_part_alone(st, layers):
    """With the shared expert gated off and no residual the routed int4 experts are all that is left."""
    l = ffi.lib()
    host, dev = layers(1)
    x = synth.make_x(11, 1, 2048)[0]
    xh = orc.rmsnorm(x[None], host["post_norm"], 1e-6, np.float64)
    idx = np.array([5, 250, 17, 0, 255, 128, 64, 33], dtype=np.int32)
    wts = np.array([0.3, 0.2, 0.15, 0.1, 0.1, 0.05, 0.05, 0.05], dtype=np.float32)
    ref = np.zeros(2048)
    for k in range(8):
        ref += wts[k] * orc.expert_forward(host, int(idx[k]), xh, np.float64)[0]
    dx, didx, dw = DevBuf.from_array(x, st), DevBuf.from_array(idx, st), DevBuf.from_array(wts, st)
    dsg = DevBuf.from_array(np.array([-1e4], np.float32), st)  # sigmoid -> 0
    dres, dact, dy = DevBuf.zeros(2048 * 4, st), DevBuf(9 * 512 * 4), DevBuf(2048 * 4)
    gq, gs = dev.gate_up.expert(0)
    dq, ds = dev.down.expert(0)
    sgq, sgs = dev.shared_gate_up.rows(0)
    sdq, sds = dev.shared_down.rows(0)
    launched(
        l.dr_moe_decode(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dres.at(0), dact.at(0),
                        dy.at(0), 2048, 512, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw), "moe_decode")
    y = dy.download(np.float32, 2048, st)
    a, r = assert_parity(y, ref, "routed experts alone", max_abs=1e-4, rel_l2=1e-5)
    assert l.dr_moe_decode(gq, gs, dq, ds, sgq, sgs, sdq, sds, dx.at(0), didx.at(0), dw.at(0), dsg.at(0), dres.at(0),
                           dact.at(0), dy.at(0), 2048, 256, 8, dev.post_norm.at(0), 1e-6, NULL, 0, st.raw) == -1


def test_moe_decode_stack_of_layers(st, layers):
    """Three layers carried x -> x + moe(rmsnorm(x)) in one graph, against the fp64 oracle."""
    pairs = [layers(s) for s in (0, 1, 0)]
    x = synth.make_x(21, 1, 2048)[0]
    ref = x.astype(np.float64)[None]
    for host, _ in pairs:
        ref = orc.moe_layer(host, ref, 8, 1e-6, np.float64)[0]
    dec = MoeDecoder([d for _, d in pairs], st=st)
    dec.capture()
    dec.set_x(x)
    y = dec.step()
    scale = np.abs(ref).max()
    a, r = assert_parity(y, ref[0], "3-layer stack", max_abs=max(1e-2, 4e-6 * scale))
    assert device_error_word() == 0


def test_moe_decode_shared_expert_extreme_codes(st):
    """The shared expert's int8 codes all at +127 against a constant hidden state: every 32-value slice of the
    normalised row sits at full scale, and a chunk's integer sum (32 * 127 * 2^20) exceeds int32. Per-layer entry
    points and the persistent kernel against the fp64 oracle."""
    shape = synth.MoeShape(experts=16)
    host = dict(synth.make_layer(5, shape))
    host["moe.shared_gate_up.q8"] = np.full_like(host["moe.shared_gate_up.q8"], 127)
    host["moe.shared_gate_up.s"] = np.full_like(host["moe.shared_gate_up.s"], 2e-5)
    host["post_norm"] = np.ones_like(host["post_norm"])
    dev = MoeLayer.upload(host, st)
    x = np.full(shape.hidden, 3.0, dtype=np.float32)
    ref, ridx, _, _, _ = orc.moe_layer(host, x[None], shape.topk, shape.eps, np.float64)
    scale = np.abs(ref).max()
    dec = MoeDecoder([dev], st=st)
    dec.set_x(x)
    y = dec.step_eager()
    assert np.array_equal(dec.routing()[0], ridx[0])
    assert_parity(y, ref[0], "per-layer decode, saturated shared expert", max_abs=max(1e-2, 4e-6 * scale))
    stack = MoeStackDecoder([dev], st=st)
    stack.set_x(x)
    assert_parity(stack.step(), ref[0], "stack decode, saturated shared expert", max_abs=max(1e-2, 4e-6 * scale))
    assert device_error_word() == 0


def test_moe_stack_persistent_kernel(st, layers, golden_dir):
    """drb_moe_stack_decode: four layers in one persistent kernel, eager and from a graph, against the fp64
    oracle (routing of every layer bit-exact) and against the per-layer entry points."""
    pairs = [layers(s) for s in (0, 1, 0, 1)]
    x = synth.make_x(21, 1, 2048)[0]
    ref = x.astype(np.float64)[None]
    ref_idx = []
    for host, _ in pairs:
        ref, ridx, _, _, _ = orc.moe_layer(host, ref, 8, 1e-6, np.float64)
        ref_idx.append(ridx[0])
    sd = MoeStackDecoder([d for _, d in pairs], st=st)
    sd.set_x(x)
    y = sd.step()
    assert device_error_word() == 0
    idx, wts = sd.routing()
    assert np.array_equal(idx, np.stack(ref_idx))
    scale = np.abs(ref).max()
    assert_parity(y, ref[0], "4-layer persistent stack", max_abs=max(1e-2, 4e-6 * scale))
    dec = MoeDecoder([d for _, d in pairs], st=st)
    dec.set_x(x)
    y_layers = dec.step_eager()
    assert np.abs(y - y_layers).max() <= 4e-6 * scale
    sd.capture()
    for _ in range(3):
        sd.set_x(x)
        assert np.array_equal(sd.step(), y), "graph replay of the persistent kernel differs from the eager launch"
    # one layer against the golden vectors of the reference's own code
    g = np.load(os.path.join(golden_dir, "moe_decode_seed0.npz"))
    one = MoeStackDecoder([pairs[0][1]], st=st)
    x0 = synth.make_x(0, 1, 2048)[0]
    one.set_x(x0)
    y0 = one.step()
    assert np.array_equal(one.routing()[0][0], g["idx"][0])
    assert_parity(y0, x0.astype(np.float64) + g["out_hf64"][0], "persistent kernel, golden layer")
    assert device_error_word() == 0


def test_moe_stack_40_layers_against_the_oracle(st, layers):
    """The benchmark's decode step at its real depth: 40 layers (two seeded layers alternating, so the stack is 40
    pointers) in one persistent kernel against the fp64 oracle, every layer's routing bit-exact. The per-layer entry
    points are held to the same bar on the same stack."""
    pairs = [layers(s) for s in (0, 1)] * 20
    x = synth.make_x(21, 1, 2048)[0]
    ref = x.astype(np.float64)[None]
    ref_idx, margins = [], []
    for host, _ in pairs:
        ref, ridx, _, _, logits = orc.moe_layer(host, ref, 8, 1e-6, np.float64)
        ref_idx.append(ridx[0])
        margins.append(float(orc.route_margin(logits, 256, 8)[0]))
    ref_idx = np.stack(ref_idx)
    # a margin below ~1e-6 of probability is within fp32 rounding of the logits themselves: such a layer's routing is
    # not decidable in single precision (none occurs on this seed; the assertion documents the premise)
    assert min(margins) > 1e-6, min(margins)
    scale = float(np.abs(ref).max())
    sd = MoeStackDecoder([d for _, d in pairs], st=st)
    sd.capture()
    sd.set_x(x)
    y = sd.step()
    assert device_error_word() == 0
    idx, _ = sd.routing()
    assert np.array_equal(idx, ref_idx), np.nonzero((idx != ref_idx).any(axis=1))[0]
    # one layer is held to 4e-6 of the largest output (the fp32 noise of the reference block); over 40 layers of an
    # fp32 hidden state that compounds, so the stack is held to 1e-5 and the reference's own fp32 kernels are run on
    # the same stack to show where the floor lies
    bar = max(1e-2, 1e-5 * scale)
    a, r = assert_parity(y, ref[0], "40-layer persistent stack", max_abs=bar)
    dec = MoeDecoder([d for _, d in pairs], st=st, trace_routing=True)
    dec.capture()
    dec.set_x(x)
    y2 = dec.step()
    assert np.array_equal(dec.routing_trace(), ref_idx)
    a2, r2 = assert_parity(y2, ref[0], "40-layer stack, per-layer entry points", max_abs=bar)
    note = ""
    if os.path.exists(REF_LIB):
        rdec = MoeDecoder([d for _, d in pairs], st=st, lib=ffi.bind(REF_LIB))
        rdec.set_x(x)
        a3, r3 = parity(rdec.step_eager(), ref[0])
        note = f"; the reference's fp32 kernels max-abs {a3:.3e} rel-L2 {r3:.3e}"
    print(f"40 layers, |x| {scale:.3e}: persistent max-abs {a:.3e} rel-L2 {r:.3e}; per-layer max-abs {a2:.3e} rel-L2 {r2:.3e}{note}; smallest routing margin {min(margins):.2e}")
    assert device_error_word() == 0


def test_moe_prefill_grouped_kernel_direct(st, layers):
    """dr_moe_prefill alone on hand-made groups: one expert with more tokens than one accumulator holds (300),
    empty experts, groups of 1, 16 and 17 tokens. Each output row against the fp64 expert on the same bf16 row."""
    l = ffi.lib()
    host, dev = layers(3, 16)
    counts = np.array([300, 0, 1, 17, 16, 5, 0, 33, 2, 0, 7, 64, 3, 1, 0, 9], dtype=np.int32)
    offsets = (np.cumsum(counts) - counts).astype(np.int32)
    n = int(counts.sum())
    rng = np.random.Generator(np.random.PCG64(77))
    xb = synth.f32_to_bf16_bits(rng.standard_normal((n, 2048), dtype=np.float32))
    dxp, dcnt, doff = DevBuf.from_array(xb, st), DevBuf.from_array(counts, st), DevBuf.from_array(offsets, st)
    dact, dy = DevBuf(n * 512 * 2), DevBuf(n * 2048 * 4)
    dy.fill(0xFF, st)
    gq, gs = dev.gate_up.expert(0)
    dq, ds = dev.down.expert(0)
    launched(l.dr_moe_prefill(gq, gs, dq, ds, dxp.at(0), doff.at(0), dcnt.at(0), dact.at(0), dy.at(0), 16, 2048, 512, st.raw), "moe_prefill")
    y = dy.download(np.float32, n * 2048, st).reshape(n, 2048)
    assert device_error_word() == 0
    x = synth.bf16_bits_to_f32(xb).astype(np.float64)
    worst = 0.0
    for e in range(16):
        if counts[e] == 0:
            continue
        rows = slice(offsets[e], offsets[e] + counts[e])
        ref = orc.expert_forward(host, e, x[rows], np.float64)
        rel = np.linalg.norm(y[rows] - ref, axis=1) / np.linalg.norm(ref, axis=1)
        assert np.isfinite(rel).all()  # max() below would let a NaN row pass
        worst = max(worst, float(rel.max()))
    # fp16 weights and fp16 intermediate: a few 1e-4 per row
    assert worst <= 8e-4, worst


def test_router_logits_do_not_depend_on_the_batch(st, layers):
    """drb_router_logits / drb_router_logits_f16: a row's logits are bit-identical whether it is computed alone, in a
    batch of 7 or of 300 (what lets expert-parallel ranks with different row counts route identically), and agree
    with cuBLAS on the same bf16 rows."""
    host, dev = layers(2)
    x = synth.make_x(8, 300, 2048)
    for rows_f16 in (True, False):
        runs = {}
        for name, sl in (("all", slice(0, 300)), ("seven", slice(100, 107)), ("one", slice(103, 104))):
            pre = MoePrefill(dev, 300, st=st)
            pre.rows_f16 = rows_f16
            pre.run(x[sl])
            n = sl.stop - sl.start
            runs[name] = (pre.rlog.download(np.float32, n * 257, st).reshape(n, 257), pre.idx.download(np.int32, n * 8, st).reshape(n, 8))
        assert np.array_equal(runs["all"][0][100:107].view(np.uint32), runs["seven"][0].view(np.uint32))
        assert np.array_equal(runs["all"][0][103:104].view(np.uint32), runs["one"][0].view(np.uint32))
        assert np.array_equal(runs["all"][1][100:107], runs["seven"][1])
        xh = orc.rmsnorm(x, host["post_norm"], 1e-6)
        xh = xh.astype(np.float16).astype(np.float32) if rows_f16 else orc.round_bf16(xh)
        ref = orc.router_logits(host, xh.astype(np.float64), np.float64)
        # the device's RMSNorm sums in another order, so a few normalised values round to the neighbouring 16-bit value
        assert np.abs(ref - runs["all"][0]).max() <= (3e-4 if rows_f16 else 2e-3) * np.abs(ref).max()
    blas = MoePrefill(dev, 300, st=st, reference_calls=True)
    blas.run(x)
    lb = blas.rlog.download(np.float32, 300 * 257, st).reshape(300, 257)
    assert np.abs(lb - runs["all"][0]).max() <= 1e-5 * np.abs(lb).max()
    assert ffi.lib().drb_router_logits(NULL, NULL, NULL, 4, 257, 1024, 0.0, st.raw) == -1
    assert ffi.lib().drb_router_logits_f16(NULL, NULL, NULL, 4, 257, 1024, 0.0, st.raw) == -1


def prefill_bar(ref):
    """The prefill bar: relative L2 1e-3, and max-abs 1e-2 scaled to the outputs where they are large. The grouped
    GEMMs run on the tensor cores with fp16 operands (11 significant bits where the decode path's integer dot
    products are exact), so the absolute error is 2^-11 of the largest output, not the decode path's 4e-6."""
    return dict(max_abs=max(MAX_ABS, 2.0 ** -11 * float(np.abs(ref).max())), rel_l2=REL_L2)


# Relative L2 of the reference call sequence: the shared expert runs through cuBLAS on weights dequantised to bf16 and
# a bf16 intermediate, exactly as the reference's prefill does (src/engine.rs:351-355, 560-562); that rounding sets it.
REL_PREFILL_CUBLAS = 4e-3


def test_moe_prefill_golden_rows40(st, layers, golden_dir):
    """40 rows through the prefill block: this library's own sequence (grouping kernel, grouped tensor-core GEMMs that
    also run the int8 shared expert, no library GEMM) held to the layer bar; the reference's call sequence (shared
    expert through cuBLAS on bf16-dequantised weights) to the looser figure that rounding sets."""
    g = np.load(os.path.join(golden_dir, "moe_rows40_seed2.npz"))
    host, dev = layers(2)
    x = synth.make_x(2, 40, 2048)
    ref = x.astype(np.float64) + g["out_hf64"]
    for reference_calls in (False, True):
        # the reference's prefill rounds the normalised rows to bf16, this library's own sequence keeps fp16: the oracle
        # is fed the rows as the sequence sees them, so routing is compared on equal terms
        xh = orc.rmsnorm(x, host["post_norm"], 1e-6)
        xh = orc.round_bf16(xh) if reference_calls else xh.astype(np.float16).astype(np.float32)
        out, oidx, _, _, logits = orc.moe_block(host, xh.astype(np.float64), 8, np.float64)
        safe = orc.route_margin(logits, 256, 8) > 1e-6
        same = (oidx == g["idx"]).all(axis=1)
        pre = MoePrefill(dev, 64, st=st, reference_calls=reference_calls)
        y = pre.run(x)
        idx = pre.idx.download(np.int32, 40 * 8, st).reshape(40, 8)
        assert safe.all() and np.array_equal(idx, oidx)
        assert same.mean() >= 0.9 and np.array_equal(idx[same], g["idx"][same])
        what = "reference call sequence" if reference_calls else "own sequence"
        bar = dict(max_abs=np.inf, rel_l2=REL_PREFILL_CUBLAS) if reference_calls else prefill_bar(out)
        a, r = assert_parity(y - x, out, f"prefill 40 rows, {what}, vs the oracle on the same 16-bit rows", **bar)
        a2, r2 = parity(y[same], ref[same])
        print(f"{what}: vs same-rows oracle max-abs {a:.3e} rel-L2 {r:.3e}; vs the reference block on fp32 rows max-abs {a2:.3e} rel-L2 {r2:.3e}")
        # the bar of the layer against the reference block itself (fp32 rows, fp64 arithmetic): relative L2 1e-3
        assert r2 <= (REL_PREFILL_CUBLAS if reference_calls else REL_L2)
        assert device_error_word() == 0


def test_moe_prefill_reference_calls_device_scan_and_graph(st, layers):
    """Reference call sequence: with the offsets computed on the device the whole block is one captured graph; its
    result equals the sequence with the host scan. Own sequence: a captured graph equals the eager launches."""
    from drama_rs_b200.gpu import Graph

    host, dev = layers(2)
    x = synth.make_x(5, 64, 2048)
    pre = MoePrefill(dev, 64, st=st, reference_calls=True)
    y_host_scan = pre.run(x)
    pre.device_scan = True
    y_dev_scan = pre.run(x)
    assert np.array_equal(y_host_scan, y_dev_scan)
    g = Graph(st, lambda: pre.run_device(64))
    pre.x.upload(x, st)
    g.launch(st)
    y_graph = pre.x.download(np.float32, 64 * 2048, st).reshape(64, 2048)
    assert np.array_equal(y_graph, y_host_scan)
    own = MoePrefill(dev, 64, st=st)
    y_own = own.run(x)
    g2 = Graph(st, lambda: own.run_device(64))
    for _ in range(2):
        own.x.upload(x, st)
        g2.launch(st)
        assert np.array_equal(own.x.download(np.float32, 64 * 2048, st).reshape(64, 2048), y_own)
    assert parity(y_own, y_host_scan)[1] <= 5e-3  # the two sequences differ by the rounding of rows and shared-expert weights to bf16
    assert device_error_word() == 0


def test_moe_group_matches_count_scan_permute(st, layers):
    """drb_moe_group against numpy: counts, exclusive scan, a valid slot assignment (every expert's slots are its
    range, each used once), row_of inverse of slot_of; an expert-parallel slice (e_lo, e_n) marks foreign pairs -1."""
    l = ffi.lib()
    rng = np.random.Generator(np.random.PCG64(5))
    for rows, topk, e, e_lo, e_n in ((300, 8, 256, 0, 256), (1, 8, 256, 0, 256), (77, 4, 64, 16, 32), (513, 8, 1024, 0, 1024)):
        idx = np.stack([rng.permutation(e)[:topk] for _ in range(rows)]).astype(np.int32)
        didx = DevBuf.from_array(idx, st)
        dc, do, ds, dr = DevBuf(e_n * 4), DevBuf(e_n * 4), DevBuf(rows * topk * 4), DevBuf(rows * topk * 4)
        dr.fill(0xFF, st)
        launched(l.drb_moe_group(didx.at(0), rows, topk, e_lo, e_n, dc.at(0), do.at(0), ds.at(0), dr.at(0), st.raw), "moe_group")
        counts, offsets = dc.download(np.int32, e_n, st), do.download(np.int32, e_n, st)
        slot_of, row_of = ds.download(np.int32, rows * topk, st), dr.download(np.int32, rows * topk, st)
        local = idx.reshape(-1) - e_lo
        mine = (local >= 0) & (local < e_n)
        assert np.array_equal(counts, np.bincount(local[mine], minlength=e_n))
        assert np.array_equal(offsets, np.cumsum(counts) - counts)
        assert (slot_of[~mine] == -1).all()
        s = slot_of[mine]
        assert np.array_equal(np.sort(s), np.arange(mine.sum()))
        assert ((s >= offsets[local[mine]]) & (s < offsets[local[mine]] + counts[local[mine]])).all()
        assert np.array_equal(row_of[s], np.nonzero(mine)[0] // topk)
    assert l.drb_moe_group(didx.at(0), 1, 8, 0, 2048, dc.at(0), do.at(0), ds.at(0), dr.at(0), st.raw) == -1


def test_moe_prefill_outliers_beyond_fp16_range_stay_finite(st, layers):
    """The tensor-core operands are fp16: a row with values above 65504 is clamped, not turned into infinities."""
    host, dev = layers(2)
    x = synth.make_x(9, 8, 2048)
    pre = MoePrefill(dev, 8, st=st)
    y0 = pre.run(x)
    # overwrite the normalised rows with outliers of 7e4 and -9e4 and run everything behind the routing
    l = ffi.lib()
    pre.x.upload(x, st)
    pre.route_device(8)
    pre.rows_f16 = False  # bf16 rows can hold such values; the fp16 operands they are converted to cannot
    pre.route_device(8)
    hb = synth.bf16_bits_to_f32(pre.hn_b.download(np.uint16, 8 * 2048, st)).reshape(8, 2048)
    hb[3, 100] = 7e4
    hb[3, 101] = -9e4
    pre.hn_b.upload(synth.f32_to_bf16_bits(hb), st)
    launched(l.drb_moe_group(pre.idx.at(0), 8, 8, 0, 256, pre.counts.at(0), pre.offsets.at(0), pre.slot_of.at(0), pre.row_of.at(0), st.raw), "group")
    gq, gs = dev.gate_up.expert(0)
    dq, ds = dev.down.expert(0)
    sgq, sgs = dev.shared_gate_up.rows(0)
    sdq, sds = dev.shared_down.rows(0)
    launched(l.drb_moe_prefill_block(gq, gs, dq, ds, sgq, sgs, sdq, sds, pre.hn_b.at(0), pre.row_of.at(0), pre.offsets.at(0), pre.counts.at(0),
                                     pre.ap.at(0), pre.yp.at(0), pre.sh_act_b.at(0), pre.sh_out.at(0), 8, 256, 2048, 512, 0, NULL, st.raw), "block")
    sh = pre.sh_out.download(np.float32, 8 * 2048, st)
    yp = pre.yp.download(np.float32, 64 * 2048, st)
    assert np.isfinite(sh).all() and np.isfinite(yp).all()
    assert np.isfinite(y0).all() and device_error_word() == 0


def test_moe_prefill_zipf_300(st, layers):
    host, dev = layers(2)
    x = synth.make_x(33, 300, 2048)
    bias = synth.zipf_router_bias(33, 256, 1.1)
    pre = MoePrefill(dev, 300, st=st)
    y = pre.run(x, logit_bias=bias)
    xh = orc.rmsnorm(x, host["post_norm"], 1e-6).astype(np.float16).astype(np.float32)  # the rows as the own sequence keeps them
    out, idx, wts, sgate, logits = orc.moe_block(host, xh.astype(np.float64), 8, np.float64, logit_bias=bias)
    got_idx = pre.idx.download(np.int32, 300 * 8, st).reshape(300, 8)
    margin = orc.route_margin(logits, 256, 8)
    safe = margin > 1e-6
    assert np.array_equal(got_idx[safe], idx[safe]) and safe.mean() > 0.99
    counts = pre.counts.download(np.int32, 256, st)
    assert counts.sum() == 2400 and np.array_equal(counts, orc.moe_count(got_idx, 256))
    assert_parity((y - x)[safe], out[safe], "prefill zipf 300", **prefill_bar(out[safe]))
    assert device_error_word() == 0
