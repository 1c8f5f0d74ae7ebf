"""Router, MoE decode and MoE prefill through the C ABI against the oracle and the golden vectors."""

import os

import numpy as np
import pytest

from drama_rs_b200 import ffi, synth
from drama_rs_b200.engine import MoeDecoder, MoePrefill, MoeStackDecoder
from drama_rs_b200.gpu import DevBuf, Stream, launched
from drama_rs_b200.model import MoeLayer
from oracle import moe_oracle as orc
from tests.helpers import NULL, assert_parity, device_error_word

pytestmark = pytest.mark.gpu

SHAPE = synth.MoeShape()


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


def test_moe_decode_chained_routing(st, layers):
    """drb_moe_decode_chained: the down kernel of layer l also produces the routing of layer l + 1. Four layers (256 experts) and three layers of 16 experts: every layer's routing bit-exact against the
    fp64 oracle, the hidden state within the layer bar, eager == graph replay, and within fp32 noise of the plain
    dr_router_topk + dr_moe_decode sequence."""
    for experts, seeds in ((256, (0, 1, 0, 1)), (16, (3, 4, 3))):
        pairs = [layers(s, experts) for s in seeds]
        x = synth.make_x(21, 1, 2048)[0]
        ref = x.astype(np.float64)[None]
        ref_idx = []
        for host, _ in pairs:
            ref, ridx, _, _, _ = orc.moe_layer(host, ref, 8, 1e-6, np.float64)
            ref_idx.append(ridx[0])
        dec = MoeDecoder([d for _, d in pairs], st=st, chained=True, trace_routing=True)
        dec.set_x(x)
        y = dec.step_eager()
        assert device_error_word() == 0
        assert np.array_equal(dec.routing_trace(), np.stack(ref_idx)), f"routing, {experts} experts"
        scale = np.abs(ref).max()
        assert_parity(y, ref[0], f"chained stack, {experts} experts", max_abs=max(1e-2, 4e-6 * scale))
        plain = MoeDecoder([d for _, d in pairs], st=st)
        plain.set_x(x)
        assert np.abs(y - plain.step_eager()).max() <= 4e-6 * scale
        dec.capture()
        for _ in range(3):
            dec.set_x(x)
            assert np.array_equal(dec.step(), y), "graph replay of the chained sequence differs from the eager launches"
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
        worst = max(worst, float(rel.max()))
    # fp16 weights and fp16 intermediate: a few 1e-4 per row
    assert worst <= 8e-4, worst


def test_router_logits_do_not_depend_on_the_batch(st, layers):
    """drb_router_logits: a row's logits are bit-identical whether it is computed alone, in a batch of 7 or of 300
    (what lets expert-parallel ranks with different row counts route identically), and agree with cuBLAS."""
    host, dev = layers(2)
    x = synth.make_x(8, 300, 2048)
    runs = {}
    for name, sl in (("all", slice(0, 300)), ("seven", slice(100, 107)), ("one", slice(103, 104))):
        pre = MoePrefill(dev, 300, st=st)
        pre.invariant_router = True
        pre.run(x[sl])
        n = sl.stop - sl.start
        runs[name] = (pre.rlog.download(np.float32, n * 257, st).reshape(n, 257), pre.idx.download(np.int32, n * 8, st).reshape(n, 8))
    assert np.array_equal(runs["all"][0][100:107].view(np.uint32), runs["seven"][0].view(np.uint32))
    assert np.array_equal(runs["all"][0][103:104].view(np.uint32), runs["one"][0].view(np.uint32))
    assert np.array_equal(runs["all"][1][100:107], runs["seven"][1])
    blas = MoePrefill(dev, 300, st=st)
    blas.run(x)
    lb = blas.rlog.download(np.float32, 300 * 257, st).reshape(300, 257)
    assert np.abs(lb - runs["all"][0]).max() <= 1e-5 * np.abs(lb).max()
    xh = orc.round_bf16(orc.rmsnorm(x, host["post_norm"], 1e-6))
    ref = orc.router_logits(host, xh.astype(np.float64), np.float64)
    # the device's RMSNorm sums in another order, so a few normalised values round to the neighbouring bf16
    assert np.abs(ref - runs["all"][0]).max() <= 2e-3 * np.abs(ref).max()
    assert ffi.lib().drb_router_logits(NULL, NULL, NULL, 4, 257, 1024, 0.0, st.raw) == -1


def test_moe_prefill_golden_rows40(st, layers, golden_dir):
    g = np.load(os.path.join(golden_dir, "moe_rows40_seed2.npz"))
    host, dev = layers(2)
    x = synth.make_x(2, 40, 2048)
    pre = MoePrefill(dev, 64, st=st)
    y = pre.run(x)
    idx = pre.idx.download(np.int32, 40 * 8, st).reshape(40, 8)
    # The prefill ABI carries the normalised rows in bf16 (src/engine.rs:499, 554), so routing is decided on
    # bf16-rounded activations: compare with the oracle fed the same rows, and with the reference's fp32-input
    # routing wherever the two oracles agree.
    xh = orc.round_bf16(orc.rmsnorm(x, host["post_norm"], 1e-6))
    out, oidx, _, _, logits = orc.moe_block(host, xh.astype(np.float64), 8, np.float64)
    safe = orc.route_margin(logits, 256, 8) > 1e-6
    assert safe.all() and np.array_equal(idx, oidx)
    same = (oidx == g["idx"]).all(axis=1)
    assert same.mean() >= 0.9 and np.array_equal(idx[same], g["idx"][same])
    ref = x.astype(np.float64) + g["out_hf64"]
    a, r = assert_parity(y[same], ref[same], "prefill 40 rows vs the reference (fp32 inputs)", max_abs=np.inf, rel_l2=REL_PREFILL)
    assert_parity(y - x, out, "prefill 40 rows vs bf16-input oracle", max_abs=np.inf, rel_l2=REL_PREFILL)
    assert device_error_word() == 0


# Relative L2 of the prefill output. The shared expert runs through cuBLAS on weights dequantised to bf16 and
# a bf16 intermediate, exactly as the reference's prefill does (src/engine.rs:351-355, 560-562); that rounding,
# not the routed int4 path, sets this figure.
REL_PREFILL = 4e-3


def test_moe_prefill_device_scan_and_graph(st, layers):
    """With the offsets computed on the device the whole prefill block is one captured graph; its result equals
    the reference-style sequence with the host scan."""
    from drama_rs_b200.gpu import Graph

    host, dev = layers(2)
    x = synth.make_x(5, 64, 2048)
    pre = MoePrefill(dev, 64, st=st)
    y_host_scan = pre.run(x)
    pre.device_scan = True
    y_dev_scan = pre.run(x)
    assert np.array_equal(y_host_scan, y_dev_scan)
    g = Graph(st, lambda: pre.run_device(64))
    pre.x.upload(x, st)
    g.launch(st)
    y_graph = pre.x.download(np.float32, 64 * 2048, st).reshape(64, 2048)
    assert np.array_equal(y_graph, y_host_scan)
    assert device_error_word() == 0


def test_moe_prefill_zipf_300(st, layers):
    host, dev = layers(2)
    x = synth.make_x(33, 300, 2048)
    bias = synth.zipf_router_bias(33, 256, 1.1)
    pre = MoePrefill(dev, 300, st=st)
    y = pre.run(x, logit_bias=bias)
    xh = orc.round_bf16(orc.rmsnorm(x, host["post_norm"], 1e-6))
    out, idx, wts, sgate, logits = orc.moe_block(host, xh.astype(np.float64), 8, np.float64, logit_bias=bias)
    got_idx = pre.idx.download(np.int32, 300 * 8, st).reshape(300, 8)
    margin = orc.route_margin(logits, 256, 8)
    safe = margin > 1e-6
    assert np.array_equal(got_idx[safe], idx[safe]) and safe.mean() > 0.99
    counts = pre.counts.download(np.int32, 256, st)
    assert counts.sum() == 2400 and np.array_equal(counts, orc.moe_count(got_idx, 256))
    assert_parity((y - x)[safe], out[safe], "prefill zipf 300", max_abs=np.inf, rel_l2=REL_PREFILL)
    assert device_error_word() == 0
