#!/usr/bin/env python3
"""Benchmark of the routed-expert MoE decode path on B200.

    python bench.py --gpus 1 --steps K --warmup W             # this library
    python bench.py --impl reference --steps K --warmup W     # the CPU implementation, host cores

Workload ("decode_stack40_b1"): the full 40-layer MoE stack decode step at batch 1 — per layer the
bf16 router over 256 experts with fused RMSNorm and top-8, the 8 chosen int4 experts (SwiGLU
gate/up then down), the int8 shared expert with its sigmoid gate, and the residual — one persistent
kernel per step (drb_moe_stack_decode) inside a CUDA graph, replayed once per step on the same input.
18.1 GB of expert weights are resident; one step reads 736 MB of them, far more than the 126 MB L2,
so every step streams from HBM. Inputs are synthetic from a seed (there is no dataset on this path).

One JSON line is printed by rank 0. `value` is microseconds per layer with everything resident in
HBM; `e2e` is the same through the public call with host buffers (pinned host x in, host x out,
copies inside the timed region). The other keys of the line: the per-layer entry points of the
reference's ABI on the same stack, a parity check of the timed kernel at its real depth against the
fp64 oracle, the int8 GEMV sweep, the 300-row prefill layer, the expert-parallel legs at this N, and
(N = 1, when the checker library was built) the reference's own CUDA kernels on the same buffers.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from drama_rs_b200 import synth  # noqa: E402

SHAPE = synth.MoeShape()
LAYERS = 40
FALLBACK_HBM_GBS = 6650.0
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libdrama_ref.so")
TRAFFIC_JSON = os.path.join(ROOT, "profiles", "decode_stack_traffic.json")
NULL = C.c_void_p(0)


def peaks_json() -> dict:
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def peaks() -> tuple[float, str]:
    p = peaks_json()
    if "hbm_gbs" in p:
        return float(p["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        mhz, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = max(mx, float(r[1]))
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ----------------------------------------------------------------------------- CPU arm

_HOST_LAYERS = None


def host_layers():
    """Two seeded config-0 layers on the host (the CPU legs and the parity checks alternate them)."""
    global _HOST_LAYERS
    if _HOST_LAYERS is None:
        _HOST_LAYERS = [synth.make_layer(1000 + i, SHAPE) for i in range(2)]
    return _HOST_LAYERS


def cpu_stack_times(n_layers: int, batches: int, budget_s: float, threads: int | None = None) -> tuple[list[float], int]:
    """Seconds per `n_layers`-layer decode step of the plain-C restatement of the reference's decode layer, all
    OpenMP threads, two seeded layers alternating; at least `batches` steps, more while the budget lasts."""
    from oracle import c_oracle

    lib = c_oracle.lib()
    if threads:
        lib.orc_set_threads.argtypes = [C.c_int]
        lib.orc_set_threads.restype = None
        lib.orc_set_threads(threads)
    structs = [c_oracle.layer_struct(t, SHAPE.topk, SHAPE.eps) for t in host_layers()]
    x0 = synth.make_x(1000, 1, SHAPE.hidden)[0]
    x = x0.copy()

    def step():
        x[:] = x0
        for i in range(n_layers):
            lib.orc_moe_decode_layer(C.byref(structs[i % 2]), x.ctypes.data, None, None)

    step()  # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < batches or (time.perf_counter() < t_end and len(times) < 400):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return times, int(lib.orc_threads())


def cpu_decode_baseline(budget_s: float = 15.0) -> dict:
    times, cores = cpu_stack_times(LAYERS, 5, budget_s)
    us = float(np.median(times) / LAYERS * 1e6)
    return {"value": us, "unit": "us/layer", "cores": cores, "kind": "port",
            "sample": f"median of {len(times)} steps of the {LAYERS}-layer stack (2 seeded config-0 layers alternating), plain-C "
                      f"restatement of the reference's CUDA decode kernels with OpenMP; it stands in for the reference's two "
                      f"PyTorch CPU paths (HF block 2.8 ms/layer, tools/reference.py 65.7 ms/layer on 8 threads): the reference has no "
                      f"CPU engine, and a checkout of it is not assumed where this runs",
            "min_us_per_layer": float(min(times) / LAYERS * 1e6), "max_us_per_layer": float(max(times) / LAYERS * 1e6)}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is the CPU path with every host thread
    threads = len(os.sched_getaffinity(0))
    from oracle import c_oracle

    lib = c_oracle.lib()
    lib.orc_set_threads.argtypes = [C.c_int]
    lib.orc_set_threads.restype = None
    lib.orc_set_threads(threads)
    structs = [c_oracle.layer_struct(t, SHAPE.topk, SHAPE.eps) for t in host_layers()]
    x0 = synth.make_x(1000, 1, SHAPE.hidden)[0]
    x = x0.copy()

    def step():
        x[:] = x0
        for i in range(args.layers):
            lib.orc_moe_decode_layer(C.byref(structs[i % 2]), x.ctypes.data, None, None)

    for _ in range(args.warmup):
        step()
    per = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        t1 = time.perf_counter()
        step()
        per.append(time.perf_counter() - t1)
    dt = time.perf_counter() - t0
    # the line's value is the median step (a host shared with other jobs makes single steps wander by 30 %)
    us = float(np.median(per)) / args.layers * 1e6
    cores = int(lib.orc_threads())
    line = {
        "impl": "reference", "metric": "int4_moe_decode_us_per_layer", "value": us, "unit": "us/layer", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.median(per)) * 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "decode_stack40_b1", "layers": args.layers, "hidden": SHAPE.hidden,
                   "experts": SHAPE.experts, "topk": SHAPE.topk, "inter": SHAPE.inter},
        "cpu_baseline": {"value": us, "unit": "us/layer", "cores": cores, "kind": "port",
                         "sample": f"median of {args.steps} steps of the {args.layers}-layer stack (2 seeded layers alternating), plain-C "
                                   f"restatement of the reference kernels, OpenMP over {cores} threads; mean {dt / args.steps / args.layers * 1e6:.1f} us/layer"},
        "e2e": {"value": us, "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ----------------------------------------------------------------------------- GPU arm


def device_layers(torch, n_layers: int, seed: int, st):
    """n_layers config-0 layers generated on the device (same distributions as drama_rs_b200.synth)."""
    from drama_rs_b200.gpu import ExtBuf
    from drama_rs_b200.model import Q4, Q8, MoeLayer

    g = torch.Generator(device="cuda")
    h, i, e = SHAPE.hidden, SHAPE.inter, SHAPE.experts

    def ext(t):
        return ExtBuf(t.data_ptr(), t.numel() * t.element_size(), keep=t)

    def q4(n, k):
        q = torch.randint(0, 256, (e, n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        s = (torch.randn((e, n, k // 64), device="cuda", generator=g) * 0.01).abs().clamp_min(1e-4).half()
        sm = torch.stack((s, (s.float() * -8.0).half()), dim=-1).contiguous()
        return Q4(ext(q), ext(sm), e, n, k)

    def q8(n, k):
        q = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
        row = (torch.randn((n, 1), device="cuda", generator=g) * 0.005).abs().clamp_min(1e-4).half()
        return Q8(ext(q), ext(row.expand(n, k // 128).contiguous()), n, k)

    out = []
    for li in range(n_layers):
        g.manual_seed(seed + li)
        router = (torch.randn((e + 1, h), device="cuda", generator=g) * 0.02).bfloat16()
        pn = (1.0 + torch.randn(h, device="cuda", generator=g) * 0.1).float()
        out.append(MoeLayer(ext(router), ext(pn), q8(2 * i, h), q8(h, i), q4(2 * i, h), q4(h, i), e, h, i))
    torch.cuda.synchronize()
    return out


def time_on_stream(torch, st, ext_stream, fn, iters: int, warm: int = 3) -> float:
    """Microseconds per call of fn(i), CUDA events on the library's stream."""
    for i in range(warm):
        fn(i)
    st.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext_stream)
    for i in range(iters):
        fn(i)
    e1.record(ext_stream)
    st.sync()
    return e0.elapsed_time(e1) / iters * 1e3


def parity_check(st) -> dict:
    """The timed kernel at the workload's real depth against the fp64 oracle, outside any timed region: 40 layers over
    two host-generated layers alternating, every layer's routing compared index by index."""
    from drama_rs_b200.engine import MoeStackDecoder
    from drama_rs_b200.model import MoeLayer
    from oracle import moe_oracle as orc

    hosts = host_layers()
    devs = [MoeLayer.upload(h, st) for h in hosts]
    x = synth.make_x(21, 1, SHAPE.hidden)[0]
    ref = x.astype(np.float64)[None]
    ref_idx, margin = [], 1.0
    for li in range(LAYERS):
        ref, ridx, _, _, logits = orc.moe_layer(hosts[li % 2], ref, SHAPE.topk, SHAPE.eps, np.float64)
        ref_idx.append(ridx[0])
        margin = min(margin, float(orc.route_margin(logits, SHAPE.experts, SHAPE.topk)[0]))
    sd = MoeStackDecoder([devs[li % 2] for li in range(LAYERS)], st=st)
    sd.capture()
    sd.set_x(x)
    y = sd.step()
    idx, _ = sd.routing()
    diff = y.astype(np.float64) - ref[0]
    scale = float(np.abs(ref).max())
    return {"what": f"{LAYERS}-layer persistent stack (2 host layers alternating) against the fp64 oracle",
            "routing_bit_exact_layers": int((idx == np.stack(ref_idx)).all(axis=1).sum()), "layers": LAYERS,
            "max_abs": float(np.abs(diff).max()), "rel_l2": float(np.linalg.norm(diff) / np.linalg.norm(ref[0])),
            "output_scale": scale, "max_abs_over_scale": float(np.abs(diff).max() / scale), "smallest_routing_margin": margin}


def prefill_extra(torch, layers, st, ext_stream) -> dict:
    """Benchmark configuration 3 on this GPU: 300 rows through one MoE layer, Zipf(1.1) expert popularity. The library's
    own sequence (seven launches, no library GEMM) from a graph, its two grouped tensor-core GEMMs alone, and the
    reference's call sequence (src/engine.rs:544-604) with host rows in. Four layers are rotated so the expert weights
    come from HBM."""
    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import DevBuf, Graph, check, launched

    rows = 300
    x = synth.make_x(33, rows, SHAPE.hidden)
    bias = synth.zipf_router_bias(33, SHAPE.experts, 1.1)
    pres = [MoePrefill(ly, rows, st=st) for ly in layers[:4]]
    y0 = None
    for p in pres:
        y = p.run(x, logit_bias=bias)
        y0 = y if y0 is None else y0
    counts = pres[0].counts.download(np.int32, SHAPE.experts, st)
    hit = int((counts > 0).sum())
    x_keep = DevBuf.from_array(x.astype(np.float32), st)
    graphs = []
    for p in pres:

        def record(p=p):
            check(p.l.dr_d2d(p.x.at(0), x_keep.at(0), rows * SHAPE.hidden * 4, st.raw), "d2d")
            p.run_device(rows)

        graphs.append(Graph(st, record))
    us_graph = time_on_stream(torch, st, ext_stream, lambda i: graphs[i % len(graphs)].launch(st), 40)

    def grouped(i):
        p = pres[i % len(pres)]
        ly = p.layer
        gq, gs = ly.gate_up.expert(0)
        dq, ds = ly.down.expert(0)
        sgq, sgs = ly.shared_gate_up.rows(0)
        sdq, sds = ly.shared_down.rows(0)
        launched(p.l.drb_moe_prefill_block(gq, gs, dq, ds, sgq, sgs, sdq, sds, p.hn_b.at(0), p.row_of.at(0), p.offsets.at(0), p.counts.at(0),
                                           p.ap.at(0), p.yp.at(0), p.sh_act_b.at(0), p.sh_out.at(0), rows, SHAPE.experts, SHAPE.hidden,
                                           SHAPE.inter, 1, NULL, st.raw), "moe_prefill_block", debug=False)

    us_grouped = time_on_stream(torch, st, ext_stream, grouped, 40)
    refs = [MoePrefill(ly, rows, st=st, reference_calls=True) for ly in layers[:4]]

    def full(i):
        p = refs[i % len(refs)]
        p.x.upload(x, st)  # 2.4 MB of host rows in: the block is in place, so every call needs fresh input
        p.run_device(rows)

    for p in refs:
        p.run(x, logit_bias=bias)
    us_full = time_on_stream(torch, st, ext_stream, full, 20)
    wbytes = hit * SHAPE.expert_bytes + SHAPE.shared_bytes
    flops = 2.0 * rows * (SHAPE.topk + 1) * 3 * SHAPE.hidden * SHAPE.inter
    tf_peak = float(peaks_json().get("bf16_tflops", 1590.0))
    hbm_peak = peaks()[0]
    return {
        "workload": "prefill_300rows_zipf1.1_one_layer", "rows": rows, "experts_hit": hit, "max_group": int(counts.max()),
        "output_sum": float(y0.astype(np.float64).sum()),
        "rows_per_s": rows / us_graph * 1e6, "us_layer_device_graph": us_graph, "launches_per_layer": 7,
        "sequence": "rmsnorm_f16, router_logits_f16, moe_topk, moe_group, 2 x grouped tcgen05 GEMM (routed int4 + shared int8), combine",
        "rows_per_s_reference_call_sequence": rows / us_full * 1e6, "us_layer_reference_call_sequence_host_rows_in": us_full,
        "grouped_gemm_us": us_grouped, "grouped_gemm_rows_per_s": rows / us_grouped * 1e6,
        "grouped_gemm_includes": "8 routed experts per row and the shared expert (both GEMMs)",
        "grouped_gemm_tflops": flops / us_grouped / 1e6, "tensor_pipe_frac_of_measured_bf16_peak": flops / us_grouped / 1e6 / tf_peak,
        "grouped_gemm_hbm_gbs": wbytes / us_grouped / 1e3, "hbm_frac_of_measured": wbytes / us_grouped / 1e3 / hbm_peak,
        "binding_bound": "hbm (33 FLOP/B against a ridge of ~213)",
    }


def fp8_extra(torch, layers, st, ext_stream) -> dict:
    """Batch-1 decode with block-FP8 routed experts (dr_moe_decode_fp8): eight layers in one graph, the router, norm
    and shared expert of the int4 layers, E4M3 codes and block scales generated on the device (uniform codes below
    2^5, scales ~1e-4). 8 x 28 MB of selected rows per step: more than L2, so the rows stream from HBM."""
    from drama_rs_b200.engine import MoeDecoder
    from drama_rs_b200.gpu import ExtBuf
    from drama_rs_b200.model import Fp8Experts

    n_layers = min(8, len(layers))
    h, i, e = SHAPE.hidden, SHAPE.inter, SHAPE.experts
    g = torch.Generator(device="cuda")
    g.manual_seed(88)
    f8s, keep = [], []
    for _ in range(n_layers):
        t = []
        for n, k in ((2 * i, h), (h, i)):
            code = torch.randint(0, 0x60, (e, n, k), dtype=torch.uint8, device="cuda", generator=g)
            sign = torch.randint(0, 2, (e, n, k), dtype=torch.uint8, device="cuda", generator=g) << 7
            w = code | sign
            sc = (torch.rand((e, n // 128, k // 128), device="cuda", generator=g) + 0.5) * 1e-4
            t += [w, sc.float().contiguous()]
        keep.append(t)
        f8s.append(Fp8Experts(ExtBuf(t[0].data_ptr(), t[0].numel()), ExtBuf(t[1].data_ptr(), t[1].numel() * 4),
                              ExtBuf(t[2].data_ptr(), t[2].numel()), ExtBuf(t[3].data_ptr(), t[3].numel() * 4), e, h, i))
    torch.cuda.synchronize()
    dec = MoeDecoder(layers[:n_layers], st=st, fp8=f8s)
    x0 = synth.make_x(99, 1, h)[0]
    dec.set_x(x0)
    dec.capture()
    us = time_on_stream(torch, st, ext_stream, lambda k: dec.graph.launch(st), 100) / n_layers
    y = dec.x.download(np.float32, h, st)
    layer_bytes = SHAPE.router_bytes + SHAPE.topk * (3 * h * i + 4 * ((2 * i // 128) * (h // 128) + (h // 128) * (i // 128))) + SHAPE.shared_bytes
    gbs = layer_bytes / us / 1e3
    # Prefill over the same FP8 experts (dr_moe_prefill_fp8): the grouping of configuration 3 (300 rows, Zipf 1.1), the
    # layers' FP8 tensors rotated so that the weights stream from HBM.
    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import launched

    rows = 300
    pre = MoePrefill(layers[0], rows, st=st, reference_calls=True)
    pre.run(synth.make_x(33, rows, h), logit_bias=synth.zipf_router_bias(33, e, 1.1))  # leaves xp, offsets, counts behind
    hit = int((pre.counts.download(np.int32, e, st) > 0).sum())
    lib = pre.l

    def grouped(k):
        f8 = f8s[k % n_layers]
        launched(lib.dr_moe_prefill_fp8(f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), pre.xp.at(0), pre.offsets.at(0),
                                        pre.counts.at(0), pre.ap.at(0), pre.yp.at(0), e, h, i, st.raw), "moe_prefill_fp8", debug=False)

    us_pf = time_on_stream(torch, st, ext_stream, grouped, 40)
    pf_bytes = hit * (3 * h * i + 4 * ((2 * i // 128) * (h // 128) + (h // 128) * (i // 128)))
    yp = pre.yp.download(np.float32, rows * SHAPE.topk * h, st)
    del keep
    return {"workload": f"decode_stack{n_layers}_b1_fp8_experts", "us_per_layer": us, "algorithmic_bytes_per_layer": layer_bytes,
            "hbm_gbs": gbs, "frac_of_measured_hbm": gbs / peaks()[0], "finite": bool(np.isfinite(y).all()),
            "prefill_300rows_grouped_gemm_us": us_pf, "prefill_experts_hit": hit, "prefill_hbm_gbs": pf_bytes / us_pf / 1e3,
            "prefill_frac_of_measured_hbm": pf_bytes / us_pf / 1e3 / peaks()[0], "prefill_finite": bool(np.isfinite(yp).all())}


def gemv_extra(torch, st, ext_stream, lib, what: str = "this library") -> list:
    """Benchmark configuration 1: int8 GEMV sweep, batch 1; >= 8 copies of each matrix rotated per launch so the reads
    come from HBM, not L2 (the method of the reference's bench/gemv_bench.cu:49-55). The rotated launches of a shape
    are captured in ONE CUDA graph and the graph is replayed (a captured chain, as bench/pf_bench.cu times it): what is
    timed is the kernels, not the host's launch rate."""
    from drama_rs_b200.gpu import Graph, launched

    hbm_peak = peaks()[0]
    out = []
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    for n, k in ((4096, 2048), (2048, 4096), (8192, 2048), (151936, 2048)):
        copies = max(8, int(1.5e9 // (n * k)) if n * k < 2e8 else 8)
        w = torch.randint(-127, 128, (copies, n, k), dtype=torch.int8, device="cuda", generator=g)
        s = (torch.randn((copies, n, 1), device="cuda", generator=g) * 0.005).abs().clamp_min(1e-4).half().expand(copies, n, k // 128).contiguous()
        x = torch.randn(k, device="cuda", generator=g).bfloat16().float()
        y = torch.empty(n, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        wb, sb = n * k, n * (k // 128) * 2
        launches = max(64, copies)

        def record(w=w, s=s, x=x, y=y, n=n, k=k, wb=wb, sb=sb, copies=copies, launches=launches):
            for i in range(launches):
                c = i % copies
                launched(lib.dr_gemv_q8(C.c_void_p(w.data_ptr() + c * wb), C.c_void_p(s.data_ptr() + c * sb), C.c_void_p(x.data_ptr()),
                                        None, C.c_void_p(y.data_ptr()), n, k, None, 0.0, None, 0, st.raw), "gemv_q8", debug=False)

        record()  # per-device setup happens outside the capture
        st.sync()
        graph = Graph(st, record)
        us = time_on_stream(torch, st, ext_stream, lambda i: graph.launch(st), 10, warm=3) / launches
        gbs = (wb + sb) / us / 1e3
        out.append({"n": n, "k": k, "us": us, "gbs": gbs, "frac_of_measured_hbm": gbs / hbm_peak, "copies_rotated": copies,
                    "launches_per_graph": launches, "by": what})
        graph.destroy()
        del w, s
        torch.cuda.empty_cache()
    return out


def reference_cuda_extra(torch, layers, st, ext_stream) -> dict | None:
    """The reference's own kernels/drama.cu, compiled unchanged for sm_100 as a checker library, timed on the same
    buffers with the same graph method: the 40-layer decode step, the four GEMVs, and its prefill call sequence.
    Checker code: it never enters the headline region; it is here so that the ratio to the reference's kernels on
    the same GPU is a measured figure."""
    if not os.path.exists(REF_LIB):
        return None
    from drama_rs_b200 import ffi
    from drama_rs_b200.engine import MoeDecoder, MoePrefill
    from drama_rs_b200.gpu import Graph, check

    ref = ffi.bind(REF_LIB)
    own = ffi.lib()
    dec = MoeDecoder(layers, st=st, lib=ref)
    x0 = synth.make_x(99, 1, SHAPE.hidden)[0]
    dec.set_x(x0)
    dec.step_eager()
    keep = torch.from_numpy(x0).cuda()

    def rec():
        check(own.dr_d2d(dec.x.at(0), C.c_void_p(keep.data_ptr()), SHAPE.hidden * 4, st.raw), "d2d")
        dec.record_step()

    g = Graph(st, rec)
    us_decode = time_on_stream(torch, st, ext_stream, lambda i: g.launch(st), 50) / len(layers)
    g.destroy()
    out = {"library": "oracle/_ref/libdrama_ref.so (kernels/drama.cu compiled with nvcc -arch=sm_100, unchanged)",
           "decode_us_per_layer": us_decode, "gemv_q8_sweep": gemv_extra(torch, st, ext_stream, ref, "reference kernels")}
    try:
        rows = 300
        x = synth.make_x(33, rows, SHAPE.hidden)
        bias = synth.zipf_router_bias(33, SHAPE.experts, 1.1)
        pres = [MoePrefill(ly, rows, st=st, reference_calls=True, lib=ref) for ly in layers[:4]]
        for p in pres:
            p.run(x, logit_bias=bias)

        def full(i):
            p = pres[i % len(pres)]
            p.x.upload(x, st)
            p.run_device(rows)

        def grouped(i):
            p = pres[i % len(pres)]
            gq, gs = p.layer.gate_up.expert(0)
            dq, ds = p.layer.down.expert(0)
            ref.dr_moe_prefill(gq, gs, dq, ds, p.xp.at(0), p.offsets.at(0), p.counts.at(0), p.ap.at(0), p.yp.at(0), SHAPE.experts,
                               SHAPE.hidden, SHAPE.inter, st.raw)

        out["prefill_us_layer_call_sequence_host_rows_in"] = time_on_stream(torch, st, ext_stream, full, 10)
        out["prefill_grouped_gemm_us"] = time_on_stream(torch, st, ext_stream, grouped, 10)
    except Exception as exc:  # noqa: BLE001 - the decode and GEMV figures stand without it
        out["prefill_error"] = f"{type(exc).__name__}: {exc}"
    return out


def _ep_time(torch, dist, world, ext_stream, stream, step, restore, iters: int) -> tuple[float, bool]:
    """Device time of step() in us (max over ranks). The step is captured in a CUDA graph (collectives included)
    when capture works; restore() puts the input back and runs inside the timed region either way."""
    restore()
    step()
    torch.cuda.synchronize()
    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        restore()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            step()
        graph = g
    except Exception as exc:  # noqa: BLE001 - the eager sequence is the same work
        sys.stderr.write(f"bench: expert-parallel graph capture failed ({type(exc).__name__}: {exc}); timing eager launches\n")
    run = graph.replay if graph is not None else step
    for _ in range(3):
        restore()
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext_stream)
    for _ in range(iters):
        restore()
        run()
    e1.record(ext_stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    graphed = graph is not None
    # a live graph that holds captured collectives keeps the communicator busy at shutdown: drop it here
    del graph, run
    torch.cuda.synchronize()
    return float(t[0]), graphed


def _reduce(torch, dist, world, vals, op="max"):
    t = torch.tensor(vals, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN if op == "min" else dist.ReduceOp.SUM)
    torch.cuda.synchronize()
    return t.cpu().tolist()


def prefill_ep_extra(torch, dist, layer, st, ext_stream, rank: int, world: int) -> dict:
    """Configuration 3 expert-parallel: the 300 rows are split over the ranks, every rank owns 256 / N experts of
    the (identical) layer, rows travel to their experts and back with two all-to-alls of fixed size
    (drama_rs_b200/ep.py; the layer replays from a CUDA graph). Timed on the device with events on every rank; max over
    ranks. Every rank's routing and rows are compared with the single-GPU block (every rank holds the whole layer)."""
    from drama_rs_b200 import ep
    from drama_rs_b200.engine import MoePrefill

    rows = 300
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    max_rows = -(-rows // world)
    cap = ep.capacity(max_rows, SHAPE.topk, world)
    x_all = synth.make_x(33, rows, SHAPE.hidden)
    bias = synth.zipf_router_bias(33, SHAPE.experts, 1.1)
    ops = ep.EpGpu(layer, rank, world, max_rows, cap, st=st)
    with torch.cuda.stream(ops.stream):
        ops.logit_bias = torch.from_numpy(bias).cuda()
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()
        single = MoePrefill(layer, rows, st=st)
        ref = single.run(x_all, logit_bias=bias)[lo:hi]
        ref_idx = single.idx.download(np.int32, rows * SHAPE.topk, st).reshape(rows, SHAPE.topk)[lo:hi]
        ep.ep_moe_block(x, ops, cap)
        torch.cuda.synchronize()
        idx_equal = bool(np.array_equal(ops.idx[: hi - lo].cpu().numpy(), ref_idx))
        diff_eager = float(np.abs(x.cpu().numpy() - ref).max())
        us, graphed = _ep_time(torch, dist, world, ext_stream, ops.stream, lambda: ep.ep_moe_block(x, ops, cap), lambda: x.copy_(x0), 20)
        diff_graph = float(np.abs(x.cpu().numpy() - ref).max())
        over = ops.overflow()
        d = _reduce(torch, dist, world, [diff_eager, diff_graph, float(np.abs(ref).max()), float(over), float(not idx_equal)])
        cs = _reduce(torch, dist, world, [float(x.double().sum())], "sum")
    return {"workload": "prefill_300rows_zipf1.1_one_layer_expert_parallel", "rows": rows, "experts_per_rank": SHAPE.experts // world,
            "us_layer": us, "rows_per_s": rows / us * 1e6, "output_sum": cs[0], "cuda_graph": graphed,
            "routing_equals_single_gpu_on_every_rank": d[4] == 0.0,
            "max_abs_diff_to_single_gpu": {"eager": d[0], "graph_replay": d[1], "output_scale": d[2]},
            "capacity_slots_per_peer": cap, "capacity_worst_case": max_rows * SHAPE.topk, "overflow": bool(d[3]),
            "exchange": f"2 fixed-size exchanges per layer (fp16 rows + expert ids out, f32 results back) by {ops.exchange_kind}"}


def decode64_ep_extra(torch, dist, layers, st, ext_stream, rank: int, world: int) -> dict:
    """Configuration 4: 64 independent streams, one row each, through the whole stack; experts sharded 256 / N per GPU;
    per layer one all-to-all out and one back (uniform routing, no bias); the whole 40-layer step is one CUDA graph.
    The first two layers are also run over two host-generated layers and compared with the fp64 oracle on this rank's
    rows (routing index by index where the oracle's margin is decidable in fp16 rows, outputs to the prefill bar)."""
    from drama_rs_b200 import ep
    from drama_rs_b200.model import MoeLayer
    from oracle import moe_oracle as orc

    rows = 64
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    max_rows = -(-rows // world)
    cap = ep.capacity(max_rows, SHAPE.topk, world)
    x_all = synth.make_x(64, rows, SHAPE.hidden)
    ops = ep.EpGpu(layers[0], rank, world, max_rows, cap, st=st)
    with torch.cuda.stream(ops.stream):
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()

        def step():
            for ly in layers:
                ops.layer = ly
                ep.ep_moe_block(x, ops, cap)

        us, graphed = _ep_time(torch, dist, world, ext_stream, ops.stream, step, lambda: x.copy_(x0), 5)
        finite = bool(torch.isfinite(x).all())
        over = ops.overflow()
        # oracle check: two layers of host-generated weights
        hosts = host_layers()
        devs = [MoeLayer.upload(h, st) for h in hosts]
        x.copy_(x0)
        ref = x_all[lo:hi].astype(np.float64)
        idx_ok, rel = True, 0.0
        for li in range(2):
            ops.layer = devs[li]
            ep.ep_moe_block(x, ops, cap)
            torch.cuda.synchronize()
            xh = orc.rmsnorm(ref, hosts[li]["post_norm"], SHAPE.eps, np.float64).astype(np.float16).astype(np.float64)
            out, oidx, _, _, logits = orc.moe_block(hosts[li], xh, SHAPE.topk, np.float64)
            safe = orc.route_margin(logits, SHAPE.experts, SHAPE.topk) > 1e-5
            got = ops.idx[: hi - lo].cpu().numpy()
            idx_ok = idx_ok and bool(np.array_equal(got[safe], oidx[safe]))
            ref = ref + out
            y = x.cpu().numpy().astype(np.float64)
            rel = max(rel, float(np.linalg.norm(y - ref) / np.linalg.norm(ref)))
            ref = y  # carry the device's state so that the second layer is checked on its own
        d = _reduce(torch, dist, world, [rel, float(not idx_ok), float(over), float(not finite)])
    return {"workload": "decode_64streams_stack_expert_parallel", "streams": rows, "layers": len(layers),
            "us_per_step": us, "us_per_layer": us / len(layers), "cuda_graph": graphed,
            "stream_layers_per_s": rows * len(layers) / us * 1e6, "finite": d[3] == 0.0, "overflow": bool(d[2]),
            "capacity_slots_per_peer": cap,
            "oracle_check_first_2_layers": {"routing_equal_where_decidable": d[1] == 0.0, "max_rel_l2_over_ranks": d[0]}}


def run_gpu(args) -> None:
    import torch

    from drama_rs_b200 import ffi
    from drama_rs_b200.engine import MoeDecoder, MoeStackDecoder
    from drama_rs_b200.gpu import Graph, Stream, check

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = ffi.lib()  # raises if the CUDA library is missing: there is no fallback
    st = Stream()
    ext_stream = torch.cuda.ExternalStream(st.raw.value)
    layers = device_layers(torch, args.layers, 1234, st)  # the same seed on every rank: replicas for decode, shards for the expert-parallel legs
    x0 = synth.make_x(99, 1, SHAPE.hidden)[0]
    x0_dev = torch.from_numpy(x0).cuda()
    hidden_bytes = SHAPE.hidden * 4

    # Headline: the whole stack as one persistent kernel per step. Device-resident step: restore the step's input with
    # a device copy, then the kernel.
    sd = MoeStackDecoder(layers, st=st)
    sd.set_x(x0)
    sd.step()  # per-device setup outside the capture

    def record():
        check(lib.dr_d2d(sd.x.at(0), C.c_void_p(x0_dev.data_ptr()), hidden_bytes, st.raw), "d2d")
        sd.launch()

    graph = Graph(st, record)
    sd.capture()  # the public step: the kernel only; x comes from the host each step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.launch(st)
    st.sync()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clocks:
        ev0.record(ext_stream)
        for _ in range(args.steps):
            graph.launch(st)
        ev1.record(ext_stream)
        st.sync()
        barrier()
        ms = ev0.elapsed_time(ev1)
        # keep the sampler alive long enough to see the loaded clocks
        if ms < 300:
            t_end = time.perf_counter() + 0.4
            while time.perf_counter() < t_end:
                graph.launch(st)
            st.sync()
    y_resident = sd.x.download(np.float32, SHAPE.hidden, st)

    # The per-layer entry points of the reference's ABI on the same layers (dr_router_topk + dr_moe_decode per layer,
    # src/engine.rs:959-1042): what a host that keeps the reference's call sites gets.
    per_layer = MoeDecoder(layers, st=st)

    def record_pl():
        check(lib.dr_d2d(per_layer.x.at(0), C.c_void_p(x0_dev.data_ptr()), hidden_bytes, st.raw), "d2d")
        per_layer.record_step()

    per_layer.set_x(x0)
    per_layer.step_eager()
    pl_graph = Graph(st, record_pl)
    pl_us = time_on_stream(torch, st, ext_stream, lambda i: pl_graph.launch(st), args.steps) / args.layers
    y_pl = per_layer.x.download(np.float32, SHAPE.hidden, st)
    pl_info = {"sequence": "dr_router_topk + dr_moe_decode per layer (src/engine.rs:959-1042), one CUDA graph of 3 kernels per layer",
               "us_per_layer": pl_us, "max_abs_diff_to_persistent_kernel": float(np.abs(y_pl - y_resident).max()),
               "hidden_state_scale": float(np.abs(y_resident).max())}

    # End to end through the public call: pinned host x -> device, graph, device -> pinned host.
    hx = torch.from_numpy(x0).pin_memory()
    hy = torch.empty(SHAPE.hidden, dtype=torch.float32).pin_memory()

    def e2e_step():
        check(lib.dr_h2d(sd.x.at(0), C.c_void_p(hx.data_ptr()), hidden_bytes, st.raw), "h2d")
        sd.graph.launch(st)
        check(lib.dr_d2h(C.c_void_p(hy.data_ptr()), sd.x.at(0), hidden_bytes, st.raw), "d2h")
        st.sync()

    for _ in range(max(args.warmup, 3)):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext_stream)
    for _ in range(args.steps):
        e2e_step()
    e1.record(ext_stream)
    st.sync()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    assert np.array_equal(hy.numpy(), y_resident), "the host-buffer step and the resident step disagree"
    assert np.isfinite(y_resident).all()

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    word = C.c_uint(0)
    lib.drb_device_error(C.byref(word))
    ep_info = ep_info64 = None
    if not args.no_extras and set(args.extras.split(",")) & {"all", "ep"}:
        ep_info = prefill_ep_extra(torch, dist, layers[0], st, ext_stream, rank, world)
        ep_info64 = decode64_ep_extra(torch, dist, layers, st, ext_stream, rank, world)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    step_ms = ms / args.steps
    us_layer = step_ms * 1e3 / args.layers
    layer_bytes = SHAPE.decode_layer_bytes
    step_bytes = layer_bytes * args.layers
    gbs = step_bytes / (step_ms * 1e-3) / 1e9
    peak, peak_kind = peaks()
    e2e_us = ms_e2e / args.steps * 1e3 / args.layers
    traffic, traffic_source = None, "no ncu capture summary at profiles/decode_stack_traffic.json"
    try:
        tj = json.load(open(TRAFFIC_JSON))
        traffic = float(tj["dram_bytes_per_layer"]) * args.layers
        traffic_source = tj["source"]
    except Exception:
        pass
    line = {
        "metric": "int4_moe_decode_us_per_layer", "value": us_layer, "unit": "us/layer", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": False,
        "scaling": "weak (N independent replicas of the batch-1 stack, no collective: batch-1 decode does not shard; the sharded path is under ep_scaling)",
        "vs_baseline": None, "dtype": "int4/int8 weights x 21-bit block-fixed activations (dp4a, exact int32) -> f32", "data": "synthetic",
        "config": {"workload": "decode_stack40_b1", "layers": args.layers, "hidden": SHAPE.hidden, "experts": SHAPE.experts,
                   "topk": SHAPE.topk, "inter": SHAPE.inter, "weights": "int4 g64 (scale,min) routed + int8 g128 shared",
                   "graph": "one CUDA graph per step: one persistent cooperative kernel for the 40 layers (drb_moe_stack_decode)",
                   "replicas": world,
                   "cache": "inputs larger than L2: 736 MB of weights read per step, 18.1 GB resident"},
        "hbm_gbs": gbs,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "kernel": "stack::k_moe_stack (one launch = 40 layers)",
                     "algorithmic_bytes_per_launch": step_bytes, "traffic": traffic, "traffic_source": traffic_source},
        "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": hidden_bytes, "d2h_bytes_per_step": hidden_bytes},
        "gpu_launches": args.steps,
        "clocks": clocks.summary(),
        "device_error_word": int(word.value),
        "decode_per_layer_abi": pl_info,
    }
    if ep_info is not None:
        line["ep_scaling"] = {"n_gpus": world, "prefill_300rows": ep_info, "decode_64streams": ep_info64}
    want = set(args.extras.split(","))
    if not args.no_extras:
        def extra(key, fn):
            """An extra leg's failure is reported under its key; the headline figures above are already measured."""
            try:
                line[key] = fn()
            except Exception as exc:  # noqa: BLE001
                line[key] = {"error": f"{type(exc).__name__}: {exc}"}

        if want & {"all", "parity"}:
            extra("parity_check", lambda: parity_check(st))
        if want & {"all", "prefill"}:
            extra("prefill", lambda: prefill_extra(torch, layers, st, ext_stream))
        if want & {"all", "gemv"}:
            extra("gemv_q8_sweep", lambda: gemv_extra(torch, st, ext_stream, lib))
        if want & {"all", "fp8"}:
            extra("decode_fp8", lambda: fp8_extra(torch, layers, st, ext_stream))
        if world == 1 and want & {"all", "reference"}:
            try:
                r = reference_cuda_extra(torch, layers, st, ext_stream)
            except Exception as exc:  # noqa: BLE001 - a checker's failure must not take the bench line with it
                r = {"error": f"{type(exc).__name__}: {exc}"}
            if r is not None:
                if "decode_us_per_layer" in r:
                    r["ratio_decode_reference_kernels_over_this_library"] = r["decode_us_per_layer"] / us_layer
                line["reference_cuda_sm100"] = r
    if not args.no_cpu and world == 1:  # the CPU baseline is a single-GPU-run figure (torchrun also pins OMP to one thread)
        line["cpu_baseline"] = cpu_decode_baseline()
    emit(line)
    if world > 1:
        dist.destroy_process_group()


_RESULT_FD = None


def keep_stdout_for_the_result() -> None:
    """Libraries write to file descriptor 1 behind Python's back (NCCL prints its version there): everything but the
    result line goes to stderr, the line itself to the descriptor stdout had when the program started."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main() -> None:
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip everything but the headline decode step")
    ap.add_argument("--extras", default="all", help="comma list of the extra legs to run: ep, parity, prefill, gemv, fp8, reference "
                                                    "(default all); small profiling cases pick one")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
