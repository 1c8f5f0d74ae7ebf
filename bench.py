#!/usr/bin/env python3
"""Benchmark of the routed-expert MoE decode path on B200.

    python bench.py --gpus 1 --steps K --warmup W             # this library
    python bench.py --impl reference --steps K --warmup W     # the CPU implementation, host cores

Workload ("decode_stack40_b1"): the full 40-layer MoE stack decode step at batch 1 — per layer the
bf16 router over 256 experts with fused RMSNorm and top-8, the 8 chosen int4 experts (SwiGLU
gate/up then down), the int8 shared expert with its sigmoid gate, and the residual — captured as one
CUDA graph through the library's C ABI and replayed once per step on the same input. 18.1 GB of
expert weights are resident; one step reads 736 MB of them, far more than the 126 MB L2, so every
step streams from HBM. Inputs are synthetic from a seed (there is no dataset on this path).

One JSON line is printed by rank 0. `value` is microseconds per layer with everything resident in
HBM; `e2e` is the same through the public call with host buffers (pinned host x in, host x out,
copies inside the timed region).
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


def peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
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


def cpu_decode_baseline(budget_s: float = 15.0) -> dict:
    """The plain-C restatement of the reference's decode layer on the host cores, all OpenMP threads,
    on a bounded sample of the workload: two distinct seeded config-0 layers applied alternately."""
    from oracle import c_oracle

    layers = [synth.make_layer(1000 + i, SHAPE) for i in range(2)]
    structs = [c_oracle.layer_struct(t, SHAPE.topk, SHAPE.eps) for t in layers]
    x0 = synth.make_x(1000, 1, SHAPE.hidden)[0]
    lib = c_oracle.lib()
    x = x0.copy()
    for s in structs:  # warm-up
        lib.orc_moe_decode_layer(C.byref(s), x.ctypes.data, None, None)
    times = []
    t_end = time.perf_counter() + budget_s
    while time.perf_counter() < t_end and len(times) < 2000:
        x[:] = x0
        t0 = time.perf_counter()
        for s in structs:
            lib.orc_moe_decode_layer(C.byref(s), x.ctypes.data, None, None)
        times.append((time.perf_counter() - t0) / len(structs))
    us = float(np.median(times) * 1e6)
    return {"value": us, "unit": "us/layer", "cores": int(lib.orc_threads()), "kind": "port",
            "sample": f"{len(times) * len(structs)} single-layer decode calls over 2 seeded config-0 layers (median)"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = []
    from oracle import c_oracle

    layers = [synth.make_layer(1000 + i, SHAPE) for i in range(2)]
    structs = [c_oracle.layer_struct(t, SHAPE.topk, SHAPE.eps) for t in layers]
    lib = c_oracle.lib()
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is the CPU path with every host thread
    lib.orc_set_threads.argtypes = [C.c_int]
    lib.orc_set_threads.restype = None
    lib.orc_set_threads(len(os.sched_getaffinity(0)))
    x0 = synth.make_x(1000, 1, SHAPE.hidden)[0]
    x = x0.copy()
    sample_layers = 8  # one step of the reference arm = 8 layers of the 40-layer stack (bounded sample)

    def step():
        x[:] = x0
        for i in range(sample_layers):
            lib.orc_moe_decode_layer(C.byref(structs[i % 2]), x.ctypes.data, None, None)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    us = dt / args.steps / sample_layers * 1e6
    cores = int(lib.orc_threads())
    line = {
        "impl": "reference", "metric": "int4_moe_decode_us_per_layer", "value": us, "unit": "us/layer", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "decode_stack40_b1", "layers_per_step": sample_layers, "hidden": SHAPE.hidden,
                   "experts": SHAPE.experts, "topk": SHAPE.topk, "inter": SHAPE.inter},
        "cpu_baseline": {"value": us, "unit": "us/layer", "cores": cores, "kind": "port",
                         "sample": f"each step = {sample_layers} layers of the stack (2 seeded layers alternating), plain-C "
                                   f"restatement of the reference kernels, OpenMP over {cores} threads"},
        "e2e": {"value": us, "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


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


def prefill_extra(torch, layers, st, ext_stream) -> dict:
    """Benchmark configuration 3 on this GPU: 300 rows through one MoE layer, Zipf(1.1) expert popularity,
    the reference's call sequence (src/engine.rs:544-604) with the expert-grouped tcgen05 GEMMs inside.
    Four layers are rotated so the expert weights come from HBM."""
    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import launched

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

    def full(i):
        p = pres[i % len(pres)]
        p.x.upload(x, st)  # 2.4 MB of host rows in: the block is in place, so every call needs fresh input
        p.run_device(rows)

    def grouped(i):
        p = pres[i % len(pres)]
        gq, gs = p.layer.gate_up.expert(0)
        dq, ds = p.layer.down.expert(0)
        launched(p.l.dr_moe_prefill(gq, gs, dq, ds, p.xp.at(0), p.offsets.at(0), p.counts.at(0), p.ap.at(0), p.yp.at(0),
                                    SHAPE.experts, SHAPE.hidden, SHAPE.inter, st.raw), "moe_prefill")

    us_full = time_on_stream(torch, st, ext_stream, full, 20)
    # The same layer with the offsets scanned on the device, captured once: rows restored by a device copy inside
    # the graph, no host round trip between the launches.
    from drama_rs_b200.gpu import DevBuf, Graph, check

    x_keep = DevBuf.from_array(x.astype(np.float32), st)
    graphs = []
    for p in pres:
        p.device_scan = True

        def record(p=p):
            check(p.l.dr_d2d(p.x.at(0), x_keep.at(0), rows * SHAPE.hidden * 4, st.raw), "d2d")
            p.run_device(rows)

        graphs.append(Graph(st, record))
    us_graph = time_on_stream(torch, st, ext_stream, lambda i: graphs[i % len(graphs)].launch(st), 40)
    for p in pres:
        p.device_scan = False
    us_grouped = time_on_stream(torch, st, ext_stream, grouped, 40)
    wbytes = hit * SHAPE.expert_bytes
    flops = 2.0 * rows * SHAPE.topk * 3 * SHAPE.hidden * SHAPE.inter
    peaks_json = {}
    try:
        peaks_json = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    tf_peak = float(peaks_json.get("bf16_tflops", 1590.0))
    hbm_peak = peaks()[0]
    return {
        "workload": "prefill_300rows_zipf1.1_one_layer", "rows": rows, "experts_hit": hit, "max_group": int(counts.max()),
        "output_sum": float(y0.astype(np.float64).sum()),
        "rows_per_s": rows / us_graph * 1e6, "us_layer_device_graph": us_graph,
        "rows_per_s_reference_call_sequence": rows / us_full * 1e6, "us_layer_reference_call_sequence_host_rows_in": us_full,
        "grouped_gemm_us": us_grouped, "grouped_gemm_rows_per_s": rows / us_grouped * 1e6,
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
    del keep
    return {"workload": f"decode_stack{n_layers}_b1_fp8_experts", "us_per_layer": us, "algorithmic_bytes_per_layer": layer_bytes,
            "hbm_gbs": gbs, "frac_of_measured_hbm": gbs / peaks()[0], "finite": bool(np.isfinite(y).all())}


def gemv_extra(torch, st, ext_stream) -> list:
    """Benchmark configuration 1: int8 GEMV sweep, batch 1; >= 8 copies of each matrix rotated per launch so
    the reads come from HBM, not L2 (the method of the reference's bench/gemv_bench.cu:49-55)."""
    from drama_rs_b200 import ffi
    from drama_rs_b200.gpu import launched

    lib = ffi.lib()
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

        def call(i, w=w, s=s, x=x, y=y, n=n, k=k, wb=wb, sb=sb, copies=copies):
            c = i % copies
            launched(lib.dr_gemv_q8(C.c_void_p(w.data_ptr() + c * wb), C.c_void_p(s.data_ptr() + c * sb), C.c_void_p(x.data_ptr()),
                                    None, C.c_void_p(y.data_ptr()), n, k, None, 0.0, None, 0, st.raw), "gemv_q8", debug=False)

        us = time_on_stream(torch, st, ext_stream, call, 64, warm=8)
        gbs = (wb + sb) / us / 1e3
        out.append({"n": n, "k": k, "us": us, "gbs": gbs, "frac_of_measured_hbm": gbs / hbm_peak, "copies_rotated": copies})
        del w, s
        torch.cuda.empty_cache()
    return out


def _ep_time(torch, dist, ext_stream, stream, step, restore, iters: int) -> tuple[float, bool]:
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
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext_stream)
    for _ in range(iters):
        restore()
        run()
    e1.record(ext_stream)
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    graphed = graph is not None
    # a live graph that holds captured collectives keeps the communicator busy at shutdown: drop it here
    del graph, run
    torch.cuda.synchronize()
    return float(t[0]), graphed


def prefill_ep_extra(torch, dist, layer, st, ext_stream, rank: int, world: int) -> dict:
    """Configuration 3 expert-parallel: the 300 rows are split over the ranks, every rank owns 256 / N experts of
    the (identical) layer, rows travel to their experts and back with NCCL all-to-all at a fixed capacity
    (drama_rs_b200/ep.py ep_moe_block_fixed: no size is read on the host, the layer replays from a CUDA graph).
    Timed on the device with events on every rank; max over ranks."""
    from drama_rs_b200 import ep

    rows = 300
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    max_rows = -(-rows // world)
    cap = max_rows * SHAPE.topk
    x_all = synth.make_x(33, rows, SHAPE.hidden)
    ops = ep.EpGpuFixed(layer, rank, world, max_rows, cap, st=st)
    with torch.cuda.stream(ops.stream):
        ops.logit_bias = torch.from_numpy(synth.zipf_router_bias(33, SHAPE.experts, 1.1)).cuda()
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()
        # this rank's rows through the single-GPU sequence (every rank holds the whole layer): the check for what follows
        from drama_rs_b200.engine import MoePrefill

        ref = MoePrefill(layer, rows, st=st).run(x_all, logit_bias=synth.zipf_router_bias(33, SHAPE.experts, 1.1))[lo:hi]
        ep.ep_moe_block_fixed(x, ops, SHAPE.experts, SHAPE.topk, cap)
        torch.cuda.synchronize()
        diff_eager = float(np.abs(x.cpu().numpy() - ref).max())
        us, graphed = _ep_time(torch, dist, ext_stream, ops.stream, lambda: ep.ep_moe_block_fixed(x, ops, SHAPE.experts, SHAPE.topk, cap),
                               lambda: x.copy_(x0), 20)
        diff_graph = float(np.abs(x.cpu().numpy() - ref).max())
        d = torch.tensor([diff_eager, diff_graph, float(np.abs(ref).max())], dtype=torch.float64, device="cuda")
        dist.all_reduce(d, op=dist.ReduceOp.MAX)
        # checksum of the result, summed over ranks: identical for every N when the routing and the sums are
        cs = torch.tensor([float(x.double().sum())], dtype=torch.float64, device="cuda")
        dist.all_reduce(cs)
        # read the reduced values while this stream is current: the default stream does not wait for it
        torch.cuda.synchronize()
        cs, d = cs.cpu(), d.cpu()
    return {"workload": "prefill_300rows_zipf1.1_one_layer_expert_parallel", "rows": rows, "experts_per_rank": SHAPE.experts // world,
            "us_layer": us, "rows_per_s": rows / us * 1e6, "output_sum": float(cs[0]), "cuda_graph": graphed,
            "max_abs_diff_to_single_gpu": {"eager": float(d[0]), "graph_replay": float(d[1]), "output_scale": float(d[2])},
            "exchange": f"NCCL all_to_all_single at fixed capacity ({cap} row slots per peer): bf16 rows out, f32 rows back"}


def decode64_ep_extra(torch, dist, layers, st, ext_stream, rank: int, world: int) -> dict:
    """Configuration 4: 64 independent streams, one row each, through the whole stack; experts sharded
    256 / N per GPU; per layer one all-to-all out and one back (uniform routing, no bias); the whole 40-layer step
    is one CUDA graph."""
    from drama_rs_b200 import ep

    rows = 64
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    max_rows = -(-rows // world)
    cap = max_rows * SHAPE.topk
    x_all = synth.make_x(64, rows, SHAPE.hidden)
    ops = ep.EpGpuFixed(layers[0], rank, world, max_rows, cap, st=st)
    with torch.cuda.stream(ops.stream):
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()

        def step():
            for ly in layers:
                ops.layer = ly
                ep.ep_moe_block_fixed(x, ops, SHAPE.experts, SHAPE.topk, cap)

        us, graphed = _ep_time(torch, dist, ext_stream, ops.stream, step, lambda: x.copy_(x0), 5)
        finite = bool(torch.isfinite(x).all())
    return {"workload": "decode_64streams_stack_expert_parallel", "streams": rows, "layers": len(layers),
            "us_per_step": us, "us_per_layer": us / len(layers), "cuda_graph": graphed,
            "stream_layers_per_s": rows * len(layers) / us * 1e6, "finite": finite}


def run_gpu(args) -> None:
    import torch

    from drama_rs_b200 import ffi
    from drama_rs_b200.engine import MoeDecoder
    from drama_rs_b200.gpu import Stream, check

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = ffi.lib()  # raises if the CUDA library is missing: there is no fallback
    st = Stream()
    ext_stream = torch.cuda.ExternalStream(st.raw.value)
    layers = device_layers(torch, args.layers, 1234, st)  # the same seed on every rank: replicas for decode, shards for the expert-parallel legs
    chained = args.sequence == "chained"
    dec = MoeDecoder(layers, st=st, chained=chained)
    x0 = synth.make_x(99, 1, SHAPE.hidden)[0]
    x0_dev = torch.from_numpy(x0).cuda()
    hidden_bytes = SHAPE.hidden * 4

    # Device-resident step: restore the step's input with a device copy, then the 40 layers.
    def record():
        check(lib.dr_d2d(dec.x.at(0), C.c_void_p(x0_dev.data_ptr()), hidden_bytes, st.raw), "d2d")
        dec.record_step()

    from drama_rs_b200.gpu import Graph

    graph = Graph(st, record)
    dec.capture()  # the public step: graph of the layers only; x comes from the host each step

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
    y_resident = dec.x.download(np.float32, SHAPE.hidden, st)

    # The other call sequence on the same layers, for comparison (device-resident step only).
    alt = MoeDecoder(layers, st=st, chained=not chained)

    def record_alt():
        check(lib.dr_d2d(alt.x.at(0), C.c_void_p(x0_dev.data_ptr()), hidden_bytes, st.raw), "d2d")
        alt.record_step()

    alt_graph = Graph(st, record_alt)
    alt_us = time_on_stream(torch, st, ext_stream, lambda i: alt_graph.launch(st), args.steps) / args.layers
    y_alt = alt.x.download(np.float32, SHAPE.hidden, st)
    alt_info = {"sequence": "chained" if not chained else "reference", "us_per_layer": alt_us,
                "max_abs_diff_to_headline_sequence": float(np.abs(y_alt - y_resident).max()),
                "hidden_state_scale": float(np.abs(y_resident).max())}

    # End to end through the public call: pinned host x -> device, graph, device -> pinned host.
    hx = torch.from_numpy(x0).pin_memory()
    hy = torch.empty(SHAPE.hidden, dtype=torch.float32).pin_memory()

    def e2e_step():
        check(lib.dr_h2d(dec.x.at(0), C.c_void_p(hx.data_ptr()), hidden_bytes, st.raw), "h2d")
        dec.graph.launch(st)
        check(lib.dr_d2h(C.c_void_p(hy.data_ptr()), dec.x.at(0), hidden_bytes, st.raw), "d2h")
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
    if world > 1 and not args.no_extras:
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
    line = {
        "metric": "int4_moe_decode_us_per_layer", "value": us_layer, "unit": "us/layer", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4/int8 weights x 21-bit block-fixed activations (dp4a, exact int32) -> f32", "data": "synthetic",
        "config": {"workload": "decode_stack40_b1", "layers": args.layers, "hidden": SHAPE.hidden, "experts": SHAPE.experts,
                   "topk": SHAPE.topk, "inter": SHAPE.inter, "weights": "int4 g64 (scale,min) routed + int8 g128 shared",
                   "graph": "one CUDA graph per step, 3 kernels per layer", "replicas": world,
                   "sequence": ("chained: dr_router_topk for layer 0, then drb_moe_decode_chained + drb_router_topk_chained per layer"
                                if chained else "reference: dr_router_topk + dr_moe_decode per layer (src/engine.rs:959-1042)"),
                   "multi_gpu": "batch-1 decode does not shard: N independent replicas, no collective; the expert-parallel path is reported under prefill_expert_parallel",
                   "cache": "inputs larger than L2: 736 MB of weights read per step, 18.1 GB resident"},
        "hbm_gbs": gbs,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "kernel": "decode step graph (router, gate_up, down per layer)",
                     "algorithmic_bytes_per_launch": step_bytes,
                     # dram__bytes_read+write per step from the ncu capture summarised in profiles/decode_kernels_ncu_full.md
                     # (19.62 MB per layer, measured on a 4-layer case; traffic is proportional to the layer count)
                     "traffic": 19.623e6 * args.layers},
        "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": hidden_bytes, "d2h_bytes_per_step": hidden_bytes},
        "gpu_launches": args.steps * args.layers * 3,
        "clocks": clocks.summary(),
        "device_error_word": int(word.value),
        "decode_other_sequence": alt_info,
    }
    if ep_info is not None:
        line["prefill_expert_parallel"] = ep_info
        line["decode_64streams_expert_parallel"] = ep_info64
    if not args.no_extras:
        line["prefill"] = prefill_extra(torch, layers, st, ext_stream)
        line["gemv_q8_sweep"] = gemv_extra(torch, st, ext_stream)
        line["decode_fp8"] = fp8_extra(torch, layers, st, ext_stream)
    if not args.no_cpu and world == 1:  # the CPU baseline is a single-GPU-run figure (torchrun also pins OMP to one thread)
        line["cpu_baseline"] = cpu_decode_baseline()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--sequence", default="reference", choices=["reference", "chained"],
                    help="decode call sequence of the headline number: the reference engine's, or the chained entry points")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill and GEMV-sweep figures")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
