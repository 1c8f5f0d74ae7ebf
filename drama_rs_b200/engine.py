"""Host-side orchestration of the MoE path, call for call as the reference's engine issues it.

Decode: `MoeDecoder.record_step` collects one op per launch, chains each weight-streaming op's
region to the op before it for L2 prefetch (the last wraps to the first), and is captured once
into a graph that `step` replays — src/engine.rs:136-150 (`Op`), 674-708 (`record_step`),
946-1042 (router + moe_decode per layer, x == res == y), 1047-1066 (`step`).

Prefill: `MoePrefill` has two forms. `reference_calls=True` is src/engine.rs:544-604 call for call:
cuBLAS router logits, dr_moe_topk, shared expert through dequant + cuBLAS, count, counts to the
host, host exclusive scan, permute, grouped expert kernel, combine. The default is this library's
own sequence of seven launches with no library GEMM and no host round trip: rmsnorm, router logits
in a fixed order, top-k, one grouping kernel, the two grouped tensor-core GEMMs (which also run the
int8 shared expert and read their rows in place), combine.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np

from . import ffi
from .gpu import DevBuf, Graph, Stream, check, launched
from .model import MoeLayer

NULL = C.c_void_p(0)
# src/engine.rs:18 has this switch off. Measured here as well: the warm-up runs in the router's single tail
# block, and 14 MB of prefetches through one multiprocessor take ~55 us, so it stays off.
ROUTER_PREFETCH = False
GEMV_PREFETCH = True  # src/engine.rs:19


@dataclass
class Op:
    """One recorded decode launch. `weights` is the region it streams (for the previous op to
    prefetch); `run` gets the region of the next weight-streaming op to prefetch itself."""

    weights: Optional[tuple[int, int]]
    run: Callable[[C.c_void_p, int], None]


class MoeDecoder:
    """Batch-1 decode over a stack of MoE layers: x <- x + moe_l(rmsnorm(x)) for each layer."""

    def __init__(self, layers: list[MoeLayer], topk: int = 8, eps: float = 1e-6, st: Stream | None = None,
                 trace_routing: bool = False, fp8: list | None = None, lib=None) -> None:
        """trace_routing copies every layer's idx to `idx_trace` (tests). lib: another library with the same ABI (ffi.bind) to issue the launches to; buffers
        and streams still come from this one."""
        self.l = lib or ffi.lib()
        self.st = st or Stream()
        self.layers = layers
        self.topk, self.eps = topk, eps
        self.trace_routing = trace_routing
        # fp8[l] (model.Fp8Experts) replaces layer l's int4 routed experts: src/engine.rs:949, 996-1003 (`Experts::Fp8`)
        self.fp8 = fp8
        h, i, e = layers[0].hidden, layers[0].inter, layers[0].experts
        self.hidden = h
        f32 = 4
        self.idx_trace = DevBuf(len(layers) * topk * 4) if trace_routing else None
        self.x = DevBuf((h) * f32)
        self.rlog = DevBuf((e + 1) * f32)
        self.idx = DevBuf(topk * 4)
        self.wts = DevBuf(topk * f32)
        self.sgate = DevBuf(f32)
        self.act = DevBuf((topk + 1) * i * f32)
        self.counter = DevBuf.zeros(16, self.st)
        self.graph: Graph | None = None

    def ops(self) -> list[Op]:
        ops: list[Op] = []
        l, st = self.l, self.st.raw
        for li, layer in enumerate(self.layers):
            gq, gs = layer.gate_up.expert(0)
            dq, ds = layer.down.expert(0)
            sizes = (layer.gate_up.q_bytes_per_expert, layer.gate_up.sm_bytes_per_expert,
                     layer.down.q_bytes_per_expert, layer.down.sm_bytes_per_expert)

            def router(pf, pfb, layer=layer, gq=gq, gs=gs, dq=dq, ds=ds, sizes=sizes):
                launched(
                    l.dr_router_topk(
                        layer.router.at(0), self.x.at(0), layer.post_norm.at(0), self.eps, self.rlog.at(0), layer.experts,
                        self.topk, layer.hidden, self.idx.at(0), self.wts.at(0), self.sgate.at(0), self.counter.at(0),
                        gq if ROUTER_PREFETCH else NULL, gs, dq, ds, *sizes, st,
                    ),
                    "router_topk",
                )

            ops.append(Op((layer.router.ptr, (layer.experts + 1) * layer.hidden * 2), router))
            if self.trace_routing:
                ops.append(Op(None, lambda pf, pfb, li=li: check(
                    l.dr_d2d(self.idx_trace.at(li * self.topk * 4), self.idx.at(0), self.topk * 4, st), "d2d")))
            sgq, sgs = layer.shared_gate_up.rows(0)
            sdq, sds = layer.shared_down.rows(0)

            def decode(pf, pfb, layer=layer, gq=gq, gs=gs, dq=dq, ds=ds, sgq=sgq, sgs=sgs, sdq=sdq, sds=sds):
                launched(
                    l.dr_moe_decode(
                        gq, gs, dq, ds, sgq, sgs, sdq, sds, self.x.at(0), self.idx.at(0), self.wts.at(0), self.sgate.at(0),
                        self.x.at(0), self.act.at(0), self.x.at(0), layer.hidden, layer.inter, self.topk,
                        layer.post_norm.at(0), self.eps, pf, pfb, st,
                    ),
                    "moe_decode",
                )

            def decode_fp8(pf, pfb, li=li, layer=layer, sgq=sgq, sgs=sgs, sdq=sdq, sds=sds):
                f8 = self.fp8[li]
                launched(
                    l.dr_moe_decode_fp8(
                        f8.gu_w.at(0), f8.gu_s.at(0), f8.d_w.at(0), f8.d_s.at(0), sgq, sgs, sdq, sds, self.x.at(0), self.idx.at(0),
                        self.wts.at(0), self.sgate.at(0), self.x.at(0), self.act.at(0), self.x.at(0), layer.hidden, layer.inter,
                        self.topk, layer.post_norm.at(0), self.eps, pf, pfb, st,
                    ),
                    "moe_decode_fp8",
                )

            ops.append(Op(None, decode_fp8 if self.fp8 else decode))
        return ops

    def record_step(self) -> None:
        ops = self.ops()
        first = next((o.weights for o in ops if o.weights), None)
        for k, op in enumerate(ops):
            nxt = next((o.weights for o in ops[k + 1:] if o.weights), None) or first
            if GEMV_PREFETCH and nxt:
                op.run(C.c_void_p(nxt[0]), nxt[1])
            else:
                op.run(NULL, 0)

    def capture(self) -> None:
        self.graph = Graph(self.st, self.record_step)

    def set_x(self, x: np.ndarray) -> None:
        self.x.upload(x.astype(np.float32), self.st)

    def step(self) -> np.ndarray:
        """Replays the captured step on the current x and returns the new hidden state."""
        assert self.graph is not None, "capture first"
        self.graph.launch(self.st)
        return self.x.download(np.float32, self.hidden, self.st)

    def step_eager(self) -> np.ndarray:
        self.record_step()
        return self.x.download(np.float32, self.hidden, self.st)

    def routing_trace(self) -> np.ndarray:
        assert self.idx_trace is not None
        return self.idx_trace.download(np.int32, len(self.layers) * self.topk, self.st).reshape(len(self.layers), self.topk)

    def routing(self) -> tuple[np.ndarray, np.ndarray, float]:
        """The last layer's idx, wts and sgate (for tests)."""
        return (self.idx.download(np.int32, self.topk, self.st), self.wts.download(np.float32, self.topk, self.st),
                float(self.sgate.download(np.float32, 1, self.st)[0]))


class MoePrefill:
    """The prefill-side MoE block over n <= max_rows rows, with the reference's buffers
    (src/engine.rs:263-305): x f32, hn_b bf16, rlog, idx/wts/sgate, shared-expert temporaries,
    counts/offsets/fill/slot_of, xp/ap/yp in expert-sorted order, and one bf16 weight buffer for
    the dequantised int8 matrices."""

    def __init__(self, layer: MoeLayer, max_rows: int, topk: int = 8, eps: float = 1e-6, st: Stream | None = None,
                 reference_calls: bool = False, lib=None) -> None:
        """lib: another library with the same ABI (ffi.bind) to issue the launches to (reference_calls only)."""
        self.l = lib or ffi.lib()
        self.st = st or Stream()
        self.layer, self.topk, self.eps, self.max_rows = layer, topk, eps, max_rows
        self.reference_calls = reference_calls
        # own sequence: the normalised rows stay in fp16 (eleven significant bits; the reference's prefill rounds them to bf16)
        self.rows_f16 = not reference_calls
        h, i, e = layer.hidden, layer.inter, layer.experts
        n = max_rows
        self.blas = C.c_void_p()
        if reference_calls:
            check(self.l.dr_cublas_create(C.byref(self.blas), self.st.raw), "cublas_create")
        else:
            check(self.l.drb_init(), "init")
        self.x = DevBuf(n * h * 4)
        self.hn_b = DevBuf(n * h * 2)
        self.rlog = DevBuf(n * (e + 1) * 4)
        self.idx = DevBuf(n * topk * 4)
        self.wts = DevBuf(n * topk * 4)
        self.sgate = DevBuf(n * 4)
        self.shh = DevBuf(n * 2 * i * 4) if reference_calls else None
        self.sh_act_b = DevBuf(n * i * 2)
        self.sh_out = DevBuf(n * h * 4)
        self.counts = DevBuf(e * 4)
        self.offsets = DevBuf(e * 4)
        self.fill = DevBuf(e * 4)
        self.slot_of = DevBuf(n * topk * 4)
        self.row_of = DevBuf(n * topk * 4)
        self.xp = DevBuf(n * topk * h * 2) if reference_calls else None
        self.ap = DevBuf(n * topk * i * 2)
        self.yp = DevBuf(n * topk * h * 4)
        self.wbuf = DevBuf(2 * i * h * 2) if reference_calls else None
        self.device_scan = False  # reference calls only: offsets by drb_moe_offsets on the device instead of the host scan
        self.invariant_router = not reference_calls  # router logits by drb_router_logits (independent of the batch size) instead of cuBLAS
        self.logit_bias: DevBuf | None = None  # [n, E + 1] f32 rows the router GEMM accumulates onto (not in the reference)

    def gemm_q8(self, a, w, c, m: int, beta: float) -> None:
        """C = A . dequant(W)^T + beta C for a q8 weight. src/engine.rs:351-355."""
        q, s = w.rows(0)
        launched(self.l.dr_dequant_q8(q, s, self.wbuf.at(0), w.n, w.k, self.st.raw), "dequant_q8")
        check(self.l.dr_gemm(self.blas, a, self.wbuf.at(0), c, m, w.n, w.k, beta), "gemm")

    def run(self, x: np.ndarray, logit_bias: np.ndarray | None = None) -> np.ndarray:
        """x [n, H] f32 on the host -> x + moe(rmsnorm(x, post_norm)). src/engine.rs:499-500 and 544-604.
        logit_bias ([E] f32, tests and the benchmark's Zipf routing only) is added to the router logits."""
        n, h = x.shape
        e = self.layer.experts
        assert n <= self.max_rows
        self.x.upload(x.astype(np.float32), self.st)
        if logit_bias is not None:
            rows = np.zeros((n, e + 1), dtype=np.float32)
            rows[:, :e] = logit_bias.astype(np.float32)
            self.logit_bias = DevBuf.from_array(rows, self.st)
        else:
            self.logit_bias = None
        self.run_device(n)
        return self.x.download(np.float32, n * h, self.st).reshape(n, h)

    def route_device(self, n: int) -> None:
        """rmsnorm -> hn_b, router logits, top-k, on the n rows in self.x."""
        l, st, layer = self.l, self.st.raw, self.layer
        h, e, topk = layer.hidden, layer.experts, self.topk
        if self.rows_f16:
            launched(l.drb_rmsnorm_f16(self.x.at(0), layer.post_norm.at(0), self.hn_b.at(0), n, h, self.eps, st), "rmsnorm_f16")
        else:
            launched(l.dr_rmsnorm(self.x.at(0), layer.post_norm.at(0), NULL, self.hn_b.at(0), n, h, self.eps, st), "rmsnorm")
        beta = 0.0
        if self.logit_bias is not None:
            check(l.dr_d2d(self.rlog.at(0), self.logit_bias.at(0), n * (e + 1) * 4, st), "d2d")
            beta = 1.0
        if self.rows_f16:
            launched(l.drb_router_logits_f16(self.hn_b.at(0), layer.router.at(0), self.rlog.at(0), n, e + 1, h, beta, st), "router_logits_f16")
        elif self.invariant_router:
            launched(l.drb_router_logits(self.hn_b.at(0), layer.router.at(0), self.rlog.at(0), n, e + 1, h, beta, st), "router_logits")
        else:
            check(l.dr_gemm(self.blas, self.hn_b.at(0), layer.router.at(0), self.rlog.at(0), n, e + 1, h, beta), "gemm")
        launched(l.dr_moe_topk(self.rlog.at(0), n, e, topk, e + 1, self.idx.at(0), self.wts.at(0), self.sgate.at(0), st), "moe_topk")

    def run_device(self, n: int) -> None:
        """The block on the n rows already in self.x (device), in place. With a logit bias the router logits are
        accumulated onto the bias rows (beta = 1) instead of overwriting them."""
        if self.reference_calls:
            return self.run_device_reference_calls(n)
        l, st, layer = self.l, self.st.raw, self.layer
        h, e, topk, i = layer.hidden, layer.experts, self.topk, layer.inter
        self.route_device(n)
        launched(l.drb_moe_group(self.idx.at(0), n, topk, 0, e, self.counts.at(0), self.offsets.at(0), self.slot_of.at(0),
                                 self.row_of.at(0), st), "moe_group")
        gq, gs = layer.gate_up.expert(0)
        dq, ds = layer.down.expert(0)
        sgq, sgs = layer.shared_gate_up.rows(0)
        sdq, sds = layer.shared_down.rows(0)
        launched(
            l.drb_moe_prefill_block(gq, gs, dq, ds, sgq, sgs, sdq, sds, self.hn_b.at(0), self.row_of.at(0), self.offsets.at(0),
                                    self.counts.at(0), self.ap.at(0), self.yp.at(0), self.sh_act_b.at(0), self.sh_out.at(0), n, e, h, i,
                                    1 if self.rows_f16 else 0, NULL, st), "moe_prefill_block")
        launched(
            l.dr_moe_combine(self.x.at(0), self.yp.at(0), self.slot_of.at(0), self.wts.at(0), self.sgate.at(0),
                             self.sh_out.at(0), n, topk, h, st), "moe_combine")

    def run_device_reference_calls(self, n: int) -> None:
        """Call for call the reference's sequence (src/engine.rs:544-604)."""
        l, st, layer = self.l, self.st.raw, self.layer
        h, e, topk, i = layer.hidden, layer.experts, self.topk, layer.inter
        self.route_device(n)
        # Shared expert.
        self.gemm_q8(self.hn_b.at(0), layer.shared_gate_up, self.shh.at(0), n, 0.0)
        launched(l.dr_swiglu_rows(self.shh.at(0), self.sh_act_b.at(0), n, i, st), "swiglu")
        self.gemm_q8(self.sh_act_b.at(0), layer.shared_down, self.sh_out.at(0), n, 0.0)
        # Group (row, k) pairs by expert.
        self.counts.zero(self.st)
        launched(l.dr_moe_count(self.idx.at(0), n * topk, self.counts.at(0), st), "moe_count")
        if self.device_scan:
            launched(l.drb_moe_offsets(self.counts.at(0), e, self.offsets.at(0), st), "moe_offsets")
        else:
            counts = self.counts.download(np.int32, e, self.st)
            offsets = (np.cumsum(counts) - counts).astype(np.int32)
            self.offsets.upload(offsets, self.st)
        self.fill.zero(self.st)
        launched(
            l.dr_moe_permute(self.idx.at(0), n, topk, self.offsets.at(0), self.fill.at(0), self.slot_of.at(0),
                             self.hn_b.at(0), self.xp.at(0), h, st), "moe_permute")
        gq, gs = layer.gate_up.expert(0)
        dq, ds = layer.down.expert(0)
        launched(
            l.dr_moe_prefill(gq, gs, dq, ds, self.xp.at(0), self.offsets.at(0), self.counts.at(0), self.ap.at(0),
                             self.yp.at(0), e, h, i, st), "moe_prefill")
        launched(
            l.dr_moe_combine(self.x.at(0), self.yp.at(0), self.slot_of.at(0), self.wts.at(0), self.sgate.at(0),
                             self.sh_out.at(0), n, topk, h, st), "moe_combine")


class MoeStackDecoder:
    """The same stack as MoeDecoder through drb_moe_stack_decode: one persistent kernel per step."""

    def __init__(self, layers: list[MoeLayer], topk: int = 8, eps: float = 1e-6, st: Stream | None = None) -> None:
        self.l = ffi.lib()
        self.st = st or Stream()
        self.layers, self.topk, self.eps = layers, topk, eps
        self.hidden, self.inter, self.experts = layers[0].hidden, layers[0].inter, layers[0].experts
        table = np.zeros((len(layers), 10), dtype=np.uint64)
        for i, ly in enumerate(layers):
            table[i] = [ly.router.ptr, ly.post_norm.ptr, ly.gate_up.q.ptr, ly.gate_up.sm.ptr, ly.down.q.ptr, ly.down.sm.ptr,
                        ly.shared_gate_up.q.ptr, ly.shared_gate_up.s.ptr, ly.shared_down.q.ptr, ly.shared_down.s.ptr]
        self.table = DevBuf.from_array(table, self.st)
        self.x = DevBuf(self.hidden * 4)
        self.ws = DevBuf.zeros(self.l.drb_moe_stack_workspace_bytes(), self.st)
        self.idx_trace = DevBuf(len(layers) * topk * 4)
        self.wts_trace = DevBuf(len(layers) * topk * 4)
        self.graph: Graph | None = None

    def launch(self) -> None:
        launched(
            self.l.drb_moe_stack_decode(self.table.at(0), len(self.layers), self.x.at(0), self.ws.at(0), self.experts, self.topk,
                                        self.hidden, self.inter, self.eps, self.idx_trace.at(0), self.wts_trace.at(0), self.st.raw),
            "moe_stack_decode")

    def capture(self) -> None:
        self.graph = Graph(self.st, self.launch)

    def set_x(self, x: np.ndarray) -> None:
        self.x.upload(x.astype(np.float32), self.st)

    def step(self) -> np.ndarray:
        if self.graph is not None:
            self.graph.launch(self.st)
        else:
            self.launch()
        return self.x.download(np.float32, self.hidden, self.st)

    def routing(self) -> tuple[np.ndarray, np.ndarray]:
        n = len(self.layers) * self.topk
        return (self.idx_trace.download(np.int32, n, self.st).reshape(-1, self.topk),
                self.wts_trace.download(np.float32, n, self.st).reshape(-1, self.topk))
