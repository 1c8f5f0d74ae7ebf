"""Expert-parallel MoE block over N ranks (one process per GPU, torch.distributed for the exchange).

The reference is single-GPU (it has no distributed code at all); this is the multi-GPU form of its
prefill-side MoE block (src/engine.rs:544-604) that the benchmark configurations ask for:

  * rank r owns experts [r * E/N, (r + 1) * E/N): contiguous slices of gate_up.q4/.sm and down.q4/.sm
    along their leading dimension (the layout has E outermost, src/model.rs:31-43);
  * router, post_norm and the shared expert are replicated; tokens are data-parallel (each rank routes its
    own rows, so the routing is the single-GPU routing by construction);
  * dispatch: every (row, k) pair travels as one bf16 row to the rank that owns its expert
    (all_to_all_single with split sizes, after a small all_to_all of the counts);
  * the owner groups what it received by expert (dr_moe_count / host scan / dr_moe_permute, exactly the
    reference's bookkeeping) and runs the grouped expert kernel (dr_moe_prefill) on its slice;
  * combine: the f32 results travel back the same way and the home rank sums them in fixed k order with
    the shared expert and the residual (dr_moe_combine), so the result does not depend on N.

The exchange is NCCL over NVLink on GPUs (gloo on CPU in the tests). Received rows land in this rank's
own memory before any kernel reads them; nothing here reads a peer's memory directly.

`ops` supplies the per-rank compute (the C-ABI kernels on a GPU; the tests plug in the oracle on CPU), so
the bookkeeping below is the same code on both.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class EpPlan:
    """Where every (row, k) pair of this rank goes and where its result comes back."""

    order: torch.Tensor        # [pairs] permutation of the local pairs, sorted by expert (hence by owner rank)
    send_counts: list[int]     # pairs sent to each rank
    recv_counts: list[int]     # pairs received from each rank
    recv_expert: torch.Tensor  # [recv pairs] local expert index (0 .. E/N - 1) of every received row


def owner_of(expert: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    return expert // (experts // world)


def make_plan(idx: torch.Tensor, experts: int, group=None) -> EpPlan:
    """idx [rows, topk] int32 on the compute device. One count exchange, one expert-id exchange."""
    world = dist.get_world_size(group)
    flat = idx.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    send = torch.bincount(owner_of(sorted_e, experts, world), minlength=world)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    send_counts, recv_counts = send.tolist(), recv.tolist()
    recv_expert = torch.empty(sum(recv_counts), dtype=torch.int64, device=idx.device)
    dist.all_to_all_single(recv_expert, sorted_e, recv_counts, send_counts, group=group)
    per = experts // world
    recv_expert = (recv_expert - dist.get_rank(group) * per).to(torch.int32)
    return EpPlan(order, send_counts, recv_counts, recv_expert)


def dispatch(rows_b: torch.Tensor, topk: int, plan: EpPlan, group=None) -> torch.Tensor:
    """rows_b [rows, H] (bf16 on GPUs) -> the rows this rank's experts must process, [recv pairs, H]."""
    src_row = plan.order // topk
    out = rows_b.new_empty((sum(plan.recv_counts), rows_b.shape[1]))
    dist.all_to_all_single(out, rows_b.index_select(0, src_row), plan.recv_counts, plan.send_counts, group=group)
    return out


def combine_exchange(y_recv: torch.Tensor, plan: EpPlan, group=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Results of the received rows travel home. Returns (Y [pairs, H] in sorted-pair order, slot_of [pairs])
    where slot_of[p] is the row of Y that holds pair p = row * topk + k."""
    y_home = y_recv.new_empty((sum(plan.send_counts), y_recv.shape[1]))
    dist.all_to_all_single(y_home, y_recv, plan.send_counts, plan.recv_counts, group=group)
    slot_of = torch.empty_like(plan.order)
    slot_of[plan.order] = torch.arange(plan.order.numel(), device=plan.order.device)
    return y_home, slot_of.to(torch.int32)


def ep_moe_block(x: torch.Tensor, ops, experts: int, topk: int, group=None) -> torch.Tensor:
    """x [rows, H] f32 (this rank's rows) -> x + moe(rmsnorm(x)); `ops` is this rank's compute.

    ops.route(x) -> (hn_b [rows, H], idx [rows, topk] i32, wts [rows, topk] f32, sgate [rows] f32, shared [rows, H] f32)
    ops.experts(rows_b [n, H], local_expert [n] i32) -> y [n, H] f32      (grouped by expert inside)
    ops.combine(x, y_home, slot_of, wts, sgate, shared) -> x'             (fixed k order)
    """
    hn_b, idx, wts, sgate, shared = ops.route(x)
    plan = make_plan(idx, experts, group)
    recv_rows = dispatch(hn_b, topk, plan, group)
    y_recv = ops.experts(recv_rows, plan.recv_expert)
    y_home, slot_of = combine_exchange(y_recv, plan, group)
    return ops.combine(x, y_home, slot_of, wts, sgate, shared)


class EpGpuOps:
    """This rank's compute through the C ABI: routing and shared expert on the local rows, the grouped
    int4 expert kernel on the local expert slice. Buffers are torch tensors on the current CUDA device;
    the kernels run on `st`, which is also made torch's current stream for the collectives."""

    def __init__(self, layer, rank: int, world: int, max_rows: int, topk: int = 8, eps: float = 1e-6, st=None) -> None:
        import ctypes as C

        from . import ffi
        from .gpu import Stream, check

        self.C, self.l = C, ffi.lib()
        self.st = st or Stream()
        self.layer, self.rank, self.world, self.topk, self.eps = layer, rank, world, topk, eps
        self.per = layer.experts // world
        self.blas = C.c_void_p()
        check(self.l.dr_cublas_create(C.byref(self.blas), self.st.raw), "cublas_create")
        self.wbuf = torch.empty(2 * layer.inter * layer.hidden, dtype=torch.bfloat16, device="cuda")
        self.stream = torch.cuda.ExternalStream(self.st.raw.value)
        self.logit_bias = None  # optional [E] f32 tensor added to the router logits (benchmark's Zipf routing)

    def _p(self, t: torch.Tensor):
        return self.C.c_void_p(t.data_ptr())

    def _gemm_q8(self, a: torch.Tensor, w, m: int) -> torch.Tensor:
        from .gpu import check, launched

        q, s = w.rows(0)
        launched(self.l.dr_dequant_q8(q, s, self._p(self.wbuf), w.n, w.k, self.st.raw), "dequant_q8")
        c = torch.empty((m, w.n), dtype=torch.float32, device="cuda")
        check(self.l.dr_gemm(self.blas, self._p(a), self._p(self.wbuf), self._p(c), m, w.n, w.k, 0.0), "gemm")
        return c

    def route(self, x: torch.Tensor):
        from .gpu import check, launched

        l, st, ly = self.l, self.st.raw, self.layer
        n, h = x.shape
        e, topk, i = ly.experts, self.topk, ly.inter
        NULL = self.C.c_void_p(0)
        hn_b = torch.empty((n, h), dtype=torch.bfloat16, device="cuda")
        launched(l.dr_rmsnorm(self._p(x), ly.post_norm.at(0), NULL, self._p(hn_b), n, h, self.eps, st), "rmsnorm")
        rlog = torch.zeros((n, e + 1), dtype=torch.float32, device="cuda")
        beta = 0.0
        if self.logit_bias is not None:  # the GEMM accumulates onto the bias rows
            rlog[:, :e] = self.logit_bias
            beta = 1.0
        check(l.dr_gemm(self.blas, self._p(hn_b), ly.router.at(0), self._p(rlog), n, e + 1, h, beta), "gemm")
        idx = torch.empty((n, topk), dtype=torch.int32, device="cuda")
        wts = torch.empty((n, topk), dtype=torch.float32, device="cuda")
        sgate = torch.empty(n, dtype=torch.float32, device="cuda")
        launched(l.dr_moe_topk(self._p(rlog), n, e, topk, e + 1, self._p(idx), self._p(wts), self._p(sgate), st), "moe_topk")
        shh = self._gemm_q8(hn_b, ly.shared_gate_up, n)
        sh_act = torch.empty((n, i), dtype=torch.bfloat16, device="cuda")
        launched(l.dr_swiglu_rows(self._p(shh), self._p(sh_act), n, i, st), "swiglu")
        shared = self._gemm_q8(sh_act, ly.shared_down, n)
        return hn_b, idx, wts, sgate, shared

    def experts(self, rows_b: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
        from .gpu import launched

        l, st, ly = self.l, self.st.raw, self.layer
        n, h = rows_b.shape
        y = torch.empty((n, h), dtype=torch.float32, device="cuda")
        if n == 0:
            return y
        counts = torch.zeros(self.per, dtype=torch.int32, device="cuda")
        launched(l.dr_moe_count(self._p(local_expert), n, self._p(counts), st), "moe_count")
        offsets = (torch.cumsum(counts, 0) - counts).to(torch.int32)  # on the device: no host round trip
        fill = torch.zeros(self.per, dtype=torch.int32, device="cuda")
        slot_of = torch.empty(n, dtype=torch.int32, device="cuda")
        xp = torch.empty((n, h), dtype=torch.bfloat16, device="cuda")
        launched(l.dr_moe_permute(self._p(local_expert), n, 1, self._p(offsets), self._p(fill), self._p(slot_of), self._p(rows_b),
                                  self._p(xp), h, st), "moe_permute")
        gq, gs = ly.gate_up.expert(self.rank * self.per)
        dq, ds = ly.down.expert(self.rank * self.per)
        ap = torch.empty((n, ly.inter), dtype=torch.bfloat16, device="cuda")
        yp = torch.empty((n, h), dtype=torch.float32, device="cuda")
        launched(l.dr_moe_prefill(gq, gs, dq, ds, self._p(xp), self._p(offsets), self._p(counts), self._p(ap), self._p(yp),
                                  self.per, h, ly.inter, st), "moe_prefill")
        return yp.index_select(0, slot_of.to(torch.int64))

    def combine(self, x, y_home, slot_of, wts, sgate, shared):
        from .gpu import launched

        n, h = x.shape
        launched(self.l.dr_moe_combine(self._p(x), self._p(y_home), self._p(slot_of), self._p(wts), self._p(sgate),
                                       self._p(shared), n, self.topk, h, self.st.raw), "moe_combine")
        return x


# ------------------------------------------------------------------------------------------------------------
# Fixed-capacity exchange: no size ever leaves the device, so a whole layer (or a whole stack of layers) is a
# fixed sequence of launches and collectives that a CUDA graph can hold.


def ep_moe_block_fixed(x: torch.Tensor, ops, experts: int, topk: int, cap: int, group=None) -> torch.Tensor:
    """x [rows, H] f32 -> x + moe(rmsnorm(x)) with every exchange at a fixed size.

    Every rank sends every peer a block of `cap` row slots (cap >= rows * topk on every rank, the worst case of
    all pairs going to one owner), filled from the front; unused slots carry the local expert id `E/N`, one past
    the owner's last expert, so the owner's grouping puts them in a bucket that the expert kernel never visits.
    Three collectives per layer, all of them all_to_all_single without split sizes: rows out, expert ids out,
    results back. Nothing is read on the host.

    ops.route(x) as for ep_moe_block.
    ops.pack(hn_b, idx, cap) -> (send_rows [N * cap, H], send_e [N * cap] i32, slot_of [rows * topk] i32)
    ops.experts_padded(recv_rows [N * cap, H], recv_e [N * cap] i32) -> y [N * cap, H] f32 (padding rows: anything)
    ops.exchange_buffers() -> (recv_rows, recv_e, y_home) to receive into, or None to allocate here
    ops.combine as for ep_moe_block; slot_of indexes the rows of y_home.
    """
    hn_b, idx, wts, sgate, shared = ops.route(x)
    send_rows, send_e, slot_of = ops.pack(hn_b, idx, cap)
    bufs = ops.exchange_buffers() if hasattr(ops, "exchange_buffers") else None
    recv_rows, recv_e, y_home = bufs if bufs is not None else (torch.empty_like(send_rows), torch.empty_like(send_e), None)
    dist.all_to_all_single(recv_rows, send_rows, group=group)
    dist.all_to_all_single(recv_e, send_e, group=group)
    y_send = ops.experts_padded(recv_rows, recv_e)
    if y_home is None:
        y_home = torch.empty_like(y_send)
    dist.all_to_all_single(y_home, y_send, group=group)
    return ops.combine(x, y_home, slot_of, wts, sgate, shared)


def pack_fixed(rows_b: torch.Tensor, idx: torch.Tensor, world: int, per: int, cap: int):
    """Device-agnostic packing with torch ops (what the CPU tests run; the GPU path uses the C-ABI kernels):
    pair p = row * topk + k goes to block idx[p] // per, slots handed out in pair order."""
    flat = idx.reshape(-1).to(torch.int64)
    owner = flat // per
    onehot = torch.nn.functional.one_hot(owner, world)
    rank_in_block = (torch.cumsum(onehot, 0) - onehot).gather(1, owner[:, None])[:, 0]
    slot_of = owner * cap + rank_in_block
    send_rows = rows_b.new_zeros((world * cap, rows_b.shape[1]))
    send_rows[slot_of] = rows_b[torch.arange(flat.numel(), device=idx.device) // idx.shape[1]]
    send_e = torch.full((world * cap,), per, dtype=torch.int32, device=idx.device)
    send_e[slot_of] = (flat - owner * per).to(torch.int32)
    return send_rows, send_e, slot_of.to(torch.int32)


class EpGpuFixed:
    """This rank's compute for ep_moe_block_fixed through the C ABI, on preallocated buffers (fixed addresses, so
    the launches can be captured). One workspace serves every layer of a stack: `layer` is switched per call."""

    def __init__(self, layer, rank: int, world: int, max_rows: int, cap: int, topk: int = 8, eps: float = 1e-6, st=None) -> None:
        import ctypes as C

        from . import ffi
        from .gpu import Stream, check

        self.C, self.l = C, ffi.lib()
        self.st = st or Stream()
        self.layer, self.rank, self.world, self.topk, self.eps, self.cap = layer, rank, world, topk, eps, cap
        e, h, i = layer.experts, layer.hidden, layer.inter
        self.per = per = e // world
        if cap < max_rows * topk:
            raise ValueError("cap must cover every pair of this rank going to one owner")
        self.blas = C.c_void_p()
        check(self.l.dr_cublas_create(C.byref(self.blas), self.st.raw), "cublas_create")
        self.stream = torch.cuda.ExternalStream(self.st.raw.value)
        self.logit_bias = None
        self.wcache: dict[int, torch.Tensor] = {}  # bf16 copies of the shared experts' int8 matrices, by matrix
        n, r = world * cap, max_rows
        dev = "cuda"
        f32, bf16, i32 = torch.float32, torch.bfloat16, torch.int32
        self.hn_b = torch.empty((r, h), dtype=bf16, device=dev)
        self.rlog = torch.empty((r, e + 1), dtype=f32, device=dev)
        self.idx = torch.empty((r, topk), dtype=i32, device=dev)
        self.wts = torch.empty((r, topk), dtype=f32, device=dev)
        self.sgate = torch.empty(r, dtype=f32, device=dev)
        self.shh = torch.empty((r, 2 * i), dtype=f32, device=dev)
        self.sh_act = torch.empty((r, i), dtype=bf16, device=dev)
        self.shared = torch.empty((r, h), dtype=f32, device=dev)
        self.owner = torch.empty(r * topk, dtype=i32, device=dev)
        self.local = torch.empty(r * topk, dtype=i32, device=dev)
        self.slot_of = torch.empty(r * topk, dtype=i32, device=dev)
        self.block_base = (torch.arange(world, dtype=i32, device=dev) * cap).contiguous()
        # [fill of the send blocks | counts | fill of the expert buckets]: zeroed with one memset per layer
        self.zeros = torch.zeros(world + 2 * (per + 1), dtype=i32, device=dev)
        self.offsets = torch.empty(per + 1, dtype=i32, device=dev)
        # Padding slots of the send block are never written: zero them once so that what travels is finite.
        self.send_rows = torch.zeros((n, h), dtype=bf16, device=dev)
        self.send_e = torch.empty(n, dtype=i32, device=dev)
        self.recv_rows = torch.empty((n, h), dtype=bf16, device=dev)
        self.recv_e = torch.empty(n, dtype=i32, device=dev)
        self.slot_of2 = torch.empty(n, dtype=i32, device=dev)
        self.xp = torch.empty((n, h), dtype=bf16, device=dev)
        self.ap = torch.empty((n, i), dtype=bf16, device=dev)
        self.yp = torch.zeros((n, h), dtype=f32, device=dev)
        self.y_send = torch.empty((n, h), dtype=f32, device=dev)
        self.y_home = torch.empty((n, h), dtype=f32, device=dev)

    def _p(self, t: torch.Tensor):
        return self.C.c_void_p(t.data_ptr())

    def exchange_buffers(self):
        return self.recv_rows, self.recv_e, self.y_home

    def _gemm_q8(self, a: torch.Tensor, w, c: torch.Tensor, m: int) -> None:
        """C = A . dequant(W)^T. The reference dequantises into one scratch buffer before every GEMM
        (src/engine.rs:351-355); here the bf16 copy of a shared-expert matrix is kept after its first use
        (6 MB per layer), which takes two launches out of every layer."""
        from .gpu import check, launched

        wb = self.wcache.get(id(w))
        if wb is None:
            q, s = w.rows(0)
            wb = torch.empty(w.n * w.k, dtype=torch.bfloat16, device="cuda")
            launched(self.l.dr_dequant_q8(q, s, self._p(wb), w.n, w.k, self.st.raw), "dequant_q8", debug=False)
            self.wcache[id(w)] = wb
        check(self.l.dr_gemm(self.blas, self._p(a), self._p(wb), self._p(c), m, w.n, w.k, 0.0), "gemm")

    def route(self, x: torch.Tensor):
        from .gpu import check, launched

        l, st, ly = self.l, self.st.raw, self.layer
        n, h = x.shape
        e, topk, i = ly.experts, self.topk, ly.inter
        NULL = self.C.c_void_p(0)
        hn_b, rlog, idx, wts, sgate = self.hn_b[:n], self.rlog[:n], self.idx[:n], self.wts[:n], self.sgate[:n]
        launched(l.dr_rmsnorm(self._p(x), ly.post_norm.at(0), NULL, self._p(hn_b), n, h, self.eps, st), "rmsnorm", debug=False)
        beta = 0.0
        if self.logit_bias is not None:  # the GEMM accumulates onto the bias rows
            rlog.zero_()
            rlog[:, :e] = self.logit_bias
            beta = 1.0
        # batch-invariant logits: the routing of a row must not depend on how many rows this rank holds
        launched(l.drb_router_logits(self._p(hn_b), ly.router.at(0), self._p(rlog), n, e + 1, h, beta, st), "router_logits", debug=False)
        launched(l.dr_moe_topk(self._p(rlog), n, e, topk, e + 1, self._p(idx), self._p(wts), self._p(sgate), st), "moe_topk", debug=False)
        self._gemm_q8(hn_b, ly.shared_gate_up, self.shh, n)
        launched(l.dr_swiglu_rows(self._p(self.shh), self._p(self.sh_act), n, i, st), "swiglu", debug=False)
        self._gemm_q8(self.sh_act, ly.shared_down, self.shared, n)
        return hn_b, idx, wts, sgate, self.shared[:n]

    def pack(self, hn_b: torch.Tensor, idx: torch.Tensor, cap: int):
        from .gpu import launched

        assert cap == self.cap
        n, h = hn_b.shape
        pairs = n * self.topk
        owner, local, slot_of = self.owner[:pairs], self.local[:pairs], self.slot_of[:pairs]
        flat = idx.reshape(-1)
        torch.div(flat, self.per, rounding_mode="floor", out=owner)
        torch.sub(flat, owner * self.per, out=local)
        self.zeros.zero_()
        fill = self.zeros[: self.world]
        launched(self.l.dr_moe_permute(self._p(owner), n, self.topk, self._p(self.block_base), self._p(fill), self._p(slot_of),
                                       self._p(hn_b), self._p(self.send_rows), h, self.st.raw), "moe_permute", debug=False)
        self.send_e.fill_(self.per)
        self.send_e.index_copy_(0, slot_of.to(torch.int64), local)
        return self.send_rows, self.send_e, slot_of

    def experts_padded(self, recv_rows: torch.Tensor, recv_e: torch.Tensor) -> torch.Tensor:
        from .gpu import launched

        l, st, ly, per = self.l, self.st.raw, self.layer, self.per
        n, h = recv_rows.shape
        counts = self.zeros[self.world: self.world + per + 1]
        fill = self.zeros[self.world + per + 1:]
        launched(l.dr_moe_count(self._p(recv_e), n, self._p(counts), st), "moe_count", debug=False)
        launched(l.drb_moe_offsets(self._p(counts), per + 1, self._p(self.offsets), st), "moe_offsets", debug=False)
        launched(l.dr_moe_permute(self._p(recv_e), n, 1, self._p(self.offsets), self._p(fill), self._p(self.slot_of2),
                                  self._p(recv_rows), self._p(self.xp), h, st), "moe_permute", debug=False)
        gq, gs = ly.gate_up.expert(self.rank * per)
        dq, ds = ly.down.expert(self.rank * per)
        launched(l.dr_moe_prefill(gq, gs, dq, ds, self._p(self.xp), self._p(self.offsets), self._p(counts), self._p(self.ap),
                                  self._p(self.yp), per, h, ly.inter, st), "moe_prefill", debug=False)
        torch.index_select(self.yp, 0, self.slot_of2.to(torch.int64), out=self.y_send)
        return self.y_send

    def combine(self, x, y_home, slot_of, wts, sgate, shared):
        from .gpu import launched

        n, h = x.shape
        launched(self.l.dr_moe_combine(self._p(x), self._p(y_home), self._p(slot_of), self._p(wts), self._p(sgate),
                                       self._p(shared), n, self.topk, h, self.st.raw), "moe_combine", debug=False)
        return x
