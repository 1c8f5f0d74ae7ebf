"""Expert-parallel MoE block over N ranks (one process per GPU, torch.distributed for the exchange).

The reference is single-GPU (it has no distributed code at all); this is the multi-GPU form of its
prefill-side MoE block (src/engine.rs:544-604) that the benchmark configurations ask for:

  * rank r owns experts [r * E/N, (r + 1) * E/N): contiguous slices of gate_up.q4/.sm and down.q4/.sm
    along their leading dimension (the layout has E outermost, src/model.rs:31-43);
  * router, post_norm and the shared expert are replicated; tokens are data-parallel (each rank routes its
    own rows with logits summed in a fixed order, so the routing is the single-GPU routing at every split);
  * dispatch: every (row, k) pair travels as one 16-bit row to the rank that owns its expert, in ONE
    all-to-all of fixed size: every rank sends every peer a block of `cap` row slots followed by the local
    expert ids of those rows; unused slots carry the id E/N, one past the owner's last expert, which the owner's
    grouping skips. No size is ever read on the host, so a layer (or a whole stack of layers with its collectives)
    is a fixed sequence of launches that a CUDA graph can hold;
  * `cap` is a capacity factor times the mean load of a (sender, owner) pair, not the worst case. A block that
    fills up drops the pair and raises a device-side overflow word that the host reads after the step (the
    result is void then and the step is repeated with a larger capacity); nothing waits and nothing faults;
  * the owner groups what it received by expert and runs the grouped tensor-core GEMMs on its slice, reading
    the rows where they arrived and writing the results in arrival order (no permuted copies);
  * combine: the f32 results travel back in a second all-to-all and the home rank sums them in fixed k order with
    the shared expert and the residual (dr_moe_combine), so the result does not depend on N;
  * the replicated shared expert runs on a second stream beside the dispatch exchange.

The exchange is, on GPUs, this library's own and fused with the kernels on either side of it: the pack kernels
store rows and ids straight into the owners' receive buffers over NVLink (symmetric memory), the down GEMM's
epilogue stores every result row straight into its home rank's buffer, and a step counter announces each
(drb_ep_sync, bounded); `EpGpu(p2p=False)`, and the CPU tests over gloo, use the library
collective instead. Received rows
land in this rank's own memory before any kernel reads them: nothing here loads from a peer's memory.

`ops` supplies the per-rank compute (the C-ABI kernels on a GPU; the tests plug in the oracle on CPU), so
the bookkeeping below is the same code on both.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist


def owner_of(expert: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    return expert // (experts // world)


def capacity(max_rows: int, topk: int, world: int, factor: float = 3.0) -> int:
    """Row slots per (sender, owner) block: `factor` times the mean load, at most the worst case (every pair of
    the sender going to one owner), and the same on every rank."""
    worst = max_rows * topk
    return max(1, min(worst, math.ceil(factor * worst / world)))


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, group=None) -> None:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        out.copy_(inp)
    else:
        dist.all_to_all_single(out, inp, group=group)


def ep_moe_block(x: torch.Tensor, ops, cap: int, group=None) -> torch.Tensor:
    """x [rows, H] f32 (this rank's rows) -> x + moe(rmsnorm(x)); `ops` is this rank's compute. Two collectives.

    ops.route(x) -> (rows16 [rows, H], idx [rows, topk] i32, wts [rows, topk] f32, sgate [rows] f32)
    ops.shared_begin(rows16) / ops.shared_end() -> shared [rows, H] f32   (may run beside the exchange)
    ops.pack(rows16, idx, cap) -> (send [N, block...], slot_of [rows * topk] i32); sets ops' overflow word when a block is full
    ops.experts(recv) -> y_send [N * cap, H] f32 in arrival order (rows of unused slots: anything)
    ops.combine(x, y_home, slot_of, wts, sgate, shared) -> x'             (fixed k order)
    ops.recv_like(send) / ops.home_like(y_send): buffers to receive into
    """
    exchange = getattr(ops, "exchange", None)  # an exchange of the ops' own (peer stores over NVLink) instead of the collective
    rows16, idx, wts, sgate = ops.route(x)
    ops.shared_begin(rows16)
    send, slot_of = ops.pack(rows16, idx, cap)
    recv = ops.recv_like(send)
    if exchange is None or not exchange(0, recv, send):
        _all_to_all(recv, send, group)
    y_send = ops.experts(recv)
    y_home = ops.home_like(y_send)
    if exchange is None or not exchange(1, y_home, y_send):
        _all_to_all(y_home, y_send, group)
    shared = ops.shared_end()
    return ops.combine(x, y_home, slot_of, wts, sgate, shared)


def pack_blocks(rows: torch.Tensor, idx: torch.Tensor, world: int, per: int, cap: int):
    """Device-agnostic packing with torch ops (what the CPU tests run; the GPU path is drb_ep_pack): the layout of the
    kernel with one id per element. Returns (send [world, cap + id rows, H], slot_of [pairs] i32, overflow bool);
    pair p = row * topk + k goes to block idx[p] // per, slots handed out in pair order."""
    h = rows.shape[1]
    id_rows = -(-cap // h)
    flat = idx.reshape(-1).to(torch.int64)
    owner = flat // per
    onehot = torch.nn.functional.one_hot(owner, world)
    rank_in_block = (torch.cumsum(onehot, 0) - onehot).gather(1, owner[:, None])[:, 0]
    fits = rank_in_block < cap
    send = rows.new_zeros((world, cap + id_rows, h))
    ids = torch.full((world, id_rows * h), float(per), dtype=rows.dtype)
    src = torch.arange(flat.numel()) // idx.shape[1]
    send[owner[fits], rank_in_block[fits]] = rows[src[fits]]
    ids[owner[fits], rank_in_block[fits]] = (flat - owner * per)[fits].to(rows.dtype)
    send[:, cap:] = ids.reshape(world, id_rows, h)
    slot_of = torch.where(fits, owner * cap + rank_in_block, owner * cap)
    return send, slot_of.to(torch.int32), bool((~fits).any())


def unpack_blocks(recv: torch.Tensor, cap: int):
    """(rows [world * cap, H], local expert ids [world * cap] i64) of a received buffer in pack_blocks' layout."""
    world, _, h = recv.shape
    rows = recv[:, :cap].reshape(world * cap, h)
    ids = recv[:, cap:].reshape(world, -1)[:, :cap].reshape(-1).to(torch.int64)
    return rows, ids


class EpGpu:
    """This rank's compute for ep_moe_block through the C ABI, on preallocated buffers (fixed addresses, so the
    launches can be captured). One workspace serves every layer of a stack: `layer` is switched per call. The
    kernels run on `st`, which is also made torch's current stream for the collectives (`stream`)."""

    def __init__(self, layer, rank: int, world: int, max_rows: int, cap: int, topk: int = 8, eps: float = 1e-6, st=None,
                 p2p: bool = True, group=None) -> None:
        import ctypes as C

        from . import ffi
        from .gpu import Stream, check

        self.C, self.l = C, ffi.lib()
        self.st = st or Stream()
        self.side = Stream()  # the shared expert runs here, beside the dispatch exchange
        check(self.l.drb_init(), "init")
        self.layer, self.rank, self.world, self.topk, self.eps, self.cap = layer, rank, world, topk, eps, cap
        e, h, i = layer.experts, layer.hidden, layer.inter
        self.per = per = e // world
        self.stream = torch.cuda.ExternalStream(self.st.raw.value)
        self.side_stream = torch.cuda.ExternalStream(self.side.raw.value)
        self.fork, self.join = torch.cuda.Event(), torch.cuda.Event()
        self.logit_bias = None  # optional [E] f32 tensor added to the router logits (the benchmark's Zipf routing)
        self.blk_rows = int(self.l.drb_ep_block_rows(cap, h * 2))
        n, r = world * cap, max_rows
        dev = "cuda"
        f32, f16, i32 = torch.float32, torch.float16, torch.int32
        self.rows16 = torch.empty((r, h), dtype=f16, device=dev)
        self.rlog = torch.empty((r, e + 1), dtype=f32, device=dev)
        self.idx = torch.empty((r, topk), dtype=i32, device=dev)
        self.wts = torch.empty((r, topk), dtype=f32, device=dev)
        self.sgate = torch.empty(r, dtype=f32, device=dev)
        self.sh_act = torch.empty((r, i), dtype=f16, device=dev)
        self.shared = torch.empty((r, h), dtype=f32, device=dev)
        self.sh_act2 = torch.empty((1, i), dtype=f16, device=dev)   # never written: stand-ins for the shared expert's buffers
        self.shared2 = torch.empty((1, h), dtype=f32, device=dev)   # in the launch that runs the routed experts only
        self.slot_of = torch.empty(r * topk, dtype=i32, device=dev)
        self.dst_row = torch.empty(r * topk, dtype=i32, device=dev)
        self.overflow_word = torch.zeros(1, dtype=i32, device=dev)
        # Row slots that are never written travel as they are: zero them once so that what travels is finite.
        self.send = torch.zeros((world, self.blk_rows, h), dtype=f16, device=dev)
        self.p2p = bool(p2p) and world > 1 and dist.is_initialized()
        self.exchange_kind = "all_to_all_single (NCCL)"
        if self.p2p:
            try:
                self._symmetric_buffers(world, n, h, dev, group)
                self.exchange_kind = ("peer stores over NVLink into symmetric memory, issued by the pack kernels and by the down GEMM's "
                                      "epilogue, + step flags (drb_ep_sync)")
            except Exception as exc:  # noqa: BLE001 - no symmetric memory on this system: the collective does the exchange
                self.p2p = False
                self.exchange_kind += f" (symmetric memory unavailable: {type(exc).__name__})"
        if not self.p2p:
            self.recv = torch.zeros((world, self.blk_rows, h), dtype=f16, device=dev)
        self.counts = torch.empty(per, dtype=i32, device=dev)
        self.offsets = torch.empty(per, dtype=i32, device=dev)
        self.slot2 = torch.empty(n, dtype=i32, device=dev)
        self.row_of = torch.empty(n, dtype=i32, device=dev)
        self.pair_of = torch.empty(n, dtype=i32, device=dev)
        self.ap = torch.empty((n, i), dtype=f16, device=dev)
        self.y_send = torch.zeros((n, h), dtype=f32, device=dev)
        if not self.p2p:
            self.y_home = torch.zeros((n, h), dtype=f32, device=dev)
        self.n_rows = 0

    def _symmetric_buffers(self, world: int, n: int, h: int, dev: str, group) -> None:
        """Receive buffers and flag words in symmetric memory, and the tables of every rank's addresses of them."""
        import torch.distributed._symmetric_memory as symm_mem

        g = group if group is not None else dist.group.WORLD
        self.recv = symm_mem.empty((world, self.blk_rows, h), dtype=torch.float16, device=dev)
        self.y_home = symm_mem.empty((n, h), dtype=torch.float32, device=dev)
        self.flags = symm_mem.empty((2, 64), dtype=torch.int32, device=dev)  # [dispatch | results][source rank]
        self.recv.zero_()
        self.y_home.zero_()
        self.flags.zero_()
        torch.cuda.synchronize()
        handles = [symm_mem.rendezvous(t, g) for t in (self.recv, self.y_home, self.flags)]
        i64 = torch.int64
        self.peer_bufs = [torch.tensor(list(hd.buffer_ptrs), dtype=i64, device=dev) for hd in handles[:2]]
        fl = list(handles[2].buffer_ptrs)
        self.peer_flags = [torch.tensor([p + 256 * which for p in fl], dtype=i64, device=dev) for which in (0, 1)]
        self.steps = torch.zeros(4, dtype=torch.int32, device=dev)  # signalled / awaited step of each direction
        self._handles = handles
        torch.cuda.synchronize()
        dist.barrier(group=g)  # nobody stores into a peer before that peer has cleared its flags

    def exchange(self, which: int, out: torch.Tensor, inp: torch.Tensor) -> bool:
        """Direction `which` (0: rows to the owners, 1: results home) by peer stores; False when this object uses the
        collective."""
        if not self.p2p:
            return False
        from .gpu import launched

        l, st = self.l, self.st.raw
        # the data is already in the peers' memory: the pack kernels and the down GEMM's epilogue store it there
        launched(l.drb_ep_sync(self._p(self.peer_flags[which]), self.C.c_void_p(self.flags.data_ptr() + 256 * which), self.world, self.rank,
                               self.C.c_void_p(self.steps.data_ptr() + 8 * which), 1 << 24, st), "ep_sync", debug=False)
        return True

    def _p(self, t: torch.Tensor):
        return self.C.c_void_p(t.data_ptr())

    def recv_like(self, send):
        return self.recv

    def home_like(self, y_send):
        return self.y_home

    def overflow(self) -> bool:
        """Reads and clears the overflow word (synchronises)."""
        v = bool(self.overflow_word.item())
        self.overflow_word.zero_()
        return v

    def route(self, x: torch.Tensor):
        from .gpu import launched

        l, st, ly = self.l, self.st.raw, self.layer
        n, h = x.shape
        e, topk = ly.experts, self.topk
        self.n_rows = n
        rows16, rlog, idx, wts, sgate = self.rows16[:n], self.rlog[:n], self.idx[:n], self.wts[:n], self.sgate[:n]
        launched(l.drb_rmsnorm_f16(self._p(x), ly.post_norm.at(0), self._p(rows16), n, h, self.eps, st), "rmsnorm_f16", debug=False)
        beta = 0.0
        if self.logit_bias is not None:  # the logits accumulate onto the bias rows
            rlog.zero_()
            rlog[:, :e] = self.logit_bias
            beta = 1.0
        # logits summed in a fixed order: the routing of a row does not depend on how many rows this rank holds
        launched(l.drb_router_logits_f16(self._p(rows16), ly.router.at(0), self._p(rlog), n, e + 1, h, beta, st), "router_logits_f16", debug=False)
        launched(l.dr_moe_topk(self._p(rlog), n, e, topk, e + 1, self._p(idx), self._p(wts), self._p(sgate), st), "moe_topk", debug=False)
        return rows16, idx, wts, sgate

    def shared_begin(self, rows16: torch.Tensor) -> None:
        from .gpu import launched

        ly, n = self.layer, rows16.shape[0]
        self.fork.record(self.stream)
        self.side_stream.wait_event(self.fork)
        sgq, sgs = ly.shared_gate_up.rows(0)
        sdq, sds = ly.shared_down.rows(0)
        gq, gs = ly.gate_up.expert(self.rank * self.per)
        dq, ds = ly.down.expert(self.rank * self.per)
        # E = 0: only the shared expert runs. Every pointer is still a valid device address (the arrays of the routed
        # part are simply not used): the kernel's loads must be safe to issue ahead of the branch that selects them.
        launched(self.l.drb_moe_prefill_block(gq, gs, dq, ds, sgq, sgs, sdq, sds, self._p(rows16), self._p(self.row_of), self._p(self.offsets),
                                              self._p(self.counts), self._p(self.ap), self._p(self.y_send), self._p(self.sh_act),
                                              self._p(self.shared), n, 0, ly.hidden, ly.inter, 1, self._p(self.pair_of), self.side.raw),
                 "shared expert", debug=False)
        self.join.record(self.side_stream)

    def shared_end(self) -> torch.Tensor:
        self.stream.wait_event(self.join)
        return self.shared[: self.n_rows]

    def pack(self, rows16: torch.Tensor, idx: torch.Tensor, cap: int):
        from .gpu import launched

        assert cap == self.cap
        n, h = rows16.shape
        pairs = n * self.topk
        if self.p2p:
            launched(self.l.drb_ep_pack_peers(self._p(rows16), self._p(idx), n, self.topk, self.per, self.world, cap, h * 2,
                                              self._p(self.peer_bufs[0]), self.rank, self._p(self.slot_of), self._p(self.dst_row),
                                              self._p(self.overflow_word), self.st.raw), "ep_pack_peers", debug=False)
            return self.send, self.slot_of[:pairs]
        launched(self.l.drb_ep_pack(self._p(rows16), self._p(idx), n, self.topk, self.per, self.world, cap, h * 2, self._p(self.send),
                                    self._p(self.slot_of), self._p(self.dst_row), self._p(self.overflow_word), self.st.raw), "ep_pack", debug=False)
        return self.send, self.slot_of[:pairs]

    def experts(self, recv: torch.Tensor) -> torch.Tensor:
        from .gpu import launched

        l, st, ly, per = self.l, self.st.raw, self.layer, self.per
        h = ly.hidden
        launched(l.drb_ep_group(self._p(recv), self.world, self.cap, h * 2, per, self._p(self.counts), self._p(self.offsets),
                                self._p(self.slot2), self._p(self.row_of), self._p(self.pair_of), st), "ep_group", debug=False)
        gq, gs = ly.gate_up.expert(self.rank * per)
        dq, ds = ly.down.expert(self.rank * per)
        sgq, sgs = ly.shared_gate_up.rows(0)
        sdq, sds = ly.shared_down.rows(0)
        # rows_sh = 0: only the routed experts run here (the shared expert is on the side stream); its pointers stay valid
        if self.p2p:
            launched(l.drb_moe_prefill_block_peers(gq, gs, dq, ds, sgq, sgs, sdq, sds, self._p(recv), self._p(self.row_of), self._p(self.offsets),
                                                   self._p(self.counts), self._p(self.ap), self._p(self.y_send), self._p(self.sh_act2),
                                                   self._p(self.shared2), 0, per, h, ly.inter, self._p(self.pair_of), self._p(self.peer_bufs[1]),
                                                   self.cap, self.rank, st), "moe_prefill_block_peers", debug=False)
            return self.y_send
        launched(l.drb_moe_prefill_block(gq, gs, dq, ds, sgq, sgs, sdq, sds, self._p(recv), self._p(self.row_of), self._p(self.offsets),
                                         self._p(self.counts), self._p(self.ap), self._p(self.y_send), self._p(self.sh_act2),
                                         self._p(self.shared2), 0, per, h, ly.inter, 1, self._p(self.pair_of), st), "moe_prefill_block", debug=False)
        return self.y_send

    def combine(self, x, y_home, slot_of, wts, sgate, shared):
        from .gpu import launched

        n, h = x.shape
        launched(self.l.dr_moe_combine(self._p(x), self._p(y_home), self._p(slot_of), self._p(wts), self._p(sgate),
                                       self._p(shared), n, self.topk, h, self.st.raw), "moe_combine", debug=False)
        return x
