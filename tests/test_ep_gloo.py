"""Expert-parallel dispatch / combine bookkeeping on CPU: world_size 2, 4 and 8 over gloo, with the numpy
oracle standing in for the per-rank kernels. The result must equal the single-process block; a capacity that is
too small must be reported, not waited on."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from drama_rs_b200 import ep, synth
from oracle import moe_oracle as orc

SHAPE = synth.MoeShape(experts=16, topk=4)
ROWS = 22


class OracleOps:
    def __init__(self, host, rank, world, cap):
        self.host, self.rank, self.world, self.per, self.cap = host, rank, world, SHAPE.experts // world, cap
        self.overflowed = False

    def route(self, x):
        xh = orc.rmsnorm(x.numpy(), self.host["post_norm"], SHAPE.eps).astype(np.float16).astype(np.float32)
        logits = orc.router_logits(self.host, xh, np.float64)
        idx, wts, sgate = orc.route(logits, SHAPE.experts, SHAPE.topk, np.float64)
        t = torch.from_numpy
        return t(xh.astype(np.float32)), t(idx), t(wts), t(sgate)

    def shared_begin(self, rows16):
        self.sh = torch.from_numpy(orc.shared_forward(self.host, rows16.numpy(), np.float64))

    def shared_end(self):
        return self.sh

    def pack(self, rows16, idx, cap):
        send, slot_of, over = ep.pack_blocks(rows16, idx, self.world, self.per, cap)
        self.overflowed |= over
        return send, slot_of

    def recv_like(self, send):
        return torch.empty_like(send)

    def home_like(self, y_send):
        return torch.empty_like(y_send)

    def experts(self, recv):
        rows, le = ep.unpack_blocks(recv, self.cap)
        le = le.numpy()
        y = np.full((rows.shape[0], SHAPE.hidden), np.nan)  # rows of unused slots must never reach the result
        for e in np.unique(le[le < self.per]):
            sel = np.nonzero(le == e)[0]
            y[sel] = orc.expert_forward(self.host, int(e) + self.rank * self.per, rows.numpy()[sel], np.float64)
        return torch.from_numpy(y)

    def combine(self, x, y_home, slot_of, wts, sgate, shared):
        return torch.from_numpy(orc.moe_combine(x.numpy(), y_home.numpy(), slot_of.numpy().reshape(-1, SHAPE.topk), wts.numpy(),
                                                sgate.numpy(), shared.numpy(), np.float64))


def worker(rank, world, port, out, cap):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    host = synth.make_layer(11, SHAPE)
    x = synth.make_x(11, ROWS, SHAPE.hidden)
    lo, hi = ROWS * rank // world, ROWS * (rank + 1) // world  # ragged split on purpose
    ops = OracleOps(host, rank, world, cap)
    y = ep.ep_moe_block(torch.from_numpy(x[lo:hi].copy()), ops, cap)
    np.save(os.path.join(out, f"y{rank}.npy"), y.numpy())
    np.save(os.path.join(out, f"over{rank}.npy"), np.array([ops.overflowed]))
    dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def reference():
    host = synth.make_layer(11, SHAPE)
    x = synth.make_x(11, ROWS, SHAPE.hidden)
    xh = orc.rmsnorm(x, host["post_norm"], SHAPE.eps).astype(np.float16).astype(np.float32)
    return x + orc.moe_block(host, xh.astype(np.float64), SHAPE.topk, np.float64)[0]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_block_matches_single_process(tmp_path, world):
    cap = -(-ROWS // world) * SHAPE.topk  # the worst case: the largest share of rows, all pairs to one owner
    mp.spawn(worker, args=(world, free_port(), str(tmp_path), cap), nprocs=world, join=True)
    y = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    ref = reference()
    assert np.abs(y - ref).max() <= 1e-9 * np.abs(ref).max()
    assert not any(np.load(tmp_path / f"over{r}.npy")[0] for r in range(world))


def test_ep_overflow_is_reported_not_waited_on(tmp_path):
    """With two slots per block some pairs find their block full: every rank still finishes the step (nothing
    waits), at least one rank reports the overflow, and with the capacity raised the step is exact again."""
    world = 2
    mp.spawn(worker, args=(world, free_port(), str(tmp_path), 2), nprocs=world, join=True)
    assert any(np.load(tmp_path / f"over{r}.npy")[0] for r in range(world))
    cap = ep.capacity(-(-ROWS // world), SHAPE.topk, world, factor=2.0)
    mp.spawn(worker, args=(world, free_port(), str(tmp_path), cap), nprocs=world, join=True)
    if not any(np.load(tmp_path / f"over{r}.npy")[0] for r in range(world)):
        y = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
        ref = reference()
        assert np.abs(y - ref).max() <= 1e-9 * np.abs(ref).max()


def test_pack_blocks_layout():
    idx = torch.tensor([[0, 5], [4, 1], [6, 7]], dtype=torch.int32)  # 8 experts, 2 ranks: owners 0 1 | 1 0 | 1 1
    rows = torch.arange(3, dtype=torch.float32)[:, None].repeat(1, 2)
    send, slot_of, over = ep.pack_blocks(rows, idx, world=2, per=4, cap=6)
    assert not over and slot_of.tolist() == [0, 6, 7, 1, 8, 9]
    got_rows, ids = ep.unpack_blocks(send, 6)
    assert ids.tolist() == [0, 1, 4, 4, 4, 4, 1, 0, 2, 3, 4, 4]
    assert got_rows[:, 0].tolist() == [0, 1, 0, 0, 0, 0, 0, 1, 2, 2, 0, 0]
    send, slot_of, over = ep.pack_blocks(rows, idx, world=2, per=4, cap=3)  # owner 1 gets four pairs: one is dropped
    assert over and slot_of.tolist() == [0, 3, 4, 1, 5, 3]
    assert ep.unpack_blocks(send, 3)[1].tolist() == [0, 1, 4, 1, 0, 2]


def test_owner_mapping_and_capacity():
    e = torch.tensor([0, 3, 4, 7, 15, 8])
    assert ep.owner_of(e, 16, 4).tolist() == [0, 0, 1, 1, 3, 2]
    assert ep.capacity(38, 8, 8, 3.0) == 114 and ep.capacity(300, 8, 1, 3.0) == 2400 and ep.capacity(8, 8, 2, 3.0) == 64
