"""Expert-parallel dispatch / combine bookkeeping on CPU: world_size 2 and 4 over gloo, with the numpy
oracle standing in for the per-rank kernels. The result must equal the single-process block."""

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
    def __init__(self, host, rank, world):
        self.host, self.rank, self.per = host, rank, SHAPE.experts // world

    def route(self, x):
        xh = orc.round_bf16(orc.rmsnorm(x.numpy(), self.host["post_norm"], SHAPE.eps))
        logits = orc.router_logits(self.host, xh, np.float64)
        idx, wts, sgate = orc.route(logits, SHAPE.experts, SHAPE.topk, np.float64)
        shared = orc.shared_forward(self.host, xh, np.float64)
        t = torch.from_numpy
        return t(xh.astype(np.float32)), t(idx), t(wts), t(sgate), t(shared)

    def experts(self, rows, local_expert):
        y = np.zeros((rows.shape[0], SHAPE.hidden))
        le = local_expert.numpy()
        for e in np.unique(le):
            sel = np.nonzero(le == e)[0]
            y[sel] = orc.expert_forward(self.host, int(e) + self.rank * self.per, rows.numpy()[sel], np.float64)
        return torch.from_numpy(y)

    def pack(self, hn_b, idx, cap):
        return ep.pack_fixed(hn_b, idx, SHAPE.experts // self.per, self.per, cap)

    def experts_padded(self, rows, local_expert):
        le = local_expert.numpy()
        y = np.full((rows.shape[0], SHAPE.hidden), np.nan)  # padding rows must never reach the result
        real = np.nonzero(le < self.per)[0]
        y[real] = self.experts(rows[real], local_expert[real]).numpy()
        return torch.from_numpy(y)

    def combine(self, x, y_home, slot_of, wts, sgate, shared):
        return torch.from_numpy(orc.moe_combine(x.numpy(), y_home.numpy(), slot_of.numpy().reshape(-1, SHAPE.topk), wts.numpy(),
                                                sgate.numpy(), shared.numpy(), np.float64))


def worker(rank, world, port, out, fixed=False):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    host = synth.make_layer(11, SHAPE)
    x = synth.make_x(11, ROWS, SHAPE.hidden)
    lo, hi = ROWS * rank // world, ROWS * (rank + 1) // world  # ragged split on purpose
    ops = OracleOps(host, rank, world)
    if fixed:
        cap = -(-ROWS // world) * SHAPE.topk  # the same on every rank: the largest share of rows, all pairs to one owner
        y = ep.ep_moe_block_fixed(torch.from_numpy(x[lo:hi].copy()), ops, SHAPE.experts, SHAPE.topk, cap)
    else:
        y = ep.ep_moe_block(torch.from_numpy(x[lo:hi].copy()), ops, SHAPE.experts, SHAPE.topk)
    np.save(os.path.join(out, f"y{rank}.npy"), y.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("fixed", [False, True], ids=["split-sizes", "fixed-capacity"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_block_matches_single_process(tmp_path, world, fixed):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(worker, args=(world, port, str(tmp_path), fixed), nprocs=world, join=True)
    y = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    host = synth.make_layer(11, SHAPE)
    x = synth.make_x(11, ROWS, SHAPE.hidden)
    xh = orc.round_bf16(orc.rmsnorm(x, host["post_norm"], SHAPE.eps))
    ref = x + orc.moe_block(host, xh.astype(np.float64), SHAPE.topk, np.float64)[0]
    assert np.abs(y - ref).max() <= 1e-9 * np.abs(ref).max()


def test_pack_fixed_layout():
    idx = torch.tensor([[0, 5], [4, 1], [6, 7]], dtype=torch.int32)  # 8 experts, 2 ranks: owners 0 1 | 1 0 | 1 1
    rows = torch.arange(3, dtype=torch.float32)[:, None].repeat(1, 2)
    send_rows, send_e, slot_of = ep.pack_fixed(rows, idx, world=2, per=4, cap=6)
    assert slot_of.tolist() == [0, 6, 7, 1, 8, 9]
    assert send_e.tolist() == [0, 1, 4, 4, 4, 4, 1, 0, 2, 3, 4, 4]
    assert send_rows[:, 0].tolist() == [0, 1, 0, 0, 0, 0, 0, 1, 2, 2, 0, 0]


def test_plan_owner_mapping():
    e = torch.tensor([0, 3, 4, 7, 15, 8])
    assert ep.owner_of(e, 16, 4).tolist() == [0, 0, 1, 1, 3, 2]
