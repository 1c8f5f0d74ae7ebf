"""Expert parallelism on real GPUs: 1 and 2 ranks over NCCL, eager and replayed from a CUDA graph, every output row
and every routing index against the single-GPU block. The 2-rank case needs two GPUs; skipped otherwise."""

import os
import socket

import numpy as np
import pytest
import torch

from drama_rs_b200 import synth

pytestmark = pytest.mark.gpu

ROWS = 37
SHAPE = synth.MoeShape(experts=16)


def _watchdog(seconds: int = 120) -> None:
    """A rank that stops making progress dumps every thread's stack and exits instead of waiting forever."""
    import faulthandler
    import sys

    faulthandler.dump_traceback_later(seconds, exit=True, file=sys.stderr)


def worker(rank, world, port, out, cap, p2p=True):
    """One layer through ep_moe_block: eager once, then captured in a CUDA graph and replayed twice. p2p: the exchange by
    this library's peer stores (falls back to the collective where symmetric memory is unavailable), else NCCL."""
    import torch.distributed as dist

    _watchdog()

    from drama_rs_b200 import ep
    from drama_rs_b200.gpu import Stream
    from drama_rs_b200.model import MoeLayer

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    st = Stream()
    layer = MoeLayer.upload(synth.make_layer(11, SHAPE), st)
    x_all = synth.make_x(11, ROWS, SHAPE.hidden)
    lo, hi = ROWS * rank // world, ROWS * (rank + 1) // world
    max_rows = -(-ROWS // world)
    ops = ep.EpGpu(layer, rank, world, max_rows, cap, st=st, p2p=p2p)
    if rank == 0:
        print("exchange:", ops.exchange_kind, flush=True)
    with torch.cuda.stream(ops.stream):
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()
        ep.ep_moe_block(x, ops, cap)
        torch.cuda.synchronize()
        eager = x.cpu().numpy()
        idx = ops.idx[: hi - lo].cpu().numpy()
        over_eager = ops.overflow()
        x.copy_(x0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=ops.stream, capture_error_mode="thread_local"):
            ep.ep_moe_block(x, ops, cap)
        for _ in range(2):  # the second replay starts from the same input again
            x.copy_(x0)
            g.replay()
        torch.cuda.synchronize()
        replay = x.cpu().numpy()
        over_replay = ops.overflow()
        del g  # a live graph that holds captured collectives keeps the communicator busy at shutdown
    np.save(os.path.join(out, f"eager{rank}.npy"), eager)
    np.save(os.path.join(out, f"replay{rank}.npy"), replay)
    np.save(os.path.join(out, f"idx{rank}.npy"), idx)
    np.save(os.path.join(out, f"over{rank}.npy"), np.array([over_eager, over_replay]))
    if rank == 0:
        with open(os.path.join(out, "exchange.txt"), "w") as f:
            f.write(ops.exchange_kind)
    from tests.helpers import device_error_word

    assert device_error_word() == 0, "a bounded wait of the exchange ran out"
    dist.destroy_process_group()


def _single_gpu_reference():
    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import Stream
    from drama_rs_b200.model import MoeLayer

    st = Stream()
    layer = MoeLayer.upload(synth.make_layer(11, SHAPE), st)
    pre = MoePrefill(layer, ROWS, st=st)
    y = pre.run(synth.make_x(11, ROWS, SHAPE.hidden))
    return y, pre.idx.download(np.int32, ROWS * SHAPE.topk, st).reshape(ROWS, SHAPE.topk)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,p2p", [(1, True), (2, True), (2, False)])
def test_ep_eager_and_graph_match_the_single_gpu_block(tmp_path, world, p2p):
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from drama_rs_b200 import ep

    cap = ep.capacity(-(-ROWS // world), SHAPE.topk, world)
    mp.spawn(worker, args=(world, _free_port(), str(tmp_path), cap, p2p), nprocs=world, join=True)
    print("exchange:", open(tmp_path / "exchange.txt").read())
    ref, ref_idx = _single_gpu_reference()
    assert not any(np.load(tmp_path / f"over{r}.npy").any() for r in range(world))
    # the routing is the single-GPU routing, bit for bit, at every split
    assert np.array_equal(np.concatenate([np.load(tmp_path / f"idx{r}.npy") for r in range(world)]), ref_idx)
    for kind in ("eager", "replay"):
        y = np.concatenate([np.load(tmp_path / f"{kind}{r}.npy") for r in range(world)])
        # same kernels, same routing, sums in the same k order: the expert-parallel result is the single-GPU result
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max(), kind


def test_ep_overflow_word_on_the_gpu(tmp_path):
    """A capacity of two slots per block overflows: the step still completes, the word is set, the results are finite."""
    import torch.multiprocessing as mp

    mp.spawn(worker, args=(1, _free_port(), str(tmp_path), 2), nprocs=1, join=True)
    assert np.load(tmp_path / "over0.npy").all()
    assert np.isfinite(np.load(tmp_path / "eager0.npy")).all()
