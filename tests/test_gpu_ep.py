"""Expert parallelism on real GPUs: 2 ranks over NCCL, every output row against the single-GPU block.
Needs two GPUs; skipped otherwise."""

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


def _stage(rank: int, what: str) -> None:
    import sys

    print(f"[rank {rank}] {what}", file=sys.stderr, flush=True)


def fixed_worker(rank, world, port, out):
    """The fixed-capacity exchange: eager once, then the same layer captured in a CUDA graph and replayed."""
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
    cap = max_rows * SHAPE.topk
    ops = ep.EpGpuFixed(layer, rank, world, max_rows, cap, st=st)
    with torch.cuda.stream(ops.stream):
        x0 = torch.from_numpy(x_all[lo:hi].copy()).cuda()
        x = x0.clone()
        _stage(rank, "eager layer")
        ep.ep_moe_block_fixed(x, ops, SHAPE.experts, SHAPE.topk, cap)
        torch.cuda.synchronize()
        eager = x.cpu().numpy()
        x.copy_(x0)
        _stage(rank, "capture")
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=ops.stream, capture_error_mode="thread_local"):
            ep.ep_moe_block_fixed(x, ops, SHAPE.experts, SHAPE.topk, cap)
        _stage(rank, "replay")
        for _ in range(2):  # the second replay starts from the same input again
            x.copy_(x0)
            g.replay()
        torch.cuda.synchronize()
        replay = x.cpu().numpy()
        _stage(rank, "done")
        del g
    np.save(os.path.join(out, f"eager{rank}.npy"), eager)
    np.save(os.path.join(out, f"replay{rank}.npy"), replay)
    dist.destroy_process_group()


def _single_gpu_reference():
    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import Stream
    from drama_rs_b200.model import MoeLayer

    st = Stream()
    layer = MoeLayer.upload(synth.make_layer(11, SHAPE), st)
    return MoePrefill(layer, ROWS, st=st).run(synth.make_x(11, ROWS, SHAPE.hidden))


@pytest.mark.parametrize("world", [1, 2])
def test_ep_fixed_capacity_eager_and_graph(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(fixed_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    ref = _single_gpu_reference()
    for kind in ("eager", "replay"):
        y = np.concatenate([np.load(tmp_path / f"{kind}{r}.npy") for r in range(world)])
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max(), kind


def worker(rank, world, port, out):
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
    host = synth.make_layer(11, SHAPE)
    layer = MoeLayer.upload(host, st)
    x = synth.make_x(11, ROWS, SHAPE.hidden)
    lo, hi = ROWS * rank // world, ROWS * (rank + 1) // world
    ops = ep.EpGpuOps(layer, rank, world, ROWS, st=st)
    with torch.cuda.stream(ops.stream):
        y = ep.ep_moe_block(torch.from_numpy(x[lo:hi].copy()).cuda(), ops, SHAPE.experts, SHAPE.topk)
        torch.cuda.synchronize()
    np.save(os.path.join(out, f"y{rank}.npy"), y.cpu().numpy())
    dist.destroy_process_group()


def test_ep_two_gpus_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from drama_rs_b200.engine import MoePrefill
    from drama_rs_b200.gpu import Stream
    from drama_rs_b200.model import MoeLayer

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    y = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(2)])
    st = Stream()
    layer = MoeLayer.upload(synth.make_layer(11, SHAPE), st)
    ref = MoePrefill(layer, ROWS, st=st).run(synth.make_x(11, ROWS, SHAPE.hidden))
    # same kernels, same routing, sums in the same k order: the expert-parallel result is the single-GPU result
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
