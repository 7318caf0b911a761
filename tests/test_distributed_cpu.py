"""The batch split and the single gather of the multi-GPU path, run as two gloo ranks on the CPU."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from daceml_b200 import distributed as D
    try:
        r, w, _ = D.init_from_env(backend="gloo", timeout_s=20)
        gen = torch.Generator().manual_seed(0)
        x_global = torch.randn(w * 3, 5, 7, generator=gen)
        if mode == "gather":
            model = lambda shard: shard * 2 + r  # noqa: E731  a per-rank stand-in for the layer stack
            y = D.ShardedEncoder(model, r, w)(x_global)
            expect = torch.cat([x_global[i * 3:(i + 1) * 3] * 2 + i for i in range(w)])
            ret[rank] = bool(torch.equal(y, expect))
        elif mode == "uneven":
            try:
                D.shard_batch(torch.zeros(w * 3 + 1, 2), r, w)
                ret[rank] = False
            except ValueError:
                ret[rank] = True
        elif mode == "rank_raises":
            # rank 1 fails before the gather; rank 0 must get an exception from the collective, not hang
            if r == 1:
                ret[rank] = True
                raise RuntimeError("injected failure before the gather")
            try:
                D.gather_outputs(torch.zeros(3, 4))
                ret[rank] = False
            except Exception:
                ret[rank] = True
        elif mode == "peer_unavailable":
            # without a GPU the peer all-gather cannot be set up: every rank gets the exception (none is left waiting in a
            # collective), and the NCCL / gloo gather still works afterwards
            try:
                D.PeerGather((3, 8), torch.float16, torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu"), r, w)
                ok = torch.cuda.is_available()
            except Exception:
                ok = not torch.cuda.is_available()
            y = D.gather_outputs(torch.full((2, 4), float(r)))
            ret[rank] = ok and bool(torch.equal(y, torch.cat([torch.full((2, 4), float(i)) for i in range(w)])))
        dist.barrier() if mode != "rank_raises" else None
    finally:
        if dist.is_initialized() and mode != "rank_raises":
            dist.destroy_process_group()


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        if p.is_alive():
            p.kill()
            pytest.fail("rank did not finish")
    return dict(ret)


def test_shard_and_gather_preserve_order():
    assert _run("gather") == {0: True, 1: True}


def test_uneven_batch_is_rejected():
    assert _run("uneven") == {0: True, 1: True}


def test_failed_rank_surfaces_as_exception():
    assert _run("rank_raises") == {0: True, 1: True}


def test_peer_gather_without_a_gpu_fails_on_every_rank_and_leaves_the_group_usable():
    assert _run("peer_unavailable") == {0: True, 1: True}


def test_single_process_paths():
    from daceml_b200 import distributed as D
    assert D.shard_bounds(64, 3, 8) == (24, 32)
    x = torch.arange(12.0).view(4, 3)
    assert torch.equal(D.gather_outputs(x), x)
    assert torch.equal(D.shard_batch(x, 1, 2), x[2:])
