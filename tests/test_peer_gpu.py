"""The all-gather over peer memory (``b200ml_peer_allgather``): one rank alone, and two ranks on two GPUs."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_one_rank_gathers_its_own_block_eagerly_and_in_a_replayed_graph():
    from daceml_b200 import lib as L
    dev = torch.device("cuda:0")
    ctx = L.get_context(dev)
    n = 3 * 1024 * 1024 + 16  # bytes; not a multiple of the kernel's stride
    storage = torch.zeros(n + 256, dtype=torch.uint8, device=dev)
    src = torch.randint(0, 255, (n, ), dtype=torch.uint8, device=dev)
    grp = L.PeerGroup()
    grp.rank, grp.world = 0, 1
    grp.gathered[0] = storage.data_ptr()
    grp.flags[0] = storage.data_ptr() + n
    for _ in range(2):
        L.check(ctx.lib.b200ml_peer_allgather(ctx.handle, ctypes.byref(grp), ctypes.c_void_p(src.data_ptr()), n, L.current_stream()))
    torch.cuda.synchronize()
    assert torch.equal(storage[:n], src)
    flags = storage[n:].view(torch.int32)
    assert int(flags[32]) == 2 and int(flags[33]) == 0, "two steps counted, arrival counter back at zero"
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            L.check(ctx.lib.b200ml_peer_allgather(ctx.handle, ctypes.byref(grp), ctypes.c_void_p(src.data_ptr()), n, L.current_stream()))
        for _ in range(3):
            src.add_(1)
            g.replay()
        side.synchronize()
    assert torch.equal(storage[:n], src)
    assert int(flags[32]) == 5
    assert ctx.device_status() == 0
    # a block that is not a multiple of 16 bytes is refused
    with pytest.raises(L.B200Error):
        L.check(ctx.lib.b200ml_peer_allgather(ctx.handle, ctypes.byref(grp), ctypes.c_void_p(src.data_ptr()), 24, L.current_stream()))


def test_ipc_export_reports_the_offset_inside_the_allocation():
    from daceml_b200 import lib as L
    dev = torch.device("cuda:0")
    ctx = L.get_context(dev)
    t = torch.zeros(4 << 20, dtype=torch.uint8, device=dev)
    handle = (ctypes.c_ubyte * 64)()
    off0, off1 = ctypes.c_int64(-1), ctypes.c_int64(-1)
    L.check(ctx.lib.b200ml_ipc_export(ctx.handle, ctypes.c_void_p(t.data_ptr()), handle, ctypes.byref(off0)))
    L.check(ctx.lib.b200ml_ipc_export(ctx.handle, ctypes.c_void_p(t.data_ptr() + 4096), handle, ctypes.byref(off1)))
    assert off0.value >= 0 and off1.value == off0.value + 4096
    assert any(handle), "an all-zero handle"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus():
    """Two processes, one GPU each: every rank's gathered buffer holds both blocks after each step, eagerly and from a
    replayed CUDA graph; nothing is left in the status word."""
    here = os.path.dirname(os.path.abspath(__file__))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29641",
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(here, "peer_worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=150)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n(timed out)"
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % rank in out, "rank %d:\n%s" % (rank, out[-3000:])
