"""One rank of the peer all-gather test (started by tests/test_peer_gpu.py with RANK / WORLD_SIZE / MASTER_* set)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from daceml_b200 import distributed as D, lib as L


def main():
    rank, world, local_rank = D.init_from_env(backend="nccl", timeout_s=60)
    dev = torch.device("cuda", local_rank)
    rows, cols = 96, 1000  # 192 000 bytes per rank: not a multiple of the kernel's stride, a multiple of 16
    peer = D.PeerGather((rows, cols), torch.float16, dev, rank, world)

    def block(r, step):
        return (torch.arange(rows * cols, dtype=torch.float32).view(rows, cols) % 251 + 1000 * r + step).half()

    def expected(step):
        return torch.cat([block(r, step) for r in range(world)])

    y = torch.empty(rows, cols, dtype=torch.float16, device=dev)
    for step in range(3):  # eager launches
        y.copy_(block(rank, step))
        out = peer.gather(y)
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), expected(step)), "rank %d: eager step %d" % (rank, step)
        dist.barrier()  # nobody starts the next step's copy into y ... (y is local; the barrier keeps the check and the next push apart)
    # the same launch inside a CUDA graph, replayed: the step counter lives on the device
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            peer.gather(y)
        for step in range(3, 6):
            y.copy_(block(rank, step))
            g.replay()
            side.synchronize()
            assert torch.equal(peer.gathered.cpu(), expected(step)), "rank %d: replay %d" % (rank, step)
            dist.barrier()
    assert L.get_context(dev).device_status() == 0
    g = None
    torch.cuda.synchronize()
    dist.barrier()
    peer.close()
    dist.destroy_process_group()
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
