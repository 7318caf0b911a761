"""Batch-sharded inference across the GPUs of one box.

The reference has no multi-device path at all.  Every operator on the path is independent across
the batch dimension, so each rank (one process per GPU, ``torch.distributed``) runs the whole
layer stack on its own samples with replicated weights and no per-layer collective; the outputs
are gathered once at the end (NCCL over NVLink / NVSwitch on GPUs, gloo in the CPU tests).
"""
import os

import torch
import torch.distributed as dist


def init_from_env(backend=None, timeout_s=120):
    """Joins the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.

    Returns ``(rank, world_size, local_rank)``; a single process without those variables is rank 0 of 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        import datetime
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
    return rank, world, local_rank


def bind_to_gpu_numa_node(local_rank):
    """Restricts this process to the CPU cores next to its GPU (NVML's CPU affinity of the device, intersected with the
    cores the process may already use), so that pinned host buffers allocated afterwards and the copy threads sit on
    the GPU's own NUMA node.  With one process per GPU this keeps eight ranks from pulling their host traffic through
    one socket.  Best effort: returns the number of cores bound to, or 0 if nothing was changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        index = local_rank
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if local_rank < len(ids) and ids[local_rank].isdigit():
                index = int(ids[local_rank])
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {i * 64 + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        allowed = near & set(os.sched_getaffinity(0))
        if not allowed or allowed == set(os.sched_getaffinity(0)):
            return 0
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return 0


def shard_bounds(global_batch, rank, world):
    """Rank r of R takes the contiguous samples [lo, hi); the batch must split evenly."""
    if global_batch % world != 0:
        raise ValueError("global batch {} does not split evenly over {} ranks".format(global_batch, world))
    per = global_batch // world
    return rank * per, (rank + 1) * per


def shard_batch(x_global, rank, world):
    lo, hi = shard_bounds(x_global.shape[0], rank, world)
    return x_global[lo:hi]


def gather_outputs(y_local, out=None, group=None):
    """All-gathers the per-rank outputs along the batch dimension, in rank order."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        if out is None:
            return y_local
        out.copy_(y_local)
        return out
    if out is None:
        out = torch.empty((world * y_local.shape[0], ) + tuple(y_local.shape[1:]), dtype=y_local.dtype,
                          device=y_local.device)
    y_local = y_local.contiguous()
    if hasattr(dist, "all_gather_into_tensor") and (y_local.is_cuda or dist.get_backend(group) != "gloo"):
        dist.all_gather_into_tensor(out, y_local, group=group)
    else:
        parts = list(out.chunk(world, dim=0))
        dist.all_gather(parts, y_local, group=group)
    return out


class ShardedEncoder:
    """Wraps a per-rank model (``model(x_shard) -> y_shard``) with the batch split and the final gather."""

    def __init__(self, model, rank, world, group=None):
        self.model, self.rank, self.world, self.group = model, rank, world, group

    def __call__(self, x_global, gather=True):
        y = self.model(shard_batch(x_global, self.rank, self.world))
        return gather_outputs(y, group=self.group) if gather else y


class PeerGather:
    """The final all-gather as one kernel per rank that stores its block into every peer's memory over NVLink
    (``b200ml_peer_allgather``), instead of an NCCL collective.

    Construction is collective: every rank allocates ``gathered`` (``[world * rows_per_rank, ...]``) and its flag
    words in one device allocation, exports it through CUDA IPC, exchanges handles with ``all_gather_object`` and maps
    the peers' allocations.  ``gather(y_local)`` launches the kernel on the current stream and returns ``gathered``; it
    may be captured in a CUDA graph.  Raises if the mapping cannot be set up (the caller then stays with NCCL)."""

    FLAG_BYTES = 256

    def __init__(self, shape_per_rank, dtype, device, rank, world, group=None):
        import ctypes
        from . import lib as L
        if world > L.MAX_PEERS:
            raise ValueError("at most {} ranks".format(L.MAX_PEERS))
        self.rank, self.world, self.group = rank, world, group
        self.ctx = L.get_context(device)
        per = 1
        for d in shape_per_rank:
            per *= int(d)
        self.bytes_per_rank = per * torch.empty((), dtype=dtype).element_size()
        if self.bytes_per_rank % 16:
            raise ValueError("the rank block must be a multiple of 16 bytes")
        total = world * self.bytes_per_rank
        # one allocation of its own (at least 2 MB: the caching allocator gives such a request its own segment), zeroed
        self.storage = torch.zeros(max(total + self.FLAG_BYTES, 2 << 20), dtype=torch.uint8, device=device)
        self.gathered = self.storage[:total].view(dtype).view((world * int(shape_per_rank[0]), ) + tuple(shape_per_rank[1:]))
        torch.cuda.synchronize(device)
        # every step below is collective: a rank that fails still takes part in the exchanges, and all ranks raise together
        mine = None
        try:
            handle = (ctypes.c_ubyte * 64)()
            offset = ctypes.c_int64(0)
            L.check(self.ctx.lib.b200ml_ipc_export(self.ctx.handle, ctypes.c_void_p(self.storage.data_ptr()), handle, ctypes.byref(offset)))
            mine = (bytes(handle), int(offset.value))
        except Exception:  # noqa: BLE001 - every rank learns of it from the None this rank sends
            mine = None
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        self._opened = []
        self.peers = L.PeerGroup()
        self.peers.rank, self.peers.world = rank, world
        problem = None
        if any(e is None for e in everyone):
            problem = "rank(s) {} could not export their buffer".format([r for r, e in enumerate(everyone) if e is None])
        else:
            try:
                for r in range(world):
                    if r == rank:
                        base = self.storage.data_ptr()
                    else:
                        h = (ctypes.c_ubyte * 64).from_buffer_copy(everyone[r][0])
                        ptr = ctypes.c_void_p()
                        L.check(self.ctx.lib.b200ml_ipc_open(self.ctx.handle, h, everyone[r][1], ctypes.byref(ptr)))
                        self._opened.append((ptr.value, everyone[r][1]))
                        base = ptr.value
                    self.peers.gathered[r] = base
                    self.peers.flags[r] = base + total
            except Exception as e:  # noqa: BLE001
                problem = "rank {}: {}".format(rank, e)
        # also the barrier behind the mapping: every rank has mapped every buffer before anyone stores into one
        problems = [None] * world
        dist.all_gather_object(problems, problem, group=group)
        if any(problems):
            self.close()
            raise RuntimeError("peer all-gather not available: " + "; ".join(p for p in problems if p))

    def gather(self, y_local):
        import ctypes
        from . import lib as L
        if not y_local.is_contiguous() or y_local.numel() * y_local.element_size() != self.bytes_per_rank:
            raise ValueError("the local block must be contiguous and of the size given at construction")
        L.check(self.ctx.lib.b200ml_peer_allgather(self.ctx.handle, ctypes.byref(self.peers), ctypes.c_void_p(y_local.data_ptr()),
                                                   self.bytes_per_rank, L.current_stream()))
        return self.gathered

    def close(self):
        """Unmaps the peers' allocations.  Collective in effect: call it on every rank once no launch is in flight."""
        for ptr, off in self._opened:
            self.ctx.lib.b200ml_ipc_close(self.ctx.handle, ptr, off)
        self._opened = []
