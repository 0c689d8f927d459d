"""Synchronized batch-norm across the GPUs of one node: host side.

One process per GPU (torch.distributed is the plumbing: it carries the 128-byte NCCL unique
id to the other ranks and nothing else; the per-step exchange is enqueued by the C ABI on the
caller's stream).  The reference has no synchronized batch-norm; its data-parallel training
keeps per-process statistics and all-reduces gradients through host memory
(src/proc_mpi.rs:138-148, src/ops_gpu.rs:538-545).

`shard_range` and `merge_moments` are plain host code (no GPU): the sharding rule of the
benchmark and a numpy restatement of the device-side merge, used by the CPU tests of the
multi-rank logic.
"""
import ctypes

import numpy as np

from . import _lib
from ._lib import check


def shard_range(extent, rank, world):
    """[lo, hi) of `extent` items owned by `rank`: contiguous, sizes differing by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world %d" % (rank, world))
    base, rem = divmod(extent, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def merge_moments(records):
    """Merges per-rank (count, mean, M2) records, shape [world, C, 3], in rank order in float64,
    exactly as the device merge does (two passes: weighted mean, then M2 about it).
    Returns (count, mean, M2) per channel."""
    r = np.asarray(records, dtype=np.float64)
    n = r[:, :, 0].sum(axis=0)
    mean = (r[:, :, 0] * r[:, :, 1]).sum(axis=0) / n
    d = r[:, :, 1] - mean[None, :]
    m2 = (r[:, :, 2] + r[:, :, 0] * d * d).sum(axis=0)
    return n, mean, m2


def local_moments(x):
    """(count, mean, M2) per channel of a local shard [N, C, *spatial] (float64, host)."""
    x64 = np.asarray(x, dtype=np.float64)
    ax = (0,) + tuple(range(2, x64.ndim))
    n = np.full(x64.shape[1], x64.size / x64.shape[1])
    mean = x64.mean(axis=ax)
    bs = (1, -1) + (1,) * (x64.ndim - 2)
    m2 = ((x64 - mean.reshape(bs)) ** 2).sum(axis=ax)
    return np.stack([n, mean, m2], axis=1)


def check_same_on_every_rank(values, what, group=None):
    """Host-side guard of the collective contract: every rank must bring the same `values` (e.g. the
    channel count of a synchronized layer).  All-gathers them over torch.distributed (any backend)
    and raises AnodeError(ANODE_E_COMM) on every rank when they differ, before anything is enqueued."""
    import torch
    import torch.distributed as dist
    from ._lib import AnodeError
    world = dist.get_world_size(group)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.tensor([int(v) for v in values], dtype=torch.int64, device=dev)
    allv = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allv, mine, group=group)
    if any(not torch.equal(a, allv[0]) for a in allv[1:]):
        raise AnodeError(-5, "%s differs across ranks: %s" % (what, [a.tolist() for a in allv]))


def wait_for_ranks(store, world, rank, key, timeout_s):
    """Bounded rendezvous on a torch.distributed store before the first synchronized call: every rank
    announces itself under `key` and waits until all `world` ranks have; a rank that never arrives
    turns into AnodeError(ANODE_E_COMM) after `timeout_s` seconds instead of a kernel that waits for
    its records."""
    import datetime
    from ._lib import AnodeError
    store.set("%s/%d" % (key, rank), "1")
    try:
        store.wait(["%s/%d" % (key, r) for r in range(world)], datetime.timedelta(seconds=timeout_s))
    except Exception as e:      # the store raises its own timeout type
        raise AnodeError(-5, "rendezvous %r: not all %d ranks arrived within %g s (%s)" % (key, world, timeout_s, type(e).__name__))


class SyncComm:
    """Communicator of the synchronized entry points (wraps AnodeSyncComm of the C ABI)."""

    def __init__(self, handle, rank, world):
        self.handle, self.rank, self.world = handle, rank, world

    @classmethod
    def from_torch_distributed(cls, group=None):
        """Collective over `group`: rank 0 creates the unique id, torch.distributed broadcasts it,
        every rank builds its communicator on its current CUDA device."""
        import torch
        import torch.distributed as dist
        lib = _lib.load()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = int(lib.anode_gpu_sync_unique_id_bytes())
        buf = (ctypes.c_ubyte * nbytes)()
        if rank == 0:
            check(lib.anode_gpu_sync_get_unique_id(buf), "anode_gpu_sync_get_unique_id")
        t = torch.tensor(list(buf), dtype=torch.uint8, device="cuda" if dist.get_backend(group) == "nccl" else "cpu")
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        raw = bytes(t.cpu().tolist())
        handle = ctypes.c_void_p()
        check(lib.anode_gpu_sync_comm_create(raw, rank, world, ctypes.byref(handle)), "anode_gpu_sync_comm_create")
        return cls(handle, rank, world)

    @classmethod
    def exchange_only(cls, rank, world):
        """A communicator without NCCL (anode_gpu_sync_comm_create_exchange_only): usable once
        attach_exchange_pointers has been given the world's buffers.  Nothing blocks on the host."""
        handle = ctypes.c_void_p()
        check(_lib.load().anode_gpu_sync_comm_create_exchange_only(rank, world, ctypes.byref(handle)),
              "anode_gpu_sync_comm_create_exchange_only")
        return cls(handle, rank, world)

    def attach_exchange_pointers(self, buffers, max_channels):
        """Hands the world's exchange buffers (CUDA uint8 tensors addressable from this process,
        indexed by rank, each of anode_gpu_sync_exchange_bytes bytes and zeroed once) to the C ABI."""
        ptrs = (ctypes.c_void_p * self.world)(*[int(b.data_ptr()) for b in buffers])
        check(_lib.load().anode_gpu_sync_comm_attach_exchange(self.handle, ptrs, max_channels),
              "anode_gpu_sync_comm_attach_exchange")
        self._exchange = (buffers, None)
        return self

    def attach_exchange(self, max_channels, group=None):
        """Collective: allocates a peer-visible exchange buffer on every rank (torch symmetric
        memory is the allocator and the rendezvous; it is not on the data path) and hands the
        world's pointers to the C ABI, which switches the synchronized calls to the one-kernel
        form with the exchange inside the kernel."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        lib = _lib.load()
        nbytes = int(lib.anode_gpu_sync_exchange_bytes(max_channels, self.world))
        if nbytes == 0:
            raise ValueError("exchange supports 1..8 ranks")
        buf = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        buf.zero_()
        hdl = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier(group)
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        check(lib.anode_gpu_sync_comm_attach_exchange(self.handle, ptrs, max_channels),
              "anode_gpu_sync_comm_attach_exchange")
        self._exchange = (buf, hdl)          # keep the mapping alive
        return self

    def allreduce_sum(self, buf):
        """In-place sum of a float32 CUDA tensor over the ranks, on the current stream: the
        device-side counterpart of SumSpmdOp's host-staged MPI_Allreduce (src/ops_gpu.rs:538-545)."""
        import torch
        if not (buf.is_cuda and buf.dtype == torch.float32 and buf.is_contiguous()):
            raise ValueError("expected a contiguous float32 CUDA tensor")
        stream = ctypes.c_void_p(torch.cuda.current_stream(buf.device).cuda_stream)
        check(_lib.load().anode_gpu_sync_allreduce_sum_f32(self.handle, ctypes.c_void_p(buf.data_ptr()),
                                                           buf.numel(), stream), "anode_gpu_sync_allreduce_sum_f32")
        return buf

    def destroy(self):
        if self.handle:
            _lib.load().anode_gpu_sync_comm_destroy(self.handle)
            self.handle = None
