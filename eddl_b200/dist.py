"""Host-side plumbing for one-process-per-GPU data parallel runs.

torch.distributed (gloo) is used only to rendezvous, to hand rank 0's NCCL unique id to the other
ranks and to reduce timings; parameter traffic goes through the backend's own NCCL communicator
(``eddlb200_comm_init_rank`` / ``eddl_b200::avg_weights_distributed``).
"""
import os

import numpy as np


def shard_rows(global_batch, nranks, rank):
    """Rows [start, end) of the global batch that replica `rank` trains on.

    EDDL's partitioning (Net::resize, src/net/net_build.cpp:428-461; Net::train_batch,
    src/net/net_api.cpp:1261-1285): every replica gets floor(B/N) consecutive rows, the last one
    also takes the remainder."""
    if nranks < 1 or not 0 <= rank < nranks:
        raise ValueError("bad rank %d of %d" % (rank, nranks))
    if global_batch < nranks:
        raise ValueError("batch_size lower than computing service parallelism")
    per = global_batch // nranks
    start = rank * per
    end = global_batch if rank == nranks - 1 else start + per
    return start, end


def env_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


class RankFailure(RuntimeError):
    """A rank is missing, or the ranks do not agree on what they are about to exchange.  Raised on the host, before any
    collective has been enqueued on a GPU."""


def rendezvous(backend="gloo", timeout_s=None):
    """Initialises torch.distributed from the torchrun environment; returns (rank, world, local_rank).
    A rank that never joins ends the rendezvous of the others with RankFailure after `timeout_s` seconds
    (default: EDDL_B200_RENDEZVOUS_TIMEOUT or 600)."""
    rank, world, local = env_world()
    if world > 1:
        import datetime
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if timeout_s is None:
            timeout_s = float(os.environ.get("EDDL_B200_RENDEZVOUS_TIMEOUT", "600"))
        if not dist.is_initialized():
            try:
                dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
            except Exception as e:          # torch raises DistStoreError / DistNetworkError / RuntimeError depending on where it gave up
                raise RankFailure("rank %d: rendezvous of %d ranks did not complete within %.0f s (%s)" % (rank, world, timeout_s, type(e).__name__)) from e
    return rank, world, local


def check_same_layout(sizes, what="parameter tensors"):
    """Every rank must be about to exchange the same sequence of tensor sizes: a collective whose ranks disagree on the
    byte count never completes.  Compared over gloo on the host; RankFailure on EVERY rank when they differ."""
    rank, world, _ = env_world()
    if world == 1:
        return
    import zlib
    import torch
    import torch.distributed as dist
    sizes = [int(s) for s in sizes]
    mine = torch.tensor([len(sizes), sum(sizes), zlib.crc32(repr(sizes).encode())], dtype=torch.int64)
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    rows = [tuple(int(v) for v in t) for t in every]
    if len(set(rows)) != 1:
        raise RankFailure("%s differ between ranks (count, floats, checksum per rank): %s" % (what, rows))


def broadcast_bytes(payload, nbytes, src=0):
    """Every rank returns rank `src`'s `payload` (bytes of length nbytes)."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        return bytes(payload)
    t = torch.zeros(nbytes, dtype=torch.uint8)
    if dist.get_rank() == src:
        t = torch.frombuffer(bytearray(payload), dtype=torch.uint8).clone()
    dist.broadcast(t, src=src)
    return bytes(t.numpy().tobytes())


def share_unique_id(make_id):
    """Rank 0 calls make_id() -> 128 bytes (eddlb200_comm_unique_id); everyone gets the same bytes."""
    rank, world, _ = env_world()
    if world == 1:
        return make_id()
    return broadcast_bytes(make_id() if rank == 0 else b"", 128, src=0)


def max_over_ranks(value):
    if env_world()[1] == 1:
        return float(value)
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier():
    if env_world()[1] == 1:
        return
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def average_replicas_host(replicas):
    """Host statement of the averaging every rank must end up with (Net::sync_weights,
    src/net/net_func.cpp:111-127): fp32 sum in replica order, times 1.0f/N.  Used by tests."""
    acc = np.zeros_like(replicas[0], dtype=np.float32)
    for r in replicas:
        acc = (acc + np.asarray(r, np.float32)).astype(np.float32)
    return (acc * (np.float32(1.0) / np.float32(len(replicas)))).astype(np.float32)
