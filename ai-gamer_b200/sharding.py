"""Data-parallel plumbing of the frame path: the path shards by independent frames, so the only
inter-rank traffic is one broadcast of the checkpoint bytes at start-up and one max-reduction of the
timing at the end.  Backend-agnostic (NCCL on GPUs, gloo in the CPU tests)."""
import numpy as np


def shard_range(n_units, world, rank):
    """Contiguous slice [lo, hi) of n_units independent units (frames or frame sequences) owned by rank:
    the first n_units % world ranks take one extra unit."""
    if world <= 0 or not (0 <= rank < world) or n_units < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def broadcast_bytes(blob, nbytes, src=0, device="cpu"):
    """Rank `src` passes the checkpoint bytes, the others pass None; every rank returns the same bytes.
    One collective, before the step loop."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        if blob is None or len(blob) != nbytes:
            raise ValueError("single process needs the blob itself")
        return bytes(blob)
    if dist.get_rank() == src:
        if blob is None or len(blob) != nbytes:
            raise ValueError("source rank must supply %d bytes" % nbytes)
        t = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(device)
    else:
        t = torch.empty(nbytes, dtype=torch.uint8, device=device)
    dist.broadcast(t, src)
    return t.cpu().numpy().tobytes()


def max_over_ranks(values, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (the timing rule: a step takes as long as
    the slowest rank)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]
