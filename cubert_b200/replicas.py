"""Rank bookkeeping for running one model replica per process (one process per GPU).

The forward pass has no cross-GPU exchange: sequences are independent, every replica holds
the whole model, and the only things ranks ever agree on are which slice of the work each
one takes and, when measuring, the slowest rank's time. That is all this module does; it
works with any torch.distributed backend (NCCL on GPUs, gloo on CPU) and without one when
there is a single process. The in-process counterpart is BertM's round-robin over replicas
(src/cuBERT/BertM.cpp:69-76).
"""
import os


def rank_info():
    """(rank, local_rank, world_size) from the launcher's environment (torchrun)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def shard_range(total, rank, world):
    """[begin, end) of `total` independent units for `rank`: contiguous, sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError("bad shard request: total=%r rank=%r world=%r" % (total, rank, world))
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def stream_seed(base_seed, rank):
    """Seed of rank's own input stream (weak scaling: every rank draws its own batch)."""
    return base_seed + 1000 * rank


def _dist():
    try:
        import torch.distributed as dist
    except ImportError:
        return None
    return dist if dist.is_available() and dist.is_initialized() else None


def _reduce(value, op_name, device):
    dist = _dist()
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
    return float(t.item())


def max_over_ranks(value, device="cpu"):
    """The slowest rank's time: what a whole-job throughput has to be divided by."""
    return _reduce(value, "MAX", device)


def sum_over_ranks(value, device="cpu"):
    return _reduce(value, "SUM", device)


def job_throughput(units_this_rank, seconds_this_rank, device="cpu"):
    """Whole-job units per second: all ranks' units over the slowest rank's time."""
    total = sum_over_ranks(units_this_rank, device)
    slowest = max_over_ranks(seconds_this_rank, device)
    return total / slowest if slowest > 0 else float("inf")
