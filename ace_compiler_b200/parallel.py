"""Host logic of the multi-GPU arrangement: independent encrypted images are
dealt out to ranks (one process per GPU, no data-path communication, as the
reference's OpenMP loop over images does within one process), and a job's time
is the slowest rank's time.

Works on any torch.distributed backend: NCCL on the GPUs, gloo in the CPU
tests.
"""
import os


def rank_world():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def images_of_rank(total, rank, world):
    """Indices of the images rank `rank` infers when `total` images are dealt
    out round-robin over `world` ranks."""
    return list(range(rank, total, world))


def slowest_rank(values, device="cpu"):
    """Element-wise maximum of a list of per-rank floats over all ranks."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [float(v) for v in values]
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def job_throughput(items_per_rank, world, slowest_ms):
    """Whole-job items per second when every rank processed items_per_rank items
    and the slowest rank needed slowest_ms milliseconds."""
    return items_per_rank * world / (slowest_ms * 1e-3)


def gather_logits(local, device="cpu"):
    """All ranks' result vectors on every rank: the only exchange of the job,
    after the encrypted work is done (a few dozen bytes per image)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [list(local)]
    t = torch.tensor(list(local), dtype=torch.float64, device=device)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [x.tolist() for x in out]
