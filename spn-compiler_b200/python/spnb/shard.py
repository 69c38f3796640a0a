"""Batch sharding across GPUs: samples are independent and the model is read-only, so the batch is
cut into contiguous row blocks, one per rank (or per device of one process), and nothing is exchanged
on the data path.  The only collective is the optional dataset-mean log-likelihood."""


def shard_rows(n, world, rank, align=1024):
    """Rows [r0, r1) of an n-row batch owned by `rank` of `world`: equal blocks rounded up to `align`
    rows (so every shard starts on a tile boundary), the last ones possibly shorter or empty.  Same rule
    as the C++ sharder behind spnb_execute_sharded."""
    per = (n + world - 1) // world
    per = (per + align - 1) // align * align
    r0 = min(n, rank * per)
    return r0, min(n, r0 + per)


def dataset_mean(local_sum, local_count, group=None):
    """Mean log-likelihood over all ranks: one all-reduce of (sum, count) in float64.
    Works on whichever backend the process group uses (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(local_sum), float(local_count)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t[0].item() / max(t[1].item(), 1.0))


def max_over_ranks(value, group=None):
    """Largest `value` over all ranks (used for the device time of a multi-GPU step)."""
    import torch
    import torch.distributed as dist
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
