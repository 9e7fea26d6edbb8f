"""Host-side helpers for running the path on several GPUs of one node (one process per GPU).

Batch sharding needs no communication: rows are independent, so a rank simply owns a contiguous block of
rows with their curand states, history and runtime arguments.  The vocabulary-parallel path exchanges one
fixed-size record per row (see vocab_parallel.py).
"""
import numpy as np


def shard_rows(batch, world_size, rank):
    """Contiguous block of rows owned by `rank`: (first_row, n_rows); sizes differ by at most one."""
    base, extra = divmod(batch, world_size)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def gather_rows(shard_logits, rows, n_shards, group=None):
    """Second round of the vocabulary-parallel path: the full-vocabulary logits of the rows the merge left
    undecided.  Every rank passes its own `[batch, shard]` tensor and the same `rows` (the merge is the same
    computation everywhere); one all-gather of `[len(rows), shard]` per rank, then the shards of a row are put
    side by side.  Returns `[len(rows), n_shards * shard]`.  Works on any backend (the CPU tests run it on gloo)."""
    import torch
    import torch.distributed as dist
    mine = shard_logits.index_select(0, rows).contiguous()
    parts = [torch.empty_like(mine) for _ in range(n_shards)]
    dist.all_gather(parts, mine, group=group)
    return torch.cat(parts, dim=1).contiguous()
