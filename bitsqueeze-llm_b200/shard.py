"""Work partition for more than one GPU (one process per GPU).

The path shards over independent matrices (one activation matrix per layer or per batch entry):
matrix i goes to rank i % world, every rank compresses its own matrices on its own device through the
unchanged interface, and nothing crosses NVLink on the data path.  Only measurements are exchanged
(a barrier and a max over ranks)."""


def layers_for_rank(n_layers, rank, world):
    """Round-robin assignment: the matrices rank `rank` of `world` handles, in order."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank/world out of range")
    return list(range(rank, n_layers, world))


def max_over_ranks(values, device=None):
    """Element-wise maximum over all ranks of a list of floats (identity without a process group)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


def gather_objects(obj):
    """All ranks' objects, in rank order (a one-element list without a process group)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, obj)
        return out
    return [obj]
