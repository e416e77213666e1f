"""Batch sharding across ranks (one process per GPU).

Images are independent, so a batch is cut into contiguous slices, one per rank; the layer stack
needs no communication. The only exchange of the whole path is the gather of the final logits,
which goes through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests)."""


def shard_bounds(n_items, rank, world):
    """[first, last) of the contiguous slice of rank `rank`; slices differ by at most one item."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside 0..%d" % (rank, world - 1))
    base, extra = divmod(n_items, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def gather_rows(local, n_total, group=None):
    """All-gather row slices produced with shard_bounds back into one [n_total, ...] tensor, in
    rank order, on every rank. Uneven slices are padded to the largest one for the collective."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return local
    sizes = [shard_bounds(n_total, r, world) for r in range(world)]
    biggest = max(b - a for a, b in sizes)
    padded = local
    if local.shape[0] < biggest:
        pad = torch.zeros((biggest - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=local.device)
        padded = torch.cat([local, pad])
    out = torch.empty((world * biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    if all(b - a == biggest for a, b in sizes):
        return out
    return torch.cat([out[r * biggest:r * biggest + (b - a)] for r, (a, b) in enumerate(sizes)])
