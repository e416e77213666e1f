"""Batch sharding across ranks (one process per GPU).

Images are independent, so a batch is cut into contiguous slices, one per rank; the layer stack
needs no communication. The only exchange of the whole path is the gather of the final logits.
Three forms of it live here:

* ``gather_rows``       a plain all-gather through ``torch.distributed`` (NCCL on GPUs, gloo in
                        the CPU tests), blocking the stream it is issued on;
* ``OverlappedGather``  the same collective on a side stream, under the next step's compute;
* ``PeerLogits``        no collective at all: every rank's last layer stores its rows straight
                        into the root rank's buffer through peer-mapped memory (ordinary global
                        stores over NVLink from the library's own kernel), so the gather is the
                        epilogue of the fully connected layer.
"""


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


class OverlappedGather:
    """The logits all-gather taken off the critical path: step i's rows are gathered on a side
    stream while step i+1 computes. Two local buffers alternate; a buffer is written again only
    once the gather that read it has finished. Outputs are preallocated."""

    def __init__(self, n_total, cols, dtype, rank, world, device, group=None):
        import torch
        self.torch, self.group = torch, group
        self.sizes = [shard_bounds(n_total, r, world) for r in range(world)]
        self.rows = max(b - a for a, b in self.sizes)
        self.local_rows = self.sizes[rank][1] - self.sizes[rank][0]
        self.locals = [torch.zeros((self.rows, cols), dtype=dtype, device=device) for _ in range(2)]
        self.outs = [torch.empty((world * self.rows, cols), dtype=dtype, device=device) for _ in range(2)]
        self.stream = torch.cuda.Stream(device=device)
        self.done = [None, None]
        self.i = 0

    def target(self):
        """Where this step's last layer writes (waits, on the current stream, for the gather that
        last read this buffer)."""
        b = self.i & 1
        if self.done[b] is not None:
            self.torch.cuda.current_stream().wait_event(self.done[b])
        return self.locals[b]

    def publish(self):
        """Call after the step's kernels are enqueued: gathers this step's rows on the side stream."""
        import torch.distributed as dist
        torch = self.torch
        b = self.i & 1
        ready = torch.cuda.Event()
        ready.record()
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            dist.all_gather_into_tensor(self.outs[b], self.locals[b], group=self.group)
            self.done[b] = torch.cuda.Event()
            self.done[b].record()
        self.i += 1

    def finish(self):
        """Makes the current stream wait for every gather issued so far; returns the last result."""
        self.torch.cuda.current_stream().wait_stream(self.stream)
        return self.outs[(self.i - 1) & 1]

    kind = "NCCL all-gather on a side stream, overlapped with the next step"


class PeerLogits:
    """The gather as the last layer's epilogue: rank r's rows [first_r, last_r) of the root's
    [n_total, cols] buffer are written by rank r's own kernel through a peer mapping of that
    buffer (torch symmetric memory: one allocation per rank, mapped into every rank). No kernel of
    one rank waits on another; completion is known on the root after the step's barrier."""

    def __init__(self, n_total, cols, dtype, rank, world, device, root=0, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.buffer = symm_mem.empty((n_total, cols), dtype=dtype, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        first, last = shard_bounds(n_total, rank, world)
        self.local_rows = last - first
        self.slice = self.handle.get_buffer(root, (last - first, cols), dtype, first * cols)
        self.root = root

    def target(self):
        return self.slice

    def publish(self):
        pass

    def finish(self):
        return self.buffer          # complete on the root once every rank's stream has drained

    kind = "last layer stores into the root rank's buffer through peer-mapped memory (NVLink), no collective"
