"""The multi-rank path on CPU: two gloo ranks each take their slice of a batch, run the layer
chain (on the CPU checker here; on a GPU each rank runs the CUDA library), and all-gather the
logits. Sharding must not change any image's result, also when the batch does not divide evenly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import pulpnn

wl = pulpnn.workloads
sharding = __import__("importlib").import_module("pulpnn_b200.sharding")


def test_shard_bounds_cover_the_batch():
    for n in (0, 1, 7, 8, 1024, 1027):
        for world in (1, 2, 3, 8):
            cuts = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in cuts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 2, 2)


def _tiny_net(cpu, x):
    """conv 3x3 s2 -> depthwise 3x3 -> pointwise -> global average pool -> linear (int32)."""
    c = wl.conv_case(61, 16, 16, 3, 8, strides=(2, 2), batch=1, out_shift=7)
    d = wl.depthwise_case(62, 8, 8, 8, batch=1, out_shift=5, hwc=True)
    p = wl.pointwise_case(63, 8, 8, 8, 16, batch=1, out_shift=6)
    l = wl.linear_case(64, 16, 10, batch=1)
    y = cpu.conv(32, x, c["w"], c["k"], c["lam"], out_shift=7, out_hw=(8, 8), kernel=(3, 3),
                 pads=(1, 1, 1, 1), strides=(2, 2))
    y = cpu.depthwise(32, y, d["w"], d["k"], d["lam"], out_shift=5, out_hw=(8, 8), kernel=(3, 3),
                      pads=(1, 1, 1, 1), strides=(1, 1), in_is_hwc=True)
    y = cpu.pointwise(32, y, p["w"], p["k"], p["lam"], out_shift=6)
    y = cpu.avgpool(32, y, out_hw=(1, 1), kernel=(8, 8), pads=(0, 0, 0, 0), strides=(8, 8))
    return cpu.linear_out_32(np.ascontiguousarray(y.reshape(y.shape[0], -1)), l["w"])


def _worker(rank, world, port, n_images, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import bindings
        cpu = bindings.Restatement()
        x = np.random.default_rng(65).integers(0, 256, size=(n_images, 16, 16, 3), dtype=np.uint8)
        a, b = sharding.shard_bounds(n_images, rank, world)
        local = _tiny_net(cpu, np.ascontiguousarray(x[a:b])) if b > a else np.zeros((0, 10), np.int32)
        full = sharding.gather_rows(torch.from_numpy(local), n_images)
        if rank == 0:
            q.put(full.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_images", [6, 7])
def test_two_ranks_give_the_unsharded_logits(n_images, restatement):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_images, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.random.default_rng(65).integers(0, 256, size=(n_images, 16, 16, 3), dtype=np.uint8)
    want = _tiny_net(restatement, x)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert len(np.unique(want)) > 10
