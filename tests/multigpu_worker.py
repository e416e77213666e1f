"""One rank of the two-GPU sharding test (launched by test_gpu_multigpu.py through
torch.distributed.run): MobileNetV1 on this rank's slice of a batch, the logits gathered on rank 0
by each of the three gather forms, compared there with a one-GPU run of the whole batch and with
the CPU checker. Prints MULTIGPU-OK on rank 0 when everything matched."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import __graft_entry__ as entry  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    api, wl = pkg.api, pkg.workloads
    sharding = __import__("importlib").import_module("pulpnn_b200.sharding")
    api.set_device(local)
    G = 50                                              # uneven over 4 ranks, even over 2
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
    x = wl.mobilenet_input(21, G)
    first, last = sharding.shard_bounds(G, rank, world)
    B = last - first
    net = api.build_mobilenet_v1(params, bits=32, max_batch=G)
    xs = torch.from_numpy(np.ascontiguousarray(x[first:last])).cuda()
    results = {}

    peer = sharding.PeerLogits(G, 1000, torch.int32, rank, world, dev)
    net.run(xs, peer.target(), B)
    peer.publish()
    api.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    results["peer"] = peer.finish().cpu().numpy() if rank == 0 else None

    if all(b - a == B for a, b in (sharding.shard_bounds(G, r, world) for r in range(world))):
        ov = sharding.OverlappedGather(G, 1000, torch.int32, rank, world, dev)
        for _ in range(3):                              # three steps through the two alternating buffers
            net.run(xs, ov.target()[:B], B)
            ov.publish()
        got = ov.finish()
        torch.cuda.synchronize()
        results["overlapped"] = got.cpu().numpy()[:G]

    local_logits = torch.zeros((B, 1000), dtype=torch.int32, device="cuda")
    net.run(xs, local_logits, B)
    api.synchronize()
    results["all_gather"] = sharding.gather_rows(local_logits, G).cpu().numpy()
    assert api.device_status() == 0

    if rank == 0:
        whole = torch.zeros((G, 1000), dtype=torch.int32, device="cuda")
        net.run(torch.from_numpy(x).cuda(), whole, G)
        api.synchronize()
        whole = whole.cpu().numpy()
        for name, got in results.items():
            assert got is not None and np.array_equal(got, whole), "%s gather differs from the one-GPU run" % name
        from oracle import bindings
        from oracle.netref import mobilenet_chain
        sample = [0, first, last - 1, G - 1]
        want = mobilenet_chain(bindings.Restatement(), params, np.ascontiguousarray(x[sample]))[-1]
        assert np.array_equal(whole[sample], want), "logits differ from the CPU checker"
        assert len(np.unique(want)) > 100
        print("MULTIGPU-OK %s" % ",".join(sorted(results)), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
