"""MobileNetV1 through the network runner, layer by layer against the CPU checker."""
import numpy as np
import pytest

from conftest import pulpnn
from oracle.netref import mobilenet_chain

pytestmark = pytest.mark.gpu
wl = pulpnn.workloads
api = pulpnn.api


def _device_run(net, x, out_shape, out_dtype, n_layers=None):
    import torch
    dx = torch.from_numpy(x).cuda()
    dout = torch.zeros(out_shape, dtype={np.uint8: torch.uint8, np.int32: torch.int32}[out_dtype],
                       device="cuda")
    net.run(dx, dout, x.shape[0], n_layers)
    api.synchronize()
    return dout.cpu().numpy()


@pytest.mark.parametrize("shift_bias,micro", [(1, 0), (11, 2)])
def test_mobilenet_every_layer(shift_bias, micro, restatement):
    """shift_bias=11 is the benchmark's literal requantisation (activations die out after a few
    layers); shift_bias=1 keeps them alive through all 29 calls."""
    pulpnn.GpuKernels()
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=shift_bias)
    x = wl.mobilenet_input(5, 3)
    want = mobilenet_chain(restatement, params, x)
    net = api.build_mobilenet_v1(params, bits=32, max_batch=4, micro_batch=micro)
    assert net.num_layers() == 29
    for l, w in enumerate(want):
        got = _device_run(net, x, w.shape, w.dtype.type, n_layers=l + 1)
        assert np.array_equal(got, w), "layer %d (%s) differs" % (l, params[l]["name"])
    if shift_bias == 1:
        assert np.count_nonzero(want[-3]) > want[-3].size // 20     # still alive at pw13
        assert len(np.unique(want[-1])) > 100
    assert api.device_status() == 0
    # host buffers in and out give the same logits
    logits = np.zeros_like(want[-1])
    net.run(x, logits, x.shape[0])
    assert np.array_equal(logits, want[-1])
    net.close()


def test_batch_split_gives_identical_logits(restatement):
    """Sharding the batch (what multi-GPU runs do) cannot change any image's logits."""
    pulpnn.GpuKernels()
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
    x = wl.mobilenet_input(6, 6)
    net = api.build_mobilenet_v1(params, bits=32, max_batch=6)
    full = _device_run(net, x, (6, 1000), np.int32)
    parts = [_device_run(net, np.ascontiguousarray(x[i:i + 2]), (2, 1000), np.int32) for i in (0, 2, 4)]
    assert np.array_equal(full, np.concatenate(parts))
    assert np.array_equal(full[:1], mobilenet_chain(restatement, params, x[:1])[-1])
    net.close()


def test_mobilenet_at_the_benchmark_batch(restatement):
    """MobileNetV1 at batch 1024 -- the benchmark's own shape, where every kernel takes its
    large-batch branch (several images per depthwise CTA, full waves of GEMM tiles) -- with live
    parameters, from device memory and through the sliced host-input path. The logits of sampled
    images (first, last, the boundaries of the four host-input slices) must equal the CPU
    checker's, and every image's logits must equal the same image's logits in a batch of 8."""
    import torch
    pulpnn.GpuKernels()
    B = 1024
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
    x = wl.mobilenet_input(9, B)
    net = api.build_mobilenet_v1(params, bits=32, max_batch=B)
    dx = torch.from_numpy(x).cuda()
    dout = torch.zeros((B, 1000), dtype=torch.int32, device="cuda")
    net.run(dx, dout, B)
    api.synchronize()
    dev_logits = dout.cpu().numpy()
    host_logits = np.zeros((B, 1000), np.int32)
    net.run(x, host_logits, B)
    assert api.device_status() == 0
    assert np.array_equal(dev_logits, host_logits), "host-input path differs from the device-input path"
    sample = [0, 1, 127, 128, 255, 256, 257, 511, 512, 513, 767, 768, 769, 1000, 1022, 1023]
    want = mobilenet_chain(restatement, params, np.ascontiguousarray(x[sample]))[-1]
    assert len(np.unique(want)) > 100
    assert np.array_equal(dev_logits[sample], want), "batch-1024 logits differ from the CPU checker"
    # batch invariance: the same images in a small batch
    small = np.ascontiguousarray(x[504:512])
    dsmall = torch.zeros((8, 1000), dtype=torch.int32, device="cuda")
    net.run(torch.from_numpy(small).cuda(), dsmall, 8)
    api.synchronize()
    assert np.array_equal(dsmall.cpu().numpy(), dev_logits[504:512])
    net.close()


def test_mobilenet_prefixes_at_a_large_batch(restatement):
    """Layer-by-layer outputs at batch 160 (large enough for the several-images-per-CTA branch of
    the late depthwise layers) for four sampled images against the CPU checker."""
    import torch
    pulpnn.GpuKernels()
    B = 160
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
    x = wl.mobilenet_input(10, B)
    sample = [0, 79, 80, 159]
    want = mobilenet_chain(restatement, params, np.ascontiguousarray(x[sample]))
    net = api.build_mobilenet_v1(params, bits=32, max_batch=B)
    dx = torch.from_numpy(x).cuda()
    for l in (0, 1, 2, 3, 4, 6, 8, 10, 12, 14, 16, 24, 26, 27, 28):
        w = want[l]
        dout = torch.zeros((B,) + w.shape[1:], dtype={np.uint8: torch.uint8, np.int32: torch.int32}[w.dtype.type],
                           device="cuda")
        net.run(dx, dout, B, l + 1)
        api.synchronize()
        got = dout.cpu().numpy()[sample]
        assert np.array_equal(got, w), "layer %d (%s) differs at batch %d" % (l, params[l]["name"], B)
    assert api.device_status() == 0
    net.close()


def test_pipelined_host_batches_match_one_call_at_a_time(restatement):
    """pulpnn_net_submit / pulpnn_net_wait with two batches in flight: five different batches (sizes
    that change from one to the next) must give the logits of pulpnn_net_run, and the first image of
    every batch the CPU checker's."""
    import torch
    pulpnn.GpuKernels()
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
    net = api.build_mobilenet_v1(params, bits=32, max_batch=24)
    sizes = [24, 7, 16, 24, 1]
    xs = [torch.from_numpy(wl.mobilenet_input(30 + i, n)).pin_memory() for i, n in enumerate(sizes)]
    outs = [torch.full((n, 1000), -1, dtype=torch.int32).pin_memory() for n in sizes]
    prev = None
    for x, o, n in zip(xs, outs, sizes):
        t = net.submit(x, o, n)
        if prev is not None:
            net.wait(prev)
        prev = t
    net.wait(prev)
    assert api.device_status() == 0
    for i, (x, o, n) in enumerate(zip(xs, outs, sizes)):
        want = np.zeros((n, 1000), np.int32)
        net.run(x.numpy(), want, n)
        assert np.array_equal(o.numpy(), want), "batch %d differs from the one-call-at-a-time run" % i
        first = mobilenet_chain(restatement, params, x.numpy()[:1])[-1]
        assert np.array_equal(o.numpy()[:1], first)
    # device buffers are refused: they need no staging
    d = torch.zeros((1, 224, 224, 3), dtype=torch.uint8, device="cuda")
    with pytest.raises(pulpnn.PulpNNError):
        net.submit(d, outs[4], 1)
    net.close()
