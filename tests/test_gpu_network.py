"""MobileNetV1 through the network runner, layer by layer against the CPU checker."""
import numpy as np
import pytest

from conftest import pulpnn
from netref import mobilenet_chain

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
