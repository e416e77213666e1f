"""B200-native (sm_100a) implementation of the PULP-NN 8-bit HWC inference kernels.

The product is the C-ABI shared library built from ``csrc/`` (declared in ``include/``); this
package is the thin Python side of it: build/load (``_lib``), a mirror of the reference entry
points (``api``), an array-level front end for tests (``harness``) and the seeded synthetic
workloads (``workloads``).
"""
from . import workloads  # noqa: F401
from ._lib import build_library, load_library, load_dropin, declared_symbols  # noqa: F401
from . import api  # noqa: F401
from .api import PulpNNError  # noqa: F401
from .harness import GpuKernels  # noqa: F401


def smoke():
    """One small call of each hot-path kernel family on cuda:0, checked bit-for-bit against the
    CPU checker (oracle/): a pointwise layer on the tensor-core kernel, a 3x3 convolution, a
    depthwise layer in both layouts and a 3-layer network through the runner."""
    import numpy as np
    from oracle import bindings

    wl = workloads
    cpu = bindings.Restatement()
    gpu = GpuKernels(host_buffers=False)
    launches0 = api.launch_count()

    c = wl.pointwise_case(101, 28, 28, 128, 256, batch=4, bits=32, out_shift=10)
    want = cpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], out_shift=c["out_shift"])
    got = gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], out_shift=c["out_shift"])
    assert api.device_status() == 0, "a bounded wait in the tensor-core kernel ran out"
    assert np.array_equal(got, want), "pointwise (tensor-core path) differs from the checker"
    assert np.count_nonzero(want) > want.size // 10

    c = wl.conv_case(102, 32, 32, 32, 64, batch=2, bits=32, out_shift=12)
    kw = dict(out_shift=c["out_shift"], out_hw=c["out_hw"], kernel=c["kernel"], pads=c["pads"],
              strides=c["strides"])
    assert np.array_equal(gpu.conv(32, c["x"], c["w"], c["k"], c["lam"], **kw),
                          cpu.conv(32, c["x"], c["w"], c["k"], c["lam"], **kw)), "conv differs"

    for hwc in (False, True):
        c = wl.depthwise_case(103, 28, 28, 64, strides=(2, 2), batch=2, bits=64, out_shift=14,
                              w_range=(-64, 63), k_range=(1, 256), lam_range=(-2 ** 20, 2 ** 20),
                              hwc=hwc)
        kw = dict(out_shift=c["out_shift"], out_hw=c["out_hw"], kernel=c["kernel"], pads=c["pads"],
                  strides=c["strides"], in_is_hwc=hwc)
        assert np.array_equal(gpu.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **kw),
                              cpu.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **kw)), "depthwise differs"

    # a three-layer network through the runner: depthwise 3x3 -> pointwise -> global average pool
    rng = np.random.default_rng(104)
    B, H, Cc, Co = 4, 14, 64, 128
    x = rng.integers(0, 256, size=(B, H, H, Cc), dtype=np.uint8)
    dw = wl.depthwise_case(105, H, H, Cc, batch=1, bits=32, out_shift=9, hwc=True)
    pw = wl.pointwise_case(106, H, H, Cc, Co, batch=1, bits=32, out_shift=10)
    net = api.Net(32, B)
    net.add_layer(api.LAYER_DEPTHWISE, dim_in=(H, H), ch_in=Cc, dim_out=(H, H), ch_out=Cc, kernel=(3, 3),
                  pads=(1, 1, 1, 1), out_shift=9, weights=dw["w"], k=dw["k"], lam=dw["lam"])
    net.add_layer(api.LAYER_POINTWISE, dim_in=(H, H), ch_in=Cc, dim_out=(H, H), ch_out=Co, out_shift=10,
                  weights=pw["w"], k=pw["k"], lam=pw["lam"])
    net.add_layer(api.LAYER_AVGPOOL, dim_in=(H, H), ch_in=Co, dim_out=(1, 1), ch_out=Co, kernel=(H, H), strides=(H, H))
    net.finalize()
    got = np.zeros((B, 1, 1, Co), np.uint8)
    net.run(x, got, B)
    net.close()
    t = cpu.depthwise(32, x, dw["w"], dw["k"], dw["lam"], out_shift=9, out_hw=(H, H), kernel=(3, 3),
                      pads=(1, 1, 1, 1), strides=(1, 1), in_is_hwc=True)
    t = cpu.pointwise(32, t, pw["w"], pw["k"], pw["lam"], out_shift=10)
    t = cpu.avgpool(32, t, out_hw=(1, 1), kernel=(H, H), pads=(0, 0, 0, 0), strides=(H, H))
    assert np.array_equal(got, t), "the network runner differs from the chain of checker calls"
    assert np.count_nonzero(t) > t.size // 4
    assert api.device_status() == 0, "a bounded wait inside a kernel ran out"

    assert api.launch_count() > launches0, "no kernel of this library was launched"
    print("smoke ok: %d kernel launches, outputs identical to the CPU checker"
          % (api.launch_count() - launches0))
