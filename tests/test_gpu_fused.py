"""The fused depthwise + pointwise kernel (one kernel for a 3x3 stride-1 depthwise layer and the
pointwise layer behind it), through the network runner of the C ABI: bit-exact against the chain
of two CPU-checker calls and against the library's own two-kernel chain."""
import numpy as np
import pytest

from conftest import pulpnn

pytestmark = pytest.mark.gpu
wl = pulpnn.workloads
api = pulpnn.api

MODES = [(1, 1), (1, 0), (0, 0), (0, 1), (2, 0)]
SHAPES = [(32, 64, 1), (128, 128, 1), (256, 256, 1), (64, 128, 2), (128, 256, 2)]      # ch_in, ch_out, depthwise stride


@pytest.fixture(autouse=True)
def _clean():
    yield
    api.set_option(api.OPT_FUSE_DWPW, 1)
    assert api.device_status() == 0, "a bounded wait inside a kernel ran out"


def _pair(seed, H, W, C, N, bits, relu, bn, dw_shift=9, pw_shift=None, with_bias=True, stride=1):
    dw = wl.depthwise_case(seed, H, W, C, strides=(stride, stride), batch=1, bits=bits, out_shift=dw_shift,
                           with_bias=with_bias, out_mult=3, relu=relu, bn=bn, hwc=True)
    Ho, Wo = dw["out_hw"]
    pw = wl.pointwise_case(seed + 1, Ho, Wo, C, N, batch=1, bits=bits,
                           out_shift=(wl.ceil_log2(C) + 4) if pw_shift is None else pw_shift, with_bias=with_bias,
                           out_mult=5, relu=relu, bn=bn)
    return dw, pw


def _net(dw, pw, H, W, C, N, bits, relu, bn, max_batch):
    dt = np.int32 if bits == 32 else np.int64
    net = api.Net(bits, max_batch)
    Ho, Wo = dw["out_hw"]
    net.add_layer(api.LAYER_DEPTHWISE, dim_in=(H, W), ch_in=C, dim_out=(Ho, Wo), ch_out=C, kernel=(3, 3),
                  pads=(1, 1, 1, 1), strides=dw["strides"], out_mult=3, out_shift=dw["out_shift"], relu=relu, bn=bn,
                  weights=dw["w"], bias=dw["bias"], k=np.ascontiguousarray(dw["k"], dt),
                  lam=np.ascontiguousarray(dw["lam"], dt))
    net.add_layer(api.LAYER_POINTWISE, dim_in=(Ho, Wo), ch_in=C, dim_out=(Ho, Wo), ch_out=N, out_mult=5,
                  out_shift=pw["out_shift"], relu=relu, bn=bn, weights=pw["w"], bias=pw["bias"],
                  k=np.ascontiguousarray(pw["k"], dt), lam=np.ascontiguousarray(pw["lam"], dt))
    net.finalize()
    return net


def _chain(cpu, dw, pw, x, bits, relu, bn):
    t = cpu.depthwise(bits, x, dw["w"], dw["k"], dw["lam"], bias=dw["bias"], out_mult=3, out_shift=dw["out_shift"],
                      out_hw=dw["out_hw"], kernel=(3, 3), pads=(1, 1, 1, 1), strides=dw["strides"], relu=relu, bn=bn,
                      in_is_hwc=True)
    return t, cpu.pointwise(bits, t, pw["w"], pw["k"], pw["lam"], bias=pw["bias"], out_mult=5,
                            out_shift=pw["out_shift"], relu=relu, bn=bn)


def _run(net, x, N, out_hw=None):
    import torch
    B, H, W, _ = x.shape
    if out_hw is not None:
        H, W = out_hw
    out = torch.zeros((B, H, W, N), dtype=torch.uint8, device="cuda")
    net.run(torch.from_numpy(x).cuda(), out, B)
    api.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("C,N,stride", SHAPES)
def test_fused_pair_all_modes(C, N, stride, relu, bn, bits, restatement):
    """Every requantisation mode in both trees, on images that are smaller than a patch, not a
    multiple of it, and several patches wide and high."""
    pulpnn.GpuKernels()
    rng = np.random.default_rng(70 + C)
    for (H, W, B) in ((5, 4, 2), (19, 37, 3), (33, 30, 2)):
        if stride == 2 and W < 8:
            W = 9
        dw, pw = _pair(71, H, W, C, N, bits, relu, bn, stride=stride)
        x = rng.integers(0, 256, size=(B, H, W, C), dtype=np.uint8)
        mid, want = _chain(restatement, dw, pw, x, bits, relu, bn)
        net = _net(dw, pw, H, W, C, N, bits, relu, bn, B)
        api.set_option(api.OPT_FUSE_DWPW, 1)
        got = _run(net, x, N, dw["out_hw"])
        # flag_relu = 2 selects different modes in the two layers (the depthwise kernel tests the flag's
        # truth, the pointwise one compares it with 1: 32bit/src/pulp_nn_depthwise_generic.c:171,
        # pulp_nn_matmul.c:178), and a pair whose layers requantise differently is not fused
        fused = relu != 2
        assert [net.layer_role(0), net.layer_role(1)] == ([1, 2] if fused else [0, 0]), "unexpected kernel choice"
        assert np.array_equal(got, want), "fused kernel differs from the chain of checker calls (%dx%d)" % (H, W)
        api.set_option(api.OPT_FUSE_DWPW, 0)
        two = _run(net, x, N, dw["out_hw"])
        assert [net.layer_role(0), net.layer_role(1)] == [0, 0]
        assert np.array_equal(two, want)
        net.close()


@pytest.mark.parametrize("C,N,H,B,stride", [(32, 64, 112, 24, 1), (128, 128, 56, 40, 1), (256, 256, 28, 96, 1),
                                            (64, 128, 112, 20, 2), (128, 256, 56, 36, 2)])
def test_fused_pair_mobilenet_shapes_many_units(C, N, H, B, stride, restatement, reference32):
    """MobileNet's own pairs (dw1+pw1, dw2+pw2, dw3+pw3, dw5+pw5) with many more patches than SMs, live
    requantisation; sampled images also against the reference's own code."""
    pulpnn.GpuKernels()
    rng = np.random.default_rng(72)
    dw, pw = _pair(73, H, H, C, N, 32, 1, 1, with_bias=False, stride=stride)
    x = rng.integers(0, 256, size=(B, H, H, C), dtype=np.uint8)
    mid, want = _chain(restatement, dw, pw, x, 32, 1, 1)
    assert np.count_nonzero(want) > want.size // 10
    net = _net(dw, pw, H, H, C, N, 32, 1, 1, B)
    got = _run(net, x, N, dw["out_hw"])
    assert net.layer_role(0) == 1
    assert np.array_equal(got, want)
    for sl in (slice(0, 1), slice(B - 1, B)):
        _, ref = _chain(reference32, dw, pw, np.ascontiguousarray(x[sl]), 32, 1, 1)
        assert np.array_equal(got[sl], ref)
    # the prefix that ends on the depthwise layer cannot be fused and must still be right
    import torch
    out = torch.zeros((B,) + tuple(dw["out_hw"]) + (C,), dtype=torch.uint8, device="cuda")
    net.run(torch.from_numpy(x).cuda(), out, B, 1)
    api.synchronize()
    assert np.array_equal(out.cpu().numpy(), mid)
    net.close()


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", [(1, 1), (0, 0), (1, 0)])
def test_32_channel_pair_has_two_fused_kernels(bits, relu, bn, restatement):
    """The 32 -> 64 pair runs with its depthwise sums made by the builders' dp4a (the default) or by
    tensor-core MMAs (PULPNN_OPT_TUNE bit 5): both must equal the chain of checker calls, on images that are
    not a multiple of the 28 x 16 patch and on more patches than SMs (the tensor-core form takes widths that
    are a multiple of four pixels)."""
    pulpnn.GpuKernels()
    rng = np.random.default_rng(76)
    try:
        for (H, W, B) in ((21, 12, 3), (35, 60, 2), (112, 112, 4)):
            dw, pw = _pair(77, H, W, 32, 64, bits, relu, bn)
            x = rng.integers(0, 256, size=(B, H, W, 32), dtype=np.uint8)
            x[0, :3] = 255                      # saturated rows: the largest sums the layer can make
            _, want = _chain(restatement, dw, pw, x, bits, relu, bn)
            net = _net(dw, pw, H, W, 32, 64, bits, relu, bn, B)
            for tune, kernel in ((32, "dwpw_tcdw_kernel"), (0, "dwpw_fused_kernel")):
                api.set_option(api.OPT_TUNE, tune)
                got = _run(net, x, 64)
                assert net.layer_kernel(0) == kernel
                assert np.array_equal(got, want), "%s differs from the checker (%dx%d)" % (kernel, H, W)
            net.close()
    finally:
        api.set_option(api.OPT_TUNE, 0)


def test_mixed_modes_fall_back_to_two_kernels(restatement):
    """A pair whose layers requantise differently has no fused kernel: the runner must use two."""
    pulpnn.GpuKernels()
    H, W, C, N, B = 12, 16, 128, 128, 2
    dw, _ = _pair(74, H, W, C, N, 32, 1, 1)
    _, pw = _pair(74, H, W, C, N, 32, 0, 0)
    net = api.Net(32, B)
    net.add_layer(api.LAYER_DEPTHWISE, dim_in=(H, W), ch_in=C, dim_out=(H, W), ch_out=C, kernel=(3, 3),
                  pads=(1, 1, 1, 1), out_mult=3, out_shift=dw["out_shift"], relu=1, bn=1, weights=dw["w"],
                  bias=dw["bias"], k=dw["k"], lam=dw["lam"])
    net.add_layer(api.LAYER_POINTWISE, dim_in=(H, W), ch_in=C, dim_out=(H, W), ch_out=N, out_mult=5,
                  out_shift=pw["out_shift"], relu=0, bn=0, weights=pw["w"], bias=pw["bias"], k=pw["k"], lam=pw["lam"])
    net.finalize()
    x = np.random.default_rng(75).integers(0, 256, size=(B, H, W, C), dtype=np.uint8)
    t = restatement.depthwise(32, x, dw["w"], dw["k"], dw["lam"], bias=dw["bias"], out_mult=3,
                              out_shift=dw["out_shift"], out_hw=(H, W), kernel=(3, 3), pads=(1, 1, 1, 1),
                              strides=(1, 1), relu=1, bn=1, in_is_hwc=True)
    want = restatement.pointwise(32, t, pw["w"], pw["k"], pw["lam"], bias=pw["bias"], out_mult=5,
                                 out_shift=pw["out_shift"], relu=0, bn=0)
    got = _run(net, x, N)
    assert [net.layer_role(0), net.layer_role(1)] == [0, 0]
    assert np.array_equal(got, want)
    net.close()
