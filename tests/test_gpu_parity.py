"""Bit-exact parity of the CUDA kernels with the CPU checker, through the C ABI.

Integer arithmetic only, so the bar is byte equality (tolerance 0). Every case runs the seeded
inputs through the C restatement (and, where oracle/_ref was built, spot-checks against the
compiled reference itself) and through the library with device pointers; a subset repeats with
host pointers (the staged path) and with the tensor-core kernel switched off, so both contraction
kernels are held to the same checker.
"""
import numpy as np
import pytest

from conftest import pulpnn

pytestmark = pytest.mark.gpu
wl = pulpnn.workloads
api = pulpnn.api

MODES = [(1, 1), (1, 0), (0, 0), (0, 1), (2, 0)]


@pytest.fixture(scope="module")
def gpu():
    return pulpnn.GpuKernels(host_buffers=False)


@pytest.fixture(scope="module")
def gpu_host():
    return pulpnn.GpuKernels(host_buffers=True)


@pytest.fixture(autouse=True)
def _clean_status():
    yield
    assert api.device_status() == 0, "a bounded wait inside a tensor-core kernel ran out"
    api.set_option(api.OPT_FORCE_GENERIC, 0)
    api.set_option(api.OPT_SPLIT_K, 0)


def conv_kw(c):
    return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])


def pw_kw(c):
    return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"],
                bn=c["bn"])


def same(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError("%d of %d bytes differ; first at %s: got %d want %d"
                             % (len(bad), a.size, tuple(bad[0]), a[tuple(bad[0])], b[tuple(bad[0])]))


# ---- the five configurations against both checkers ----------------------------------------------
@pytest.fixture(params=["restatement", "reference"])
def checker(request, restatement):
    """The CPU side of a comparison: our restatement, or the reference's own code compiled in
    place (skipped where that library was not built)."""
    if request.param == "restatement":
        return lambda bits: restatement
    r32, r64 = request.getfixturevalue("reference32"), request.getfixturevalue("reference64")
    return lambda bits: r32 if bits == 32 else r64


def test_configurations_against_both_checkers(checker, gpu):
    """Configurations 1-4 (literal and live requantisation) and the pooling / add kernels, GPU
    against the restatement AND against the compiled reference, in the GPU run itself."""
    for shift in (None, 12):
        c = wl.conv_case(0, 32, 32, 32, 64, bits=32, out_shift=shift, batch=2)
        same(gpu.conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)),
             checker(32).conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)))
    for shift in (None, 10):
        c = wl.pointwise_case(1, 56, 56, 128, 256, batch=3, bits=32, out_shift=shift)
        same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)),
             checker(32).pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)))
    c = wl.config_c3(batch=3)
    same(gpu.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)),
         checker(64).depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)))
    c = wl.config_c4(batch=6)
    for shift in (c["out_shift"], 14):
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=shift, relu=c["relu"], bn=c["bn"])
        same(gpu.linear(32, c["x"], c["w"], c["k"], c["lam"], **kw),
             checker(32).linear(32, c["x"], c["w"], c["k"], c["lam"], **kw))
    same(gpu.linear_out_32(c["x"], c["w"], bias32=c["bias32"]),
         checker(32).linear_out_32(c["x"], c["w"], bias32=c["bias32"]))
    # MobileNet's own pair shapes with live parameters
    c = wl.depthwise_case(61, 28, 28, 256, batch=5, bits=32, out_shift=9, hwc=True)
    same(gpu.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)),
         checker(32).depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)))
    c = wl.pointwise_case(62, 14, 14, 512, 512, batch=4, bits=32, out_shift=12)
    same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)),
         checker(32).pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)))
    rng = np.random.default_rng(63)
    x = rng.integers(0, 256, size=(3, 7, 7, 1024), dtype=np.uint8)
    pk = dict(out_hw=(1, 1), kernel=(7, 7), pads=(0, 0, 0, 0), strides=(7, 7))
    same(gpu.avgpool(32, x, **pk), checker(32).avgpool(32, x, **pk))
    a = rng.integers(0, 256, size=(2, 9, 9, 48), dtype=np.uint8)
    b = rng.integers(0, 256, size=(2, 9, 9, 48), dtype=np.uint8)
    same(gpu.add(a, b, m1=37, m2=91, out_shift=6), checker(32).add(a, b, m1=37, m2=91, out_shift=6))


# ---- standard convolution ------------------------------------------------------------------
@pytest.mark.parametrize("variant", ["Ho", "HoWo"])
def test_conv_config1_literal(variant, gpu, restatement):
    c = wl.config_c1()
    want = restatement.conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
    same(gpu.conv(32, c["x"], c["w"], c["k"], c["lam"], variant=variant, **conv_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
def test_conv_config1_live_parameters(bits, gpu, gpu_host, restatement):
    c = wl.conv_case(0, 32, 32, 32, 64, bits=bits, out_shift=12, batch=3, with_bias=True)
    want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
    assert np.count_nonzero(want) > want.size // 10
    same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)
    same(gpu_host.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_conv_ragged_all_modes(bits, relu, bn, gpu, restatement):
    c = wl.conv_case(11, 13, 11, 5, 7, kernel=(3, 5), strides=(2, 1), pads=(1, 0, 2, 1), batch=3,
                     bits=bits, out_shift=9, with_bias=True, out_mult=5, relu=relu, bn=bn,
                     k_range=(-64, 64), lam_range=(-2 ** 20, 2 ** 20))
    want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
    same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)


def test_conv_bn_wraparound(gpu, restatement):
    for bits in (32, 64):
        c = wl.conv_case(12, 9, 9, 16, 8, bits=bits, out_shift=12, w_range=(-128, 127),
                         k_range=(2 ** 20, 2 ** 24), lam_range=(-2 ** 30, 2 ** 30))
        want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
        same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)


def test_conv_mobilenet_first_layer(gpu, restatement):
    c = wl.conv_case(13, 224, 224, 3, 32, strides=(2, 2), batch=2, bits=32, out_shift=9)
    want = restatement.conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
    same(gpu.conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_conv_first_layer_tensor_core_kernel(bits, relu, bn, gpu, restatement):
    """3x3 kernels on at most 3 input channels with 32 or 64 filters take the kernel that builds
    the im2col tiles in shared memory: both strides, 1 to 3 input channels, left/top padding 0 to
    2, widths up to the 128 columns of a tile, heights that are not a multiple of the four rows a
    unit covers, more units than SMs."""
    cases = [  # H, W, Cin, Cout, strides, pads (top, bottom, left, right), batch
        (20, 32, 3, 32, (2, 2), (1, 1, 1, 1), 3),
        (9, 16, 3, 64, (1, 1), (1, 1, 1, 1), 2),
        (13, 64, 1, 32, (1, 1), (1, 1, 1, 1), 2),
        (10, 48, 2, 32, (2, 1), (0, 1, 2, 1), 2),
        (6, 256, 3, 32, (2, 2), (1, 1, 1, 1), 1),
        (7, 128, 3, 64, (1, 1), (2, 1, 0, 2), 2),
        (8, 16, 3, 32, (2, 2), (1, 1, 1, 1), 160),
    ]
    for (H, W, Cin, Cout, strides, pads, batch) in cases:
        c = wl.conv_case(40, H, W, Cin, Cout, strides=strides, pads=pads, batch=batch, bits=bits,
                         out_shift=9, with_bias=True, out_mult=5, relu=relu, bn=bn,
                         k_range=(-64, 64), lam_range=(-2 ** 20, 2 ** 20))
        want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
        same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)
    assert api.device_status() == 0


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_conv_spatial_tensor_core_kernel(bits, relu, bn, gpu, restatement):
    """Spatial kernels on a multiple of 32 input channels take the tensor-core GEMM with the im2col
    done by 4-D TMA boxes: every K-slab width, 64-, 128- and 256-column tiles (plain and TMA
    stores), strides 1 and 2 in either direction, 3x3 / 5x5 / 3x1 kernels, asymmetric padding,
    ragged filter counts, patches that hang over the image's edge, more patches than SMs."""
    cases = [  # H, W, Cin, Cout, kernel, strides, pads (top, bottom, left, right), batch
        (32, 32, 32, 64, (3, 3), (1, 1), (1, 1, 1, 1), 2),
        (14, 14, 64, 128, (3, 3), (1, 1), (1, 1, 1, 1), 3),
        (9, 13, 32, 48, (3, 3), (2, 2), (1, 1, 1, 1), 2),
        (12, 20, 128, 256, (3, 3), (1, 1), (1, 1, 1, 1), 2),
        (11, 10, 32, 32, (5, 5), (1, 1), (2, 2, 2, 2), 2),
        (10, 17, 64, 80, (3, 1), (1, 2), (1, 1, 0, 0), 2),
        (7, 7, 256, 160, (3, 3), (1, 1), (0, 2, 2, 0), 2),
        (16, 40, 32, 64, (3, 3), (2, 1), (1, 1, 1, 1), 40),
    ]
    for (H, W, Cin, Cout, kernel, strides, pads, batch) in cases:
        c = wl.conv_case(41, H, W, Cin, Cout, kernel=kernel, strides=strides, pads=pads, batch=batch, bits=bits,
                         out_shift=12, with_bias=True, out_mult=5, relu=relu, bn=bn,
                         k_range=(-64, 64), lam_range=(-2 ** 20, 2 ** 20))
        want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
        same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)
    assert api.device_status() == 0


def test_conv_against_compiled_reference(gpu, reference32):
    c = wl.conv_case(14, 17, 19, 8, 12, batch=2, bits=32, out_shift=10, with_bias=True)
    want = reference32.conv(32, c["x"], c["w"], c["k"], c["lam"], variant="HoWo", **conv_kw(c))
    same(gpu.conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)), want)


# ---- pointwise -----------------------------------------------------------------------------
@pytest.mark.parametrize("force_generic", [0, 1])
def test_pointwise_config2_literal_and_live(force_generic, gpu, restatement):
    api.set_option(api.OPT_FORCE_GENERIC, force_generic)
    for shift in (None, 10):
        c = wl.pointwise_case(1, 56, 56, 128, 256, batch=4, bits=32, out_shift=shift)
        want = restatement.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
        same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_pointwise_tensor_core_all_modes(bits, relu, bn, gpu, restatement):
    # K = 80 (not a multiple of the 128-byte stage), N = 48 (< one tile), M = 3*9*7 = 189 (ragged)
    c = wl.pointwise_case(22, 9, 7, 80, 48, batch=3, bits=bits, out_shift=8, with_bias=True,
                          out_mult=3, relu=relu, bn=bn, w_range=(-128, 127))
    want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    same(gpu.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)


@pytest.mark.parametrize("cin,cout", [(16, 16), (32, 64), (64, 128), (256, 512), (512, 520),
                                      (1024, 1024), (48, 1000), (144, 24)])
def test_pointwise_tensor_core_shapes(cin, cout, gpu, restatement):
    c = wl.pointwise_case(23, 14, 14, cin, cout, batch=5, bits=32,
                          out_shift=wl.ceil_log2(cin) + 3, w_range=(-128, 127))
    want = restatement.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    assert np.count_nonzero(want) > want.size // 20
    same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)


@pytest.mark.parametrize("relu,bn", MODES)
def test_pointwise_ragged_generic_path(relu, bn, gpu, gpu_host, restatement):
    c = wl.pointwise_case(21, 9, 7, 22, 13, batch=2, bits=32, out_shift=8, with_bias=True,
                          out_mult=3, relu=relu, bn=bn)
    want = restatement.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)
    same(gpu_host.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)


def test_pointwise_against_compiled_reference(gpu, reference64):
    c = wl.pointwise_case(24, 12, 12, 64, 96, batch=2, bits=64, out_shift=9, with_bias=True)
    want = reference64.pointwise(64, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    same(gpu.pointwise(64, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_pointwise_short_reduction_folded_rows(bits, relu, bn, gpu, restatement):
    """Many pixels with at most 64 input and 128 output channels: the GEMM folds 2, 4 or 8 pixels
    into one row against a block-diagonal copy of the weights. Filter counts that are not a power
    of two (the per-channel parameters wrap around inside a folded row), a pixel count that is odd
    (no folding), and every requantisation mode."""
    for (H, W, cin, cout, batch) in ((112, 112, 32, 64, 16), (56, 56, 64, 128, 32), (112, 112, 16, 32, 25),
                                     (112, 112, 32, 48, 16), (113, 113, 32, 64, 13), (112, 112, 64, 16, 16)):
        c = wl.pointwise_case(25, H, W, cin, cout, batch=batch, bits=bits, out_shift=9, with_bias=True,
                              out_mult=3, relu=relu, bn=bn)
        want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
        same(gpu.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)
    assert api.device_status() == 0


def test_pointwise_many_tiles_property(gpu, restatement):
    """Full config-2 batch: too large for the CPU checker in seconds, so check a size-independent
    property instead: the batched result equals the per-image results (images are independent),
    and the first and last images equal the checker."""
    c = wl.config_c2(batch=64)
    c["out_shift"] = 10
    got = gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    for i in (0, 63):
        want = restatement.pointwise(32, c["x"][i:i + 1], c["w"], c["k"], c["lam"], **pw_kw(c))
        same(got[i:i + 1], want)
    one = gpu.pointwise(32, c["x"][17:18], c["w"], c["k"], c["lam"], **pw_kw(c))
    same(got[17:18], one)


# ---- depthwise -----------------------------------------------------------------------------
def dw_kw(c):
    return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"],
                in_is_hwc=c["hwc"])


@pytest.mark.parametrize("hwc", [False, True])
def test_depthwise_config3(hwc, gpu, restatement):
    c = wl.config_c3(batch=3)
    if hwc:
        c["x"] = np.ascontiguousarray(c["x"].transpose(0, 2, 3, 1))
        c["hwc"] = True
    want = restatement.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    assert np.count_nonzero(want) > want.size // 4
    same(gpu.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("hwc", [False, True])
def test_depthwise_modes(bits, relu, bn, stride, hwc, gpu, restatement):
    c = wl.depthwise_case(31, 15, 14, 8, strides=(stride, stride), batch=2, bits=bits, out_shift=7,
                          with_bias=True, out_mult=3, relu=relu, bn=bn, hwc=hwc)
    want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    same(gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


@pytest.mark.parametrize("hwc", [False, True])
@pytest.mark.parametrize("C", [6, 37, 64])
def test_depthwise_ragged_and_5x5(hwc, C, gpu, gpu_host, restatement):
    for kernel, pads in (((3, 3), (1, 1, 1, 1)), ((5, 5), (2, 2, 2, 2)), ((2, 3), (0, 1, 1, 1))):
        c = wl.depthwise_case(32, 13, 12, C, kernel=kernel, pads=pads, batch=2, out_shift=8, hwc=hwc)
        want = restatement.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)
    same(gpu_host.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_chw_row_kernel(bits, relu, bn, stride, gpu, restatement):
    """CHW input with a width that is a multiple of 4 (8 for stride 2) takes the row-wise kernel:
    ragged channel counts, several channel tiles, widths that leave the last column group partly
    empty, large k that does not fit 32 bits in the 64-bit tree."""
    for (H, W, C) in ((13, 16, 12), (9, 24, 4), (20, 40, 72), (7, 128, 8)):
        c = wl.depthwise_case(35, H, W, C, strides=(stride, stride), batch=2, bits=bits, out_shift=9,
                              with_bias=True, out_mult=3, relu=relu, bn=bn,
                              k_range=(1, 2 ** 33) if bits == 64 else (1, 64),
                              lam_range=(-2 ** 34, 2 ** 34) if bits == 64 else (-32768, 32767))
        if bits == 64:
            c["out_shift"] = 30
        want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_hwc_tma_kernel(bits, relu, bn, stride, gpu, restatement):
    """HWC input with a multiple of 32 channels takes the TMA-staged kernel: 128-, 64- and 32-byte
    channel chunks, every tile width, images narrower and shorter than a tile, several column tiles
    with a ragged last one, heights that are not a multiple of the rows a group completes, several
    channel chunks, and (64-bit tree) k that does not fit 32 bits."""
    for (H, W, C) in ((14, 14, 128), (7, 7, 256), (5, 4, 128), (33, 61, 128), (28, 28, 128), (16, 30, 128),
                      (14, 14, 32), (9, 30, 64), (12, 20, 96), (8, 115, 32), (6, 112 * stride, 32),
                      (10, 56 * stride, 64), (7, 40, 192)):
        c = wl.depthwise_case(36, H, W, C, strides=(stride, stride), batch=3, bits=bits, out_shift=9,
                              with_bias=True, out_mult=3, relu=relu, bn=bn, hwc=True,
                              k_range=(1, 2 ** 33) if (bits == 64 and H == 7) else (1, 64),
                              lam_range=(-2 ** 34, 2 ** 34) if (bits == 64 and H == 7) else (-32768, 32767))
        if bits == 64 and H == 7:
            c["out_shift"] = 30
        want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)
    assert api.device_status() == 0


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_chw_tma_kernel(bits, relu, bn, stride, gpu, restatement):
    """CHW input whose rows are a multiple of 16 bytes and wider than 16 outputs takes the
    TMA-staged kernel: 16 and 32 lanes per channel quad, a partly empty last column group, a
    ragged last chunk of 32 channels, heights that are not a multiple of the rows a group
    completes, strips (batch 1), and (64-bit tree) k that does not fit 32 bits."""
    for (H, W, C, B) in ((9, 32 * stride, 8, 2), (13, 48 * stride, 36, 2), (7, 80 * stride, 12, 2), (56, 112, 64, 1),
                         (10, 128, 4, 3), (33, 64, 32, 1)):
        big = bits == 64 and H == 7
        c = wl.depthwise_case(38, H, W, C, strides=(stride, stride), batch=B, bits=bits, out_shift=9,
                              with_bias=True, out_mult=3, relu=relu, bn=bn,
                              k_range=(1, 2 ** 33) if big else (1, 64),
                              lam_range=(-2 ** 34, 2 ** 34) if big else (-32768, 32767))
        if big:
            c["out_shift"] = 30
        want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)
    assert api.device_status() == 0


def test_depthwise_hwc_tma_small_batch_strips(gpu, restatement):
    """Batch 1 splits the height into strips (each with its own opening group of rows)."""
    for (H, W, C, s) in ((56, 56, 128, 1), (56, 56, 128, 2), (112, 20, 128, 1)):
        c = wl.depthwise_case(37, H, W, C, strides=(s, s), batch=1, out_shift=9, hwc=True)
        want = restatement.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)
    assert api.device_status() == 0


@pytest.mark.parametrize("H,C,s,B", [(14, 512, 1, 256), (7, 1024, 1, 250), (28, 256, 2, 128), (112, 32, 1, 67),
                                     (56, 128, 1, 131), (14, 512, 2, 301), (28, 256, 1, 203), (112, 64, 2, 75)])
def test_depthwise_hwc_tma_several_images_per_cta(H, C, s, B, gpu, restatement):
    """Large batches: more whole-image columns than CTAs fit on the GPU at once, so a CTA works
    through several consecutive images with its ring of row groups running on from one image to
    the next (the branch every depthwise layer of the batch-1024 benchmark takes). Batches that
    do not divide by the images per CTA leave the last CTA short."""
    c = wl.depthwise_case(41, H, H, C, strides=(s, s), batch=B, bits=32, out_shift=9, hwc=True)
    want = restatement.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    assert np.count_nonzero(want) > want.size // 4
    same(gpu.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)
    assert api.device_status() == 0


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_depthwise_hwc_tma_several_images_per_cta_modes(bits, relu, bn, gpu, restatement, reference32, reference64):
    """The same branch in every epilogue mode and both trees; the first and the last images are
    also held to the compiled reference itself."""
    c = wl.depthwise_case(42, 14, 14, 512, batch=250, bits=bits, out_shift=9, with_bias=True, out_mult=3,
                          relu=relu, bn=bn, hwc=True)
    want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    got = gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    same(got, want)
    ref = reference32 if bits == 32 else reference64
    for sl in (slice(0, 2), slice(248, 250)):
        r = ref.depthwise(bits, np.ascontiguousarray(c["x"][sl]), c["w"], c["k"], c["lam"], **dw_kw(c))
        same(got[sl], r)


def test_depthwise_mobilenet_shapes(gpu, restatement):
    for (H, C, s) in ((112, 32, 1), (112, 64, 2), (14, 512, 1), (7, 1024, 1)):
        c = wl.depthwise_case(33, H, H, C, strides=(s, s), batch=2, out_shift=9, hwc=True)
        want = restatement.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
        same(gpu.depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


def test_depthwise_against_compiled_reference(gpu, reference64):
    c = wl.config_c3(batch=1)
    want = reference64.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c))
    same(gpu.depthwise(64, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)), want)


# ---- the remaining entry points of the reference header ------------------------------------------
@pytest.mark.parametrize("bits", [32, 64])
def test_slicing_variants_and_short_kernels(bits, gpu, restatement, reference32, reference64):
    """pulp_nn_conv_Co_parallel, pulp_nn_pointwise_Ho_parallel / _Co_parallel and
    pulp_nn_depthwise_generic_less_4_weights through the C ABI: the checker is the compiled
    reference wherever it computes the convolution (it does not for pointwise_Co), and the
    restatement everywhere."""
    ref = reference32 if bits == 32 else reference64
    c = wl.conv_case(60, 11, 9, 8, 20, strides=(2, 1), batch=3, bits=bits, with_bias=True, out_shift=10)
    want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c))
    same(ref.conv(bits, c["x"], c["w"], c["k"], c["lam"], variant="Co", **conv_kw(c)), want)
    same(gpu.conv(bits, c["x"], c["w"], c["k"], c["lam"], variant="Co", **conv_kw(c)), want)
    c = wl.pointwise_case(61, 6, 10, 32, 48, batch=3, bits=bits, with_bias=True)
    want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
    same(ref.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], variant="Ho", **pw_kw(c)), want)
    for variant in ("Ho", "Co"):
        same(gpu.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], variant=variant, **pw_kw(c)), want)
    for kernel, pads in (((1, 3), (0, 0, 1, 1)), ((3, 1), (1, 1, 0, 0)), ((1, 1), (0, 0, 0, 0)), ((3, 3), (1, 1, 1, 1))):
        c = wl.depthwise_case(62, 9, 12, 8, kernel=kernel, pads=pads, batch=2, bits=bits, out_shift=6, with_bias=True)
        want = ref.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], less4=True, **dw_kw(c))
        same(gpu.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], less_4_weights=True, **dw_kw(c)), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_depthwise_3x3_s1_and_matmul(bits, relu, bn, gpu, gpu_host, restatement, reference32, reference64):
    """The last two symbols of the reference header through the C ABI, against the compiled
    reference and the restatement: pulp_nn_depthwise_3x3_s1 (CHW in, no vertical padding) and
    pulp_nn_matmul (two im2col columns; adjacent and separate output rows; device and host
    buffers; the returned pointer is checked inside the harness)."""
    ref = reference32 if bits == 32 else reference64
    for (R, Cw, CH, B) in ((9, 12, 6, 3), (20, 32, 8, 2), (3, 2, 1, 1)):
        c = wl.depthwise_case(64, R, Cw, CH, pads=(0, 0, 1, 1), batch=B, bits=bits, out_shift=6, out_mult=3,
                              relu=relu, bn=bn)
        kw = dict(out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
        want = ref.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        same(restatement.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
        same(gpu.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
    same(gpu_host.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
    for (K, N) in ((288, 64), (27, 7), (64, 1), (1024, 96)):
        c = wl.linear_case(65, K, N, batch=2, bits=bits, out_shift=8, out_mult=3, relu=relu, bn=bn)
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
        want = ref.matmul(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        same(gpu.matmul(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
        same(gpu.matmul(bits, c["x"], c["w"], c["k"], c["lam"], adjacent=False, **kw), want)
    same(gpu_host.matmul(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
    same(gpu_host.matmul(bits, c["x"], c["w"], c["k"], c["lam"], adjacent=False, **kw), want)


def test_depthwise_3x3_s1_rejects_what_the_reference_gets_wrong(gpu):
    """Without left/right padding flags, or with an odd width, the reference's row loop runs into
    the next row (32bit/src/pulp_nn_depthwise_3x3_s1.c:140): rejected, nothing is enqueued."""
    c = wl.depthwise_case(66, 9, 12, 4, pads=(0, 0, 1, 1), batch=1, out_shift=6)
    for p_l, p_r, x in ((0, 1, c["x"]), (1, 0, c["x"]), (1, 1, c["x"][:, :, :, :11].copy())):
        with pytest.raises(api.PulpNNError):
            gpu.depthwise_3x3_s1(32, x, c["w"], c["k"], c["lam"], out_shift=6, p_l=p_l, p_r=p_r)


@pytest.mark.parametrize("bits_per_value,signed", [(4, False), (2, False), (4, True), (2, True)])
def test_subbyte_unpack(bits_per_value, signed, gpu, gpu_host, restatement, reference32):
    """pulp_nn_im2col_u4_to_u8 / _u2_to_u8 and their sign-extending counterparts: whole words, a
    byte-wise tail, host buffers; an element count that is not a whole number of bytes is refused
    (the reference's tail loop would never end)."""
    rng = np.random.default_rng(67)
    for n_in in (4, 64, 1001, 1 << 20):
        packed = rng.integers(0, 256, size=n_in, dtype=np.uint8)
        want = restatement.unpack(packed, bits_per_value, signed)
        if n_in % 4 == 0:
            same(reference32.unpack(packed, bits_per_value, signed), want)
        same(gpu.unpack(packed, bits_per_value, signed), want)
    same(gpu_host.unpack(packed[:1001], bits_per_value, signed), restatement.unpack(packed[:1001], bits_per_value, signed))
    fn = {(4, False): api.pulp_nn_im2col_u4_to_u8, (2, False): api.pulp_nn_im2col_u2_to_u8,
          (4, True): api.pulpnn_i4_to_i8, (2, True): api.pulpnn_i2_to_i8}[(bits_per_value, signed)]
    with pytest.raises(api.PulpNNError):
        fn(packed, np.zeros(16, np.uint8), 8 // bits_per_value + 1)


def test_layout_change(gpu, gpu_host):
    """CHW <-> HWC against numpy's transpose: whole tiles, ragged tiles, sizes that rule out 32-bit
    accesses on either side, and the round trip."""
    rng = np.random.default_rng(63)
    for (B, Cc, H, W) in ((2, 64, 8, 16), (3, 5, 7, 9), (1, 130, 3, 67), (2, 32, 56, 56), (1, 3, 224, 224),
                          (2, 144, 20, 20), (1, 256, 16, 24), (3, 64, 112, 112)):
        x = rng.integers(0, 256, size=(B, Cc, H, W), dtype=np.uint8)
        hwc = gpu.chw_to_hwc(x)
        same(hwc, np.ascontiguousarray(x.transpose(0, 2, 3, 1)))
        same(gpu.hwc_to_chw(hwc), x)
    same(gpu_host.chw_to_hwc(x), np.ascontiguousarray(x.transpose(0, 2, 3, 1)))


# ---- linear --------------------------------------------------------------------------------
def lin_kw(c):
    return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"],
                bn=c["bn"])


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_linear_modes_generic(bits, relu, bn, gpu, restatement):
    c = wl.linear_case(41, 203, 37, batch=3, bits=bits, out_shift=6, out_mult=3, relu=relu, bn=bn,
                       w_range=(-128, 127))
    want = restatement.linear(bits, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c))
    same(gpu.linear(bits, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c)), want)


@pytest.mark.parametrize("split_k", [0, 1, 4])
@pytest.mark.parametrize("relu,bn,shift", [(1, 0, None), (1, 1, 16), (0, 0, 14)])
def test_linear_config4(split_k, relu, bn, shift, gpu, restatement):
    api.set_option(api.OPT_SPLIT_K, split_k)
    c = wl.config_c4(batch=32)
    c.update(relu=relu, bn=bn)
    if shift is not None:
        c["out_shift"] = shift
    want = restatement.linear(32, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c))
    same(gpu.linear(32, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c)), want)


@pytest.mark.parametrize("split_k", [0, 1, 3])
def test_linear_out_32_config4_raw_accumulators(split_k, gpu, gpu_host, restatement):
    api.set_option(api.OPT_SPLIT_K, split_k)
    c = wl.config_c4(batch=32)
    b32 = c["bias32"].view(np.int8)
    want = restatement.linear_out_32(c["x"], c["w"], bias32=b32)
    same(gpu.linear_out_32(c["x"], c["w"], bias32=b32), want)
    same(gpu.linear_out_32(c["x"], c["w"]), restatement.linear_out_32(c["x"], c["w"]))
    if split_k == 0:
        same(gpu_host.linear_out_32(c["x"], c["w"], bias32=b32), want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_linear_few_tiles_long_reduction(bits, relu, bn, gpu, gpu_host, restatement):
    """Few output tiles and a long reduction (the shape of a fully connected layer at a small
    batch): K split into partial sums or not, depending on the tile count; a K that is not a
    multiple of the slab, filter counts that are not a multiple of 16, one and two row tiles, every
    requantisation mode, and raw int32 output."""
    for (K, N, B) in ((2048, 256, 5), (4096, 1000, 200), (2064, 48, 130), (3072, 520, 256), (4096, 4096, 256)):
        c = wl.linear_case(26, K, N, batch=B, bits=bits, out_shift=wl.ceil_log2(K) + 4, out_mult=3,
                           relu=relu, bn=bn, w_range=(-128, 127))
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
        want = restatement.linear(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        assert np.count_nonzero(want) > want.size // 20
        same(gpu.linear(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
        if (relu, bn) == (1, 1):
            same(gpu.linear_out_32(c["x"], c["w"], bias32=c["bias32"].view(np.int8), bits=bits),
                 restatement.linear_out_32(c["x"], c["w"], bias32=c["bias32"].view(np.int8)))
    same(gpu_host.linear(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
    assert api.device_status() == 0


def test_linear_single_vector_and_odd_sizes(gpu, restatement):
    for (K, N, B) in ((4096, 4096, 1), (1024, 1000, 7), (77, 5, 1), (16, 16, 130)):
        c = wl.linear_case(43, K, N, batch=B, out_shift=wl.ceil_log2(K) + 2, relu=1, bn=1)
        want = restatement.linear(32, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c))
        same(gpu.linear(32, c["x"], c["w"], c["k"], c["lam"], **lin_kw(c)), want)
        same(gpu.linear_out_32(c["x"], c["w"]), restatement.linear_out_32(c["x"], c["w"]))


# ---- pooling and add -----------------------------------------------------------------------
@pytest.mark.parametrize("geom", [
    dict(kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0), out_hw=(7, 7)),
    dict(kernel=(3, 3), strides=(2, 2), pads=(1, 1, 1, 1), out_hw=(7, 7)),
    dict(kernel=(3, 2), strides=(3, 2), pads=(1, 0, 0, 0), out_hw=(5, 7)),
    dict(kernel=(5, 5), strides=(3, 3), pads=(2, 2, 2, 2), out_hw=(5, 5)),     # a large window
    dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(2, 2)),
])
@pytest.mark.parametrize("C", [10, 64])
def test_maxpool(geom, C, gpu, gpu_host, restatement):
    rng = np.random.default_rng(51)
    x = rng.integers(0, 256, size=(3, 14, 14, C), dtype=np.uint8)
    want, want_after = restatement.maxpool(x, want_input_after=True, **geom)
    same(gpu.maxpool(x, **geom), want)
    same(gpu_host.maxpool(x, **geom), want)
    got, got_after = gpu.maxpool(x, want_input_after=True, **geom)
    same(got, want)
    # only the columns the reference overwrites are compared: it leaves the rest untouched
    same(got_after, want_after)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("requant,lam,add,shift", [(0, 0, 0, 0), (1, 300, 128, 8), (1, -3, 5, 2),
                                                   (1, 70000, -9, 11)])
def test_avgpool(bits, requant, lam, add, shift, gpu, restatement):
    rng = np.random.default_rng(52)
    for C in (9, 32):
        x = rng.integers(0, 256, size=(2, 14, 14, C), dtype=np.uint8)
        for geom in (dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(2, 2)),
                     dict(kernel=(3, 3), strides=(2, 2), pads=(1, 1, 1, 1), out_hw=(7, 7)),
                     dict(kernel=(5, 5), strides=(2, 2), pads=(2, 2, 2, 2), out_hw=(7, 7))):
            kw = dict(lam=lam, out_shift=shift, out_add=add, requant=requant, **geom)
            same(gpu.avgpool(bits, x, **kw), restatement.avgpool(bits, x, **kw))


def test_avgpool_mobilenet_tail(gpu, restatement):
    rng = np.random.default_rng(53)
    x = rng.integers(0, 256, size=(5, 7, 7, 1024), dtype=np.uint8)
    kw = dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(1, 1))
    same(gpu.avgpool(32, x, **kw), restatement.avgpool(32, x, **kw))
    # windows of 32 pixels and more share a window among the warps of a block: a channel count that
    # leaves the last 128-channel chunk ragged, overlapping padded windows, both requantised forms
    x = rng.integers(0, 256, size=(3, 13, 12, 200), dtype=np.uint8)
    for bits in (32, 64):
        for requant in (0, 1):
            kw = dict(kernel=(6, 7), strides=(3, 4), pads=(2, 2, 3, 3), out_hw=(4, 3), lam=-77, out_shift=5,
                      out_add=1000, requant=requant)
            same(gpu.avgpool(bits, x, **kw), restatement.avgpool(bits, x, **kw))


@pytest.mark.parametrize("m1,m2,shift", [(37, 91, 6), (1, 1, 0), (65535, 3, 4), (300, 500, 1)])
def test_add(m1, m2, shift, gpu, gpu_host, restatement):
    rng = np.random.default_rng(54)
    for shape in ((2, 14, 13, 11), (4, 56, 56, 64)):
        a = rng.integers(0, 256, size=shape, dtype=np.uint8)
        b = rng.integers(0, 256, size=shape, dtype=np.uint8)
        want = restatement.add(a, b, m1=m1, m2=m2, out_shift=shift)
        same(gpu.add(a, b, m1=m1, m2=m2, out_shift=shift), want)
    same(gpu_host.add(a, b, m1=m1, m2=m2, out_shift=shift), want)


# ---- argument checking ---------------------------------------------------------------------
def test_rejects_what_the_reference_leaves_undefined(gpu):
    x = np.zeros((1, 8, 8, 16), np.uint8)
    w = np.zeros((16, 16), np.int8)
    k = np.ones(16, np.int32)
    with pytest.raises(pulpnn.PulpNNError) as e:       # shift outside 0..31
        gpu.pointwise(32, x, w, k, k, out_shift=40)
    assert e.value.code == api.ERR_INVALID_ARG
    wd = np.zeros((16, 3, 3), np.int8)
    with pytest.raises(pulpnn.PulpNNError) as e:       # pad_left != kx/2
        gpu.depthwise(32, x.transpose(0, 3, 1, 2).copy(), wd, k, k, out_hw=(8, 7), kernel=(3, 3),
                      pads=(1, 1, 0, 1), strides=(1, 1))
    assert e.value.code == api.ERR_UNSUPPORTED
    with pytest.raises(pulpnn.PulpNNError) as e:       # in-place x pass would read pooled values
        gpu.maxpool(x, out_hw=(8, 8), kernel=(3, 3), pads=(1, 1, 1, 1), strides=(1, 1))
    assert e.value.code == api.ERR_UNSUPPORTED


# ---- the GEMM computed by pairs of SMs --------------------------------------------------------------
@pytest.mark.parametrize("cin,cout,hw,batch", [(512, 512, 14, 5), (512, 1024, 7, 9), (1024, 1024, 7, 6), (512, 256, 16, 1),
                                               (1024, 768, 9, 4), (640, 512, 14, 3), (512, 512, 14, 160)])
def test_pointwise_sm_pair_kernel_shapes(cin, cout, hw, batch, gpu, restatement):
    """Wide layers with a long reduction on the tcgen05 cta_group::2 kernel (two CTAs share a 256-row
    tile, each holds half of the weight tile): one and two resident column tiles, one or several
    column groups, row counts that leave the last pair of tiles ragged or half empty, more row pairs
    than SM pairs."""
    api.set_option(api.OPT_TUNE, 8)
    try:
        c = wl.pointwise_case(81, hw, hw, cin, cout, batch=batch, bits=32, out_shift=wl.ceil_log2(cin) + 3,
                              w_range=(-128, 127))
        want = restatement.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
        assert np.count_nonzero(want) > want.size // 20
        same(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)
    finally:
        api.set_option(api.OPT_TUNE, 0)
    assert api.device_status() == 0


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_pointwise_sm_pair_kernel_modes(bits, relu, bn, gpu, restatement):
    api.set_option(api.OPT_TUNE, 8)
    try:
        c = wl.pointwise_case(82, 11, 13, 512, 512, batch=3, bits=bits, out_shift=12, with_bias=True, out_mult=3,
                              relu=relu, bn=bn, w_range=(-128, 127))
        want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c))
        same(gpu.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)), want)
    finally:
        api.set_option(api.OPT_TUNE, 0)
    assert api.device_status() == 0


# ---- the scalar sub-byte requantisers of pulp_nn_utils.h as bulk operations -------------------------
@pytest.mark.parametrize("bits", [32, 64])
def test_bulk_quantisers_against_the_compiled_reference(bits, gpu_host, reference32, reference64):
    """pulp_nn_bn_quant_u8/u4/u2, pulp_nn_quant_u8/u4/u2, pulp_nn_i4_quant / pulp_nn_i2_quant and
    pulp_nn_avg_and_replace_int8 element by element from the reference's own compiled code, both
    trees, device and host buffers, values that overflow 32 bits and cross every clip boundary."""
    import torch
    ref = reference32 if bits == 32 else reference64
    rng = np.random.default_rng(90 + bits)
    n, ch = 1537, 13
    dt = np.int32 if bits == 32 else np.int64
    phi = rng.integers(-2 ** 20, 2 ** 20, size=n).astype(np.int32)
    phi[:8] = [0, 1, -1, 2 ** 31 - 1, -2 ** 31, 255, 256, -255]
    for (krange, lrange, d) in (((1, 64), (-32768, 32767), 9), ((-2 ** 20, 2 ** 20), (-2 ** 30, 2 ** 30), 17)):
        k = rng.integers(krange[0], krange[1] + 1, size=ch).astype(dt)
        lam = rng.integers(lrange[0], lrange[1] + 1, size=ch).astype(dt)
        for out_bits in (8, 4, 2):
            want = ref.scalar_bn_quant(out_bits, phi, k, lam, d)
            for dev in (True, False):
                out = torch.zeros(n, dtype=torch.uint8, device="cuda") if dev else np.zeros(n, np.uint8)
                args = [torch.from_numpy(a).cuda() if dev else a for a in (phi, k, lam)]
                api.pulpnn_bn_quant_bulk(bits, args[0], args[1], args[2], d, out, n, ch, out_bits)
                api.synchronize()
                same(out.cpu().numpy() if dev else out, want)
    for (m, d) in ((3, 4), (-7, 2), (32767, 15), (300, 0)):
        for out_bits in (8, 4, 2):
            want = ref.scalar_quant(out_bits, phi, m, d)
            out = np.zeros(n, np.uint8)
            api.pulpnn_quant_bulk(bits, phi, m, d, out, n, out_bits)
            same(out, want)
    x = rng.integers(-40000, 40000, size=n).astype(np.int32)
    for out_bits, width in ((4, 16), (2, 4)):
        thr = np.sort(rng.integers(-32768, 32768, size=(ch, width)), axis=1).astype(np.int16)
        x[:ch * width] = thr.reshape(-1)                     # inputs equal to a threshold: "<=" decides
        want = ref.scalar_threshold_quant(out_bits, x, thr)
        out = np.zeros(n, np.int8)
        api.pulpnn_threshold_quant_bulk(x, thr, out, n, ch, out_bits)
        same(out, want)
    base = rng.integers(-128, 128, size=1003).astype(np.int8)
    target = rng.integers(-128, 128, size=1003).astype(np.int8)
    want = ref.avg_and_replace(base, target)
    got = base.copy()
    api.pulp_nn_avg_and_replace_int8(got, target, got.size)
    same(got, want)
    assert np.array_equal(got[1000:], base[1000:])           # the last three bytes are not a whole word


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_linear_few_rows_kernel(bits, relu, bn, gpu, restatement):
    """Few rows (M <= 256) and a long reduction take the dp4a kernel that keeps eight neurons' weights
    per CTA: neuron counts that are not a multiple of eight, K that is not a multiple of 512, one row,
    the largest row count; and the same calls on the tensor-core kernel (the switch bit 16) agree."""
    for (K, N, B) in ((1024, 1000, 128), (272, 1001, 3), (4096, 67, 1), (2048, 256, 256), (1040, 8, 77)):
        c = wl.linear_case(44, K, N, batch=B, bits=bits, out_shift=wl.ceil_log2(K) + 4, out_mult=3, relu=relu, bn=bn,
                           w_range=(-128, 127))
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
        want = restatement.linear(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        launches = api.launch_count()
        same(gpu.linear(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)
        assert api.launch_count() - launches == 1, "expected the one-kernel few-rows path"
        if (relu, bn) == (1, 1):
            want32 = restatement.linear_out_32(c["x"], c["w"], bias32=c["bias32"])
            same(gpu.linear_out_32(c["x"], c["w"], bias32=c["bias32"], bits=bits), want32)
            api.set_option(api.OPT_TUNE, 16)
            try:
                same(gpu.linear_out_32(c["x"], c["w"], bias32=c["bias32"], bits=bits), want32)
            finally:
                api.set_option(api.OPT_TUNE, 0)
