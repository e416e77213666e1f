"""Pins the C restatement (oracle/pulpnn_oracle.c) to the reference's own code.

The reference ships no tests or golden vectors, so the only pin available is the reference
itself: oracle/_ref holds its unmodified sources compiled in place. Every case here runs both
and demands byte equality. Skipped on machines where oracle/_ref was not built (tests/golden
carries outputs of the same compiled reference for those, see test_golden.py).
"""
import numpy as np
import pytest

from conftest import pulpnn

wl = pulpnn.workloads

MODES = [(1, 1), (1, 0), (0, 0), (0, 1), (2, 0), (2, 1)]   # (flag_relu, flag_batch_norm)


def _ref(bits, reference32, reference64):
    return reference32 if bits == 32 else reference64


def _run_conv(impl, c, variant="Ho", **kw):
    return impl.conv(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=c["bias"],
                     out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                     kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"],
                     bn=c["bn"], variant=variant, **kw)


def _run_pw(impl, c, variant="HoWo", **kw):
    return impl.pointwise(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=c["bias"],
                          out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"],
                          bn=c["bn"], variant=variant, **kw)


def _run_dw(impl, c, **kw):
    return impl.depthwise(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=c["bias"],
                          out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                          kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"],
                          bn=c["bn"], in_is_hwc=c["hwc"], **kw)


def _run_lin(impl, c):
    return impl.linear(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=c["bias"],
                       out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"], bn=c["bn"])


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("variant", ["Ho", "HoWo"])
def test_conv_config1_literal(bits, variant, restatement, reference32, reference64):
    c = wl.conv_case(0, 32, 32, 32, 64, bits=bits)
    got = _run_conv(restatement, c)
    want = _run_conv(_ref(bits, reference32, reference64), c, variant=variant)
    assert np.array_equal(got, want)
    assert 0 < np.count_nonzero(want) < want.size // 10      # literal parameters: mostly zeros


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
@pytest.mark.parametrize("variant", ["Ho", "HoWo"])
def test_conv_ragged_all_modes(bits, relu, bn, variant, restatement, reference32, reference64):
    # odd width, ch_out % 4 != 0, K % 4 != 0, asymmetric pads, non-square kernel and strides
    c = wl.conv_case(11, 13, 11, 5, 7, kernel=(3, 5), strides=(2, 1), pads=(1, 0, 2, 1), batch=3,
                     bits=bits, out_shift=9, with_bias=True, out_mult=5, relu=relu, bn=bn,
                     k_range=(-64, 64), lam_range=(-2 ** 20, 2 ** 20))
    got = _run_conv(restatement, c)
    want = _run_conv(_ref(bits, reference32, reference64), c, variant=variant)
    assert np.array_equal(got, want)
    assert np.count_nonzero(want) > want.size // 20


@pytest.mark.parametrize("bits", [32, 64])
def test_conv_bn_wraparound(bits, restatement, reference32, reference64):
    # large k so that k*acc overflows int32: the 32-bit tree wraps, the 64-bit tree does not
    c = wl.conv_case(12, 9, 9, 16, 8, bits=bits, out_shift=12, w_range=(-128, 127),
                     k_range=(2 ** 20, 2 ** 24), lam_range=(-2 ** 30, 2 ** 30))
    got = _run_conv(restatement, c)
    want = _run_conv(_ref(bits, reference32, reference64), c)
    assert np.array_equal(got, want)
    assert 0 < np.count_nonzero(want) < want.size


def test_conv_mobilenet_first_layer_shape(restatement, reference32):
    c = wl.conv_case(13, 224, 224, 3, 32, strides=(2, 2), batch=1, bits=32, out_shift=9)
    got = _run_conv(restatement, c)
    want = _run_conv(reference32, c, variant="HoWo")
    assert got.shape == (1, 112, 112, 32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_pointwise_ragged_all_modes(bits, relu, bn, restatement, reference32, reference64):
    c = wl.pointwise_case(21, 9, 7, 22, 13, batch=2, bits=bits, out_shift=8, with_bias=True,
                          out_mult=3, relu=relu, bn=bn)
    got = _run_pw(restatement, c)
    want = _run_pw(_ref(bits, reference32, reference64), c)
    assert np.array_equal(got, want)


def test_pointwise_config2_shape_one_image(restatement, reference32):
    lit = wl.pointwise_case(1, 56, 56, 128, 256, batch=1, bits=32)
    live = wl.pointwise_case(1, 56, 56, 128, 256, batch=1, bits=32, out_shift=10)
    for c in (lit, live):
        assert np.array_equal(_run_pw(restatement, c), _run_pw(reference32, c))
    nz = np.count_nonzero(_run_pw(restatement, live))
    assert nz > live["x"].shape[1] * live["x"].shape[2] * 256 // 10


@pytest.mark.parametrize("bits", [32, 64])
def test_depthwise_config3_shape(bits, restatement, reference32, reference64):
    c = wl.depthwise_case(2, 112, 112, 64, strides=(2, 2), batch=1, bits=bits, out_shift=14,
                          w_range=(-64, 63), k_range=(1, 256), lam_range=(-2 ** 20, 2 ** 20))
    got = _run_dw(restatement, c)
    want = _run_dw(_ref(bits, reference32, reference64), c)
    assert np.array_equal(got, want)
    assert np.count_nonzero(want) > want.size // 4


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", [(1, 1), (1, 0), (0, 0), (0, 1), (2, 0)])
@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_modes_and_strides(bits, relu, bn, stride, restatement, reference32, reference64):
    c = wl.depthwise_case(31, 15, 14, 6, strides=(stride, stride), batch=2, bits=bits, out_shift=7,
                          with_bias=True, out_mult=3, relu=relu, bn=bn)
    got = _run_dw(restatement, c)
    want = _run_dw(_ref(bits, reference32, reference64), c)
    assert np.array_equal(got, want)


def test_depthwise_5x5_and_hwc_glue(restatement, reference32):
    c = wl.depthwise_case(32, 12, 12, 4, kernel=(5, 5), pads=(2, 2, 2, 2), batch=1, out_shift=8)
    assert np.array_equal(_run_dw(restatement, c), _run_dw(reference32, c))
    # HWC-input variant (network runner layout): same numbers as CHW through the layout glue
    h = dict(c)
    h["x"] = np.ascontiguousarray(c["x"].transpose(0, 2, 3, 1))
    h["hwc"] = True
    assert np.array_equal(_run_dw(restatement, h), _run_dw(reference32, h))
    assert np.array_equal(_run_dw(restatement, h), _run_dw(restatement, c))


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("relu,bn", MODES)
def test_linear_modes(bits, relu, bn, restatement, reference32, reference64):
    c = wl.linear_case(41, 203, 37, batch=3, bits=bits, out_shift=6, out_mult=3, relu=relu, bn=bn,
                       w_range=(-128, 127))
    got = _run_lin(restatement, c)
    want = _run_lin(_ref(bits, reference32, reference64), c)
    assert np.array_equal(got, want)


def test_linear_out_32_int32_bias(restatement, reference32, reference64):
    c = wl.linear_case(42, 1024, 100, batch=2)
    b = c["bias32"].view(np.int8)
    for ref in (reference32, reference64):
        assert np.array_equal(restatement.linear_out_32(c["x"], c["w"], bias32=b),
                              ref.linear_out_32(c["x"], c["w"], bias32=b))
    assert np.array_equal(restatement.linear_out_32(c["x"], c["w"]),
                          reference32.linear_out_32(c["x"], c["w"]))


def test_linear_config4_one_vector(restatement, reference32):
    c = wl.linear_case(3, 4096, 4096, batch=1, bits=32)
    assert np.array_equal(_run_lin(restatement, c), _run_lin(reference32, c))
    assert np.array_equal(restatement.linear_out_32(c["x"], c["w"]),
                          reference32.linear_out_32(c["x"], c["w"]))


@pytest.mark.parametrize("geom", [
    dict(kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0), out_hw=(7, 7)),
    dict(kernel=(3, 3), strides=(2, 2), pads=(1, 1, 1, 1), out_hw=(7, 7)),
    dict(kernel=(3, 2), strides=(3, 2), pads=(1, 0, 0, 0), out_hw=(5, 7)),
])
def test_maxpool(geom, restatement, reference32, reference64):
    rng = np.random.default_rng(51)
    x = rng.integers(0, 256, size=(2, 14, 14, 10), dtype=np.uint8)
    got, got_after = restatement.maxpool(x, want_input_after=True, **geom)
    for ref in (reference32, reference64):
        want, want_after = ref.maxpool(x, want_input_after=True, **geom)
        assert np.array_equal(got, want)
        assert np.array_equal(got_after, want_after)     # the reference clobbers its input
    assert not np.array_equal(got_after, x)


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("requant,lam,add,shift", [(0, 0, 0, 0), (1, 300, 128, 8), (1, -3, 5, 2),
                                                   (1, 70000, -9, 11)])
def test_avgpool(bits, requant, lam, add, shift, restatement, reference32, reference64):
    rng = np.random.default_rng(52)
    x = rng.integers(0, 256, size=(2, 14, 14, 9), dtype=np.uint8)
    for geom in (dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(2, 2)),
                 dict(kernel=(3, 3), strides=(2, 2), pads=(1, 1, 1, 1), out_hw=(7, 7))):
        kw = dict(lam=lam, out_shift=shift, out_add=add, requant=requant, **geom)
        got = restatement.avgpool(bits, x, **kw)
        want = _ref(bits, reference32, reference64).avgpool(bits, x, **kw)
        assert np.array_equal(got, want)


def test_avgpool_mobilenet_tail(restatement, reference32):
    rng = np.random.default_rng(53)
    x = rng.integers(0, 256, size=(3, 7, 7, 1024), dtype=np.uint8)
    kw = dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(1, 1))
    got = restatement.avgpool(32, x, **kw)
    assert np.array_equal(got, reference32.avgpool(32, x, **kw))
    assert np.array_equal(got.reshape(3, 1024), x.astype(np.uint32).sum(axis=(1, 2)) // 49)


@pytest.mark.parametrize("m1,m2,shift", [(37, 91, 6), (1, 1, 0), (65535, 3, 4), (300, 500, 1)])
def test_add(m1, m2, shift, restatement, reference32, reference64):
    rng = np.random.default_rng(54)
    a = rng.integers(0, 256, size=(2, 14, 13, 11), dtype=np.uint8)
    b = rng.integers(0, 256, size=(2, 14, 13, 11), dtype=np.uint8)
    got = restatement.add(a, b, m1=m1, m2=m2, out_shift=shift)
    for ref in (reference32, reference64):
        assert np.array_equal(got, ref.add(a, b, m1=m1, m2=m2, out_shift=shift))


# ---- the remaining core-slicing variants and the short-kernel depthwise -------------------------
def test_slicing_variants_compute_the_same_function(restatement, reference32, reference64):
    """pulp_nn_conv_Co_parallel and pulp_nn_pointwise_Ho_parallel (single core) give the bytes of the
    plain convolution. pulp_nn_pointwise_Co_parallel does not, even on one core (it mis-steps its
    bias pointer, 32bit/src/pulp_nn_pointwise_Co_parallel.c): the library defines that name as the
    convolution itself, so the checker for it is the restatement."""
    for bits, ref in ((32, reference32), (64, reference64)):
        c = wl.conv_case(50, 9, 8, 8, 12, batch=2, bits=bits, with_bias=True, out_shift=10)
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                  kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])
        want = restatement.conv(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        assert np.array_equal(ref.conv(bits, c["x"], c["w"], c["k"], c["lam"], variant="Co", **kw), want)
        c = wl.pointwise_case(51, 7, 9, 16, 24, batch=2, bits=bits, with_bias=True)
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"], bn=c["bn"])
        want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        assert np.array_equal(ref.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], variant="Ho", **kw), want)


@pytest.mark.parametrize("kernel,pads", [((1, 3), (0, 0, 1, 1)), ((3, 1), (1, 1, 0, 0)), ((1, 1), (0, 0, 0, 0)),
                                         ((3, 3), (1, 1, 1, 1))])
def test_depthwise_less_4_weights(kernel, pads, restatement, reference32, reference64):
    for bits, ref in ((32, reference32), (64, reference64)):
        c = wl.depthwise_case(52, 9, 11, 6, kernel=kernel, pads=pads, batch=2, bits=bits, out_shift=6,
                              with_bias=True)
        kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                  kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])
        want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
        assert np.count_nonzero(want) > want.size // 10
        assert np.array_equal(ref.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], less4=True, **kw), want)


@pytest.mark.parametrize("relu,bn", MODES)
def test_depthwise_3x3_s1(relu, bn, restatement, reference32, reference64):
    """pulp_nn_depthwise_3x3_s1 inside its defined domain (p_l = p_r = 1, even C) equals the 3x3
    stride-1 depthwise convolution with horizontal padding only; its flags select the mode the
    way the convolutions' do (flag_relu == 1 for the multiplier mode)."""
    for bits, ref in ((32, reference32), (64, reference64)):
        for (R, Cw, CH) in ((9, 12, 6), (3, 2, 1), (17, 30, 5)):
            c = wl.depthwise_case(53, R, Cw, CH, pads=(0, 0, 1, 1), batch=2, bits=bits, out_shift=6, out_mult=3,
                                  relu=relu, bn=bn)
            kw = dict(out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
            want = restatement.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
            assert want.shape == (2, R - 2, Cw, CH)
            assert np.array_equal(ref.depthwise_3x3_s1(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)


@pytest.mark.parametrize("relu,bn", MODES)
def test_matmul_two_columns(relu, bn, restatement, reference32, reference64):
    """pulp_nn_matmul: two im2col columns against all filters, with the channel tail (ch_out & 3)
    and the reduction tail (K & 3) of the reference, and the returned pointer."""
    for bits, ref in ((32, reference32), (64, reference64)):
        for (K, N) in ((288, 64), (27, 7), (10, 3), (64, 1), (5, 9)):
            c = wl.linear_case(54, K, N, batch=2, bits=bits, out_shift=8, out_mult=3, relu=relu, bn=bn)
            kw = dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=relu, bn=bn)
            want = restatement.matmul(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
            assert np.array_equal(ref.matmul(bits, c["x"], c["w"], c["k"], c["lam"], **kw), want)


@pytest.mark.parametrize("bits_per_value,signed", [(4, False), (2, False), (4, True), (2, True)])
def test_subbyte_unpack(bits_per_value, signed, restatement, reference32):
    """The sub-byte unpack helpers: whole words and (unsigned block forms) the byte-wise tail."""
    rng = np.random.default_rng(55)
    for n_in in (4, 64, 1000) + (() if signed else (1, 7, 1001)):
        packed = rng.integers(0, 256, size=n_in, dtype=np.uint8)
        want = restatement.unpack(packed, bits_per_value, signed)
        assert want.size == n_in * (8 // bits_per_value)
        assert np.array_equal(reference32.unpack(packed, bits_per_value, signed), want)
