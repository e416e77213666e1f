"""Seeded synthetic workloads: the five benchmark configurations and the MobileNetV1 layer stack.

Everything here is numpy on the host. Inputs are synthetic by definition (uniform integers of
the stated ranges from ``numpy.random.default_rng(seed)``); no dataset is involved.

Layouts follow the reference API (32bit/include/pulp_nn_kernels.h): activations HWC uint8,
convolution weights ``[ch_out][ky][kx][ch_in]`` int8, depthwise weights ``[ch][ky][kx]`` int8
(the reference depthwise takes CHW input, 32bit/src/pulp_nn_depthwise_generic.c:74), batch-norm
``k``/``lambda`` one per output channel, int32 or int64 depending on the tree.
"""
import math

import numpy as np


def ceil_log2(n):
    return int(math.ceil(math.log2(n))) if n > 1 else 0


def out_dim(n, k, pad_a, pad_b, stride):
    return (n + pad_a + pad_b - k) // stride + 1


def _bn(rng, n, bits, k_range, lam_range):
    dt = np.int32 if bits == 32 else np.int64
    k = rng.integers(k_range[0], k_range[1] + 1, size=n).astype(dt)
    lam = rng.integers(lam_range[0], lam_range[1] + 1, size=n).astype(dt)
    return k, lam


def conv_case(seed, H, W, Cin, Cout, kernel=(3, 3), strides=(1, 1), pads=(1, 1, 1, 1), batch=1,
              bits=32, out_shift=None, w_range=(-16, 15), k_range=(1, 64),
              lam_range=(-32768, 32767), with_bias=False, out_mult=1, relu=1, bn=1):
    """A standard-convolution case (pads = top, bottom, left, right; kernel = ky, kx)."""
    rng = np.random.default_rng(seed)
    ky, kx = kernel
    K = ky * kx * Cin
    case = dict(
        kind="conv", bits=bits, batch=batch, relu=relu, bn=bn, out_mult=out_mult,
        x=rng.integers(0, 256, size=(batch, H, W, Cin), dtype=np.uint8),
        w=rng.integers(w_range[0], w_range[1] + 1, size=(Cout, ky, kx, Cin)).astype(np.int8),
        kernel=kernel, strides=strides, pads=pads,
        out_hw=(out_dim(H, ky, pads[0], pads[1], strides[0]), out_dim(W, kx, pads[2], pads[3], strides[1])),
        out_shift=ceil_log2(K) + 11 if out_shift is None else out_shift,
    )
    case["k"], case["lam"] = _bn(rng, Cout, bits, k_range, lam_range)
    case["bias"] = rng.integers(-128, 128, size=Cout).astype(np.int8) if with_bias else None
    return case


def pointwise_case(seed, H, W, Cin, Cout, batch=1, bits=32, out_shift=None, w_range=(-16, 15),
                   k_range=(1, 64), lam_range=(-32768, 32767), with_bias=False, out_mult=1,
                   relu=1, bn=1):
    rng = np.random.default_rng(seed)
    case = dict(
        kind="pointwise", bits=bits, batch=batch, relu=relu, bn=bn, out_mult=out_mult,
        x=rng.integers(0, 256, size=(batch, H, W, Cin), dtype=np.uint8),
        w=rng.integers(w_range[0], w_range[1] + 1, size=(Cout, Cin)).astype(np.int8),
        out_shift=ceil_log2(Cin) + 11 if out_shift is None else out_shift,
    )
    case["k"], case["lam"] = _bn(rng, Cout, bits, k_range, lam_range)
    case["bias"] = rng.integers(-128, 128, size=Cout).astype(np.int8) if with_bias else None
    return case


def depthwise_case(seed, H, W, C, kernel=(3, 3), strides=(1, 1), pads=(1, 1, 1, 1), batch=1,
                   bits=32, out_shift=15, w_range=(-16, 15), k_range=(1, 64),
                   lam_range=(-32768, 32767), with_bias=False, out_mult=1, relu=1, bn=1,
                   hwc=False):
    """Depthwise case. x is CHW (the reference layout) unless hwc=True."""
    rng = np.random.default_rng(seed)
    ky, kx = kernel
    shape = (batch, H, W, C) if hwc else (batch, C, H, W)
    case = dict(
        kind="depthwise", bits=bits, batch=batch, relu=relu, bn=bn, out_mult=out_mult, hwc=hwc,
        x=rng.integers(0, 256, size=shape, dtype=np.uint8),
        w=rng.integers(w_range[0], w_range[1] + 1, size=(C, ky, kx)).astype(np.int8),
        kernel=kernel, strides=strides, pads=pads,
        out_hw=(out_dim(H, ky, pads[0], pads[1], strides[0]), out_dim(W, kx, pads[2], pads[3], strides[1])),
        out_shift=out_shift,
    )
    case["k"], case["lam"] = _bn(rng, C, bits, k_range, lam_range)
    case["bias"] = rng.integers(-128, 128, size=C).astype(np.int8) if with_bias else None
    return case


def linear_case(seed, K, N, batch=1, bits=32, out_shift=None, w_range=(-16, 15), k_range=(1, 64),
                lam_range=(-32768, 32767), with_bias=True, out_mult=1, relu=1, bn=0):
    rng = np.random.default_rng(seed)
    case = dict(
        kind="linear", bits=bits, batch=batch, relu=relu, bn=bn, out_mult=out_mult,
        x=rng.integers(0, 256, size=(batch, K), dtype=np.uint8),
        w=rng.integers(w_range[0], w_range[1] + 1, size=(N, K)).astype(np.int8),
        out_shift=ceil_log2(K) + 11 if out_shift is None else out_shift,
    )
    case["k"], case["lam"] = _bn(rng, N, bits, k_range, lam_range)
    case["bias"] = rng.integers(-128, 128, size=N).astype(np.int8) if with_bias else None
    # pulp_nn_linear_out_32 reads its bias as int32 words (32bit/src/pulp_nn_linear_out_32.c:54)
    case["bias32"] = rng.integers(-2 ** 20, 2 ** 20, size=N).astype(np.int32) if with_bias else None
    return case


# ---- the five benchmark configurations --------------------------------------------------------

def config_c1(batch=1):
    """Standard conv 32x32x32 -> 64, 3x3 s1 p1, 32-bit BN, shift ceil(log2 288)+11, seed 0."""
    return conv_case(0, 32, 32, 32, 64, batch=batch, bits=32)


def config_c2(batch=64):
    """Pointwise 56x56x128 -> 256, 32-bit BN, shift ceil(log2 128)+11."""
    return pointwise_case(1, 56, 56, 128, 256, batch=batch, bits=32)


def config_c3(batch=64):
    """Depthwise 3x3 s2 p1 on 112x112x64, CHW in / HWC out, 64-bit BN, shift 14."""
    return depthwise_case(2, 112, 112, 64, strides=(2, 2), batch=batch, bits=64, out_shift=14,
                          w_range=(-64, 63), k_range=(1, 256), lam_range=(-2 ** 20, 2 ** 20))


def config_c4(batch=256):
    """Linear 4096 -> 4096 (uint8 and int32 outputs), int8 bias, shift ceil(log2 4096)+11."""
    return linear_case(3, 4096, 4096, batch=batch, bits=32)


# ---- MobileNetV1-1.0, 224x224x3 ---------------------------------------------------------------

MOBILENET_PW_CHANNELS = (64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024)
MOBILENET_STRIDE2_PAIRS = (2, 4, 6, 12)          # 1-based pair index whose depthwise has stride 2
MOBILENET_CLASSES = 1000


def mobilenet_v1_layers(in_hw=224):
    """The 29-call layer stack: conv1, 13 x (depthwise, pointwise), avgpool, fc (int32 out)."""
    layers = []
    H = in_hw
    Ho = out_dim(H, 3, 1, 1, 2)
    layers.append(dict(name="conv1", op="conv", H=H, W=H, Cin=3, Cout=32, stride=2, Ho=Ho, Wo=Ho,
                       K=27))
    H, C = Ho, 32
    for i, cout in enumerate(MOBILENET_PW_CHANNELS, start=1):
        s = 2 if i in MOBILENET_STRIDE2_PAIRS else 1
        Ho = out_dim(H, 3, 1, 1, s)
        layers.append(dict(name="dw%d" % i, op="depthwise", H=H, W=H, Cin=C, Cout=C, stride=s,
                           Ho=Ho, Wo=Ho, K=9))
        H = Ho
        layers.append(dict(name="pw%d" % i, op="pointwise", H=H, W=H, Cin=C, Cout=cout, stride=1,
                           Ho=H, Wo=H, K=C))
        C = cout
    layers.append(dict(name="avgpool", op="avgpool", H=H, W=H, Cin=C, Cout=C, stride=H, Ho=1, Wo=1,
                       K=H * H))
    layers.append(dict(name="fc", op="linear32", H=1, W=1, Cin=C, Cout=MOBILENET_CLASSES, stride=1,
                       Ho=1, Wo=1, K=C))
    return layers


def mobilenet_params(seed=4, bits=32, shift_bias=11, in_hw=224, w_range=(-16, 15),
                     k_range=(1, 64), lam_range=(-32768, 32767)):
    """Random-init parameters for every layer. out_shift = ceil(log2 K) + shift_bias.

    shift_bias=11 is the benchmark's literal setting (outputs collapse to zero after a few
    layers, which is fine for timing); a smaller value (e.g. 1) keeps activations alive through
    the whole stack and is what the parity tests use in addition.
    """
    rng = np.random.default_rng(seed)
    params = []
    for L in mobilenet_v1_layers(in_hw):
        p = dict(L)
        if L["op"] == "conv":
            p["w"] = rng.integers(w_range[0], w_range[1] + 1, size=(L["Cout"], 3, 3, L["Cin"])).astype(np.int8)
        elif L["op"] == "depthwise":
            p["w"] = rng.integers(w_range[0], w_range[1] + 1, size=(L["Cin"], 3, 3)).astype(np.int8)
        elif L["op"] in ("pointwise", "linear32"):
            p["w"] = rng.integers(w_range[0], w_range[1] + 1, size=(L["Cout"], L["Cin"])).astype(np.int8)
        if L["op"] in ("conv", "depthwise", "pointwise"):
            p["k"], p["lam"] = _bn(rng, L["Cout"], bits, k_range, lam_range)
            p["out_shift"] = ceil_log2(L["K"]) + shift_bias
        params.append(p)
    return params


def mobilenet_input(seed, batch, in_hw=224):
    rng = np.random.default_rng(seed)
    return rng.integers(0, 256, size=(batch, in_hw, in_hw, 3), dtype=np.uint8)


def mobilenet_ops_bytes(in_hw=224):
    """(ops, algorithmic bytes) per image and per layer: 2*M*N*K for the contractions,
    2*taps per output for depthwise; bytes = input + output (+ parameters once, ignored here)."""
    rows = []
    for L in mobilenet_v1_layers(in_hw):
        in_b = L["H"] * L["W"] * L["Cin"]
        out_b = L["Ho"] * L["Wo"] * L["Cout"] * (4 if L["op"] == "linear32" else 1)
        if L["op"] in ("conv", "pointwise", "linear32"):
            ops = 2 * L["Ho"] * L["Wo"] * L["Cout"] * L["K"]
        elif L["op"] == "depthwise":
            ops = 2 * L["Ho"] * L["Wo"] * L["Cout"] * 9
        else:
            ops = L["H"] * L["W"] * L["Cin"]
        rows.append(dict(name=L["name"], ops=ops, bytes=in_b + out_b))
    return rows
