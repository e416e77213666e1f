#!/usr/bin/env python
"""Generates tests/golden/vectors.npz: inputs and outputs of the UNMODIFIED reference kernels.

The reference ships no test vectors, so these were produced by running its own sources (compiled
in place by oracle/Makefile into oracle/_ref/) on small seeded inputs. Run from the repo root on
a machine that has the reference tree:

    python tests/golden/make_golden.py

The file travels with the repository, so the C restatement and the CUDA kernels can be checked
against the reference's answers on machines where the reference itself is absent.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402
from oracle import bindings  # noqa: E402

wl = entry.load_package().workloads
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vectors.npz")

ARRAYS = ("x", "w", "k", "lam", "bias", "bias32", "x2")


def pack(store, meta, name, case, **outputs):
    m = {}
    for key, val in case.items():
        if isinstance(val, np.ndarray):
            store["%s/%s" % (name, key)] = val
        elif val is not None:
            m[key] = val
    for key, val in outputs.items():
        store["%s/out_%s" % (name, key)] = val
    meta[name] = m


def main():
    bindings.build()
    ref = {32: bindings.CompiledReference(32), 64: bindings.CompiledReference(64)}
    store, meta = {}, {}

    def conv_kw(c):
        return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                    kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])

    # standard convolution: the literal first benchmark configuration and ragged shapes in all modes
    c = wl.config_c1()
    pack(store, meta, "conv_c1_literal", c,
         Ho=ref[32].conv(32, c["x"], c["w"], c["k"], c["lam"], variant="Ho", **conv_kw(c)),
         HoWo=ref[32].conv(32, c["x"], c["w"], c["k"], c["lam"], variant="HoWo", **conv_kw(c)))
    c = wl.conv_case(0, 32, 32, 32, 64, bits=64, out_shift=12, with_bias=True)
    pack(store, meta, "conv_c1_live_bn64", c,
         Ho=ref[64].conv(64, c["x"], c["w"], c["k"], c["lam"], variant="Ho", **conv_kw(c)))
    for bits in (32, 64):
        for relu, bn in ((1, 1), (1, 0), (0, 0), (0, 1), (2, 0)):
            c = wl.conv_case(11, 13, 11, 5, 7, kernel=(3, 5), strides=(2, 1), pads=(1, 0, 2, 1), batch=2,
                             bits=bits, out_shift=9, with_bias=True, out_mult=5, relu=relu, bn=bn,
                             k_range=(-64, 64), lam_range=(-2 ** 20, 2 ** 20))
            pack(store, meta, "conv_ragged_bn%d_r%d_b%d" % (bits, relu, bn), c,
                 HoWo=ref[bits].conv(bits, c["x"], c["w"], c["k"], c["lam"], variant="HoWo", **conv_kw(c)))
    c = wl.conv_case(12, 9, 9, 16, 8, bits=32, out_shift=12, w_range=(-128, 127),
                     k_range=(2 ** 20, 2 ** 24), lam_range=(-2 ** 30, 2 ** 30))
    pack(store, meta, "conv_bn32_wraparound", c,
         Ho=ref[32].conv(32, c["x"], c["w"], c["k"], c["lam"], **conv_kw(c)))

    def pw_kw(c):
        return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"],
                    bn=c["bn"])

    # pointwise: second benchmark configuration's channel counts on a small image; ragged shapes
    for name, c in (("pw_128_256_literal", wl.pointwise_case(1, 14, 14, 128, 256, batch=1, bits=32)),
                    ("pw_128_256_live", wl.pointwise_case(1, 14, 14, 128, 256, batch=1, bits=32, out_shift=10)),
                    ("pw_80_48_bn64", wl.pointwise_case(22, 9, 7, 80, 48, batch=2, bits=64, out_shift=8,
                                                        with_bias=True, w_range=(-128, 127))),
                    ("pw_ragged_mult", wl.pointwise_case(21, 9, 7, 22, 13, batch=2, bits=32, out_shift=8,
                                                         with_bias=True, out_mult=3, relu=1, bn=0))):
        b = c["bits"]
        pack(store, meta, name, c, HoWo=ref[b].pointwise(b, c["x"], c["w"], c["k"], c["lam"], **pw_kw(c)))

    def dw_kw(c):
        return dict(bias=c["bias"], out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                    kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])

    # depthwise: third benchmark configuration's parameters on a small image, both strides/trees
    for bits in (32, 64):
        for s in (1, 2):
            c = wl.depthwise_case(2, 28, 28, 16, strides=(s, s), batch=1, bits=bits, out_shift=14,
                                  w_range=(-64, 63), k_range=(1, 256), lam_range=(-2 ** 20, 2 ** 20))
            pack(store, meta, "dw_28_16_s%d_bn%d" % (s, bits), c,
                 out=ref[bits].depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)))
    c = wl.depthwise_case(32, 12, 12, 4, kernel=(5, 5), pads=(2, 2, 2, 2), batch=1, out_shift=8,
                          with_bias=True, out_mult=3, relu=1, bn=0)
    pack(store, meta, "dw_5x5_mult", c, out=ref[32].depthwise(32, c["x"], c["w"], c["k"], c["lam"], **dw_kw(c)))

    # linear, both outputs
    for bits, relu, bn in ((32, 1, 0), (64, 1, 1), (32, 0, 0)):
        c = wl.linear_case(41, 203, 37, batch=2, bits=bits, out_shift=6, out_mult=3, relu=relu, bn=bn,
                           w_range=(-128, 127))
        pack(store, meta, "linear_203_37_bn%d_r%d_b%d" % (bits, relu, bn), c,
             u8=ref[bits].linear(bits, c["x"], c["w"], c["k"], c["lam"], bias=c["bias"], out_mult=3,
                                 out_shift=6, relu=relu, bn=bn),
             i32=ref[bits].linear_out_32(c["x"], c["w"], bias32=c["bias32"].view(np.int8)))
    c = wl.linear_case(3, 4096, 64, batch=1, bits=32)
    pack(store, meta, "linear_4096_64_literal", c,
         u8=ref[32].linear(32, c["x"], c["w"], c["k"], c["lam"], bias=c["bias"], out_mult=1,
                           out_shift=c["out_shift"], relu=1, bn=0),
         i32=ref[32].linear_out_32(c["x"], c["w"]))

    # pooling and add
    rng = np.random.default_rng(51)
    x = rng.integers(0, 256, size=(1, 14, 14, 10), dtype=np.uint8)
    for i, g in enumerate((dict(kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0), out_hw=(7, 7)),
                           dict(kernel=(3, 3), strides=(2, 2), pads=(1, 1, 1, 1), out_hw=(7, 7)))):
        out, after = ref[32].maxpool(x, want_input_after=True, **g)
        pack(store, meta, "maxpool_%d" % i, dict(x=x, **g), out=out, input_after=after)
    for bits, (requant, lam, add, shift) in ((32, (0, 0, 0, 0)), (32, (1, -3, 5, 2)), (64, (1, -3, 5, 2)),
                                             (64, (1, 300, 128, 8))):
        g = dict(kernel=(7, 7), strides=(7, 7), pads=(0, 0, 0, 0), out_hw=(2, 2))
        out = ref[bits].avgpool(bits, x, lam=lam, out_shift=shift, out_add=add, requant=requant, **g)
        pack(store, meta, "avgpool_bn%d_q%d_l%d" % (bits, requant, lam),
             dict(x=x, bits=bits, lam=lam, out_shift=shift, out_add=add, requant=requant, **g), out=out)
    a = rng.integers(0, 256, size=(1, 14, 13, 11), dtype=np.uint8)
    b = rng.integers(0, 256, size=(1, 14, 13, 11), dtype=np.uint8)
    for m1, m2, shift in ((37, 91, 6), (65535, 3, 4)):
        pack(store, meta, "add_%d_%d" % (m1, m2), dict(x=a, x2=b, m1=m1, m2=m2, out_shift=shift),
             out=ref[32].add(a, b, m1=m1, m2=m2, out_shift=shift))

    store["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **store)
    print("wrote %s: %d cases, %.1f KB" % (OUT, len(meta), os.path.getsize(OUT) / 1024))


if __name__ == "__main__":
    main()
