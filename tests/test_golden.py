"""Golden vectors: tests/golden/vectors.npz holds inputs and the outputs the unmodified reference
kernels gave for them (made by tests/golden/make_golden.py). The C restatement must reproduce
them on any machine (CPU test); the CUDA library must reproduce them on a GPU (gpu test)."""
import json
import os

import numpy as np
import pytest

from conftest import pulpnn

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "vectors.npz")


def load_cases():
    z = np.load(GOLD)
    meta = json.loads(bytes(z["meta"]).decode())
    cases = {}
    for name, m in meta.items():
        c = dict(m)
        for key in z.files:
            if key.startswith(name + "/"):
                c[key[len(name) + 1:]] = z[key]
        for key in ("kernel", "strides", "pads", "out_hw"):
            if key in c:
                c[key] = tuple(c[key])
        cases[name] = c
    return cases


CASES = load_cases()


def run_case(impl, name, c):
    """Returns {output name: array} computed by impl for one golden case."""
    g = lambda key: c.get(key)   # noqa: E731
    if name.startswith("conv"):
        kw = dict(bias=g("bias"), out_mult=c["out_mult"], out_shift=c["out_shift"], out_hw=c["out_hw"],
                  kernel=c["kernel"], pads=c["pads"], strides=c["strides"], relu=c["relu"], bn=c["bn"])
        res = {}
        for v in ("Ho", "HoWo"):
            if "out_" + v in c:
                res[v] = impl.conv(c["bits"], c["x"], c["w"], c["k"], c["lam"], variant=v, **kw)
        return res
    if name.startswith("pw"):
        return {"HoWo": impl.pointwise(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=g("bias"),
                                       out_mult=c["out_mult"], out_shift=c["out_shift"],
                                       relu=c["relu"], bn=c["bn"])}
    if name.startswith("dw"):
        return {"out": impl.depthwise(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=g("bias"),
                                      out_mult=c["out_mult"], out_shift=c["out_shift"],
                                      out_hw=c["out_hw"], kernel=c["kernel"], pads=c["pads"],
                                      strides=c["strides"], relu=c["relu"], bn=c["bn"])}
    if name.startswith("linear"):
        b32 = c["bias32"].view(np.int8) if "literal" not in name else None
        return {"u8": impl.linear(c["bits"], c["x"], c["w"], c["k"], c["lam"], bias=g("bias"),
                                  out_mult=c["out_mult"], out_shift=c["out_shift"], relu=c["relu"],
                                  bn=c["bn"]),
                "i32": impl.linear_out_32(c["x"], c["w"], bias32=b32)}
    if name.startswith("maxpool"):
        out, after = impl.maxpool(c["x"], out_hw=c["out_hw"], kernel=c["kernel"], pads=c["pads"],
                                  strides=c["strides"], want_input_after=True)
        return {"out": out, "input_after": after}
    if name.startswith("avgpool"):
        return {"out": impl.avgpool(c["bits"], c["x"], lam=c["lam"], out_shift=c["out_shift"],
                                    out_add=c["out_add"], out_hw=c["out_hw"], kernel=c["kernel"],
                                    pads=c["pads"], strides=c["strides"], requant=c["requant"])}
    if name.startswith("add"):
        return {"out": impl.add(c["x"], c["x2"], m1=c["m1"], m2=c["m2"], out_shift=c["out_shift"])}
    raise KeyError(name)


def check(impl, name):
    c = CASES[name]
    res = run_case(impl, name, c)
    assert res, name
    for key, got in res.items():
        want = c["out_" + key]
        assert got.dtype == want.dtype and got.shape == want.shape
        assert np.array_equal(got, want), "%s/%s differs from the reference's output" % (name, key)


def test_fixture_is_complete():
    assert len(CASES) >= 30
    kinds = {n.split("_")[0] for n in CASES}
    assert kinds == {"conv", "pw", "dw", "linear", "maxpool", "avgpool", "add"}
    # the literal benchmark parameters give almost-all-zero outputs; the live ones do not
    assert np.count_nonzero(CASES["conv_c1_literal"]["out_Ho"]) < 2000
    assert np.count_nonzero(CASES["pw_128_256_live"]["out_HoWo"]) > 5000


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_reproduces_reference_outputs(name, restatement):
    check(restatement, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_reproduces_reference_outputs(name):
    check(pulpnn.GpuKernels(host_buffers=False), name)
    assert pulpnn.api.device_status() == 0
