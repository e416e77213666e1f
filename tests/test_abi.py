"""The C-ABI library: it loads, exports everything include/*.h declares, and refuses to compute
without a GPU (no compute call is made here)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import pulpnn, _has_gpu


def test_library_builds_and_exports_every_declared_symbol():
    pulpnn.build_library()
    lib = pulpnn.load_library()
    names = pulpnn.declared_symbols()
    assert len(names) >= 45
    d32, d64 = pulpnn.load_dropin(32), pulpnn.load_dropin(64)
    for n in names:
        suffixed = n.endswith(("_bn32", "_bn64")) or n.startswith("pulpnn_") and not n.startswith("pulpnn_depthwise_hwc")
        if suffixed or n in ("pulpnn_depthwise_hwc_bn32", "pulpnn_depthwise_hwc_bn64"):
            assert hasattr(lib, n), n
        else:
            # the reference's own names live in the two drop-in libraries
            assert hasattr(d32, n) and hasattr(d64, n), n


def test_reference_names_present():
    want = ["pulp_nn_conv_Ho_parallel", "pulp_nn_conv_HoWo_parallel", "pulp_nn_pointwise_HoWo_parallel",
            "pulp_nn_depthwise_generic", "pulp_nn_linear", "pulp_nn_linear_out_32", "pulp_nn_maxpool",
            "pulp_nn_avgpool", "pulp_nn_add"]
    lib = pulpnn.load_library()
    for n in want:
        assert hasattr(lib, n + "_bn32") and hasattr(lib, n + "_bn64")
        assert hasattr(pulpnn.load_dropin(32), n) and hasattr(pulpnn.load_dropin(64), n)


def test_context_calls_without_compute():
    lib = pulpnn.load_library()
    api = pulpnn.api
    api.set_batch(7)
    assert api.get_batch() == 7
    with pytest.raises(pulpnn.PulpNNError) as e:
        api.set_batch(0)
    assert e.value.code == api.ERR_INVALID_ARG
    assert api.get_batch() == 7
    api.set_batch(1)
    api.set_option(api.OPT_FORCE_GENERIC, 1)
    assert api.get_option(api.OPT_FORCE_GENERIC) == 1
    api.set_option(api.OPT_FORCE_GENERIC, 0)
    with pytest.raises(pulpnn.PulpNNError):
        api.set_option(99, 1)
    assert isinstance(api.launch_count(), int)
    assert lib.pulpnn_last_error() == 0


@pytest.mark.skipif(_has_gpu(), reason="checks the behaviour on a machine without a GPU")
def test_no_gpu_means_error_not_fallback():
    api = pulpnn.api
    a = np.zeros((1, 4, 4, 16), np.uint8)
    out = np.full((1, 4, 4, 16), 7, np.uint8)
    with pytest.raises(pulpnn.PulpNNError) as e:
        api.pulp_nn_add(32, a, a, out, 1, 1, 0, 4, 4, 16)
    assert e.value.code == api.ERR_NO_DEVICE
    assert (out == 7).all()          # nothing was computed anywhere
    with pytest.raises(RuntimeError):
        pulpnn.GpuKernels()


def test_dropin_header_compiles_and_links_as_documented(tmp_path):
    """INTEGRATION.md's two-line switch: a C file that includes pulpnn_b200_dropin.h and uses the
    reference's names is compiled and linked with the documented line, then run. Without a GPU the
    call must record PULPNN_ERR_NO_DEVICE and leave the output alone; with one it must compute
    pulp_nn_add (32bit/src/pulp_nn_add.c:54-60)."""
    import subprocess
    pulpnn.build_library()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "pulp-nn_b200", "lib")
    exe = str(tmp_path / "dropin_app")
    subprocess.run(["cc", os.path.join(root, "tests", "data", "dropin_app.c"), "-I" + os.path.join(root, "include"),
                    "-L" + libdir, "-lpulpnn_b200_32", "-lpulpnn_b200", "-Wl,-rpath," + libdir, "-o", exe],
                   check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "status"
    if _has_gpu():
        a = (np.arange(256) * 7).astype(np.uint8).astype(np.uint32)
        b = (255 - np.arange(256)).astype(np.uint8).astype(np.uint32)
        want = np.minimum(((a * 3 + b * 5) >> 2) & 0xffff, 255)
        assert out[1] == "0" and int(out[3]) == int(want.sum())
    else:
        assert int(out[1]) == pulpnn.api.ERR_NO_DEVICE


def test_product_does_not_reach_the_checkers():
    """Nothing under the package or include/ may import, link or name the oracle."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "pulp-nn_b200")
    for base, _, files in os.walk(pkg):
        if "build" in base or base.endswith("lib"):
            continue
        for f in files:
            if not f.endswith((".py", ".cu", ".cuh", ".c", ".h")):
                continue
            text = open(os.path.join(base, f)).read()
            if f == "__init__.py":
                # smoke() is the one sanctioned user of the checker
                text = text.split("def smoke")[0]
            assert "oracle" not in text, os.path.join(base, f)
