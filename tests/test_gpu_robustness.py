"""Robustness of the C ABI on a GPU: the drop-in libraries with the reference's own symbol names,
the bounded-wait report, a second device in the same process."""
import ctypes as C

import numpy as np
import pytest

from conftest import pulpnn

pytestmark = pytest.mark.gpu
wl = pulpnn.workloads
api = pulpnn.api


def _dev(a):
    import torch
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("bits", [32, 64])
def test_dropin_libraries_compute(bits, restatement):
    """libpulpnn_b200_32.so / _64.so export the reference's unsuffixed names: a pointwise and a
    depthwise call through them (the call a program built against pulp_nn_kernels.h makes)."""
    import torch
    pulpnn.GpuKernels()
    lib = pulpnn.load_dropin(bits)
    dt = np.int32 if bits == 32 else np.int64
    u16, vp = C.c_uint16, C.c_void_p

    def ptr(t):
        return vp(0 if t is None else t.data_ptr())

    c = wl.pointwise_case(51, 14, 14, 64, 96, batch=1, bits=bits, out_shift=9)
    want = restatement.pointwise(bits, c["x"], c["w"], c["k"], c["lam"], out_shift=9)
    x, w, k, lam = _dev(c["x"]), _dev(c["w"]), _dev(c["k"].astype(dt)), _dev(c["lam"].astype(dt))
    out = torch.zeros((1, 14, 14, 96), dtype=torch.uint8, device="cuda")
    api.set_batch(1)
    f = lib.pulp_nn_pointwise_HoWo_parallel
    f.restype = None
    f(ptr(x), vp(0), vp(0), ptr(out), ptr(w), ptr(k), ptr(lam), u16(1), u16(9), u16(14), u16(14), u16(64), u16(14),
      u16(14), u16(96), u16(1), u16(1), u16(0), u16(0), u16(0), u16(0), u16(1), u16(1), C.c_int(1), C.c_int(1))
    api.synchronize()
    assert api._lib.load_library().pulpnn_last_error() == 0
    assert np.array_equal(out.cpu().numpy(), want)

    c = wl.depthwise_case(52, 16, 16, 32, strides=(1, 1), batch=1, bits=bits, out_shift=8)
    kw = dict(out_shift=8, out_hw=c["out_hw"], kernel=c["kernel"], pads=c["pads"], strides=c["strides"])
    want = restatement.depthwise(bits, c["x"], c["w"], c["k"], c["lam"], **kw)
    x, w, k, lam = _dev(c["x"]), _dev(c["w"]), _dev(c["k"].astype(dt)), _dev(c["lam"].astype(dt))
    out = torch.zeros((1, 16, 16, 32), dtype=torch.uint8, device="cuda")
    f = lib.pulp_nn_depthwise_generic
    f.restype = None
    f(ptr(x), vp(0), vp(0), ptr(out), ptr(w), vp(0), ptr(k), ptr(lam), u16(1), u16(8), u16(16), u16(16), u16(32),
      u16(16), u16(16), u16(32), u16(3), u16(3), u16(1), u16(1), u16(1), u16(1), u16(1), u16(1), C.c_int8(1),
      C.c_int8(1))
    api.synchronize()
    assert api._lib.load_library().pulpnn_last_error() == 0
    assert np.array_equal(out.cpu().numpy(), want)


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(restatement):
    """A kernel waits 1 ms on a barrier nothing completes: the wait gives up, the kernel ends
    through its ordinary exit, the status word carries a code, the host sees
    PULPNN_ERR_DEVICE_WAIT -- and the next ordinary call is clean and correct."""
    gpu = pulpnn.GpuKernels()
    lib = api._lib.load_library()
    assert api.device_status() == 0
    lib.pulpnn_clear_error()
    assert lib.pulpnn_selftest_wait_timeout(C.c_uint(1000)) == api.OK
    api.synchronize()
    assert api.device_status() != 0
    assert lib.pulpnn_last_error() == api.ERR_DEVICE_WAIT
    lib.pulpnn_clear_error()
    assert api.device_status() == 0, "the status word must be cleared once it has been read"
    c = wl.pointwise_case(53, 14, 14, 128, 128, batch=2, bits=32, out_shift=10)
    want = restatement.pointwise(32, c["x"], c["w"], c["k"], c["lam"], out_shift=10)
    assert np.array_equal(gpu.pointwise(32, c["x"], c["w"], c["k"], c["lam"], out_shift=10), want)
    assert api.device_status() == 0


def test_second_device_in_the_same_process(restatement):
    """The large-shared-memory kernels must work on a second GPU after the first one has used them
    in the same process (their per-function settings belong to a device)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cp = wl.pointwise_case(54, 14, 14, 256, 512, batch=4, bits=32, out_shift=10)
    cd = wl.depthwise_case(55, 28, 28, 128, batch=3, bits=32, out_shift=9, hwc=True)
    dkw = dict(out_shift=9, out_hw=cd["out_hw"], kernel=cd["kernel"], pads=cd["pads"], strides=cd["strides"],
               in_is_hwc=True)
    want_p = restatement.pointwise(32, cp["x"], cp["w"], cp["k"], cp["lam"], out_shift=10)
    want_d = restatement.depthwise(32, cd["x"], cd["w"], cd["k"], cd["lam"], **dkw)
    try:
        for device in (0, 1, 0):
            gpu = pulpnn.GpuKernels(device=device)
            assert np.array_equal(gpu.pointwise(32, cp["x"], cp["w"], cp["k"], cp["lam"], out_shift=10), want_p)
            assert np.array_equal(gpu.depthwise(32, cd["x"], cd["w"], cd["k"], cd["lam"], **dkw), want_d)
            assert api.device_status() == 0
    finally:
        pulpnn.GpuKernels(device=0)
