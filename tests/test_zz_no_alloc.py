"""The split-K fully connected entry point that uses the scratch array built into the library
instead of allocated device memory (pulpnn_linear_out_32_static_scratch).

Who needs it: a caller that cannot let a library allocate -- a server whose own pool already owns
all free device memory, or a product with a fixed memory budget -- and therefore cannot use the
ordinary split-K path, which takes its partial-sum buffer from cudaMalloc. The entry point must
give exactly the int32 results of pulp_nn_linear_out_32 (integer sums: tolerance 0), on two calls in
a row (the second call finds the first call's leftovers in the shared array), and must refuse
problems larger than the built-in array. This file is collected last on purpose: a failure here
cannot hide a failure of any other test in a run that stops at the first failure.
"""
import numpy as np
import pytest

from conftest import pulpnn

pytestmark = pytest.mark.gpu
wl = pulpnn.workloads
api = pulpnn.api


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_static_scratch_linear_matches_the_allocating_entry_point():
    import torch
    pulpnn.GpuKernels()                       # binds the device
    K, N = 4096, 4096
    rng = np.random.default_rng(77)
    w = _dev(rng.integers(-128, 128, size=(N, K)).astype(np.int8))
    bias = _dev(rng.integers(-2 ** 20, 2 ** 20, size=N).astype(np.int32))
    results = []
    # two calls in a row with different inputs and shapes: 32 vectors x 4 slices, then
    # 16 vectors x 8 slices (both 524288 partial sums, half of the built-in array)
    for call, (B, slices) in enumerate(((32, 4), (16, 8))):
        x = _dev(rng.integers(0, 256, size=(B, K), dtype=np.uint8))
        want = torch.zeros((B, N), dtype=torch.int32, device="cuda")
        api.set_batch(B)
        api.set_option(api.OPT_SPLIT_K, 1)        # the existing entry point, no split, no scratch
        try:
            api.pulp_nn_linear_out_32(32, x, bias, want, w, K, N)
        finally:
            api.set_option(api.OPT_SPLIT_K, 0)
        got = torch.full((B, N), -1, dtype=torch.int32, device="cuda")
        api.pulpnn_linear_out_32_static_scratch(x, bias, got, w, K, N, B, slices)
        api.synchronize()
        assert api.device_status() == 0
        assert torch.equal(got, want), "call %d differs from pulp_nn_linear_out_32" % call
        results.append(int(want.abs().max()))
    assert min(results) > 0
    # without a bias, and a neuron count that is not a multiple of the tile width
    x = _dev(rng.integers(0, 256, size=(8, 1024), dtype=np.uint8))
    w2 = _dev(rng.integers(-16, 16, size=(1000, 1024)).astype(np.int8))
    want = torch.zeros((8, 1000), dtype=torch.int32, device="cuda")
    got = torch.zeros_like(want)
    api.set_batch(8)
    api.pulp_nn_linear_out_32(32, x, None, want, w2, 1024, 1000)
    api.pulpnn_linear_out_32_static_scratch(x, None, got, w2, 1024, 1000, 8, 2)
    api.synchronize()
    assert torch.equal(got, want)


def test_static_scratch_linear_refuses_what_does_not_fit():
    import torch
    pulpnn.GpuKernels()
    x = torch.zeros((256, 4096), dtype=torch.uint8, device="cuda")
    w = torch.zeros((4096, 4096), dtype=torch.int8, device="cuda")
    out = torch.zeros((256, 4096), dtype=torch.int32, device="cuda")
    with pytest.raises(pulpnn.PulpNNError) as e:       # 2 x 256 x 4096 partial sums > 1048576
        api.pulpnn_linear_out_32_static_scratch(x, None, out, w, 4096, 4096, 256, 2)
    assert e.value.code == api.ERR_UNSUPPORTED and "exceed" in str(e.value)
    with pytest.raises(pulpnn.PulpNNError) as e:       # nothing to split
        api.pulpnn_linear_out_32_static_scratch(x, None, out, w, 4096, 4096, 16, 1)
    assert e.value.code == api.ERR_INVALID_ARG
    host = np.zeros((16, 4096), np.uint8)              # host buffers would need staging memory
    with pytest.raises(pulpnn.PulpNNError):
        api.pulpnn_linear_out_32_static_scratch(host, None, out, w, 4096, 4096, 16, 2)
