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


def test_static_scratch_linear_matches_the_allocating_entry_point(restatement):
    import torch
    pulpnn.GpuKernels()                       # binds the device
    K, N = 4096, 4096
    rng = np.random.default_rng(77)
    w_np = rng.integers(-128, 128, size=(N, K)).astype(np.int8)
    bias_np = rng.integers(-2 ** 20, 2 ** 20, size=N).astype(np.int32)
    w, bias = _dev(w_np), _dev(bias_np)
    results = []
    # two calls in a row with different inputs and shapes: 32 vectors x 4 slices, then
    # 16 vectors x 8 slices (both 524288 partial sums, half of the built-in array)
    for call, (B, slices) in enumerate(((32, 4), (16, 8))):
        x_np = rng.integers(0, 256, size=(B, K), dtype=np.uint8)
        x = _dev(x_np)
        want = torch.zeros((B, N), dtype=torch.int32, device="cuda")
        api.set_batch(B)
        api.set_option(api.OPT_SPLIT_K, 1)        # the existing entry point, no split, no scratch
        try:
            api.pulp_nn_linear_out_32(32, x, bias, want, w, K, N)
        finally:
            api.set_option(api.OPT_SPLIT_K, 0)
        got = torch.full((B, N), -1, dtype=torch.int32, device="cuda")
        api.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        api.pulpnn_linear_out_32_static_scratch(x, bias, got, w, K, N, B, slices)
        api.synchronize()
        if call > 0:      # the first call on a device may make the driver load the module's data
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        assert api.device_status() == 0       # covers this entry point's own status word too
        assert torch.equal(got, want), "call %d differs from pulp_nn_linear_out_32" % call
        # ... and both equal the CPU checker (32bit/src/pulp_nn_linear_out_32.c:48-80)
        cpu = restatement.linear_out_32(x_np, w_np, bias32=bias_np)
        assert np.array_equal(got.cpu().numpy(), cpu), "call %d differs from the CPU checker" % call
        results.append(int(want.abs().max()))
    assert min(results) > 0
    # without a bias; neuron counts that are not a multiple of the tile width (1000) or of the
    # 16-byte store (1001: scalar stores of the partial sums); a reduction length that leaves the
    # last K slab partly empty (144 = 128 + 16)
    for (B, K2, N2, slices) in ((8, 1024, 1000, 2), (5, 1024, 1001, 4), (7, 144, 72, 2)):
        x_np = rng.integers(0, 256, size=(B, K2), dtype=np.uint8)
        w2_np = rng.integers(-16, 16, size=(N2, K2)).astype(np.int8)
        x, w2 = _dev(x_np), _dev(w2_np)
        got = torch.full((B, N2), -1, dtype=torch.int32, device="cuda")
        api.pulpnn_linear_out_32_static_scratch(x, None, got, w2, K2, N2, B, slices)
        api.synchronize()
        assert api.device_status() == 0
        assert np.array_equal(got.cpu().numpy(), restatement.linear_out_32(x_np, w2_np)), (B, K2, N2)


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
