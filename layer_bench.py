#!/usr/bin/env python
"""Single-kernel measurements: the four single-layer benchmark configurations and the layer shapes
of MobileNetV1, one C-ABI call each, timed with CUDA events on device-resident buffers.

    python layer_bench.py --case c2            # pointwise 56x56x128 -> 256, batch 64
    python layer_bench.py --case pw1 --batch 128 --reps 3
    python layer_bench.py --all

Prints one JSON line per case: milliseconds per call, GOP/s, algorithmic GB/s and the fraction of
the measured HBM bandwidth (MEASURED_PEAKS.json at the repository root, if present). With a small
batch and few repetitions it is also the command to profile one kernel in isolation.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

POINTWISE = {"pw1": (112, 32, 64), "pw2": (56, 64, 128), "pw3": (56, 128, 128), "pw4": (28, 128, 256),
             "pw5": (28, 256, 256), "pw6": (14, 256, 512), "pw7": (14, 512, 512), "pw12": (7, 512, 1024),
             "pw13": (7, 1024, 1024), "c2": (56, 128, 256)}
DEPTHWISE = {"dw1": (112, 32, 1), "dw2": (112, 64, 2), "dw3": (56, 128, 1), "dw4": (56, 128, 2),
             "dw5": (28, 256, 1), "dw6": (28, 256, 2), "dw7": (14, 512, 1), "dw12": (14, 512, 2),
             "dw13": (7, 1024, 1)}
DEFAULT_BATCH = {"c1": 1, "c2": 64, "c3": 64, "c4": 256}


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return float(json.load(open(p))["hbm_gbs"]) if os.path.exists(p) else 6650.0


def build_case(name, B, pkg):
    """Returns (callable, ops, algorithmic bytes) for one case."""
    import torch
    api, wl = pkg.api, pkg.workloads

    def dev(a):
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def out(shape, dt=torch.uint8):
        return torch.zeros(shape, dtype=dt, device="cuda")

    if name in POINTWISE:
        H, cin, cout = POINTWISE[name]
        c = wl.pointwise_case(1, H, H, cin, cout, batch=B, bits=32)
        x, w, k, lam, o = dev(c["x"]), dev(c["w"]), dev(c["k"]), dev(c["lam"]), out((B, H, H, cout))
        fn = lambda: api.pulp_nn_pointwise_HoWo_parallel(32, x, None, None, o, w, k, lam, 1, c["out_shift"], H, H,  # noqa: E731
                                                         cin, H, H, cout, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1)
        return fn, 2.0 * B * H * H * cin * cout, B * H * H * (cin + cout) + cin * cout, (x, w, k, lam, o)
    if name in DEPTHWISE or name == "c3":
        if name == "c3":
            c = wl.config_c3(batch=B)
            H, C, s, bits, hwc = 112, 64, 2, 64, False
        else:
            H, C, s = DEPTHWISE[name]
            bits, hwc = 32, True
            c = wl.depthwise_case(2, H, H, C, strides=(s, s), batch=B, bits=32, hwc=True)
        Ho = c["out_hw"][0]
        x, w, k, lam, o = dev(c["x"]), dev(c["w"]), dev(c["k"]), dev(c["lam"]), out((B, Ho, Ho, C))
        call = api.pulpnn_depthwise_hwc if hwc else api.pulp_nn_depthwise_generic
        fn = lambda: call(bits, x, None, None, o, w, None, k, lam, 1, c["out_shift"], H, H, C, Ho, Ho, C,  # noqa: E731
                          3, 3, 1, 1, 1, 1, s, s, 1, 1)
        return fn, 2.0 * B * Ho * Ho * C * 9, B * C * (H * H + Ho * Ho), (x, w, k, lam, o)
    if name == "net":
        # MobileNetV1 through the network runner, literal parameters: the device-resident benchmark step
        # alone (for a launch list of exactly one step's kernels)
        params = wl.mobilenet_params(seed=4, bits=32, shift_bias=11)
        net = api.build_mobilenet_v1(params, bits=32, max_batch=B)
        x = torch.from_numpy(wl.mobilenet_input(100, B)).cuda()
        o = out((B, 1000), torch.int32)
        rows = wl.mobilenet_ops_bytes()
        return ((lambda: net.run(x, o, B)), float(sum(r["ops"] for r in rows)) * B, sum(r["bytes"] for r in rows) * B,
                (net, x, o))
    if name.startswith("dwpw"):
        # a depthwise layer and the pointwise layer behind it through the network runner: one fused
        # kernel where the library has one (PULPNN_OPT_FUSE_DWPW), else two kernels
        idx = name[4:]
        H, C, s = DEPTHWISE["dw" + idx]
        Hp, cin, cout = POINTWISE["pw" + idx]
        dw = wl.depthwise_case(2, H, H, C, strides=(s, s), batch=1, bits=32, hwc=True)
        pw = wl.pointwise_case(1, Hp, Hp, cin, cout, batch=1, bits=32)
        net = api.Net(32, B)
        net.add_layer(api.LAYER_DEPTHWISE, dim_in=(H, H), ch_in=C, dim_out=(Hp, Hp), ch_out=C, kernel=(3, 3),
                      pads=(1, 1, 1, 1), strides=(s, s), out_shift=dw["out_shift"], weights=dw["w"], k=dw["k"], lam=dw["lam"])
        net.add_layer(api.LAYER_POINTWISE, dim_in=(Hp, Hp), ch_in=cin, dim_out=(Hp, Hp), ch_out=cout,
                      out_shift=pw["out_shift"], weights=pw["w"], k=pw["k"], lam=pw["lam"])
        net.finalize()
        x = torch.randint(0, 256, (B, H, H, C), dtype=torch.uint8, device="cuda")
        o = out((B, Hp, Hp, cout))
        ops = 2.0 * B * Hp * Hp * C * 9 + 2.0 * B * Hp * Hp * cin * cout
        return (lambda: net.run(x, o, B)), ops, B * (H * H * C + Hp * Hp * cout), (net, x, o)
    if name in ("c1", "conv1"):
        if name == "c1":
            c = wl.config_c1(batch=B)
            H, cin, cout, s = 32, 32, 64, 1
        else:
            c = wl.conv_case(3, 224, 224, 3, 32, strides=(2, 2), batch=B, bits=32)
            H, cin, cout, s = 224, 3, 32, 2
        Ho = c["out_hw"][0]
        x, w, k, lam, o = dev(c["x"]), dev(c["w"]), dev(c["k"]), dev(c["lam"]), out((B, Ho, Ho, cout))
        fn = lambda: api.pulp_nn_conv_Ho_parallel(32, x, None, None, o, w, k, lam, 1, c["out_shift"], H, H, cin,  # noqa: E731
                                                  Ho, Ho, cout, 3, 3, 1, 1, 1, 1, s, s, 1, 1)
        return (fn, 2.0 * B * Ho * Ho * cout * 9 * cin, B * (H * H * cin + Ho * Ho * cout) + cout * 9 * cin,
                (x, w, k, lam, o))
    if name in ("c4", "c4_out32"):
        c = wl.config_c4(batch=B)
        x, w, bias = dev(c["x"]), dev(c["w"]), dev(c["bias"])
        if name == "c4":
            o = out((B, 4096))
            fn = lambda: api.pulp_nn_linear(32, x, bias, o, w, None, None, 1, c["out_shift"], 4096, 4096, 1, 0)  # noqa: E731
            nbytes = B * 4096 * 2 + 4096 * 4096
        else:
            o = out((B, 4096), torch.int32)
            fn = lambda: api.pulp_nn_linear_out_32(32, x, None, o, w, 4096, 4096)  # noqa: E731
            nbytes = B * 4096 * 5 + 4096 * 4096
        return fn, 2.0 * B * 4096 * 4096, nbytes, (x, w, bias, o)
    if name == "fc":
        # MobileNet's classifier: 1024 -> 1000, raw int32 logits
        c = wl.linear_case(5, 1024, 1000, batch=B, bits=32, with_bias=False)
        x, w, o = dev(c["x"]), dev(c["w"]), out((B, 1000), torch.int32)
        fn = lambda: api.pulp_nn_linear_out_32(32, x, None, o, w, 1024, 1000)  # noqa: E731
        return fn, 2.0 * B * 1024 * 1000, B * (1024 + 4000) + 1024 * 1000, (x, w, o)
    if name in ("add", "maxpool", "avgpool"):
        # the byte movers on a 56x56x128 tensor (3 bytes per element for add; 2x2 stride-2 max pool;
        # the network's 7x7 global average pool on 7x7x1024)
        if name == "add":
            a = torch.randint(0, 256, (B, 56, 56, 128), dtype=torch.uint8, device="cuda")
            b = torch.randint(0, 256, (B, 56, 56, 128), dtype=torch.uint8, device="cuda")
            o = torch.empty_like(a)
            return (lambda: api.pulp_nn_add(32, a, b, o, 37, 91, 6, 56, 56, 128)), 0.0, 3 * a.numel(), (a, b, o)
        if name == "maxpool":
            x = torch.randint(0, 256, (B, 56, 56, 128), dtype=torch.uint8, device="cuda")
            o = torch.empty((B, 28, 28, 128), dtype=torch.uint8, device="cuda")
            return ((lambda: api.pulp_nn_maxpool(32, x, o, 56, 56, 128, 28, 28, 2, 2, 0, 0, 0, 0, 2, 2)), 0.0,
                    x.numel() + o.numel(), (x, o))
        x = torch.randint(0, 256, (B, 7, 7, 1024), dtype=torch.uint8, device="cuda")
        o = torch.empty((B, 1, 1, 1024), dtype=torch.uint8, device="cuda")
        return ((lambda: api.pulp_nn_avgpool(32, x, o, 0, 0, 0, 7, 7, 1024, 1, 1, 7, 7, 0, 0, 0, 0, 7, 7, 0)), 0.0,
                x.numel() + o.numel(), (x, o))
    if name in ("chw_to_hwc", "hwc_to_chw"):
        # the layout change a reference-style chain needs before every depthwise call: dw2's tensor
        H, C = 112, 64
        x = torch.randint(0, 256, (B, C, H, H) if name == "chw_to_hwc" else (B, H, H, C), dtype=torch.uint8, device="cuda")
        o = torch.empty((B, H, H, C) if name == "chw_to_hwc" else (B, C, H, H), dtype=torch.uint8, device="cuda")
        call = api.pulpnn_chw_to_hwc if name == "chw_to_hwc" else api.pulpnn_hwc_to_chw
        return (lambda: call(x, o, H, H, C)), 0.0, 2 * B * C * H * H, (x, o)
    raise SystemExit("unknown case %r" % name)


def int8_peak(reps):
    """Practical int8 tensor peak of this GPU: the library GEMM (torch._int_mm, cuBLASLt) on a large
    square, the denominator for the tensor-bound fraction of the GEMM layers."""
    import torch
    n = 8192
    a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (n, n), dtype=torch.int8, device="cuda").t().contiguous().t()   # column-major B
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(max(3, reps)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        torch._int_mm(a, b)
        ev1.record()
        torch.cuda.synchronize()
        best = min(best, ev0.elapsed_time(ev1))
    return {"case": "int8_peak", "how": "torch._int_mm %d^3, best of %d" % (n, max(3, reps)),
            "ms_per_call": round(best, 4), "TOPs": round(2.0 * n ** 3 / best / 1e9, 1)}


def run_case(name, B, reps, pkg, graph=False):
    import torch
    if name == "int8_peak":
        return int8_peak(reps)
    api = pkg.api
    api.set_batch(B)
    fn, ops, nbytes, keep = build_case(name, B, pkg)
    for _ in range(max(3, reps)):
        fn()
    api.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        # the calls are captured once and replayed: no host time between the kernels, which is what
        # a caller that chains layers in a CUDA graph sees (calls shorter than ~15 us are otherwise
        # paced by the Python/ctypes call, not by the GPU)
        stream = torch.cuda.Stream()
        api.set_stream(stream)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(reps):
                fn()
        api.set_stream(None)
        g.replay()
        torch.cuda.synchronize()
        ev0.record()
        g.replay()
        ev1.record()
    else:
        ev0.record()
        for _ in range(reps):
            fn()
        ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / reps
    assert api.device_status() == 0
    peak = hbm_peak()
    return {"case": name, "batch": B, "ms_per_call": round(ms, 5), "GOPs": round(ops / ms / 1e6, 1),
            "GBs": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / peak, 3),
            "timed": "graph replay" if graph else "calls", "algorithmic_bytes": int(nbytes), "working_set_larger_than_L2": bool(nbytes > 126e6)}


def print_trace(pkg):
    """clock64 stamps of CTA 0's roles per tile, and globaltimer stamps of its stations per launch."""
    import ctypes
    import numpy as np
    lib = pkg.load_library()
    if not hasattr(lib, "pulpnn_trace_read"):
        raise SystemExit("the library was built without -DPULPNN_TRACE")
    t = np.zeros((3, 64, 8), dtype=np.int64)
    lib.pulpnn_trace_read(t.ctypes.data_as(ctypes.c_void_p), t.size)
    names = {0: ["empty_seen", "load_issued"],
             1: ["start", "acc_free", "slab0", "slab1", "slab2", "slab3", "committed"],
             2: ["enter", "acc_full", "acc_returned", "round0_barrier", "round0_stored", "round1_barrier", "round1_stored"]}
    role_names = ["producer warp 0", "MMA warps", "epilogue warp 0"]
    base = t[1, 4, 0]
    for tile in range(4, 20):
        for role in (0, 1, 2):
            print("tile %2d %-16s" % (tile, role_names[role]),
                  " ".join("%s=%d" % (n, t[role, tile, k] - base) for k, n in enumerate(names[role])))
    print("cycles from tile to tile (MMA commit):", np.diff(t[1, 4:20, 6]).tolist())
    k = np.zeros((8, 8), dtype=np.int64)
    n = ctypes.c_int(0)
    lib.pulpnn_ktrace_read(k.ctypes.data_as(ctypes.c_void_p), ctypes.byref(n))
    stations = ["entry", "set up", "previous kernel complete", "first slab landed", "first tile committed",
                "first accumulator seen", "stores have read", "tensor memory freed"]
    previous = None
    for s_ in sorted(range(8), key=lambda i: k[i, 0]):
        r = k[s_]
        print("launch: " + ", ".join("%s +%d ns" % (stations[j], r[j] - r[0]) for j in range(1, 8)) +
              ("" if previous is None else "; entry %+d ns after the previous launch freed its tensor memory" % (r[0] - previous)))
        previous = r[7]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="c2")
    ap.add_argument("--batch", type=int, default=0, help="0 = the configuration's own batch (1024 for MobileNet layers)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--graph", action="store_true", help="capture the repetitions in one CUDA graph and time its replay")
    ap.add_argument("--split-k", type=int, default=0, help="force this many K-slices in the GEMM (0 = automatic)")
    ap.add_argument("--no-fuse", action="store_true", help="dwpwN cases: two kernels instead of the fused one")
    ap.add_argument("--tune", type=int, default=0, help="experimental kernel configurations (bit mask)")
    ap.add_argument("--trace", action="store_true",
                    help="print the per-role timing trace of igemm_tc_kernel (a library built with PULPNN_NVCC_FLAGS=-DPULPNN_TRACE)")
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    pkg = entry.load_package()
    pkg.api.set_device(0)
    if args.split_k:
        pkg.api.set_option(3, args.split_k)      # PULPNN_OPT_SPLIT_K
    if args.tune:
        pkg.api.set_option(pkg.api.OPT_TUNE, args.tune)
    if args.no_fuse:
        pkg.api.set_option(pkg.api.OPT_FUSE_DWPW, 0)
    names = [args.case]
    if args.all:
        names = list(dict.fromkeys(["c1", "c2", "c3", "c4", "c4_out32", "conv1"] + sorted(POINTWISE) + sorted(DEPTHWISE)))
    for n in names:
        B = args.batch or DEFAULT_BATCH.get(n, 1024)
        print(json.dumps(run_case(n, B, args.reps, pkg, args.graph)), flush=True)
    if args.trace:
        print_trace(pkg)


if __name__ == "__main__":
    main()
