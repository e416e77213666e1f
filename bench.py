#!/usr/bin/env python
"""Benchmark: MobileNetV1-int8 images/s on N B200s (one process per GPU).

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
  python bench.py --impl reference          # the reference's own C code on the host cores

A step is one pass of the 29-call layer stack over one batch of 1024 synthetic images, sharded by
batch over the GPUs (strong scaling: 1024/N images per GPU; nothing is exchanged but the final
logits gather). With N > 1 the weak-scaling figure (1024 images per GPU) is measured in the same run
and reported under "weak". `value` is measured with the batch already resident in HBM; `e2e` is the
same metric through the C ABI with host buffers (pinned input copied in, logits copied out, every
step). At N = 1 the line also carries configurations 1-4, the box's int8 GEMM and pinned-copy rates,
a sustained run and a parity check of the timed network against the CPU checker.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

WORKLOAD = "MobileNetV1-1.0 int8, 224x224x3 HWC uint8 inputs U[0,255], int8 weights U[-16,15], " \
           "32-bit BN k U[1,64] lambda U[-32768,32767], out_shift ceil(log2 K)+11"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, keep_samples=False):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        trace = []
        for ts, ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
            try:
                watts = float(f[6]) if len(f) > 6 else None
            except ValueError:
                watts = None
            trace.append((ts, sm[-1], watts))
        out = {"sm_mhz": statistics.median(sm) if sm else None,
               "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
               "samples": len(sm)}
        if keep_samples:
            out["trace"] = trace
        return out


# ---- CPU arm -----------------------------------------------------------------------------------
def cpu_chain_seconds(ref, params, x, bits=32):
    """Runs the layer chain on the compiled reference; returns (seconds in reference code incl.
    per-image buffer copies, seconds of HWC->CHW layout glue that is not reference code)."""
    total, glue = 0.0, 0.0
    cur = x
    for p in params:
        if p["op"] == "conv":
            cur = ref.conv(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"],
                           out_hw=(p["Ho"], p["Wo"]), kernel=(3, 3), pads=(1, 1, 1, 1),
                           strides=(p["stride"], p["stride"]), variant="HoWo")
        elif p["op"] == "depthwise":
            cur = ref.depthwise(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"],
                                out_hw=(p["Ho"], p["Wo"]), kernel=(3, 3), pads=(1, 1, 1, 1),
                                strides=(p["stride"], p["stride"]), in_is_hwc=True)
            glue += ref.last_glue_seconds
        elif p["op"] == "pointwise":
            cur = ref.pointwise(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"])
        elif p["op"] == "avgpool":
            cur = ref.avgpool(bits, cur, out_hw=(1, 1), kernel=(p["H"], p["W"]), pads=(0, 0, 0, 0),
                              strides=(p["H"], p["W"]))
        elif p["op"] == "linear32":
            cur = ref.linear_out_32(np.ascontiguousarray(cur.reshape(cur.shape[0], -1)), p["w"])
        total += ref.last_seconds
    return total, glue, cur


def port_chain_seconds(cpu, params, x, bits=32):
    """The same chain on the C restatement (no harness timers: wall clock)."""
    class Timed:
        last_glue_seconds = 0.0
        last_seconds = 0.0

        def __getattr__(self, name):
            fn = getattr(cpu, name)

            def call(*a, **kw):
                kw.pop("variant", None)
                t0 = time.time()
                r = fn(*a, **kw)
                self.last_seconds = time.time() - t0
                return r
            return call
    return cpu_chain_seconds(Timed(), params, x, bits)


def cpu_baseline(params, wl, budget_s=12.0, max_images=1024):
    """Times the reference's own C implementation (oracle/_ref) on the host cores, one worker
    thread per core over the images of a bounded sample. Falls back to the C restatement when the
    compiled reference is not present on this machine."""
    from oracle import bindings
    cores = os.cpu_count() or 1
    if bindings.have_reference(32):
        ref = bindings.CompiledReference(32, arena_mb=256, threads=cores)
        kind, build = "reference", ref.build_info()
        x = wl.mobilenet_input(7, min(cores, max_images))
        t, glue, _ = cpu_chain_seconds(ref, params, x)
        per_round = max(t, 1e-3)
        rounds = int(max(1, min(budget_s / per_round, max_images / x.shape[0])))
        n = x.shape[0] * rounds
        if rounds > 1:
            x = wl.mobilenet_input(7, n)
            t, glue, _ = cpu_chain_seconds(ref, params, x)
        return {"value": n / t, "unit": "images/s", "cores": cores, "kind": kind,
                "sample": "%d images through all 29 reference calls, %d threads over images, "
                          "NUM_CORES=1 per image; %.2f s of which %.2f s HWC->CHW glue outside the "
                          "reference; %s" % (n, cores, t, glue, build)}, (n, t)
    cpu = bindings.Restatement()          # OpenMP over images and pixels; only a last resort
    x = wl.mobilenet_input(7, 4)
    t, _, _ = port_chain_seconds(cpu, params, x)
    return {"value": 4 / t, "unit": "images/s", "cores": cores, "kind": "port",
            "sample": "4 images through the C restatement in %.2f s (compiled reference not built "
                      "here)" % t}, (4, t)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pkg = entry.load_package()
    wl = pkg.workloads
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=11)
    n_img, secs = 0, 0.0
    base = None
    for i in range(args.warmup + args.steps):
        # every step is a bounded sample; the whole run stays within a few minutes
        budget = args.budget or max(0.5, min(4.0, 150.0 / (args.warmup + args.steps)))
        base, (n, t) = cpu_baseline(params, wl, budget_s=budget, max_images=args.max_images)
        if i >= args.warmup:
            n_img += n
            secs += t
    value = n_img / secs
    base["value"] = value
    line = {"impl": "reference", "metric": "MobileNetV1-int8 images/s", "value": value, "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * secs / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8*s8->s32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_step": "bounded sample of <=256 images on the host cores"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- GPU arm -----------------------------------------------------------------------------------
def _event_ms(torch, fn, reps):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(reps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / reps


def measured_traffic_ratio(kernel):
    """DRAM bytes moved / algorithmic bytes of one launch, from an ncu capture of that kernel at the
    benchmark's batch (dram__bytes_read.sum + dram__bytes_write.sum); None when no capture is on file."""
    p = os.path.join(ROOT, "profiles", "dram_traffic_measured.json")
    if not os.path.exists(p):
        return None
    try:
        return json.load(open(p)).get(kernel)
    except Exception:
        return None


def single_layer_configs(pkg, torch, hbm_peak, int8_library_pops):
    """Configurations 1-4 with their literal parameters on device buffers: 200 back-to-back C-ABI
    calls between two CUDA events, and a CUDA-graph replay of the same 200 calls (calls shorter than
    about 15 us are paced by the Python call, not by the GPU)."""
    import layer_bench
    out = []
    for name, batch in (("c1", 1), ("c2", 64), ("c3", 64), ("c4", 256), ("c4_out32", 256)):
        r = layer_bench.run_case(name, batch, 200, pkg, graph=False)
        g = layer_bench.run_case(name, batch, 200, pkg, graph=True)
        us = g["ms_per_call"] * 1e3
        tops = g["GOPs"] / 1e3
        out.append({"name": name, "batch": batch, "us": round(us, 2), "us_python_calls": round(r["ms_per_call"] * 1e3, 2),
                    "GOPs": g["GOPs"], "GBs": g["GBs"], "hbm_frac": round(g["GBs"] / hbm_peak, 3),
                    "tc_frac_nominal": round(tops / 4500.0, 3),
                    "tc_frac_library": round(tops / int8_library_pops / 1e3, 3) if int8_library_pops else None,
                    "algorithmic_bytes": g["algorithmic_bytes"]})
    return out


def run_gpu_arm(args):
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer stores only, no NVLS binding
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this framework has no CPU path "
                         "(use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    api, wl = pkg.api, pkg.workloads
    api.set_device(local)
    api.set_stream(None)
    sharding = __import__("importlib").import_module("pulpnn_b200.sharding")
    params = wl.mobilenet_params(seed=4, bits=32, shift_bias=11)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def make_gather(n_total):
        if world == 1:
            return None
        if args.gather in ("auto", "peer"):
            try:
                return sharding.PeerLogits(n_total, 1000, torch.int32, rank, world, dev)
            except Exception as exc:      # no symmetric memory on this box
                if args.gather == "peer":
                    raise
                print("peer-mapped logits unavailable (%s): NCCL all-gather on a side stream" % exc)
        return sharding.OverlappedGather(n_total, 1000, torch.int32, rank, world, dev)

    class Job:
        """One scaling mode: this rank's slice of a global batch, its network and its buffers."""

        def __init__(self, global_batch):
            first, last = sharding.shard_bounds(global_batch, rank, world)
            self.B, self.global_batch = last - first, global_batch
            self.net = api.build_mobilenet_v1(params, bits=32, max_batch=self.B, micro_batch=args.micro)
            seed = 100 if world == 1 else 100 + rank
            self.x_host = torch.from_numpy(wl.mobilenet_input(seed, self.B)).pin_memory()
            self.x_dev = self.x_host.cuda()
            self.logits = torch.zeros((self.B, 1000), dtype=torch.int32, device="cuda")
            self.logits_host = torch.zeros((self.B, 1000), dtype=torch.int32).pin_memory()
            self.logits_host2 = torch.zeros((self.B, 1000), dtype=torch.int32).pin_memory()
            self.gather = make_gather(global_batch)

        def step(self):
            if self.gather is None:
                self.net.run(self.x_dev, self.logits, self.B)
            else:   # the only exchange of the whole path: the final logits gather
                self.net.run(self.x_dev, self.gather.target(), self.B)
                self.gather.publish()

        def step_e2e(self):
            self.net.run(self.x_host, self.logits_host, self.B)

        def e2e_pipelined(self, steps):
            """K steps through pulpnn_net_submit / pulpnn_net_wait, two batches in flight: every step
            copies its input from pinned host memory and its logits back, and the copy of step i+1 runs
            under the compute of step i."""
            outs = [self.logits_host, self.logits_host2]
            prev = None
            for i in range(steps):
                t = self.net.submit(self.x_host, outs[i & 1], self.B)
                if prev is not None:
                    self.net.wait(prev)
                prev = t
            self.net.wait(prev)

        def timed(self, fn, steps):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            ev0.record()
            for _ in range(steps):
                fn()
            if self.gather is not None and fn == self.step:
                self.gather.finish()
            ev1.record()
            barrier()
            ms = ev0.elapsed_time(ev1)
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

    strong = args.scaling == "strong"
    job = Job(args.batch if strong else args.batch * world)
    B, global_batch = job.B, job.global_batch
    warm = max(args.warmup, 3)

    # the clock sampler needs a moment to come up: start it before the warm-up and keep the GPU
    # busy until its first samples are in, so that the timed region is covered
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(warm):
        job.step()
    if world == 1:
        t_wait = time.time()
        while len(sampler.lines) < 2 and time.time() - t_wait < 3.0:
            job.step()
    else:
        for _ in range(200):        # same count on every rank
            job.step()
    barrier()
    launches0 = api.launch_count()
    ms = job.timed(job.step, args.steps)
    launches = api.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the C ABI with host buffers: the pipelined form (two batches in flight) is
    # the headline; the one-call-at-a-time form is reported beside it
    for _ in range(2):
        job.step_e2e()
    ms_e2e_sync = job.timed(job.step_e2e, args.steps)
    job.e2e_pipelined(3)
    ms_e2e = job.timed(lambda: job.e2e_pipelined(args.steps), 1)

    # per-layer times (events between layer calls), averaged over a few runs
    layer_ms = np.zeros(job.net.num_layers())
    reps = max(3, min(args.steps, 10))
    for _ in range(reps):
        layer_ms += np.array(job.net.run_timed(job.x_dev, job.logits, B))
    layer_ms /= reps
    assert api.device_status() == 0, "a bounded wait inside a tensor-core kernel ran out"

    # the other scaling mode, in the same run (N > 1 only; at N = 1 the two coincide)
    other = None
    if world > 1 and not args.no_extras:
        job2 = Job(args.batch * world if strong else args.batch)
        for _ in range(warm + 20):
            job2.step()
        ms2 = job2.timed(job2.step, args.steps)
        job2.e2e_pipelined(3)
        ms2_e2e = job2.timed(lambda: job2.e2e_pipelined(args.steps), 1)
        other = {"scaling": "weak" if strong else "strong", "per_gpu_batch": job2.B, "global_batch": job2.global_batch,
                 "value": round(job2.global_batch * args.steps / (ms2 / 1e3), 1), "unit": "images/s",
                 "ms_per_step": round(ms2 / args.steps, 4),
                 "e2e_value": round(job2.global_batch * args.steps / (ms2_e2e / 1e3), 1)}
        del job2

    if rank != 0:
        if world > 1:
            barrier()
            dist.destroy_process_group()
        return

    hbm_peak, peak_kind = peaks()
    rows = wl.mobilenet_ops_bytes()
    per_layer = []
    by_kernel = {}
    roles = [job.net.layer_role(l) for l in range(job.net.num_layers())]
    idx = 0
    while idx < len(params):
        L, r, t_ms = params[idx], rows[idx], float(layer_ms[idx])
        name, ops, nbytes = L["name"], r["ops"], r["bytes"]
        kname = job.net.layer_kernel(idx) or L["op"]
        step = 1
        if roles[idx] == 1:
            # a depthwise + pointwise pair run as one kernel: one entry, the pair's operations, and as
            # algorithmic bytes what the fused kernel has to move (the pair's input and output; the
            # intermediate tensor is not traffic any more)
            r2 = rows[idx + 1]
            name = L["name"] + "+" + params[idx + 1]["name"]
            t_ms += float(layer_ms[idx + 1])
            ops += r2["ops"]
            nbytes = L["H"] * L["W"] * L["Cin"] + params[idx + 1]["Ho"] * params[idx + 1]["Wo"] * params[idx + 1]["Cout"]
            step = 2
        gb, gop = nbytes * B / 1e9, ops * B / 1e9
        entry_ = {"layer": name, "ms": round(t_ms, 4),
                  "GOPs": round(gop / (t_ms / 1e3), 1), "GBs": round(gb / (t_ms / 1e3), 1),
                  "hbm_frac": round(gb / (t_ms / 1e3) / hbm_peak, 3),
                  "tc_frac_nominal": round(gop / (t_ms / 1e3) / 4.5e6, 3), "kernel": kname}
        if step == 2:
            entry_["unfused_bytes_frac"] = round((r["bytes"] + rows[idx + 1]["bytes"]) * B / 1e9 / (t_ms / 1e3) / hbm_peak, 3)
        per_layer.append(entry_)
        k = by_kernel.setdefault(kname, {"ms": 0.0, "bytes": 0.0, "launches": 0})
        k["ms"] += t_ms; k["bytes"] += nbytes * B; k["launches"] += 1
        idx += step
    top = max(by_kernel, key=lambda n: by_kernel[n]["ms"])
    tk = by_kernel[top]
    achieved = tk["bytes"] / 1e9 / (tk["ms"] / 1e3)
    traffic, traffic_src = None, None
    m = measured_traffic_ratio(top)
    if m:
        traffic = int(m["dram_over_algorithmic"] * tk["bytes"] / tk["launches"])
        traffic_src = m.get("source")
    roofline = {"bound": "hbm", "kernel": top, "achieved": round(achieved, 1), "peak": hbm_peak,
                "unit": "GB/s", "frac": round(achieved / hbm_peak, 4), "traffic": traffic,
                "traffic_source": traffic_src,
                "peak_source": "of %s" % peak_kind,
                "launches_per_step": tk["launches"], "avg_launch_ms": round(tk["ms"] / tk["launches"], 4),
                "algorithmic_bytes_per_launch": int(tk["bytes"] / tk["launches"]),
                "share_of_step": round(tk["ms"] / float(layer_ms.sum()), 3)}

    images = global_batch * args.steps
    value = images / (ms / 1e3)
    gather_kind = job.gather.kind if job.gather is not None else "none (one GPU)"
    line = {"metric": "MobileNetV1-int8 images/s", "value": round(value, 1), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "u8*s8->s32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_batch": B, "global_batch": global_batch,
                       "micro_batch": args.micro, "parallelism": "batch-sharded x%d" % world,
                       "logits_gather": gather_kind,
                       "l2": "inputs larger than L2 (154 MB of images per step)" if B * 150528 > 126e6 else
                             "per-GPU input %.0f MB: the first layer's input is re-read from HBM every step "
                             "(the 29 layers between two reads of it move %.0f MB)" % (B * 0.150528, B * 10.24)},
            "clocks": clocks,
            "e2e": {"value": round(images / (ms_e2e / 1e3), 1), "unit": "images/s",
                    "h2d_bytes_per_step": int(job.x_host.numel()), "d2h_bytes_per_step": int(job.logits_host.numel() * 4),
                    "how": "pulpnn_net_submit / pulpnn_net_wait, two batches in flight, pinned host buffers",
                    "one_call_at_a_time": round(images / (ms_e2e_sync / 1e3), 1)},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "per_layer": per_layer}
    if other:
        line[other["scaling"]] = other

    if world == 1 and not args.no_extras:
        import layer_bench
        # the box's practical int8 tensor peak and its pinned host-to-device copy rate: the
        # denominators of the tensor-bound layers and of the end-to-end figure
        ip = layer_bench.int8_peak(5)
        line["int8_peak"] = {"nominal_pops": 4.5, "library_pops": round(ip["TOPs"] / 1e3, 3), "how": ip["how"]}
        best = min(_event_ms(torch, lambda: job.x_dev.copy_(job.x_host, non_blocking=True), 1) for _ in range(5))
        h2d_gbs = job.x_host.numel() / best / 1e6
        e2e_ms = ms_e2e / args.steps
        line["e2e"].update({"h2d_gbs_measured": round(h2d_gbs, 2), "h2d_copy_ms": round(best, 4),
                            "ms_per_step": round(e2e_ms, 4), "frac_of_copy": round(best / e2e_ms, 3)})
        # what this GPU's memory system gives a pure write stream and a copy (library kernels, measured
        # here only as denominators: layers that write two or more bytes per byte read are held to the
        # write figure, not to the copy figure)
        probe = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")
        fill_ms = min(_event_ms(torch, lambda: probe.fill_(7), 1) for _ in range(5))
        half = probe.numel() // 2
        copy_ms = min(_event_ms(torch, lambda: probe[:half].copy_(probe[half:]), 1) for _ in range(5))
        line["hbm_probe"] = {"fill_gbs": round(probe.numel() / fill_ms / 1e6, 1), "copy_gbs": round(2 * half / copy_ms / 1e6, 1),
                             "how": "torch fill_ of 1 GiB; torch copy_ of 512 MiB (read + write bytes); best of 5, CUDA events"}
        del probe
        for pl in per_layer:
            pl["tc_frac_library"] = round(pl["GOPs"] / 1e3 / ip["TOPs"], 3)
        line["configs"] = single_layer_configs(pkg, torch, hbm_peak, ip["TOPs"] / 1e3)
        api.set_batch(1)

        # sustained: the same step in blocks for >= 3 s, with the clocks sampled meanwhile
        s2 = ClockSampler(local)
        s2.start()
        blocks, t_end = [], time.time() + args.sustain
        per_block = max(1, int(0.25 / (ms / args.steps / 1e3)))
        while time.time() < t_end:
            t0 = time.time()
            bms = _event_ms(torch, job.step, per_block) * per_block
            blocks.append((t0, time.time(), B * per_block / (bms / 1e3)))
        clk = s2.stop(keep_samples=True)
        out_blocks = []
        for (t0, t1, ips) in blocks:
            mhz = [v for (ts, v, _) in clk.get("trace", []) if t0 <= ts <= t1]
            out_blocks.append([round(ips, 1), statistics.median(mhz) if mhz else None])
        tail = [b for b in blocks if b[1] >= blocks[-1][1] - 1.0]
        pw = [w for (_, _, w) in clk.get("trace", []) if w is not None]
        line["sustained"] = {"seconds": round(blocks[-1][1] - blocks[0][0], 2),
                             "value": round(sum(b[2] for b in tail) / len(tail), 1), "unit": "images/s",
                             "sm_mhz_median": clk["sm_mhz"], "power_w_max": max(pw) if pw else None,
                             "reasons": clk["reasons"], "blocks": out_blocks[:: max(1, len(out_blocks) // 16)]}

        # what was timed is also what is checked: the same layer stack at the same batch, with
        # live requantisation parameters, against the CPU checker on sampled images
        line["parity_checked"] = parity_check(pkg, torch, job, params, args)

    if world == 1 and not args.no_cpu:
        # in a process of its own: the reference harness wants a low-address arena, and a process
        # that has CUDA loaded may already have that address range mapped
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "1",
                            "--warmup", "0", "--budget", "12", "--max-images", "1024"],
                           capture_output=True, text=True, timeout=600)
        try:
            line["cpu_baseline"] = json.loads(r.stdout.strip().splitlines()[-1])["cpu_baseline"]
        except Exception:
            line["cpu_baseline"] = {"value": None, "unit": "images/s", "cores": os.cpu_count(), "kind": "reference",
                                    "sample": "CPU baseline run failed: " + (r.stderr.strip().splitlines() or ["?"])[-1][:200]}
    print(json.dumps(line), flush=True)
    if world > 1:
        barrier()
        dist.destroy_process_group()


PARITY_SAMPLE = [0, 1, 255, 256, 511, 512, 767, 768, 1022, 1023]


def parity_check(pkg, torch, job, timed_params, args):
    """Runs the benchmark's layer stack once more at the benchmark's batch -- with the literal
    parameters (the timed network object itself) and with live ones (same shapes, so the same
    kernels and branches) -- and compares sampled images' logits with the CPU checker, which runs
    in a child process (`--impl parity-oracle`)."""
    import tempfile
    api, wl = pkg.api, pkg.workloads
    B = job.B
    sample = sorted({i for i in PARITY_SAMPLE if i < B} | {B - 1})
    res = {"images": 0, "equal": None}
    with tempfile.TemporaryDirectory() as tmp:
        got = {}
        job.net.run(job.x_dev, job.logits, B)
        api.synchronize()
        got["literal"] = job.logits.cpu().numpy()[sample]
        live = wl.mobilenet_params(seed=4, bits=32, shift_bias=1)
        net = api.build_mobilenet_v1(live, bits=32, max_batch=B, micro_batch=args.micro)
        net.run(job.x_dev, job.logits, B)
        api.synchronize()
        got["live"] = job.logits.cpu().numpy()[sample]
        host_logits = np.zeros((B, 1000), np.int32)
        net.run(job.x_host, host_logits, B)
        got["live_host_input"] = host_logits[sample]
        net.close()
        np.save(os.path.join(tmp, "x.npy"), job.x_host.numpy()[sample])
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "parity-oracle", "--tmp", tmp],
                           capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            res["error"] = (r.stderr.strip().splitlines() or ["?"])[-1][:200]
            return res
        want_lit, want_live = np.load(os.path.join(tmp, "literal.npy")), np.load(os.path.join(tmp, "live.npy"))
        eq = {"literal": bool(np.array_equal(got["literal"], want_lit)),
              "live": bool(np.array_equal(got["live"], want_live)),
              "live_host_input": bool(np.array_equal(got["live_host_input"], want_live))}
        res = {"images": len(sample), "image_indices": sample, "batch": B, "equal": all(eq.values()), "cases": eq,
               "distinct_logit_values_live": int(len(np.unique(want_live))),
               "checker": r.stdout.strip().splitlines()[-1] if r.stdout.strip() else "?"}
    return res


def run_parity_oracle(args):
    """Child of parity_check: the CPU checker's logits for the sampled images (the compiled
    reference when it was built on this machine, else the C restatement)."""
    from oracle import bindings
    from oracle.netref import mobilenet_chain
    pkg = entry.load_package()
    wl = pkg.workloads
    x = np.load(os.path.join(args.tmp, "x.npy"))
    if bindings.have_reference(32):
        impl, kind = bindings.CompiledReference(32, arena_mb=256, threads=os.cpu_count() or 1), "compiled reference"
    else:
        impl, kind = bindings.Restatement(), "C restatement"
    for name, sb in (("literal", 11), ("live", 1)):
        params = wl.mobilenet_params(seed=4, bits=32, shift_bias=sb)
        np.save(os.path.join(args.tmp, name + ".npy"), mobilenet_chain(impl, params, x)[-1])
    print(kind)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "parity-oracle"])
    ap.add_argument("--batch", type=int, default=1024, help="images: in total (strong scaling) or per GPU (weak)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (the configuration the metric is quoted on): --batch images in total, sliced over "
                         "the GPUs; weak: --batch images per GPU. With more than one GPU the other mode is measured "
                         "too and reported under its own key.")
    ap.add_argument("--gather", default="auto", choices=["auto", "peer", "nccl"],
                    help="final logits gather: stores into the root's peer-mapped buffer, or an NCCL all-gather "
                         "on a side stream")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the single-layer configurations, the sustained run and the parity check")
    ap.add_argument("--sustain", type=float, default=3.0, help="seconds of the sustained run")
    ap.add_argument("--tmp", default="", help="(internal) exchange directory of the parity check")
    ap.add_argument("--micro", type=int, default=0, help="images per pass through the stack (0 = all)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--budget", type=float, default=0.0, help="reference arm: seconds of CPU work per step")
    ap.add_argument("--max-images", type=int, default=256, help="reference arm: largest sample per step")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: whatever libraries print meanwhile (NCCL's version
    # banner, for one) is sent to stderr by pointing file descriptor 1 there for the run
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    global print
    _print = print

    def print(*a, **kw):          # noqa: A001 -- the two JSON lines below go to the real stdout
        os.write(real_stdout, (" ".join(str(x) for x in a) + "\n").encode())
    try:
        if args.impl == "reference":
            run_reference_arm(args)
        elif args.impl == "parity-oracle":
            run_parity_oracle(args)
        else:
            run_gpu_arm(args)
    finally:
        print = _print            # noqa: A001
        os.dup2(real_stdout, 1)


if __name__ == "__main__":
    main()
