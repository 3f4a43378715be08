#!/usr/bin/env python
"""Benchmark of the CUDA backend on kurumi's headline configurations.

    python bench.py --gpus N --steps K --warmup W            (this backend)
    python bench.py --impl reference --gpus N --steps K ...  (the reference's CPU path, restated)

A "step" is one evaluation of the workload graph over one batch of seeded synthetic input. The headline workload
is configuration 2 of the baseline (view-fused row softmax through a transpose view, f32 [8192, 8192] + bias): the
metric is achieved HBM GB/s = algorithmic bytes (one read of L, one read of the bias, one write of the output) /
device time. The other four configurations, and the decode step of a weight-only quantised projection (one GPU only),
are measured in the same run and reported under "workloads".

With N > 1 the ONE named problem is sharded by rows (ku_graph_row_split): rank r evaluates rows [r, r + 1) * M / N
on its slices of the row-wise inputs and on all of the replicated ones; there is no collective on the data path,
outputs stay device-resident shards ("scaling": "strong", value = whole-problem work / slowest rank's time). The
NCCL all-gather that assembles the shards (ku_cuda_all_gather_rows) is timed apart, as "assembly".

`e2e` is the same metric through the drop-in call with host buffers: ku_feeds_set + ku_eval_with + ku_tensor_bytes
per step, host tensors in, a host tensor out; the library streams the evaluation through the device in row chunks.
Inputs smaller than a few L2s are rotated through copies so that no device-timed step finds them cached.
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from kurumi_b200 import api, build, configs  # noqa: E402

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each workload's dominant kernel, from one
# ncu capture per kernel at the full workload size, summarised in the named file under profiles/. An entry is used only
# while the kernel source it was captured from is unchanged (first 16 hex digits of its SHA-256).
NCU_TRAFFIC = {
    ("c1_fused_reduce", "reduce_rows"): (137.9e6, "profiles/reduce_rows__c1_fused_reduce.txt", "kurumi_b200/csrc/cuda/emit.cc", "7e375c1b68033b2c"),
    ("c2_transposed_softmax", "softmax_groups_tma"): (478.7e6, "profiles/softmax_groups_tma__c2_transposed_softmax.txt", "kurumi_b200/csrc/cuda/kernels/softmax_groups_tma.cuh", "dd8c62b067697094"),
    ("c3_gemm_bias_gelu", "gemm_tc"): (1251e6, "profiles/gemm_tc2__c3_gemm_bias_gelu.txt", "kurumi_b200/csrc/cuda/kernels/gemm_tc2.cuh", "df0ad6236b887218"),
    ("c4_causal_attention", "attention_tc"): (1057.5e6, "profiles/attention_tc__c4_causal_attention.txt", "kurumi_b200/csrc/cuda/kernels/attention_tc.cuh", "e76ea16f0699bdc8"),
    ("n3_quant_gemv", "quant_gemv"): (128.2e6, "profiles/quant_gemv_mma__n3_quant_gemv.txt", "kurumi_b200/csrc/cuda/kernels/quant_gemv_mma.cuh", "b61c2994e45d6d5a"),
    ("c5_fp8_weight_gemm", "gemm_tc_f8"): (4236e6, "profiles/gemm_tc2_f8__c5_fp8_weight_gemm.txt", "kurumi_b200/csrc/cuda/kernels/gemm_tc2.cuh", "df0ad6236b887218"),
}

WORKLOADS = {
    # name: (builder, full-size args, metric kind)
    "c1_fused_reduce": (configs.fused_reduce, dict(rows=4096, cols=4096), "hbm"),
    "c2_transposed_softmax": (configs.transposed_softmax, dict(n=8192), "hbm"),
    "c3_gemm_bias_gelu": (configs.gemm_bias_gelu, dict(m=8192, n=8192, kdim=8192), "tensor"),
    "c4_causal_attention": (configs.causal_attention, dict(batch=8, heads=32, seq=4096, dh=128), "tensor"),
    "c5_fp8_weight_gemm": (configs.fp8_weight_gemm, dict(m=16384, kdim=8192, n=28672), "tensor"),
    # beyond the five configurations: the decode step of a weight-only quantised projection (one GPU; its one activation
    # row leaves nothing to cut into row shards)
    "n3_quant_gemv": (configs.quant_gemv, dict(m=1, n=28672, kdim=8192, bits=4, group=128), "hbm"),
}
ONE_GPU_ONLY = {"n3_quant_gemv"}
HEADLINE = "c2_transposed_softmax"


def algorithmic_work(name: str, kw: dict):
    """(bytes, flops) one evaluation must move / compute: inputs read once, output written once."""
    if name == "c1_fused_reduce":
        return 2 * kw["rows"] * kw["cols"] * 4 + kw["rows"] * 4, 0.0
    if name == "c2_transposed_softmax":
        n, lines = kw["n"], kw.get("lines") or kw["n"]
        return 2 * n * lines * 4 + n * 4, 0.0
    if name == "c3_gemm_bias_gelu":
        m, n, k = kw["m"], kw["n"], kw["kdim"]
        return (m * k + k * n + m * n + n) * 2, 2.0 * m * n * k
    if name == "c4_causal_attention":
        b, h, s, d = kw["batch"], kw["heads"], kw["seq"], kw["dh"]
        return 4 * b * h * s * d * 2, 4.0 * d * b * h * s * (s + 1) / 2
    if name == "n3_quant_gemv":
        m, n, k, bits, group = kw["m"], kw["n"], kw["kdim"], kw["bits"], kw["group"]
        return n * k * bits // 8 + 2 * n * (k // group) * 2 + m * k * 2 + m * n * 2, 2.0 * m * n * k
    m, k, n = kw["m"], kw["kdim"], kw["n"]
    return m * k * 2 + k * n + n * 4 + m * n * 2, 2.0 * m * n * k


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic(name: str, family: str):
    """(bytes per launch, source) from the table above, or (None, why) when the kernel changed since the capture."""
    entry = NCU_TRAFFIC.get((name, family))
    if entry is None:
        return None, "no capture for this kernel"
    nbytes, summary, source, sha = entry
    try:
        now = hashlib.sha256(open(os.path.join(ROOT, source), "rb").read()).hexdigest()[:16]
    except OSError:
        return None, f"{source} missing"
    if now != sha:
        return None, f"{source} changed since the capture summarised in {summary}"
    return nbytes, summary


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def cpu_sample(name, kw):
    """The workload, or a bounded slice of it, for the CPU evaluator: (sizes, description). Configurations 1 and 2 run at
    full size; the contractions and attention take minutes on one core, so a stated slice of their rows / heads is timed."""
    if name == "c2_transposed_softmax":
        return dict(kw), "full size"
    if name == "c1_fused_reduce":
        return dict(kw), "full size"
    if name == "c3_gemm_bias_gelu":
        m = min(kw["m"], 64)
        return dict(m=m, n=kw["n"], kdim=kw["kdim"]), f"{m} of {kw['m']} rows of A"
    if name == "c4_causal_attention":
        return dict(batch=1, heads=1, seq=min(kw["seq"], 512), dh=kw["dh"]), "1 head at seq 512"
    if name == "n3_quant_gemv":
        n = min(kw["n"], 4096)   # the interpreter widens the whole weight to f32 first: 4 bytes per weight of host memory
        return dict(kw, n=n), f"{n} of {kw['n']} output channels"
    m, n = min(kw["m"], 256), min(kw["n"], 1792)   # few rows against all of W would time the widening of W, not the contraction
    return dict(m=m, kdim=kw["kdim"], n=n, amp=False), f"{m} of {kw['m']} rows of X against {n} of {kw['n']} output channels"


def metric_name(name):
    return {"hbm": "achieved HBM GB/s (algorithmic bytes / device time)", "tensor": "achieved TFLOP/s (algorithmic FLOP / device time)"}[WORKLOADS[name][2]] + f", {name}"


def dtype_of(name):
    return {"c1_fused_reduce": "f32", "c2_transposed_softmax": "f32", "c3_gemm_bias_gelu": "bf16", "c4_causal_attention": "bf16", "c5_fp8_weight_gemm": "f8e4m3", "n3_quant_gemv": "int4 x bf16"}[name]


def unit_of(name):
    return "GB/s" if WORKLOADS[name][2] == "hbm" else "TFLOP/s"


def rate(name, nbytes, flops, seconds):
    return nbytes / seconds / 1e9 if WORKLOADS[name][2] == "hbm" else flops / seconds / 1e12


def cpu_evaluator(name, kw):
    """kurumi's own CPU path for the workload (the view-fused evaluator; it falls back to the interpreter for graphs
    outside its f32 fused path, as the reference does), restated in oracle/ because no Rust toolchain exists here.
    Single thread: the reference is single-threaded by construction. Returns (evaluate(), sample sizes, description)."""
    olib = api.Library(build.ORACLE_LIB if os.path.exists(build.ORACLE_LIB) else build.build_oracle())
    cpu = api.Backend(olib, 65)
    skw, what = cpu_sample(name, kw)
    g = api.Graph(olib)
    root, gens = WORKLOADS[name][0](g, **skw)
    # inputs of the configuration's shapes, dtypes and spreads, drawn with numpy: the evaluator's time does not depend on
    # the values, and recording the seeded draw through the CPU interpreter would take longer than the measurement
    rng = np.random.default_rng(0)
    feeds = api.Feeds(olib)
    for node in gens:
        shape, dt = g.shape(node), g.dtype(node)
        if dt == api.F8E4M3:
            feeds.set(node, rng.integers(0, 0x78, shape, dtype=np.uint8) | (rng.integers(0, 2, shape, dtype=np.uint8) << 7), dt)
        elif dt == api.U8:
            feeds.set(node, rng.integers(0, 256, shape, dtype=np.uint8), dt)
        elif dt == api.F16:
            feeds.set(node, rng.uniform(0.004, 0.012, shape).astype(np.float16).view(np.uint16), dt)
        elif dt == api.BF16:
            feeds.set(node, api.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.05 if name != "c4_causal_attention" else 1.0)), dt)
        else:
            feeds.set(node, rng.standard_normal(shape, dtype=np.float32) * np.float32(2.0 if name == "c2_transposed_softmax" else 0.5), dt)
    return (lambda: cpu.eval_with(g, root, feeds)), skw, what


def reference_arm(args, name, kw):
    """`--impl reference`: the CPU evaluator timed on this box's host, `steps` evaluations after `warmup`."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    evaluate, skw, what = cpu_evaluator(name, kw)
    t0 = time.perf_counter()
    evaluate()                      # also the first warm-up evaluation
    first = time.perf_counter() - t0
    # The run has to end within a few minutes whatever K, W and the host: when K + W evaluations of the sample would take
    # more than four, the softmax configuration is timed on a slab of its lines (softmax lines are independent, the rate
    # per byte is the same) and the sample says so.
    if name == "c2_transposed_softmax" and first * (args.steps + args.warmup) > 240.0:
        lines = max(256, int(kw["n"] * 240.0 / (first * (args.steps + args.warmup))) // 256 * 256)
        evaluate, skw, what = cpu_evaluator(name, dict(kw, lines=lines))
        what = f"{lines} of {kw['n']} softmax lines (the full size would take {first * (args.steps + args.warmup):.0f} s for {args.steps + args.warmup} evaluations)"
        evaluate()
    for _ in range(max(0, args.warmup - 1)):
        evaluate()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        evaluate()
    dt = (time.perf_counter() - t0) / args.steps
    nbytes, flops = algorithmic_work(name, skw)
    value, unit = rate(name, nbytes, flops, dt), unit_of(name)
    emit({"impl": "reference", "metric": metric_name(name), "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
          "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(name), "data": "synthetic",
          "config": {"workload": name, **kw, "sample": what},
          "cpu_baseline": {"value": value, "unit": unit, "cores": 1, "kind": "port", "sample": what},
          "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})


def cpu_baseline(name, kw, budget_s):
    """The same evaluator timed beside the GPU number for about `budget_s` seconds (one evaluation at least)."""
    evaluate, skw, what = cpu_evaluator(name, kw)
    evaluate()
    reps, t0 = 0, time.perf_counter()
    while reps < 1 or (time.perf_counter() - t0 < budget_s and reps < 20):
        evaluate()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    nbytes, flops = algorithmic_work(name, skw)
    return {"value": rate(name, nbytes, flops, dt), "unit": unit_of(name), "cores": 1, "kind": "port", "sample": what + f"; {reps} evaluations, {dt * 1e3:.1f} ms each",
            "host_cpus": os.cpu_count()}


_RESULT_FD = None


def emit(line: dict):
    """The one JSON line goes to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


class Session:
    """One rank: its GPU, the backend, the torch view of the backend's stream, and the process group when N > 1."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        if self.world > 1:
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the JSON line only
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.lib = api.Library(build.LIB)
        self.gpu = api.CudaBackend(self.lib, self.local)
        self.stream = torch.cuda.ExternalStream(self.gpu.stream, device=self.local)
        if self.world > 1:   # the library's own communicator, for the assembly column
            box = [self.gpu.comm_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            self.gpu.comm_init(box[0], self.rank, self.world)

    def barrier(self):
        self.gpu.sync()
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, v: float) -> float:
        t = self.torch.tensor([v], device=f"cuda:{self.local}", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.gpu.comm_free()
            self.dist.destroy_process_group()


def device_slice(s: Session, t, axis: int, index: int, parts: int):
    """Slice `index` of `parts` along `axis` of a device tensor, as a new device tensor."""
    step = t.shape[axis] // parts
    g = api.Graph(s.lib)
    x = g.input(list(t.shape), t.dtype)
    ranges = [(0, d) for d in t.shape]
    ranges[axis] = (index * step, (index + 1) * step)
    out = s.gpu.eval_device(g, [g.slice(x, ranges)], None, {x: t})[0]
    s.gpu.sync()
    s.gpu.release_graph(g)
    return out


def setup(s: Session, name: str, kw: dict):
    """The workload graph (its row shard when N > 1) and device-resident seeded inputs, in several copies when small."""
    builder = WORKLOADS[name][0]
    g_full = api.Graph(s.lib)
    root_full, gens = builder(g_full, **kw)
    if s.world > 1:
        g, root, inputs = api.row_split(g_full, root_full, s.world)
    else:
        g, root, inputs = g_full, root_full, [(n, n, None) for n in gens]
    in_bytes = 0
    for orig, part, axis in inputs:
        in_bytes += int(np.prod(g.shape(part))) * api.WIDTH[g.dtype(part)]
    # Inputs smaller than about three L2s (126 MB) are kept in several copies that the steps rotate through, so that a
    # step never finds its inputs in L2 from the step before.
    n_sets = max(1, min(8, int(np.ceil(3 * 126e6 / max(in_bytes, 1)))))
    first = {}
    for orig, part, axis in inputs:   # the seeded draw, generated on the device; a rank keeps its slice of it
        h = api.Graph(s.lib)
        full = s.gpu.eval_device(h, [gens[orig](h)])[0]
        s.gpu.sync()
        s.gpu.release_graph(h)
        if axis is None:
            first[part] = full
        else:
            first[part] = device_slice(s, full, axis, s.rank, s.world)
            full.free()
    sets = [first]
    for _ in range(n_sets - 1):       # further copies of the same values at other addresses
        cp = {}
        for part, t in first.items():
            gi = api.Graph(s.lib)
            x = gi.input(list(t.shape), t.dtype)
            cp[part] = s.gpu.eval_device(gi, [gi.slice(x, [(0, d) for d in t.shape])], None, {x: t})[0]   # a root that is a bare input is copied out
            s.gpu.sync()
            s.gpu.release_graph(gi)
        sets.append(cp)
    return {"g": g, "root": root, "g_full": g_full, "inputs": inputs, "sets": sets, "in_bytes": in_bytes, "n_sets": n_sets}


def teardown(s: Session, w: dict):
    s.gpu.sync()
    for st in w["sets"]:
        for t in st.values():
            t.free()
    s.gpu.release_graph(w["g"])


def measure(s: Session, name: str, kw: dict, steps: int, warmup: int, e2e_steps: int, cpu_budget: float, sample_clocks: bool):
    """Device-timed value, roofline of the dominant kernel, end-to-end value through the drop-in call, assembly column
    (N > 1) and the CPU evaluator's figure for one workload."""
    torch = s.torch
    kind = WORKLOADS[name][2]
    nbytes, flops = algorithmic_work(name, kw)     # of the WHOLE problem, whatever N
    w = setup(s, name, kw)
    g, root, sets, n_sets = w["g"], w["root"], w["sets"], w["n_sets"]
    counter = [0]
    prepared = [s.gpu.prepare_device_step(g, [root], st) for st in sets]   # argument marshalling done once per input copy
    steppers = [p[0] for p in prepared]

    def step():
        counter[0] += 1
        return steppers[counter[0] % n_sets]()

    sampler = ClockSampler(s.local) if (sample_clocks and s.rank == 0) else None
    if sampler:
        sampler.start()
    for _ in range(warmup):
        step().free()
    s.barrier()
    launches0 = s.gpu.stats()["launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s.stream)
    for _ in range(steps):
        step().free()
    e1.record(s.stream)
    s.barrier()
    ms_local = e0.elapsed_time(e1)
    launches = s.gpu.stats()["launches"] - launches0
    # nvidia-smi needs ~100 ms per sample: when the timed region is shorter than that, keep the same load running
    # (untimed) so that the clock record still describes the kernel under load
    clocks = None
    if sampler:
        t_sustain = time.perf_counter()
        while ms_local < 1500 and time.perf_counter() - t_sustain < 1.2:
            for _ in range(20):
                step().free()
            s.gpu.sync()
        clocks = sampler.stop()
        clocks["window"] = "warm-up + timed steps" + (" + 1.2 s of the same steps, untimed" if ms_local < 1500 else "")
    s.barrier()
    ms = s.max_over_ranks(ms_local)
    per_step_s = ms / 1e3 / steps
    res = {"value": rate(name, nbytes, flops, per_step_s), "unit": unit_of(name), "ms_per_step": ms / steps, "gpu_launches": int(launches), "clocks": clocks,
           "l2": f"steps rotate through {n_sets} copies of the inputs ({w['in_bytes'] * n_sets / 1e6:.0f} MB per rank in all, L2 is 126 MB): no step finds its inputs cached"}

    # dominant kernel: average launch duration from CUDA events around every launch on the backend's stream
    s.gpu.profile(True)
    n_prof = min(steps, 20)
    for _ in range(n_prof):
        step().free()
    s.gpu.sync()
    prof = s.gpu.take_profile()
    s.gpu.profile(False)
    peaks = measured_peaks()
    if prof:
        fam, p = max(prof.items(), key=lambda kv: kv[1]["ms"])
        avg_s = p["ms"] / 1e3 / p["launches"]
        duration_source = "CUDA events around each launch (a pass of its own after the timed region)"
        if len(prof) == 1 and p["launches"] == n_prof:
            # the step IS this one kernel: its average duration over the timed region (events bracket the K back-to-back
            # launches on the launching stream) is the timed region / K; launch gaps count against it
            avg_s = ms_local / 1e3 / steps
            duration_source = "timed region / launches (one launch per step; CUDA events bracket the K launches)"
        traffic, traffic_source = ncu_traffic(name, fam) if s.world == 1 else (None, "captured at one GPU only")
        if kind == "hbm":
            ach, peak, peak_source = (p["algo_bytes"] / p["launches"]) / avg_s / 1e9, peaks["hbm_gbs"], peaks["source"]
        else:
            ach, peak, peak_source = (p["flops"] / p["launches"]) / avg_s / 1e12, peaks["bf16_tflops"], peaks["source"] + " (bf16 burst)"
        res["roofline"] = {"bound": kind, "kernel": fam, "achieved": ach, "peak": peak, "unit": unit_of(name), "frac": ach / peak, "traffic": traffic, "traffic_source": traffic_source,
                           "avg_launch_us": avg_s * 1e6, "duration_source": duration_source, "peak_source": peak_source, "share_of_step": p["ms"] / sum(v["ms"] for v in prof.values()),
                           "per": "this rank's launch (its shard of the problem)" if s.world > 1 else "launch"}
        res["kernel_times"] = {k: {"launches": v["launches"], "avg_us": v["ms"] * 1e3 / v["launches"]} for k, v in prof.items()}

    w["launches_per_step"] = max(1, int(launches) // steps)
    if e2e_steps > 0:
        res["e2e"] = measure_e2e(s, name, nbytes, flops, w, e2e_steps)
    if s.world > 1:
        res["assembly"] = measure_assembly(s, step)
    if cpu_budget > 0 and s.rank == 0 and s.world == 1:
        res["cpu_baseline"] = cpu_baseline(name, kw, cpu_budget)
    for _, close in prepared:
        close()
    teardown(s, w)
    return res


def measure_e2e(s: Session, name: str, nbytes: int, flops: float, w: dict, n_steps: int):
    """The drop-in call with host buffers: ku_feeds_set for every input, ku_eval_with, ku_tensor_bytes into the caller's
    buffer, every step. Host wall clock around the steps (the calls return when the result is in host memory)."""
    g, root = w["g"], w["root"]
    L = s.lib.lib
    tensors = {}
    for part, t in w["sets"][0].items():   # this rank's inputs as host tensors (ku_tensor_new copies the caller's bytes)
        tensors[part] = api.Tensor.from_numpy(s.lib, t.numpy(), t.dtype)
    feeds = api.Feeds(s.lib)
    out_bytes = int(np.prod(g.shape(root))) * api.WIDTH[g.dtype(root)]
    host_out = np.zeros(max(out_bytes, 1), np.uint8)   # the caller's result buffer, touched once
    out_ptr = host_out.ctypes.data

    def e2e_step():
        for part, t in tensors.items():
            L.ku_feeds_set(feeds.h, C.c_uint32(part), t.h)
        r = s.gpu.eval_with(g, root, feeds)
        r.copy_into(out_ptr)
        r.free()

    before = s.gpu.stats()
    for _ in range(2):
        e2e_step()
    chunked = s.gpu.stats()["launches"] - before["launches"] > 2 * w["launches_per_step"]   # more launches than two one-piece evaluations
    s.barrier()
    t0 = time.perf_counter()
    for _ in range(n_steps):
        e2e_step()
    dt_local = (time.perf_counter() - t0) / n_steps
    s.barrier()
    dt = s.max_over_ranks(dt_local)
    # the result in the caller's buffer is the device-resident evaluation's
    ref = s.gpu.eval_device(g, [root], None, w["sets"][0])[0]
    want = ref.numpy().view(np.uint8).reshape(-1)
    ref.free()
    if name == "c2_transposed_softmax":   # a chunk of lines may take another softmax kernel (another summation order): the f32 band
        same = bool(np.allclose(host_out.view(np.float32), want.view(np.float32), rtol=1e-5, atol=1e-12))
    else:
        same = bool(np.array_equal(host_out[:out_bytes], want))
        if not same and g.dtype(root) == api.BF16:   # a chunk of few rows may take the one-SM form of the contraction kernel: one bf16 step
            fa, fb = (api.bf16_to_f32(v[:out_bytes].view(np.uint16)).astype(np.float64) for v in (host_out, want))
            same = bool((np.abs(fa - fb) <= 2.0 ** -7 * np.maximum(np.abs(fa), np.abs(fb)) + 1e-30).all())
    h2d = int(sum(t.nbytes for t in tensors.values()))
    for t in tensors.values():
        t.free()
    return {"value": rate(name, nbytes, flops, dt), "unit": unit_of(name), "h2d_bytes_per_step": h2d * s.world if s.world > 1 else h2d, "d2h_bytes_per_step": out_bytes * s.world,
            "ms_per_step": dt * 1e3, "steps": n_steps, "timing": "host wall clock around the calls, max over ranks",
            "method": "ku_feeds_set + ku_eval_with (host tensors in, host tensor out) + ku_tensor_bytes per step" +
                      ("; inside ku_eval_with the evaluation streams through the device in row chunks, upload, kernels and download overlapped" if chunked else "") +
                      ("; every rank feeds its slice of the row-wise inputs and all of the replicated ones" if s.world > 1 else ""),
            "matches_device_resident_evaluation": same}


def measure_assembly(s: Session, step):
    """N > 1: gathering the ranks' output shards into one tensor on every GPU is NOT on the data path that `value`
    times (shards stay device-resident); its cost is reported beside it."""
    torch = s.torch
    shard = step()
    for _ in range(2):
        s.gpu.all_gather_rows(shard).free()
    s.barrier()
    reps = 5
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record(s.stream)
    for _ in range(reps):
        s.gpu.all_gather_rows(shard).free()
    a1.record(s.stream)
    s.barrier()
    ms = s.max_over_ranks(a0.elapsed_time(a1) / reps)
    nb = shard.nbytes
    shard.free()
    return {"ms": ms, "bytes_per_rank": int(nb), "collective": "ncclAllGather of the output shards on the backend's stream (ku_cuda_all_gather_rows), CUDA events, max over ranks",
            "in_value": False}


def fp8_ceiling(s: Session):
    """This repository's own fp8 GEMM kernel on a plain square e4m3 x e4m3 contraction (8192^3, bf16 result, no
    epilogue): best of 10 launches, the method of the measured bf16 burst figure. There is no library fp8 figure in
    MEASURED_PEAKS.json; this is the ceiling the fp8 workload is set against, beside twice the measured bf16 peak."""
    torch = s.torch
    n = 8192
    g = api.Graph(s.lib)
    a, b = g.input([n, n], api.F8E4M3), g.input([n, n], api.F8E4M3)
    root = g.matmul(g.cast(a, api.BF16), g.cast(b, api.BF16))
    feeds = {}
    for node, seed in ((a, 11), (b, 12)):
        h = api.Graph(s.lib)
        feeds[node] = s.gpu.eval_device(h, [h.cast(h.randn([n, n], seed), api.F8E4M3)])[0]
        s.gpu.release_graph(h)
    for _ in range(3):
        s.gpu.eval_device(g, [root], None, feeds)[0].free()
    s.gpu.sync()
    best = 1e30
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s.stream)
        s.gpu.eval_device(g, [root], None, feeds)[0].free()
        e1.record(s.stream)
        s.gpu.sync()
        best = min(best, e0.elapsed_time(e1))
    for t in feeds.values():
        t.free()
    s.gpu.release_graph(g)
    return {"tflops": 2.0 * n ** 3 / (best / 1e3) / 1e12, "us": best * 1e3, "what": "own kernel, e4m3 x e4m3 8192^3 -> bf16, no epilogue, best of 10 launches (CUDA events)"}


def main():
    # libraries (NCCL's version banner, for one) write to file descriptor 1: keep it for the result line alone
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="kurumi_b200", choices=["kurumi_b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS), help="measure this workload alone (default: configuration 2 as the headline, the others beside it)")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling captures); 1.0 = the baseline's size")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only-headline", action="store_true", help="skip the other workloads")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    name = args.workload or HEADLINE

    def sizes(nm):
        kw = dict(WORKLOADS[nm][1])
        if args.scale != 1.0:
            for k in kw:
                if k != "dh" and not (nm in ONE_GPU_ONLY and k in ("m", "bits", "group")):
                    kw[k] = max(128, int(kw[k] * args.scale) // 128 * 128)
        return kw
    kw = sizes(name)
    if args.impl == "reference":
        return reference_arm(args, name, kw)

    s = Session()
    if name in ONE_GPU_ONLY and s.world > 1:
        raise SystemExit(f"{name} is measured on one GPU only")
    head = measure(s, name, kw, args.steps, args.warmup, 0 if args.no_e2e else max(3, min(args.steps, 10)), 0 if args.no_cpu_baseline else 8.0, True)
    others = {}
    if args.workload is None and not args.only_headline and args.scale == 1.0:
        for nm in WORKLOADS:
            if nm == name or (nm in ONE_GPU_ONLY and s.world > 1):
                continue
            k2 = sizes(nm)
            r = measure(s, nm, k2, max(5, min(args.steps, 20)), 3, 0 if args.no_e2e else 3, 0 if args.no_cpu_baseline else 2.0, True)
            r["config"] = {"workload": nm, **k2}
            r["dtype"] = dtype_of(nm)
            r["metric"] = metric_name(nm)
            if nm == "c5_fp8_weight_gemm" and s.world == 1:
                r["fp8_ceiling"] = fp8_ceiling(s)
                r["roofline"]["frac_of_fp8_ceiling"] = r["roofline"]["achieved"] / r["fp8_ceiling"]["tflops"]
                r["roofline"]["frac_of_twice_bf16_peak"] = r["roofline"]["achieved"] / (2 * r["roofline"]["peak"])
            others[nm] = r
    if s.rank == 0:
        line = {"metric": metric_name(name), "value": head["value"], "unit": head["unit"], "n_gpus": s.world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(name),
                "data": "synthetic (seeded threefry2x32 / Box-Muller, generated on device)",
                "config": {"workload": name, **kw, "l2": head["l2"],
                           "sharding": ("one GPU" if s.world == 1 else f"the one named problem is cut into {s.world} row shards (ku_graph_row_split), rank r evaluates shard r; no collective on the data path, "
                                        "outputs stay device-resident shards; value = whole-problem work / slowest rank's device time")},
                "clocks": head["clocks"], "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "roofline": head.get("roofline"), "cpu_baseline": head.get("cpu_baseline"),
                "assembly": head.get("assembly"), "kernel_times": head.get("kernel_times"), "workloads": others or None}
        emit(line)
    s.close()


if __name__ == "__main__":
    main()
