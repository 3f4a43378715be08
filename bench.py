#!/usr/bin/env python
"""Benchmark of the CUDA backend on kurumi's headline configurations.

    python bench.py --gpus N --steps K --warmup W            (this backend)
    python bench.py --impl reference --gpus N --steps K ...  (the reference's CPU path, restated)

A "step" is one evaluation of the workload graph over one batch of seeded synthetic input. The
default workload is configuration 2 of the baseline (view-fused row softmax through a transpose
view, f32 [8192, 8192] + bias): the metric is achieved HBM GB/s = algorithmic bytes (one read of L,
one read of the bias, one write of the output) / device time. With N > 1 every rank evaluates its
own shard of an N-times larger batch (weak scaling, no data-path collective); the value is the
sum over ranks divided by the slowest rank's time. One JSON line is printed by rank 0.

`e2e` is the same metric with every input in pinned host memory and the result read back to pinned host
memory inside the timed region, through the library's public calls: the evaluation is cut into chunks of
independent output rows (kurumi_b200/pipeline.py) so that uploads, kernels and downloads overlap; the
chunked result is compared with the single evaluation byte for byte. Inputs smaller than a few L2s are
rotated through copies so that no step finds them cached.
"""
from __future__ import annotations

import argparse
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

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each workload's dominant kernel,
# from one ncu capture per kernel at the full workload size; the captures are summarised under profiles/.
NCU_TRAFFIC = {
    ("c1_fused_reduce", "reduce_rows"): 137.8e6,
    ("c2_transposed_softmax", "softmax_groups_tma"): 481.4e6,
    ("c2_transposed_softmax", "softmax_panels_tma"): 535.7e6,
    ("c3_gemm_bias_gelu", "gemm_tc"): 1231e6,
    ("c4_causal_attention", "attention_tc"): 1057e6,
    ("c5_fp8_weight_gemm", "gemm_tc_f8"): 3556e6,
}

# how a workload's evaluation is cut into chunks of independent output rows for the end-to-end measurement:
# chunk count, the builder arguments of one chunk, and per input (in the builder's order) the axis it is
# sharded along (None = every chunk needs all of it)
CHUNKING = {
    "c1_fused_reduce": {"chunks": 8, "chunk_kw": lambda kw, c: dict(kw, rows=kw["rows"] // c), "axes": [0, 0]},
    "c2_transposed_softmax": {"chunks": 8, "chunk_kw": lambda kw, c: dict(kw, lines=kw["n"] // c), "axes": [1, None]},
    "c3_gemm_bias_gelu": {"chunks": 8, "chunk_kw": lambda kw, c: dict(kw, m=kw["m"] // c), "axes": [0, None, None]},
    "c4_causal_attention": {"chunks": 8, "chunk_kw": lambda kw, c: dict(kw, batch=kw["batch"] // c), "axes": [0, 0, 0]},
    "c5_fp8_weight_gemm": {"chunks": 8, "chunk_kw": lambda kw, c: dict(kw, m=kw["m"] // c), "axes": [0, None, None]},
}

WORKLOADS = {
    # name: (builder, full-size args, metric kind)
    "c1_fused_reduce": (configs.fused_reduce, dict(rows=4096, cols=4096), "hbm"),
    "c2_transposed_softmax": (configs.transposed_softmax, dict(n=8192), "hbm"),
    "c3_gemm_bias_gelu": (configs.gemm_bias_gelu, dict(m=8192, n=8192, kdim=8192), "tensor"),
    "c4_causal_attention": (configs.causal_attention, dict(batch=8, heads=32, seq=4096, dh=128), "tensor"),
    "c5_fp8_weight_gemm": (configs.fp8_weight_gemm, dict(m=16384, kdim=8192, n=28672), "tensor"),
}


def algorithmic_work(name: str, kw: dict):
    """(bytes, flops) one evaluation must move / compute: inputs read once, output written once."""
    if name == "c1_fused_reduce":
        return 2 * kw["rows"] * kw["cols"] * 4 + kw["rows"] * 4, 0.0
    if name == "c2_transposed_softmax":
        n = kw["n"]
        return 2 * n * n * 4 + n * 4, 0.0
    if name == "c3_gemm_bias_gelu":
        m, n, k = kw["m"], kw["n"], kw["kdim"]
        return (m * k + k * n + m * n + n) * 2, 2.0 * m * n * k
    if name == "c4_causal_attention":
        b, h, s, d = kw["batch"], kw["heads"], kw["seq"], kw["dh"]
        return 4 * b * h * s * d * 2, 4.0 * d * b * h * s * (s + 1) / 2
    m, k, n = kw["m"], kw["kdim"], kw["n"]
    return m * k * 2 + k * n + n * 4 + m * n * 2, 2.0 * m * n * k


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


def reference_arm(args, name, builder, kw):
    """The reference's own CPU path for the workload (kurumi's view-fused evaluator; it falls back to
    the interpreter for graphs outside its f32 fused path, as the reference does), restated in
    oracle/ because no Rust toolchain exists here. Single thread: the reference is single-threaded
    by construction. Each step evaluates a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    olib = api.Library(build.ORACLE_LIB if os.path.exists(build.ORACLE_LIB) else build.build_oracle())
    cpu = api.Backend(olib, 65)
    skw, frac, what = cpu_sample(name, kw)
    g = api.Graph(olib)
    root, gens = builder(g, **skw)
    gen = api.Backend(olib, 0)
    feeds = api.Feeds(olib)
    for node, mk in gens.items():
        h = api.Graph(olib)
        feeds.set(node, gen.eval(h, mk(h)))
    for _ in range(args.warmup):
        cpu.eval_with(g, root, feeds)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.eval_with(g, root, feeds)
    dt = (time.perf_counter() - t0) / args.steps
    nbytes, flops = algorithmic_work(name, skw)
    kind = WORKLOADS[name][2]
    value = nbytes / dt / 1e9 if kind == "hbm" else flops / dt / 1e12
    unit = "GB/s" if kind == "hbm" else "TFLOP/s"
    line = {"impl": "reference", "metric": metric_name(name), "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_of(name), "data": "synthetic",
            "config": {"workload": name, **kw, "sample": what},
            "cpu_baseline": {"value": value, "unit": unit, "cores": 1, "kind": "port", "sample": what},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def cpu_sample(name, kw):
    """A bounded slice of the workload for the CPU baseline: (sizes, fraction of the full work, description)."""
    if name == "c2_transposed_softmax":
        n = min(kw["n"], 2048)
        return dict(n=n), (n / kw["n"]) ** 2, f"[{n},{n}] instance of the same graph (work is linear in elements)"
    if name == "c1_fused_reduce":
        return dict(kw), 1.0, "full size"
    if name == "c3_gemm_bias_gelu":
        m = min(kw["m"], 64)
        return dict(m=m, n=kw["n"], kdim=kw["kdim"]), m / kw["m"], f"{m} of {kw['m']} rows of A"
    if name == "c4_causal_attention":
        return dict(batch=1, heads=1, seq=min(kw["seq"], 512), dh=kw["dh"]), None, "1 head at seq 512"
    m = min(kw["m"], 32)
    return dict(m=m, kdim=kw["kdim"], n=kw["n"], amp=False), m / kw["m"], f"{m} of {kw['m']} rows of X"


def metric_name(name):
    return {"hbm": "achieved HBM GB/s (algorithmic bytes / device time)", "tensor": "achieved TFLOP/s (algorithmic FLOP / device time)"}[WORKLOADS[name][2]] + f", {name}"


def dtype_of(name):
    return {"c1_fused_reduce": "f32", "c2_transposed_softmax": "f32", "c3_gemm_bias_gelu": "bf16", "c4_causal_attention": "bf16", "c5_fp8_weight_gemm": "f8e4m3"}[name]


_RESULT_FD = None


def emit(line: dict):
    """The one JSON line goes to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


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
    ap.add_argument("--workload", default="c2_transposed_softmax", choices=sorted(WORKLOADS))
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling captures); 1.0 = the baseline's size")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    name = args.workload
    builder, kw, kind = WORKLOADS[name]
    kw = dict(kw)
    if args.scale != 1.0:
        for k in kw:
            if k not in ("dh",):
                kw[k] = max(128, int(kw[k] * args.scale) // 128 * 128)
    if args.impl == "reference":
        return reference_arm(args, name, builder, kw)

    import torch
    import torch.distributed as dist
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = api.Library(build.LIB)
    gpu = api.CudaBackend(lib, local)
    stream = torch.cuda.ExternalStream(gpu.stream, device=local)

    # the workload graph and its seeded inputs, generated on the device (each rank: its own shard of
    # an N-times larger batch: the same shapes and the same seeded draw, since kernel time does not depend on the values)
    g = api.Graph(lib)
    root, gens = builder(g, **kw)
    nbytes, flops = algorithmic_work(name, kw)
    # Inputs smaller than about three L2s (126 MB) are kept in several copies that the steps rotate
    # through, so that a step never finds its inputs in L2 from the step before.
    in_bytes = sum(int(np.prod(g.shape(n))) * api.WIDTH[g.dtype(n)] for n in gens)
    n_sets = max(1, min(8, int(np.ceil(3 * 126e6 / max(in_bytes, 1)))))
    dev_sets = []
    for _ in range(n_sets):
        dev_in = {}
        for node, mk in gens.items():
            h = api.Graph(lib)
            dev_in[node] = gpu.eval_device(h, [mk(h)])[0]
        dev_sets.append(dev_in)
    dev_in = dev_sets[0]
    gpu.sync()
    counter = [0]

    def step():
        counter[0] += 1
        return gpu.eval_device(g, [root], None, dev_sets[counter[0] % n_sets])[0]

    def barrier():
        gpu.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step().free()
    barrier()
    launches0 = gpu.stats()["launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step().free()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = gpu.stats()["launches"] - launches0
    # nvidia-smi needs ~100 ms per sample: when the timed region is shorter than that, keep the same
    # load running (untimed) so the clock record still describes the kernel under load
    t_sustain = time.perf_counter()
    while rank == 0 and ms < 1500 and time.perf_counter() - t_sustain < 1.5:
        for _ in range(20):
            step().free()
        gpu.sync()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed steps" + (" + 1.5 s of the same steps, untimed" if ms < 1500 else "")
    barrier()
    t = torch.tensor([ms], device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    per_step_s = ms / 1e3 / args.steps
    unit = "GB/s" if kind == "hbm" else "TFLOP/s"
    value = world * (nbytes / per_step_s / 1e9 if kind == "hbm" else flops / per_step_s / 1e12)

    # dominant kernel: average launch duration from CUDA events around every launch on the backend's stream
    gpu.profile(True)
    for _ in range(min(args.steps, 20)):
        step().free()
    gpu.sync()
    prof = gpu.take_profile()
    gpu.profile(False)
    peaks = measured_peaks()
    roofline = None
    if prof:
        top = max(prof.items(), key=lambda kv: kv[1]["ms"])
        fam, p = top
        avg_s = p["ms"] / 1e3 / p["launches"]
        duration_source = "CUDA events around each launch (a pass of its own after the timed region)"
        if len(prof) == 1 and p["launches"] == min(args.steps, 20):
            # the step IS this one kernel: its average duration over the timed region (events bracket the K
            # back-to-back launches on the launching stream) is the timed region / K; launch gaps count against it
            avg_s = per_step_s
            duration_source = "timed region / launches (one launch per step; CUDA events bracket the K launches)"
        traffic = NCU_TRAFFIC.get((args.workload, fam)) if args.scale == 1.0 else None
        if kind == "hbm":
            ach = (p["algo_bytes"] / p["launches"]) / avg_s / 1e9
            peak = peaks["hbm_gbs"]
            roofline = {"bound": "hbm", "kernel": fam, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": traffic,
                        "avg_launch_us": avg_s * 1e6, "duration_source": duration_source, "peak_source": peaks["source"], "share_of_step": p["ms"] / sum(v["ms"] for v in prof.values())}
        else:
            ach = (p["flops"] / p["launches"]) / avg_s / 1e12
            peak = peaks["bf16_tflops"]
            roofline = {"bound": "tensor", "kernel": fam, "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": traffic,
                        "avg_launch_us": avg_s * 1e6, "duration_source": duration_source, "peak_source": peaks["source"] + " (bf16 burst)", "share_of_step": p["ms"] / sum(v["ms"] for v in prof.values())}

    # end to end through the C ABI with host buffers: pinned host inputs -> device, evaluate, result -> pinned host
    e2e = None
    if not args.no_e2e:
        host_in = {}
        for node, d in dev_in.items():
            hb = torch.empty(d.nbytes, dtype=torch.uint8).pin_memory()
            d.download_into(hb.data_ptr(), d.nbytes)
            host_in[node] = (hb, d.shape, d.dtype)
        out0 = step()
        host_out = torch.empty(out0.nbytes, dtype=torch.uint8).pin_memory()
        out_bytes, out0_shape = out0.nbytes, tuple(out0.shape)
        out0.free()

        def serial_step():
            ups = {node: gpu.upload_ptr(hb.data_ptr(), hb.numel(), shape, dt) for node, (hb, shape, dt) in host_in.items()}
            o = gpu.eval_device(g, [root], None, ups)[0]
            o.download_into(host_out.data_ptr(), out_bytes)   # waits for the result
            o.free()
            for u in ups.values():
                u.free()

        # the same step chunk by chunk over the independent output rows, uploads, kernels and downloads overlapped
        pipe, e2e_method = None, "one upload of every input, one evaluation, one download"
        plan = CHUNKING.get(name)
        if plan is not None and args.scale == 1.0:
            try:
                from kurumi_b200 import pipeline
                chunks, chunk_kw, axes = plan["chunks"], plan["chunk_kw"](kw, plan["chunks"]), plan["axes"]
                gch = api.Graph(lib)
                root_ch, gens_ch = builder(gch, **chunk_kw)
                inputs = [pipeline.HostInput(node_ch, host_in[node][0].data_ptr(), tuple(host_in[node][1]), host_in[node][2], axes[i])
                          for i, (node, node_ch) in enumerate(zip(dev_in, gens_ch))]
                out_rows = out0_shape[0]
                pipe = pipeline.RowPipeline(gpu, gch, root_ch, inputs, host_out.data_ptr(), out_rows, out_bytes // out_rows, chunks)
                pipe.step()   # a failure of the chunked path shows here, before anything is timed
                e2e_method = f"{chunks} chunks of output rows; host-to-device copies, evaluations (ku_cuda_eval_device) and device-to-host copies overlapped on three streams"
            except Exception as exc:   # the unchunked step is still a valid end-to-end measurement
                print(f"bench: chunked end-to-end path unavailable ({exc}); timing the unchunked step", file=sys.stderr)
                pipe = None
        e2e_step = pipe.step if pipe is not None else serial_step
        n_e2e = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / n_e2e
        tt = torch.tensor([dt], device=f"cuda:{local}")
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        ev = world * (nbytes / dt / 1e9 if kind == "hbm" else flops / dt / 1e12)
        e2e = {"value": ev, "unit": unit, "h2d_bytes_per_step": int(sum(hb.numel() for hb, _, _ in host_in.values())), "d2h_bytes_per_step": int(out_bytes),
               "ms_per_step": dt * 1e3, "timing": "host wall clock around upload + eval + download (download waits for the device)", "steps": n_e2e,
               "method": e2e_method}
        if pipe is not None:   # the result of the chunked step is the result of the single evaluation
            ref_out = step()
            check = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
            ref_out.download_into(check.data_ptr(), out_bytes)
            ref_out.free()
            e2e["matches_single_evaluation"] = bool(torch.equal(check, host_out))
            pipe.close()

    # N > 1: gathering the ranks' output shards into one tensor on every GPU is NOT on the data path that
    # `value` times (shards stay device-resident); its cost is reported beside it
    assembly = None
    if world > 1:
        from cuda.bindings import runtime as cudart
        o = step()
        shard = torch.empty(o.nbytes, dtype=torch.uint8, device=f"cuda:{local}")
        gpu.sync()
        (err,) = cudart.cudaMemcpy(shard.data_ptr(), o.ptr, o.nbytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
        if int(err) != 0:
            raise RuntimeError(f"cudaMemcpy of the output shard failed: {err}")
        o.free()
        whole = torch.empty(world * shard.numel(), dtype=torch.uint8, device=f"cuda:{local}")
        for _ in range(2):
            dist.all_gather_into_tensor(whole, shard)
        torch.cuda.synchronize()
        dist.barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        a0.record()
        for _ in range(reps):
            dist.all_gather_into_tensor(whole, shard)
        a1.record()
        torch.cuda.synchronize()
        at = torch.tensor([a0.elapsed_time(a1) / reps], device=f"cuda:{local}")
        dist.all_reduce(at, op=dist.ReduceOp.MAX)
        assembly = {"ms": float(at.item()), "bytes_per_rank": int(shard.numel()), "collective": "nccl all_gather of the output shards (torch.distributed), CUDA events, max over ranks",
                    "in_value": False}
        del whole, shard

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_baseline(name, builder, kw)

    if rank == 0:
        line = {"metric": metric_name(name), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_of(name),
                "data": "synthetic (seeded threefry2x32 / Box-Muller, generated on device)",
                "config": {"workload": name, **kw, "l2": f"steps rotate through {n_sets} copies of the inputs ({in_bytes * n_sets / 1e6:.0f} MB in all, L2 is 126 MB): no step finds its inputs cached",
                           "sharding": "each rank evaluates its own shard of an N-times larger batch (same shapes); no collective on the data path"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu_base, "assembly": assembly,
                "kernel_times": {k: {"launches": v["launches"], "avg_us": v["ms"] * 1e3 / v["launches"]} for k, v in prof.items()}}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(name, builder, kw):
    """kurumi's own CPU path (view-fused evaluator with interpreter fallback, one thread), restated
    in oracle/, timed on this box's host on a bounded sample of the same workload."""
    olib = api.Library(build.ORACLE_LIB)
    cpu, gen = api.Backend(olib, 65), api.Backend(olib, 0)
    skw, frac, what = cpu_sample(name, kw)
    g = api.Graph(olib)
    root, gens = builder(g, **skw)
    feeds = api.Feeds(olib)
    for node, mk in gens.items():
        h = api.Graph(olib)
        feeds.set(node, gen.eval(h, mk(h)))
    cpu.eval_with(g, root, feeds)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 10 and reps < 20):
        cpu.eval_with(g, root, feeds)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    nbytes, flops = algorithmic_work(name, skw)
    kind = WORKLOADS[name][2]
    return {"value": nbytes / dt / 1e9 if kind == "hbm" else flops / dt / 1e12, "unit": "GB/s" if kind == "hbm" else "TFLOP/s", "cores": 1, "kind": "port",
            "sample": what + f"; {reps} evaluations, {dt * 1e3:.1f} ms each", "host_cpus": os.cpu_count()}


if __name__ == "__main__":
    main()
