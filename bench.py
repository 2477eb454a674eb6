#!/usr/bin/env python
"""Benchmark of the BT4-shape forward pass: positions per second on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode bf16|int8] [--batch B]
    python bench.py --impl reference ...      # the CPU fp32 forward on the host cores
    python bench.py --impl reference-gpu      # the reference's own 291-node program on the GPU (batch <= 2047)

One "step" is one forward pass over one batch of synthetic positions (seeded planes,
N(0, 0.02) random-init weights of the BT4 shape; the trained network and lc0's benchmark
positions are not available offline).  Positions are independent, so N GPUs run N replicas
on disjoint batches with no collective on the data path ("weak" scaling: the per-GPU batch
is fixed); torch.distributed (NCCL) is used only for the barrier and the max-over-ranks of
the device-side time.  Rank 0 prints one JSON line: the bf16 batch-4096 headline with its `roofline`,
`cpu_baseline`, `e2e`, `parity_sample` (a few positions of the benchmarked batch against the CPU oracle)
and, as extra keys, the other figures the metric names: `int8` (same forward on int8 GEMMs, with the int8
tensor peak measured in the same run), `batch1024`, `bt3_b256`, `attention_sweep`, `latency_batch64` and,
for N > 1, `strong` (one global batch of 4096 / 1024 positions split over the ranks).  `--gpus N` without
a multi-process launcher drives the N GPUs from one process (`ShardedNet`).
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "positions/sec at BT4 shape"
CPU_SAMPLE_BATCH = 32  # positions per CPU step: the batch at which the CPU forward is fastest per position (8 and 128 are slower)


def _peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.lines: list[str] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def halt(self) -> None:
        """Stop sampling (the summary is made by stop())."""
        if self.proc is not None and self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.halt()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    torch.cuda.set_device(0)
    return 0, 1, 0, None


def _barrier(dist) -> None:
    if dist is not None:
        t = torch.zeros(1, device="cuda")
        dist.all_reduce(t)
    torch.cuda.synchronize()


def _max_over_ranks(value: float, dist) -> float:
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed_steps(step, warmup: int, steps: int, dist, sampler: "ClockSampler | None" = None) -> float:
    """Milliseconds for exactly `steps` calls of `step`, CUDA events on the current stream, max over ranks.
    A clock sampler, if given, runs from the first warm-up step to the end of the timed steps: every sample is
    taken with the GPU under this load (set-up, graph capture and the barriers' waits are outside)."""
    if sampler is not None:
        sampler.start()
    for _ in range(warmup):
        step()
    _barrier(dist)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.halt()
    _barrier(dist)
    return _max_over_ranks(start.elapsed_time(stop), dist)


def _cpu_forward_rate(cfg, batch: int, repeats: int, warmup: int) -> tuple[float, float]:
    """positions/s of the fp32 CPU oracle forward (the restatement of the reference graph)."""
    from lczero_triton_b200 import mapping_table
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights
    from oracle import bt4_oracle

    weights = {k: v.float() for k, v in random_weights(cfg, 0).items()}
    masks, values = synthetic_planes(batch, 0)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    times = []
    with torch.no_grad():
        for i in range(warmup + repeats):
            t0 = time.perf_counter()
            bt4_oracle.forward(weights, cfg, masks, values, table=table)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return batch / med, med * 1e3


def _config(batch: int, world: int, mode: str) -> dict:
    """The workload both arms report (the reference arm times a bounded sample of it on the CPU)."""
    return {"workload": f"BT4-shape forward (E1024 L15 H32 F1536 smolgen 32->256), batch {batch} per GPU",
            "batch_per_gpu": batch, "global_batch": batch * world, "mode": mode, "parallelism": f"replicas x{world}",
            "l2": "working set per step (several GB of activations) far exceeds the 126 MB L2"}


def run_reference(args) -> None:
    """The reference arm: the CPU fp32 forward on the host cores (the reference itself has no
    executable forward: it is a graph compiler whose runtime lives outside its tree)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from lczero_triton_b200.config import BT4

    # torchrun pins OMP_NUM_THREADS to 1; the CPU arm is meant to use every host core.
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    threads = torch.get_num_threads()
    rate, ms = _cpu_forward_rate(BT4, CPU_SAMPLE_BATCH, max(1, args.steps), max(1, args.warmup))
    sample = f"BT4 fp32 forward, batch {CPU_SAMPLE_BATCH} per step, median of {max(1, args.steps)} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": "positions/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(_config(args.batch, max(1, args.gpus), args.mode),
                       sample=f"CPU fp32 forward of the same network, {CPU_SAMPLE_BATCH} positions per step"),
        "cpu_baseline": {"value": rate, "unit": "positions/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "positions/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args) -> None:
    """An extra arm, not part of the two-arm contract: the UNMODIFIED reference package under ``baseline/_ref``
    building its own program (its graph builder, Triton kernels, compile functions, allocation plan) and that
    program replayed on this GPU by the small runtime of ``tests/golden/make_network_golden.py``.  The
    reference's batched kernels cannot be launched above 2047 positions, so the workload is the BT4 shape at
    min(batch, 2047) positions; building the program autotunes its kernels (about four minutes)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import importlib.util

    def unavailable(why: str) -> None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": why}), flush=True)

    if not (ROOT / "baseline" / "_ref" / "lczero_triton").exists():
        return unavailable("baseline/_ref holds no reference install")
    try:
        import triton  # noqa: F401
    except ImportError:
        return unavailable("triton is not importable")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    spec = importlib.util.spec_from_file_location("make_network_golden", ROOT / "tests" / "golden" / "make_network_golden.py")
    runtime = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runtime)
    runtime.stub_generated_protobuf_modules()
    from lczero_triton_b200.config import BT4
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    torch.cuda.set_device(0)
    batch = min(args.batch, 65535 // BT4.heads)
    weights = runtime.exact_in_both(random_weights(BT4, 0))
    masks, values = (x.cuda() for x in synthetic_planes(batch, 1000))
    started = time.time()
    builder, program, _ = runtime.build_program(BT4, batch, dry=False)
    built = time.time() - started
    loaded = runtime.LoadedProgram(builder, program, {n: w.float().half().cuda() for n, w in weights.items()},
                                   {"/input/plane_masks": masks, "/input/plane_values": values}, fill=0)
    loaded.launch()
    step, _ = _graph_step(loaded.launch)
    sampler = ClockSampler(0)
    ms = _timed_steps(step, args.warmup, args.steps, None, sampler)
    clocks = sampler.stop()
    rate = batch * args.steps / (ms * 1e-3)
    line = {
        "impl": "reference-gpu", "metric": METRIC, "value": rate, "unit": "positions/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"BT4-shape forward (E1024 L15 H32 F1536 smolgen 32->256), batch {batch}: the reference's "
                               f"program of {loaded.info['nodes']} kernel launches, replayed from a CUDA graph",
                   "batch_per_gpu": batch, "graph_build_s": round(built, 1),
                   "l2": "working set per step (GBs of activations) far exceeds the 126 MB L2"},
        "clocks": clocks, "gpu_launches": 0, "reference_launches": loaded.info["nodes"] * args.steps,
    }
    loaded.close()
    print(json.dumps(line), flush=True)


def _graph_step(fn):
    """`fn` captured into a CUDA graph (returns the replay callable), or `fn` itself when capture fails."""
    try:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph.replay, None
    except Exception as exc:  # noqa: BLE001 - fall back to eager launches, say so in the line
        return fn, repr(exc)[:160]


def _forward_rate(net, masks_d, values_d, batch: int, world: int, args, dist, *, graph: bool = True,
                  sampler: "ClockSampler | None" = None) -> dict:
    """Device-resident positions/s of `net` on one batch: whole-job value, max over ranks."""
    def eager() -> None:
        net.forward(masks_d, values_d)

    eager()
    step, error = _graph_step(eager) if graph else (eager, None)
    total_ms = _timed_steps(step, args.warmup, args.steps, dist, sampler)
    out = {"value": world * batch * args.steps / (total_ms * 1e-3), "unit": "positions/s",
           "ms_per_step": total_ms / args.steps, "batch_per_gpu": batch,
           "launch": "CUDA graph replay" if graph and error is None else "eager launches"}
    if error is not None:
        out["graph_error"] = error
    return out


def _e2e_rate(net, masks_h, values_h, batch: int, world: int, args, dist) -> dict:
    """The same metric through the public API with HOST buffers: every step copies the packed planes
    from pinned memory to the device, runs the forward and copies policy / WDL / moves-left back."""
    from lczero_triton_b200.config import POLICY_SIZE

    out_h = [torch.empty((batch, POLICY_SIZE), dtype=torch.float32).pin_memory(),
             torch.empty((batch, 3), dtype=torch.float32).pin_memory(),
             torch.empty((batch, 1), dtype=torch.float32).pin_memory()]
    masks_in = torch.empty(masks_h.shape, dtype=masks_h.dtype, device="cuda")
    values_in = torch.empty(values_h.shape, dtype=values_h.dtype, device="cuda")

    def step() -> None:
        masks_in.copy_(masks_h, non_blocking=True)
        values_in.copy_(values_h, non_blocking=True)
        outs = net.forward(masks_in, values_in)
        for dst, src in zip(out_h, outs):
            dst.copy_(src, non_blocking=True)

    ms = _timed_steps(step, max(1, args.warmup // 2), args.steps, dist)
    return {"value": world * batch * args.steps / (ms * 1e-3), "unit": "positions/s",
            "h2d_bytes_per_step": masks_h.numel() * 8 + values_h.numel() * 4,
            "d2h_bytes_per_step": sum(t.numel() * 4 for t in out_h), "ms_per_step": ms / args.steps}


def _int8_peak() -> dict:
    """int8 tensor-core throughput of this GPU, measured the way the bf16 figures of MEASURED_PEAKS.json
    were: the library GEMM (torch._int_mm) at 8192^3, best of 10 single launches (burst) and launched back
    to back for about two seconds (sustained, under the power cap)."""
    n = 8192
    a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    ops_per_call = 2.0 * n ** 3
    for _ in range(3):
        torch._int_mm(a, b)
    best = float("inf")
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        torch._int_mm(a, b)
        e.record()
        e.synchronize()
        best = min(best, s.elapsed_time(e))
    calls = max(50, int(2000.0 / best))
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(calls):
        torch._int_mm(a, b)
    e.record()
    e.synchronize()
    sustained_ms = s.elapsed_time(e) / calls
    return {"int8_tops": ops_per_call / best / 1e9, "int8_tops_sustained": ops_per_call / sustained_ms / 1e9,
            "how": f"torch._int_mm {n}^3: best of 10 (burst), {calls} back to back (sustained)"}


# DRAM traffic of the QKV GEMM per row of A: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture
# of a launch at 131072 rows (A 268 MB + C 805 MB, more than eight times the L2), divided by the rows.
QKV_TRAFFIC_BYTES_PER_ROW = {"bf16": 7943.0, "int8": 6714.0}


def _qkv_roofline(net, cfg, batch: int, mode: str, peaks: dict, peak_kind: str, int8_peak: dict | None) -> dict:
    """The dominant kernel, timed alone in the form the forward pass launches it: the QKV projection
    GEMM (bf16: LayerNorm of the input rows folded into the epilogue; int8: dequantising epilogue)."""
    from lczero_triton_b200 import ops

    t_rows = batch * 64
    if mode == "int8":
        layer = net.layers[0]["qkv"]
        a = torch.randint(-127, 128, (t_rows, cfg.embedding), device="cuda", dtype=torch.int8)
        extra = {"bias": layer.bias, "col_scale": layer.col_scale,
                 "row_scale": torch.rand(t_rows, device="cuda") * 0.01 + 0.001}
        kernel_name = "gemm_tcgen05_kernel<256, int8, NK, pair, plain>"
    else:
        layer = net.layers[0]["qkv_f"] if net.deferred else net.layers[0]["qkv"]
        a = torch.randn((t_rows, cfg.embedding), device="cuda").to(torch.bfloat16)
        if net.deferred:
            parts = (cfg.embedding + 63) // 64
            stats = torch.rand((parts, t_rows, 2), device="cuda") + 1.0
            extra = {"ln_in": (stats, layer.fold_c, layer.fold_d)}
            kernel_name = "gemm_tcgen05_kernel<256, bf16, NK, pair, ln_in>"
        else:
            extra = {"bias": layer.bias}
            kernel_name = "gemm_tcgen05_kernel<256, bf16, NK, pair, plain>"
    n_main = 3 * cfg.embedding
    out = torch.empty((t_rows, n_main), dtype=torch.bfloat16, device="cuda")
    if layer.n > n_main:  # smolgen's compression rides on this GEMM as trailing columns with an output of their own
        extra["out_tail"] = torch.empty((t_rows, layer.n - n_main), dtype=torch.bfloat16, device="cuda")
        extra["n_main"] = n_main
        kernel_name += " + %d trailing columns (smolgen compression)" % (layer.n - n_main)

    def gemm_once() -> None:
        ops.gemm(out, a, layer.w, m=t_rows, n=layer.n, k=layer.k, w_layout=layer.layout, **extra)

    gemm_ms = _timed_steps(gemm_once, 3, 10, None) / 10
    gemm_flops = 2.0 * t_rows * layer.n * layer.k
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    if mode == "int8":
        peak, sustained = int8_peak["int8_tops"], int8_peak["int8_tops_sustained"]
        peak_source = "measured in this run: " + int8_peak["how"]
    else:
        peak, sustained = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
        peak_source = f"{peak_kind} burst bf16"
    eb = 1 if mode == "int8" else 2
    algorithmic = float(t_rows * layer.k * eb + layer.n * layer.k * eb + t_rows * layer.n * 2)
    per_row = QKV_TRAFFIC_BYTES_PER_ROW[mode]
    traffic = per_row * t_rows if per_row is not None else None
    return {
        "bound": "tensor", "kernel": "%s (QKV projection, M=%d N=%d K=%d)" % (kernel_name, t_rows, layer.n, layer.k),
        "achieved": achieved, "peak": peak, "unit": "TFLOP/s" if mode == "bf16" else "TOP/s", "frac": achieved / peak,
        "peak_source": peak_source, "frac_of_sustained_peak": achieved / sustained,
        "ms_per_launch": gemm_ms, "flops_per_launch": gemm_flops, "algorithmic_bytes": algorithmic,
        "traffic": traffic, "traffic_over_algorithmic": None if traffic is None else traffic / algorithmic,
        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 131072 rows, scaled by rows",
    }


def _attention_sweep(peaks: dict, peak_kind: str) -> list[dict]:
    """The stand-alone edge-biased attention operator at B = 64 / 512 / 4096 (32 heads of depth 32)."""
    from lczero_triton_b200 import ops

    gen = torch.Generator(device="cuda").manual_seed(0)
    # tensor-pipe share of the kernel's cycles: ncu sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed,
    # one-pass captures of this very kernel at the three sizes (a number taken under a profiler, so a constant here)
    tensor_pipe_pct = {64: 5.7, 512: 10.4, 4096: 11.5}
    rows = []
    for b in (64, 512, 4096):
        h, d = 32, 1024
        q, k_, v = (torch.randn((b, 64, d), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(3))
        bias = (torch.randn((b, h, 64, 64), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        out = torch.empty((b, 64, d), dtype=torch.bfloat16, device="cuda")

        def once() -> None:
            ops.attention(out, q, k_, v, bias, 32 ** -0.5, b, h)

        ms = _timed_steps(once, 3, 20, None) / 20
        nbytes = 786432.0 * b
        gbs = nbytes / (ms * 1e-3) / 1e9
        rows.append({"batch": b, "ms": ms, "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
                     "peak_source": f"{peak_kind} HBM copy", "tflops": 4.0 * b * h * 64 * 64 * 32 / (ms * 1e-3) / 1e12,
                     "tensor_pipe_pct_ncu": tensor_pipe_pct.get(b),
                     "working_set": "larger than L2" if nbytes > 126e6 else "fits in L2: not an HBM figure"})
    return rows


def _parity_sample(net, masks_h, values_h, cfg, weights, mode: str, positions: int = 8) -> tuple[dict, float]:
    """A few positions of the benchmarked batch, picked across it, against the fp32 CPU oracle.
    Returns the report and the oracle's positions per second on that sample."""
    from lczero_triton_b200 import mapping_table
    from oracle import bt4_oracle

    batch = masks_h.shape[0]
    index = torch.linspace(0, batch - 1, positions).long().unique()
    outs = net.forward(masks_h.cuda(), values_h.cuda())
    got = [x[index.cuda()].float().cpu() for x in outs]
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    t0 = time.perf_counter()
    want = bt4_oracle.forward(weights, cfg, masks_h[index], values_h[index], table=table)
    oracle_s = time.perf_counter() - t0
    report = {"positions": [int(i) for i in index], "tolerance": "1e-2 absolute or 1 % relative (bf16 target)",
              "oracle": "fp32 CPU forward", "oracle_seconds": oracle_s}
    for name, g, w in zip(("policy", "wdl", "mlh"), got, want):
        err = (g - w).abs()
        outside = ~((err <= 1e-2) | (err <= 1e-2 * w.abs()))
        report[name] = {"max_abs_err": float(err.max()), "outside_tolerance": int(outside.sum()), "count": g.numel(),
                        "max_err_over_spread": float(err.max() / w.std().clamp_min(1e-12))}
    if mode == "int8":
        report["note"] = "int8 GEMMs: no end-to-end tolerance is promised; the figures are against the fp32 forward"
    return report, float(len(index)) / oracle_s


def run(args) -> None:
    rank, world, local, dist = _dist_setup(args.gpus)
    from lczero_triton_b200 import _lib, build
    from lczero_triton_b200.config import BT3, BT4
    from lczero_triton_b200.net import Bt4Net
    from lczero_triton_b200.sharded import shard_range
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    build.build()
    cfg = BT4
    batch = args.batch
    peaks, peak_kind = _peaks()
    weights = random_weights(cfg, 0)
    deferred = None if args.deferred_ln < 0 else bool(args.deferred_ln)
    net = Bt4Net(weights, cfg, mode=args.mode, deferred_layer_norm=deferred)
    masks_h, values_h = synthetic_planes(batch, seed=1000 + rank)
    masks_h, values_h = masks_h.pin_memory(), values_h.pin_memory()
    masks_d, values_d = masks_h.cuda(), values_h.cuda()

    # ---- headline: device-resident throughput, then end to end with host buffers
    net.forward(masks_d, values_d)
    torch.cuda.synchronize()
    launches_before = _lib.launch_count()
    net.forward(masks_d, values_d)
    launches_per_step = _lib.launch_count() - launches_before
    sampler = ClockSampler(local)
    head = _forward_rate(net, masks_d, values_d, batch, world, args, dist, graph=bool(args.graph), sampler=sampler)
    clocks = sampler.stop()
    e2e = _e2e_rate(net, masks_h, values_h, batch, world, args, dist)

    line = {
        "metric": METRIC, "value": head["value"], "unit": "positions/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.mode == "bf16" else "int8", "data": "synthetic",
        "config": _config(batch, world, args.mode),
        "clocks": clocks, "gpu_launches": launches_per_step * args.steps, "e2e": e2e,
    }
    line["config"]["launch"] = head["launch"]
    if "graph_error" in head:
        line["config"]["graph_error"] = head["graph_error"]
    flops = cfg.flops_per_position()
    line["forward_tflops_per_gpu"] = flops * batch / (head["ms_per_step"] * 1e-3) / 1e12
    line["forward_frac_of_sustained_bf16_peak"] = line["forward_tflops_per_gpu"] / peaks["bf16_tflops_sustained"]

    extras = not args.headline_only
    int8_peak = None
    if extras and args.mode == "bf16":
        # ---- the same forward with int8 GEMMs (weak scaling, every N), and its own peak
        int8_peak = _int8_peak()
        net8 = Bt4Net(weights, cfg, mode="int8", deferred_layer_norm=deferred)
        row = _forward_rate(net8, masks_d, values_d, batch, world, args, dist)
        row["e2e"] = _e2e_rate(net8, masks_h, values_h, batch, world, args, dist)
        row["forward_tops_per_gpu"] = flops * batch / (row["ms_per_step"] * 1e-3) / 1e12
        row["forward_frac_of_sustained_int8_peak"] = row["forward_tops_per_gpu"] / int8_peak["int8_tops_sustained"]
        row["peak"] = int8_peak
        if rank == 0 and world == 1:
            row["roofline"] = _qkv_roofline(net8, cfg, batch, "int8", peaks, peak_kind, int8_peak)
            row["parity_sample"], _ = _parity_sample(net8, masks_h, values_h, cfg, weights, "int8")
        line["int8"] = row
        del net8
        torch.cuda.empty_cache()
    if extras and world > 1:
        # ---- strong scaling: ONE global batch split by position over the ranks (no collective on the path)
        strong = {}
        for global_batch in (4096, 1024):
            lo, hi = shard_range(global_batch, rank, world)
            m_all, v_all = synthetic_planes(global_batch, seed=2000)
            m_d, v_d = m_all[lo:hi].cuda(), v_all[lo:hi].cuda()
            row = _forward_rate(net, m_d, v_d, hi - lo, 1, args, dist)
            strong[f"global_batch_{global_batch}"] = {
                "value": global_batch / (row["ms_per_step"] * 1e-3), "unit": "positions/s",
                "ms_per_step": row["ms_per_step"], "positions_per_gpu": hi - lo, "launch": row["launch"]}
        line["strong"] = strong

    if rank == 0 and world == 1:
        line["roofline"] = _qkv_roofline(net, cfg, batch, args.mode, peaks, peak_kind, int8_peak or
                                         (_int8_peak() if args.mode == "int8" else None))
        # ---- parity of the benchmarked batch, and the CPU baseline from the same oracle run
        parity, cpu_rate = _parity_sample(net, masks_h, values_h, cfg, weights, args.mode)
        line["parity_sample"] = parity
        if not args.no_cpu_baseline:
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            rate, ms = _cpu_forward_rate(cfg, CPU_SAMPLE_BATCH, 3, 1)
            line["cpu_baseline"] = {"value": rate, "unit": "positions/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": f"BT4 fp32 forward, batch {CPU_SAMPLE_BATCH}, median of 3 after 1 warm-up ({ms:.0f} ms each)"}
        if extras:
            # ---- the other configurations the metric names
            m1k, v1k = synthetic_planes(1024, seed=3000)
            line["batch1024"] = _forward_rate(net, m1k.cuda(), v1k.cuda(), 1024, 1, args, None)
            net3 = Bt4Net(random_weights(BT3, 0), BT3, mode="bf16", deferred_layer_norm=deferred)
            m256, v256 = synthetic_planes(256, seed=3001)
            row = _forward_rate(net3, m256.cuda(), v256.cuda(), 256, 1, args, None)
            row["workload"] = "BT3-shape forward (E768 L15 H24 F1024), batch 256"
            row["forward_tflops"] = BT3.flops_per_position() * 256 / (row["ms_per_step"] * 1e-3) / 1e12
            line["bt3_b256"] = row
            del net3
            line["attention_sweep"] = _attention_sweep(peaks, peak_kind)
        # ---- p50 latency at batch 64 (whole forward replayed from a CUDA graph)
        if not args.no_latency:
            try:
                m64, v64 = synthetic_planes(64, 7)
                m64, v64 = m64.cuda(), v64.cuda()
                net.forward(m64, v64)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    net.forward(m64, v64)
                samples = []
                for _ in range(10):
                    graph.replay()
                torch.cuda.synchronize()
                for _ in range(200):
                    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s.record()
                    graph.replay()
                    e.record()
                    e.synchronize()
                    samples.append(s.elapsed_time(e))
                line["latency_batch64"] = {"p50_ms": statistics.median(samples), "p99_ms": sorted(samples)[197],
                                           "how": "CUDA graph replay of the whole forward, 200 samples"}
            except Exception as exc:  # noqa: BLE001 - reported, never fatal for the throughput line
                line["latency_batch64"] = {"error": repr(exc)[:200]}
    status, detail = _lib.device_status()
    line["device_status"] = status
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_one_process(args) -> None:
    """`--gpus N` without a multi-process launcher: ONE process drives N GPUs through `ShardedNet` (a
    replica and a worker thread per device).  A global batch of N x `--batch` host-resident positions is
    split by position every step, so the H2D / D2H copies are inside the timed region and `value` is the
    end-to-end figure.  Timed with CUDA events on every device's stream; the slowest device counts."""
    from lczero_triton_b200 import build
    from lczero_triton_b200.config import BT4
    from lczero_triton_b200.sharded import ShardedNet
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    build.build()
    n = args.gpus
    if torch.cuda.device_count() < n:
        raise SystemExit(f"--gpus {n}: only {torch.cuda.device_count()} CUDA devices are visible")
    total = n * args.batch
    net = ShardedNet(random_weights(BT4, 0), BT4, max_batch=total, devices=list(range(n)), mode=args.mode)
    masks_h, values_h = synthetic_planes(total, seed=1000)
    masks_h, values_h = masks_h.pin_memory(), values_h.pin_memory()
    for _ in range(args.warmup):
        net.forward(masks_h, values_h)
    events = []
    for d in range(n):
        with torch.cuda.device(d):
            torch.cuda.synchronize()
            events.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
    sampler = ClockSampler(0)
    sampler.start()
    for d in range(n):
        with torch.cuda.device(d):
            events[d][0].record()
    for _ in range(args.steps):
        net.forward(masks_h, values_h)
    elapsed = []
    for d in range(n):
        with torch.cuda.device(d):
            events[d][1].record()
            torch.cuda.synchronize()
            elapsed.append(events[d][0].elapsed_time(events[d][1]))
    clocks = sampler.stop()
    ms = max(elapsed)
    value = total * args.steps / (ms * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": "positions/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.mode == "bf16" else "int8", "data": "synthetic",
        "config": dict(_config(args.batch, n, args.mode), parallelism=f"one process, {n} replica threads (ShardedNet)",
                       launch="eager launches, host buffers in and out every step"),
        "clocks": clocks, "gpu_launches": 170 * n * args.steps,
        "e2e": {"value": value, "unit": "positions/s", "h2d_bytes_per_step": masks_h.numel() * 8 + values_h.numel() * 4,
                "d2h_bytes_per_step": total * (1858 + 3 + 1) * 4, "ms_per_step": ms / args.steps},
        "per_device_ms": elapsed,
    }
    net.close()
    print(json.dumps(line), flush=True)


def run_kernel(args) -> None:
    """Single-kernel measurements (one GPU): the GEMM at a given shape, the stand-alone
    edge-biased attention operator (B x 64 tokens x 32 heads x 32), or the LayerNorm kernel.
    Prints one JSON line with the CUDA-event time per launch and the achieved rate against the
    measured peak that bounds the kernel."""
    torch.cuda.set_device(0)
    from lczero_triton_b200 import _lib, build, ops

    build.build()
    peaks, peak_kind = _peaks()
    gen = torch.Generator(device="cuda").manual_seed(0)
    line: dict = {"kernel": args.kernel, "iters": args.iters}
    if args.kernel == "gemm":
        m, n, k = args.m, args.n, args.k
        int8 = args.mode == "int8"
        if int8:
            a = torch.randint(-127, 128, (m, k), generator=gen, device="cuda", dtype=torch.int8)
            w = torch.randint(-127, 128, (n, k) if args.layout == "nk" else (k, n), generator=gen, device="cuda",
                              dtype=torch.int8)
        else:
            a = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
            w = (torch.randn((n, k) if args.layout == "nk" else (k, n), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)
        out_dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "s32": torch.int32}[args.out]
        out = torch.empty((m, n), dtype=out_dtype, device="cuda")
        bias = torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16) if args.epilogue != "none" else None
        rs = torch.rand(m, generator=gen, device="cuda") if int8 and args.out != "s32" else None
        cs = torch.rand(n, generator=gen, device="cuda") if int8 and args.out != "s32" else None
        act = "mish" if args.epilogue == "bias_mish" else "none"
        layout = _lib.W_NK if args.layout == "nk" else _lib.W_KN

        extra = {}
        if args.epilogue in ("res", "res_ln"):  # residual epilogue: z = alpha * (acc + b) + (LN of) skip, with row sums
            bias = torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16)
            extra = {"res_skip": torch.randn((m, n), generator=gen, device="cuda").to(torch.bfloat16), "res_alpha": 0.43,
                     "stats_out": torch.empty(((n + 63) // 64, m, 2), dtype=torch.float32, device="cuda")}
            if args.epilogue == "res_ln":
                extra["res_ln"] = (torch.rand(((n + 63) // 64, m, 2), generator=gen, device="cuda") + 1.0,
                                   torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16),
                                   torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16))
        elif args.epilogue in ("ln_in", "ln_in_mish"):  # LayerNorm of the A rows folded into the epilogue
            bias = None
            extra = {"ln_in": (torch.rand(((k + 63) // 64, m, 2), generator=gen, device="cuda") + 1.0,
                               torch.randn(n, generator=gen, device="cuda"), torch.randn(n, generator=gen, device="cuda"))}
            act = "mish" if args.epilogue == "ln_in_mish" else "none"

        def once() -> None:
            ops.gemm(out, a, w, m=m, n=n, k=k, bias=bias, activation=act, w_layout=layout, row_scale=rs, col_scale=cs,
                     **extra)

        ms = _timed_steps(once, 3, args.iters, None) / args.iters
        achieved = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        peak = _int8_peak()["int8_tops"] if int8 else peaks["bf16_tflops"]
        eb = 1 if int8 else 2
        line.update({"shape": [m, n, k], "mode": args.mode, "layout": args.layout, "epilogue": args.epilogue,
                     "out": args.out, "ms": ms, "achieved": achieved, "unit": "TFLOP/s", "peak": peak,
                     "frac": achieved / peak, "peak_source": "int8 burst measured in this run (torch._int_mm 8192^3)" if int8 else f"{peak_kind} burst bf16",
                     "algorithmic_bytes": m * k * eb + n * k * eb + m * n * out.element_size()})
    elif args.kernel in ("quantize", "normalize_quantize"):
        # int8 row quantisers: bf16 rows in, int8 rows and one f32 scale per row out
        rows, width = args.rows, args.width
        x = torch.randn((rows, width), generator=gen, device="cuda").to(torch.bfloat16)
        q = torch.empty((rows, width), dtype=torch.int8, device="cuda")
        sc = torch.empty((rows,), dtype=torch.float32, device="cuda")
        if args.kernel == "quantize":
            def once() -> None:
                ops.quantize_rows(q, sc, x, rows, width)
            nbytes = rows * (width * 3.0 + 4.0)
        else:
            groups = x.float().reshape(rows, width // 64, 64)
            stats = torch.stack((groups.sum(dim=2), (groups * groups).sum(dim=2)), dim=2).permute(1, 0, 2).contiguous()
            gamma = (1.0 + 0.1 * torch.randn(width, generator=gen, device="cuda")).to(torch.bfloat16)
            beta = (0.1 * torch.randn(width, generator=gen, device="cuda")).to(torch.bfloat16)

            def once() -> None:
                ops.normalize_quantize_rows(q, sc, x, stats, gamma, beta, rows, width)
            nbytes = rows * (width * 3.0 + 4.0 + (width // 64) * 8.0)
        ms = _timed_steps(once, 3, args.iters, None) / args.iters
        achieved = nbytes / (ms * 1e-3) / 1e9
        line.update({"rows": rows, "width": width, "ms": ms, "achieved": achieved, "unit": "GB/s",
                     "peak": peaks["hbm_gbs"], "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} HBM copy",
                     "algorithmic_bytes": nbytes})
    elif args.kernel in ("policy_tail", "embed_concat"):
        # the two HBM-bound ends of the forward: packed planes -> embedding input, records -> 1858 f32 logits
        from lczero_triton_b200 import mapping_table
        from lczero_triton_b200.synthetic import synthetic_planes

        b = args.batch
        if args.kernel == "embed_concat":
            masks, values = (t.cuda() for t in synthetic_planes(b, 0))
            position = torch.randn((b, 64 * 64), generator=gen, device="cuda").to(torch.bfloat16)
            out = torch.empty((b * 64, 112 + 64), dtype=torch.bfloat16, device="cuda")

            def once() -> None:
                ops.embed_concat(out, masks, values, position, b, 64)
            nbytes = b * (112 * 12.0 + 64 * 64 * 2.0 + 64 * 176 * 2.0)
        else:
            width = 1024
            records = torch.randn((b, 4288), generator=gen, device="cuda").to(torch.bfloat16)
            keys = torch.randn((b * 64, width), generator=gen, device="cuda").to(torch.bfloat16)
            w = torch.randn((width, 4), generator=gen, device="cuda").to(torch.bfloat16)
            table = torch.tensor(mapping_table.values(), dtype=torch.int32, device="cuda")
            out = torch.empty((b, 1858), dtype=torch.float32, device="cuda")

            def once() -> None:
                ops.policy_tail(out, records, keys, w, table, b, width)
            nbytes = b * (4288 * 2.0 + 8 * width * 2.0 + 1858 * 4.0)  # records, the eight promotion-rank key rows, logits
        ms = _timed_steps(once, 3, args.iters, None) / args.iters
        achieved = nbytes / (ms * 1e-3) / 1e9
        line.update({"batch": b, "ms": ms, "achieved": achieved, "unit": "GB/s", "peak": peaks["hbm_gbs"],
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} HBM copy", "algorithmic_bytes": nbytes})
    elif args.kernel == "attention":
        b, h, d = args.batch, 32, 1024
        q, k_, v = (torch.randn((b, 64, d), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(3))
        bias = (torch.randn((b, h, 64, 64), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        out = torch.empty((b, 64, d), dtype=torch.bfloat16, device="cuda")

        def once() -> None:
            ops.attention(out, q, k_, v, bias, 32 ** -0.5, b, h)

        ms = _timed_steps(once, 3, args.iters, None) / args.iters
        nbytes = 786432.0 * b
        achieved = nbytes / (ms * 1e-3) / 1e9
        line.update({"batch": b, "heads": h, "depth": 32, "ms": ms, "achieved": achieved, "unit": "GB/s",
                     "peak": peaks["hbm_gbs"], "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} HBM copy",
                     "algorithmic_bytes": nbytes, "tflops": 2.0 * 2 * b * h * 64 * 64 * 32 / (ms * 1e-3) / 1e12,
                     "working_set_vs_l2": "larger" if nbytes > 126e6 else "fits in L2: not an HBM measurement"})
    else:
        rows, width = args.rows, args.width
        x = torch.randn((rows, width), generator=gen, device="cuda").to(torch.bfloat16)
        skip = torch.randn((rows, width), generator=gen, device="cuda").to(torch.bfloat16) if args.skip else None
        vec = [torch.randn(width, generator=gen, device="cuda").to(torch.bfloat16) for _ in range(3)]
        alpha = torch.tensor([0.5], device="cuda").to(torch.bfloat16) if args.skip else None
        out = torch.empty_like(x)

        def once() -> None:
            ops.layer_norm(out, x, vec[0], vec[1], vec[2], row_count=rows, width=width, skip=skip, alpha=alpha)

        ms = _timed_steps(once, 3, args.iters, None) / args.iters
        nbytes = rows * width * 2.0 * (3 if args.skip else 2)
        achieved = nbytes / (ms * 1e-3) / 1e9
        line.update({"rows": rows, "width": width, "skip": bool(args.skip), "ms": ms, "achieved": achieved, "unit": "GB/s",
                     "peak": peaks["hbm_gbs"], "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} HBM copy",
                     "algorithmic_bytes": nbytes})
    status, _ = _lib.device_status()
    line["device_status"] = status
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"])
    ap.add_argument("--mode", default="bf16", choices=["bf16", "int8"])
    ap.add_argument("--batch", type=int, default=4096, help="positions per GPU per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-latency", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the extra keys (int8, batch 1024, BT3, attention sweep, strong scaling)")
    ap.add_argument("--graph", type=int, default=1, help="replay the forward from a CUDA graph in the timed loop")
    ap.add_argument("--deferred-ln", type=int, default=-1,
                    help="LayerNorm folded into the GEMM epilogues: 1 / 0, or -1 for the mode's default")
    ap.add_argument("--kernel", default=None, choices=["gemm", "attention", "layer_norm", "quantize", "normalize_quantize", "policy_tail", "embed_concat"],
                    help="measure one kernel instead of the whole forward pass")
    ap.add_argument("--m", type=int, default=262144)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--layout", default="nk", choices=["nk", "kn"])
    ap.add_argument("--epilogue", default="bias",
                    choices=["none", "bias", "bias_mish", "res", "res_ln", "ln_in", "ln_in_mish"])
    ap.add_argument("--out", default="bf16", choices=["bf16", "f32", "s32"])
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--skip", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    if args.kernel is not None:
        run_kernel(args)
        return
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    elif args.gpus > 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_one_process(args)
    else:
        run(args)


if __name__ == "__main__":
    main()
