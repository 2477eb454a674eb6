#!/usr/bin/env python
"""Time the reference's whole forward pass on this GPU, beside this library's, on the same network.

The reference (Kovax007/lczero-triton) is a graph compiler without a runtime in its tree.
``tests/golden/make_network_golden.py`` supplies the missing runtime: the reference's own graph builder,
Triton kernels, compile functions and allocation plan, with the nodes launched in program order at the
planned addresses.  This script builds that program for one network shape and batch size, replays it as a
CUDA graph (what a runtime with a static node list does) and as plain launches, then runs this library's C
network object on the same weights and planes and compares the outputs.

    python baseline/time_reference_graph.py [--config bt4] [--batch 1024] [--iters 10]

The reference's batched attention kernels put batch x heads on ``grid.z`` (limit 65535): with 32 heads the
largest batch its BT4 program can run is 2047.  Every line printed is one JSON object.  Timing: CUDA events
around ``iters`` replays after 3 warm-up replays; the working set (several GB at the default batch) is far
larger than the 126 MB L2.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import pathlib
import sys
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT)]


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _captured(fn):
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph.replay


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="bt4")
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--profile-one", action="store_true",
                    help="bracket ONE plain forward of each side with cudaProfilerStart/Stop (for a profiler run with "
                         "--profile-from-start off: the launch lists of the two programs, nothing else)")
    args = ap.parse_args()
    if not (ROOT / "baseline" / "_ref" / "lczero_triton").exists():
        print(json.dumps({"unavailable": "baseline/_ref holds no reference install"}))
        return
    spec = importlib.util.spec_from_file_location("make_network_golden", ROOT / "tests" / "golden" / "make_network_golden.py")
    runtime = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runtime)
    runtime.stub_generated_protobuf_modules()

    from lczero_triton_b200 import build, config, native, synthetic
    from lczero_triton_b200 import weights as W

    build.build()
    cfg = config.CONFIGS[args.config]
    if args.batch * cfg.heads > 65535:
        print(json.dumps({"unavailable": f"batch {args.batch} x {cfg.heads} heads exceeds grid.z of the reference's "
                                         f"batched kernels; largest batch is {65535 // cfg.heads}"}))
        return
    weights = runtime.exact_in_both(W.random_weights(cfg, args.seed))
    masks, values = synthetic.synthetic_planes(args.batch, args.seed)
    masks, values = masks.cuda(), values.cuda()

    started = time.time()
    builder, program, _ = runtime.build_program(cfg, args.batch, dry=False)
    built = time.time() - started
    loaded = runtime.LoadedProgram(builder, program, {n: w.float().half().cuda() for n, w in weights.items()},
                                   {"/input/plane_masks": masks, "/input/plane_values": values}, fill=0)
    loaded.launch()
    reference = loaded.outputs()
    assert all(bool(torch.isfinite(t).all()) for t in reference.values())
    ms_graph = _time(_captured(loaded.launch), args.iters)
    ms_plain = _time(loaded.launch, args.iters)
    if args.profile_one:
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
        loaded.launch()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
    print(json.dumps({"impl": "reference graph (Triton kernels, its allocation plan)", "config": args.config,
                      "batch": args.batch, "dtype": "fp16", "nodes": loaded.info["nodes"],
                      "kernel_specialisations": loaded.info["kernels"], "graph_build_s": round(built, 1),
                      "execution_allocation_bytes": loaded.info["execution_bytes"],
                      "ms_per_forward_cuda_graph": round(ms_graph, 3), "ms_per_forward_plain_launches": round(ms_plain, 3),
                      "positions_per_s": round(args.batch / ms_graph * 1e3, 1)}), flush=True)
    loaded.close()
    del loaded
    torch.cuda.empty_cache()

    for mode in ("bf16", "int8"):
        net = native.NativeNet(weights, cfg, max_batch=args.batch, mode=mode)
        outs = [x.float().cpu() for x in net.forward(masks, values)]
        ms_graph = _time(_captured(lambda: net.forward(masks, values)), args.iters)
        ms_plain = _time(lambda: net.forward(masks, values), args.iters)
        if args.profile_one and mode == "bf16":
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
            net.forward(masks, values)
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()
        differences = {name: float((outs[i].reshape(args.batch, -1) - reference[f"/output/{name}"].float().reshape(args.batch, -1))
                                   .abs().max()) for i, name in enumerate(("policy", "wdl", "mlh"))}
        print(json.dumps({"impl": f"this library, C network object, {mode}", "config": args.config, "batch": args.batch,
                          "dtype": mode, "ms_per_forward_cuda_graph": round(ms_graph, 3),
                          "ms_per_forward_plain_launches": round(ms_plain, 3),
                          "positions_per_s": round(args.batch / ms_graph * 1e3, 1),
                          "max_abs_difference_from_reference_outputs": differences,
                          "policy_spread": float(reference["/output/policy"].float().std())}), flush=True)
        net.close()
        del net
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
