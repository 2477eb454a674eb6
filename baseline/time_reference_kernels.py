#!/usr/bin/env python
"""Time the reference's own Triton kernels on this GPU, beside this library's kernels on the same shapes.

The reference (Kovax007/lczero-triton) has no runtime of its own: its kernels are Triton functions that
its tests launch directly through their autotuners (tests/test_matmul.py:25-138, test_fused_qkv.py:36-75,
test_batched_matmul.py:96-170, test_softmax_64.py:44-55, test_layer_norm.py:77-119).  This script does
the same with the unmodified reference package installed under ``baseline/_ref`` (its three generated
``*_pb2`` protobuf modules, which do not exist offline and which no kernel uses, are replaced by attribute
stubs as ``tests/golden/make_golden.py`` does), at the BT4 layer shapes, fp16 as the reference stores
its tensors, and then runs this library's kernel for the same operator on bf16 copies of the same values.

    python baseline/time_reference_kernels.py [--batch 4096] [--iters 10]

Every line printed is one JSON object: operator, shape, milliseconds per call for both sides (CUDA
events around ``iters`` back-to-back calls after warm-up and, for the reference, after its autotuner has
picked a configuration), and the rate in the unit that bounds the operator.  Inputs are far larger than
the 126 MB L2 at the default batch.
"""

from __future__ import annotations

import argparse
import json
import pathlib
import sys

import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT), str(ROOT / "baseline" / "_ref"), str(ROOT / "tests" / "golden")]


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    if not (ROOT / "baseline" / "_ref" / "lczero_triton").exists():
        print(json.dumps({"unavailable": "baseline/_ref holds no reference install"}))
        return
    import make_golden

    make_golden._stub_generated_protobuf_modules()
    import triton
    from lczero_triton.bt4.kernels import batched_matmul as r_bmm
    from lczero_triton.bt4.kernels import fused_qkv as r_qkv
    from lczero_triton.bt4.kernels import layer_norm as r_ln
    from lczero_triton.bt4.kernels import matmul as r_mm
    from lczero_triton.bt4.kernels import softmax_64 as r_sm

    from lczero_triton_b200 import _lib, build, ops

    build.build()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    b = args.batch
    t = b * 64
    it = args.iters
    f16, bf16 = torch.float16, torch.bfloat16

    def emit(**row) -> None:
        row["triton"] = triton.__version__
        print(json.dumps(row), flush=True)

    # ---- dense GEMMs of one encoder layer (matmul.py:57-116), reference [K,N] weight layout on both sides
    for label, m, k, n in (("ffn_dense1", t, 1024, 1536), ("ffn_dense2", t, 1536, 1024), ("mha_out", t, 1024, 1024),
                           ("smolgen_shared", b * 32, 256, 4096)):
        a = torch.randn((m, k), dtype=f16, device="cuda") * 0.05
        w = torch.randn((k, n), dtype=f16, device="cuda") * 0.05
        out = torch.empty((m, n), dtype=f16, device="cuda")
        ref_ms = _time(lambda: r_mm._matmul_kernel[r_mm._autotune_grid](out, a, w, m, n, k), it)
        a2, w2, out2 = a.to(bf16), w.to(bf16), torch.empty((m, n), dtype=bf16, device="cuda")
        our_kn_ms = _time(lambda: ops.matmul(out2, a2, w2, m, n, k), it)
        w_nk = w2.t().contiguous()
        our_nk_ms = _time(lambda: ops.gemm(out2, a2, w_nk, m=m, n=n, k=k, w_layout=_lib.W_NK), it)
        flops = 2.0 * m * n * k
        emit(op="matmul", layer=label, m=m, k=k, n=n, reference_ms=ref_ms, ours_kn_ms=our_kn_ms, ours_nk_ms=our_nk_ms,
             reference_tflops=flops / ref_ms / 1e9, ours_kn_tflops=flops / our_kn_ms / 1e9,
             ours_nk_tflops=flops / our_nk_ms / 1e9,
             reference_config=str(getattr(r_mm._matmul_kernel, "best_config", None)))
        del a, w, out, a2, w2, out2, w_nk

    # ---- fused Q/K/V projection (fused_qkv.py:30-123) against this library's single GEMM over concatenated weights
    m, k, n = t, 1024, 1024
    a = torch.randn((m, k), dtype=f16, device="cuda") * 0.05
    ws = [torch.randn((k, n), dtype=f16, device="cuda") * 0.05 for _ in range(3)]
    outs = [torch.empty((m, n), dtype=f16, device="cuda") for _ in range(3)]
    ref_ms = _time(lambda: r_qkv._fused_qkv_projection_kernel[r_qkv._projection_autotune_grid](
        outs[0], outs[1], outs[2], a, ws[0], ws[1], ws[2], m, n, n, n, k), it)
    a2 = a.to(bf16)
    w_cat = torch.cat([w.to(bf16) for w in ws], dim=1).t().contiguous()  # [3N, K]
    out2 = torch.empty((m, 3 * n), dtype=bf16, device="cuda")
    our_ms = _time(lambda: ops.gemm(out2, a2, w_cat, m=m, n=3 * n, k=k, w_layout=_lib.W_NK), it)
    flops = 2.0 * m * 3 * n * k
    emit(op="fused_qkv_projection", m=m, k=k, n=3 * n, reference_ms=ref_ms, ours_ms=our_ms,
         reference_tflops=flops / ref_ms / 1e9, ours_tflops=flops / our_ms / 1e9,
         reference_config=str(getattr(r_qkv._fused_qkv_projection_kernel, "best_config", None)))
    del a, ws, outs, a2, w_cat, out2

    # ---- attention: body_qk + softmax_64 + attention_v (batched_matmul.py:68-210, softmax_64.py:45-71), three
    #      launches with the scores in HBM, against this library's one fused kernel
    #      (the reference puts the matrix index on grid.z, which CUDA limits to 65535: 2047 positions of 32 heads
    #      is the largest batch its kernels can be launched on, so that stands in for larger batches)
    for bb in sorted({512, min(b, 65535 // 32)}):
        heads, depth, d = 32, 32, 1024
        q, kk, v = (torch.randn((bb, 64, d), dtype=f16, device="cuda") for _ in range(3))
        bias = torch.randn((bb, heads, 64, 64), dtype=f16, device="cuda") * 0.5
        scale = torch.tensor([depth ** -0.5], dtype=f16, device="cuda")
        scores = torch.empty((bb, heads, 64, 64), dtype=f16, device="cuda")
        merged = torch.empty((bb, 64, d), dtype=f16, device="cuda")
        rows = bb * heads * 64

        def qk() -> None:
            r_bmm._qk_kernel[r_bmm._autotune_grid](scores, q, kk, scale, r_bmm._OPERATIONS["body_qk"], bb * heads, heads,
                                                   64, 64, depth, 64 * 64)

        def softmax() -> None:
            r_sm._softmax_64_kernel[r_sm._autotune_grid](scores, scores, bias, rows)

        def pv() -> None:
            r_bmm._attention_v_kernel[r_bmm._autotune_grid](merged, scores, v, bb * heads, heads, 64, depth, 64)

        parts = [_time(f, it) for f in (qk, softmax, pv)]

        def all_three() -> None:
            qk()
            softmax()
            pv()

        ref_ms = _time(all_three, it)
        q2, k2, v2, bias2 = q.to(bf16), kk.to(bf16), v.to(bf16), bias.to(bf16)
        out2 = torch.empty((bb, 64, d), dtype=bf16, device="cuda")
        our_ms = _time(lambda: ops.attention(out2, q2, k2, v2, bias2, depth ** -0.5, bb, heads), it)
        nbytes = 786432.0 * bb  # Q, K, V, bias in and O out, once each: what the fused operator has to move
        emit(op="attention", batch=bb, heads=heads, reference_ms=ref_ms, reference_parts_ms=parts, ours_ms=our_ms,
             reference_gbs=nbytes / ref_ms / 1e6, ours_gbs=nbytes / our_ms / 1e6)
        del q, kk, v, bias, scores, merged, q2, k2, v2, bias2, out2

    # ---- LayerNorm with skip (layer_norm.py:37-161)
    for rows in sorted({65536, t}):
        width = 1024
        x = torch.randn((rows, width), dtype=f16, device="cuda")
        skip = torch.randn((rows, width), dtype=f16, device="cuda")
        bias, gamma, beta = (torch.randn(width, dtype=f16, device="cuda") for _ in range(3))
        alpha = torch.tensor([0.43], dtype=f16, device="cuda")
        out = torch.empty_like(x)
        block = triton.next_power_of_2(width)
        ref_ms = _time(lambda: r_ln._layer_norm_skip_kernel[r_ln._autotune_grid](
            out, x, bias, skip, gamma, beta, alpha, rows, width, 1e-3, r_ln._ACTIVATIONS["none"], block), it)
        x2, skip2, out2 = x.to(bf16), skip.to(bf16), torch.empty((rows, width), dtype=bf16, device="cuda")
        vec = [v_.to(bf16) for v_ in (bias, gamma, beta)]
        alpha2 = alpha.to(bf16)
        our_ms = _time(lambda: ops.layer_norm(out2, x2, vec[0], vec[1], vec[2], row_count=rows, width=width, skip=skip2,
                                              alpha=alpha2, epsilon=1e-3), it)
        nbytes = rows * width * 2.0 * 3
        emit(op="layer_norm_skip", rows=rows, width=width, reference_ms=ref_ms, ours_ms=our_ms,
             reference_gbs=nbytes / ref_ms / 1e6, ours_gbs=nbytes / our_ms / 1e6)
        del x, skip, out, x2, skip2, out2
    status, detail = _lib.device_status()
    emit(op="device_status", status=status)


if __name__ == "__main__":
    main()
