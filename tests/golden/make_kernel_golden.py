"""Generate ``tests/golden/reference_kernel_outputs.npz``: outputs of the reference's OWN Triton kernels.

Run on a machine with a GPU and the unmodified reference package installed under ``baseline/_ref``:

    python tests/golden/make_kernel_golden.py [output.npz]

Every kernel of the reference's forward path (``lczero_triton/bt4/kernels/*.py``) is launched through its
autotuner exactly as the reference's tests launch it, on small seeded inputs, and inputs and outputs are
stored.  The three generated ``*_pb2`` protobuf modules do not exist offline and are replaced by attribute
stubs, as in ``make_golden.py``; no kernel uses them.  The reference stores fp16 and this library bf16, so
every floating-point input value is chosen to be exactly representable in BOTH formats (rounded to bf16, tiny
magnitudes flushed to zero): the same numbers can be fed to either side.  Outputs are the reference's fp16
results.  ``tests/test_kernel_golden.py`` holds the CPU oracle to them (no GPU needed) and, on a GPU, this
library's kernels.
"""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path[:0] = [str(ROOT / "baseline" / "_ref"), str(ROOT / "tests" / "golden")]


def both(x: torch.Tensor) -> torch.Tensor:
    """fp16 tensor whose values are exact in bf16 too."""
    y = x.float().to(torch.bfloat16).float()
    y = torch.where(y.abs() < 2.0 ** -10, torch.zeros_like(y), y)
    return y.clamp(-60000.0, 60000.0).half()


def main(target: pathlib.Path) -> None:
    import make_golden

    make_golden._stub_generated_protobuf_modules()
    import triton
    from lczero_triton.bt4.kernels import (add_bias_batched, add_vectors, batched_matmul, copy_type_converted,
                                           expand_planes, fused_qkv, input_gating, layer_norm, mapping_table, matmul,
                                           nchw_to_nhwc, policy_map, preprocess_attention_body, promotion_logits,
                                           softmax_64)

    gen = torch.Generator().manual_seed(4321)
    out: dict[str, np.ndarray] = {}

    def rnd(*shape, scale=1.0):
        return both(torch.randn(shape, generator=gen) * scale)

    def put(name: str, **arrays) -> None:
        for key, value in arrays.items():
            if isinstance(value, torch.Tensor):
                value = value.detach().cpu().numpy()
            out[f"{name}/{key}"] = np.asarray(value)

    f16 = torch.float16
    dev = "cuda"

    # ---- expand_planes (expand_planes.py:26-42): out[p, sq] = bit sq of masks[p] ? fp16(values[p]) : 0
    planes = 112 * 2
    bits = torch.rand((planes, 64), generator=gen) < 0.4
    weights = torch.ones(64, dtype=torch.int64) << torch.arange(64, dtype=torch.int64)
    masks = (bits.to(torch.int64) * weights).sum(dim=-1)          # wraps into the sign bit for square 63
    values = both(torch.rand(planes, generator=gen) * 3.0).float()
    result = torch.empty((planes, 64), dtype=f16, device=dev)
    expand_planes._expand_planes_kernel[expand_planes._autotune_grid](
        result, masks.view(torch.uint64).to(dev), values.to(dev), planes, 64)
    put("expand_planes", masks=masks, values=values, y=result)

    # ---- nchw_to_nhwc (nchw_to_nhwc.py:26-44)
    x = rnd(3, 112, 8, 8)
    result = torch.empty((3, 8, 8, 12), dtype=f16, device=dev)
    nchw_to_nhwc._nchw_to_nhwc_kernel[nchw_to_nhwc._autotune_grid](result, x.to(dev), 3, 112, 12, 8, 8)
    put("nchw_to_nhwc", x=x, y=result)

    # ---- preprocess_attention_body (preprocess_attention_body.py:26-61)
    p_in, enc = rnd(3, 112, 64), rnd(3, 64, 40)
    result = torch.empty((3, 64, 152), dtype=f16, device=dev)
    preprocess_attention_body._preprocess_attention_body_kernel[preprocess_attention_body._autotune_grid](
        result, p_in.to(dev), enc.to(dev), 3, 64, 112, 40)
    put("preprocess_attention_body", planes=p_in, encoding=enc, y=result)

    # ---- input_gating (input_gating.py:26-51)
    x, mult, add = rnd(3, 64, 96), rnd(64, 96), rnd(64, 96)
    result = torch.empty((3, 64, 96), dtype=f16, device=dev)
    input_gating._input_gating_kernel[input_gating._autotune_grid](result, x.to(dev), mult.to(dev), add.to(dev), 3, 64, 96)
    put("input_gating", x=x, mult=mult, add=add, y=result)

    # ---- add_vectors (add_vectors.py:37-66) and add_bias_batched (add_bias_batched.py:35-66)
    for act in ("none", "mish", "relu"):
        x, bias = rnd(5, 64, 48, scale=1.5), rnd(48)
        result = torch.empty_like(x, device=dev)
        add_vectors._add_vectors_kernel[add_vectors._autotune_grid](result, x.to(dev), bias.to(dev), x.numel(), 48,
                                                                    add_vectors._ACTIVATIONS[act])
        put(f"add_vectors_{act}", x=x, bias=bias, y=result)
    for act in ("none", "mish"):
        x, bias = rnd(3, 7, 40, scale=1.5), rnd(3, 40)
        result = torch.empty_like(x, device=dev)
        add_bias_batched._add_bias_batched_kernel[add_bias_batched._autotune_grid](
            result, x.to(dev), bias.to(dev), 3, 7, 40, add_bias_batched._ACTIVATIONS[act])
        put(f"add_bias_batched_{act}", x=x, bias=bias, y=result)

    # ---- matmul (matmul.py:57-116): [K, N] weights; the BT4 head shape, a mid shape and the reference's tail case
    for name, m, k, n in (("mid", 200, 192, 160), ("tails", 7, 37, 11), ("deep", 70, 1024, 96)):
        a, w = rnd(m, k, scale=0.5), rnd(k, n, scale=0.5)
        result = torch.empty((m, n), dtype=f16, device=dev)
        matmul._matmul_kernel[matmul._autotune_grid](result, a.to(dev), w.to(dev), m, n, k)
        put(f"matmul_{name}", a=a, w=w, y=result)

    # ---- fused_qkv_projection / fused_qkv_bias (fused_qkv.py:30-183), the reference test's widths 11 / 13 / 9
    m, k = 70, 24
    a = rnd(m, k, scale=0.5)
    ws = [rnd(k, n, scale=0.5) for n in (11, 13, 9)]
    outs = [torch.empty((m, n), dtype=f16, device=dev) for n in (11, 13, 9)]
    fused_qkv._fused_qkv_projection_kernel[fused_qkv._projection_autotune_grid](
        outs[0], outs[1], outs[2], a.to(dev), ws[0].to(dev), ws[1].to(dev), ws[2].to(dev), m, 11, 13, 9, k)
    put("fused_qkv_projection", a=a, wq=ws[0], wk=ws[1], wv=ws[2], q=outs[0], k=outs[1], v=outs[2])
    xs = [rnd(9, n) for n in (11, 13, 9)]
    bs = [rnd(n) for n in (11, 13, 9)]
    outs = [torch.empty((9, n), dtype=f16, device=dev) for n in (11, 13, 9)]
    fused_qkv._fused_qkv_bias_kernel[fused_qkv._bias_autotune_grid](
        outs[0], xs[0].to(dev), bs[0].to(dev), outs[1], xs[1].to(dev), bs[1].to(dev), outs[2], xs[2].to(dev), bs[2].to(dev),
        9, 11, 13, 9)
    put("fused_qkv_bias", q_in=xs[0], k_in=xs[1], v_in=xs[2], q_bias=bs[0], k_bias=bs[1], v_bias=bs[2], q=outs[0], k=outs[1],
        v=outs[2])

    # ---- batched_matmul (batched_matmul.py:68-210): body_qk, body_attention_v, policy_qk
    samples, heads, depth = 3, 4, 32
    q, kk = rnd(samples, 64, heads * depth, scale=0.5), rnd(samples, 64, heads * depth, scale=0.5)
    scale = both(torch.tensor([0.173]))
    scores = torch.empty((samples, heads, 64, 64), dtype=f16, device=dev)
    batched_matmul._qk_kernel[batched_matmul._autotune_grid](
        scores, q.to(dev), kk.to(dev), scale.to(dev), batched_matmul._OPERATIONS["body_qk"], samples * heads, heads, 64, 64,
        depth, 64 * 64)
    put("body_qk", q=q, k=kk, scale=scale, y=scores)
    probs = both(torch.softmax(torch.randn((samples, heads, 64, 64), generator=gen), dim=-1))
    v = rnd(samples, 64, heads * depth)
    merged = torch.empty((samples, 64, heads * depth), dtype=f16, device=dev)
    batched_matmul._attention_v_kernel[batched_matmul._autotune_grid](
        merged, probs.to(dev), v.to(dev), samples * heads, heads, 64, depth, 64)
    put("body_attention_v", p=probs, v=v, y=merged)
    width = 128
    qp, kp = rnd(samples, 64, width, scale=0.3), rnd(samples, 64, width, scale=0.3)
    pscale = both(torch.tensor([width ** -0.5]))
    records = torch.full((samples, 4288), -123.0, dtype=f16, device=dev)
    batched_matmul._qk_kernel[batched_matmul._autotune_grid](
        records, qp.to(dev), kp.to(dev), pscale.to(dev), batched_matmul._OPERATIONS["policy_qk"], samples, 1, 64, 64, width,
        4288)
    put("policy_qk", q=qp, k=kp, scale=pscale, y=records)

    # ---- softmax_64 (softmax_64.py:45-71): random rows and the non-finite rows of its test
    qk, sg = rnd(48, 64, scale=3.0), rnd(48, 64, scale=2.0)
    result = torch.empty((48, 64), dtype=f16, device=dev)
    softmax_64._softmax_64_kernel[softmax_64._autotune_grid](result, qk.to(dev), sg.to(dev), 48)
    put("softmax_random", qk=qk, smolgen=sg, y=result)
    qk = torch.zeros((8, 64), dtype=f16)
    sg = torch.zeros_like(qk)
    qk[0, 0] = torch.inf
    qk[1, :2] = torch.inf
    qk[2] = -torch.inf
    qk[3, 0] = torch.inf
    sg[3, 0] = -torch.inf
    qk[4, 7] = torch.nan
    qk[5, 0] = 65280.0
    sg[5, 0] = 65280.0
    qk[6, 0] = -65280.0
    sg[6, 0] = -65280.0
    qk[7] = both(torch.linspace(-20.0, 20.0, 64))
    sg[7] = both(torch.linspace(3.0, -4.0, 64))
    result = torch.empty((8, 64), dtype=f16, device=dev)
    softmax_64._softmax_64_kernel[softmax_64._autotune_grid](result, qk.to(dev), sg.to(dev), 8)
    put("softmax_edges", qk=qk, smolgen=sg, y=result)

    # ---- layer_norm (layer_norm.py:37-161): the four variants the graph uses
    for name, rows, width, act, has_skip in (("mish_noskip", 6, 128, "mish", False), ("swish_noskip", 5, 256, "swish", False),
                                              ("none_skip", 7, 1024, "none", True), ("swish_wide", 2, 8192, "swish", False)):
        x, bias = rnd(rows, width), rnd(width, scale=0.5)
        gamma, beta = both(1.0 + torch.randn(width, generator=gen) * 0.1), rnd(width, scale=0.1)
        result = torch.empty((rows, width), dtype=f16, device=dev)
        block = triton.next_power_of_2(width)
        if has_skip:
            skip, alpha = rnd(rows, width), both(torch.tensor([0.4272]))
            layer_norm._layer_norm_skip_kernel[layer_norm._autotune_grid](
                result, x.to(dev), bias.to(dev), skip.to(dev), gamma.to(dev), beta.to(dev), alpha.to(dev), rows, width, 1e-3,
                layer_norm._ACTIVATIONS[act], block)
            put(f"layer_norm_{name}", x=x, bias=bias, skip=skip, alpha=alpha, gamma=gamma, beta=beta, y=result)
        else:
            layer_norm._layer_norm_kernel[layer_norm._autotune_grid](
                result, x.to(dev), bias.to(dev), gamma.to(dev), beta.to(dev), rows, width, 1e-3,
                layer_norm._ACTIVATIONS[act], block)
            put(f"layer_norm_{name}", x=x, bias=bias, gamma=gamma, beta=beta, y=result)

    # ---- promotion_logits (promotion_logits.py:67-145), in place on the records
    rec, keys, w = rnd(3, 4288), rnd(3, 64, 48, scale=0.5), rnd(48, 4, scale=0.5)
    work = rec.clone().to(dev)
    promotion_logits._promotion_logits_kernel[promotion_logits._autotune_grid](work, keys.to(dev), w.to(dev), 3, 48)
    put("promotion_logits", records=rec, keys=keys, w=w, y=work)

    # ---- policy_map (policy_map.py:28-49) with the reference's table, and copy_type_converted
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    rec = rnd(3, 4288)
    gathered = torch.empty((3, 1858), dtype=f16, device=dev)
    policy_map._policy_map_kernel[policy_map._autotune_grid](gathered, rec.to(dev), table.to(dev), 3, 4288, 1858)
    put("policy_map", records=rec, y=gathered)
    wide = torch.empty(3 * 1858, dtype=torch.float32, device=dev)
    copy_type_converted._copy_type_converted_kernel[copy_type_converted._autotune_grid](wide, gathered.reshape(-1), 3 * 1858)
    put("copy_type_converted", x=gathered.reshape(-1), y=wide)

    torch.cuda.synchronize()
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays, triton {triton.__version__})")


if __name__ == "__main__":
    main(pathlib.Path(sys.argv[1]) if len(sys.argv) > 1 else pathlib.Path(__file__).with_name("reference_kernel_outputs.npz"))
