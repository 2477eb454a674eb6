"""Outputs of the reference's own Triton kernels as the yardstick.

``tests/golden/reference_kernel_outputs.npz`` was produced by ``tests/golden/make_kernel_golden.py``: every
kernel of the reference's forward path launched on a B200 through its autotuner, as the reference's tests
launch it, on seeded inputs whose values are exact in fp16 and in bf16.  Here

* the CPU oracle is held to those outputs (no GPU needed): what the oracle restates is what the reference's
  kernels compute, not only what the reference's test helpers say they should;
* on a GPU, this library's kernel for the same operator gets the same numbers as bf16 and is held to the same
  outputs.

Tolerances: the reference rounds results to fp16 (relative step 2^-11), this library to bf16 (2^-8); layout,
gather and widening ops are exact on both sides.  The reference's GEMMs accumulate partly in fp16, so they get
the reference tests' own tolerance (rtol 1e-2, atol 2e-2, T/test_matmul.py:41-42).
"""

from __future__ import annotations

import pathlib

import numpy as np
import pytest
import torch

from oracle import bt4_oracle as O

GOLDEN = pathlib.Path(__file__).parent / "golden" / "reference_kernel_outputs.npz"
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ref() -> dict[str, torch.Tensor]:
    with np.load(GOLDEN) as data:
        return {key: torch.from_numpy(data[key]) for key in data.files}


def _case(ref: dict[str, torch.Tensor], name: str) -> dict[str, torch.Tensor]:
    prefix = name + "/"
    return {k[len(prefix):]: v for k, v in ref.items() if k.startswith(prefix)}


def _fp16_close(got: torch.Tensor, want: torch.Tensor, rtol: float = 2e-3, atol: float = 1e-3) -> None:
    torch.testing.assert_close(got.float(), want.float(), rtol=rtol, atol=atol, equal_nan=True)


# ------------------------------------------------------------------ the CPU oracle against the reference's kernels

def test_oracle_layout_and_gather_ops_equal_the_reference_kernels(ref) -> None:
    from lczero_triton_b200 import mapping_table

    c = _case(ref, "expand_planes")
    assert torch.equal(O.expand_planes(c["masks"], c["values"], torch.float16).float(), c["y"].float())
    c = _case(ref, "nchw_to_nhwc")
    assert torch.equal(O.nchw_to_nhwc(c["x"].reshape(3, 112, 64), 12).reshape(3, 8, 8, 12), c["y"])
    c = _case(ref, "preprocess_attention_body")
    assert torch.equal(O.preprocess_attention_body(c["planes"], c["encoding"]).float(), c["y"].float())
    c = _case(ref, "policy_map")
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    assert torch.equal(O.policy_map(c["records"], table).float(), c["y"].float())
    c = _case(ref, "copy_type_converted")
    assert torch.equal(c["x"].float(), c["y"])


def test_oracle_element_wise_ops_match_the_reference_kernels(ref) -> None:
    c = _case(ref, "input_gating")
    _fp16_close(O.input_gating(c["x"], c["mult"], c["add"]), c["y"])
    for act in ("none", "mish", "relu"):
        c = _case(ref, f"add_vectors_{act}")
        _fp16_close(O.add_vectors(c["x"], c["bias"], act), c["y"])
    for act in ("none", "mish"):
        c = _case(ref, f"add_bias_batched_{act}")
        _fp16_close(O.add_bias_batched(c["x"], c["bias"], act), c["y"])
    c = _case(ref, "fused_qkv_bias")
    for part in ("q", "k", "v"):
        _fp16_close(c[f"{part}_in"].float() + c[f"{part}_bias"].float(), c[part])


def test_oracle_contractions_match_the_reference_kernels(ref) -> None:
    # "deep" (K = 1024, results up to +-32 where one fp16 step is 2^-6): the reference's kernel accumulates
    # partial sums in fp16 (K/matmul.py:18), four steps of slack there.
    for name, atol in (("mid", 2e-2), ("tails", 2e-2), ("deep", 6.25e-2)):
        c = _case(ref, f"matmul_{name}")
        _fp16_close(O.matmul(c["a"], c["w"]), c["y"], rtol=1e-2, atol=atol)
    c = _case(ref, "fused_qkv_projection")
    for part in ("q", "k", "v"):
        _fp16_close(O.matmul(c["a"], c[f"w{part}"]), c[part], rtol=1e-2, atol=2e-2)
    c = _case(ref, "body_qk")
    _fp16_close(O.body_qk(c["q"], c["k"], float(c["scale"].float()), 4), c["y"], rtol=1e-2, atol=1e-2)
    c = _case(ref, "body_attention_v")
    _fp16_close(O.attention_v(c["p"], c["v"]), c["y"], rtol=1e-2, atol=1e-2)
    c = _case(ref, "policy_qk")
    want = O.policy_qk(c["q"], c["k"], float(c["scale"].float()), torch.full((3, 4288), -123.0))
    _fp16_close(want, c["y"], rtol=1e-2, atol=1e-2)
    assert torch.equal(c["y"][:, 4096:].float(), torch.full((3, 192), -123.0))  # promotion slots untouched


def test_oracle_softmax_layer_norm_and_promotion_match_the_reference_kernels(ref) -> None:
    c = _case(ref, "softmax_random")
    _fp16_close(O.softmax_64(c["qk"], c["smolgen"]), c["y"])
    c = _case(ref, "softmax_edges")
    got = O.softmax_64(c["qk"], c["smolgen"])
    assert torch.equal(torch.isnan(got), torch.isnan(c["y"].float()))
    _fp16_close(got, c["y"])
    for name, act in (("mish_noskip", "mish"), ("swish_noskip", "swish"), ("none_skip", "none"), ("swish_wide", "swish")):
        c = _case(ref, f"layer_norm_{name}")
        got = O.layer_norm(c["x"], c["bias"], c["gamma"], c["beta"], act, 1e-3, skip=c.get("skip"), alpha=c.get("alpha"))
        _fp16_close(got, c["y"], rtol=3e-3, atol=3e-3)
    c = _case(ref, "promotion_logits")
    want = c["records"].float().clone()
    want[:, 4096:] = O.promotion_logits(c["records"], c["keys"], c["w"])
    _fp16_close(want, c["y"], rtol=1e-2, atol=1e-2)
    assert torch.equal(c["y"][:, :4096], c["records"][:, :4096])  # in place: only the 192 promotion slots change


# ------------------------------------------------------------------ this library's kernels against the reference's

def _bf(x: torch.Tensor) -> torch.Tensor:
    """The same numbers as bf16 on the GPU (every golden input is exact in both formats)."""
    torch.testing.assert_close(x.float().to(BF16).float(), x.float(), rtol=0, atol=0, equal_nan=True)
    return x.float().to(BF16).cuda()


def _bf16_close(got: torch.Tensor, want: torch.Tensor, rtol: float = 8e-3, atol: float = 4e-3) -> None:
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=rtol, atol=atol, equal_nan=True)


@pytest.fixture(scope="module")
def ops():
    from lczero_triton_b200 import build, ops as module

    build.build()
    return module


@pytest.mark.gpu
def test_kernels_layout_and_gather_ops_equal_the_reference_kernels(ops, ref) -> None:
    from lczero_triton_b200 import mapping_table

    c = _case(ref, "expand_planes")
    out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
    ops.expand_planes(out, c["masks"].cuda(), c["values"].cuda())
    assert torch.equal(out.float().cpu(), c["y"].float())
    c = _case(ref, "nchw_to_nhwc")
    out = torch.empty((3, 64, 12), dtype=BF16, device="cuda")
    ops.nchw_to_nhwc(out, _bf(c["x"]), 3, 112, 12)
    assert torch.equal(out.float().cpu().reshape(3, 8, 8, 12), c["y"].float())
    c = _case(ref, "preprocess_attention_body")
    out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
    ops.preprocess_attention_body(out, _bf(c["planes"]), _bf(c["encoding"]), 3, 112, 40)
    assert torch.equal(out.float().cpu(), c["y"].float())
    c = _case(ref, "policy_map")
    table = torch.tensor(mapping_table.values(), dtype=torch.int32, device="cuda")
    out = torch.empty((3, 1858), dtype=BF16, device="cuda")
    ops.policy_map(out, _bf(c["records"]), table, 3)
    assert torch.equal(out.float().cpu(), c["y"].float())


@pytest.mark.gpu
def test_kernels_element_wise_ops_match_the_reference_kernels(ops, ref) -> None:
    c = _case(ref, "input_gating")
    out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
    ops.input_gating(out, _bf(c["x"]), _bf(c["mult"]), _bf(c["add"]), 3, 64, 96)
    _bf16_close(out, c["y"])
    for act in ("none", "mish", "relu"):
        c = _case(ref, f"add_vectors_{act}")
        out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
        ops.add_vectors(out, _bf(c["x"]), _bf(c["bias"]), act)
        _bf16_close(out, c["y"])
    for act in ("none", "mish"):
        c = _case(ref, f"add_bias_batched_{act}")
        out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
        ops.add_bias_batched(out, _bf(c["x"]), _bf(c["bias"]), 3, 7, 40, act)
        _bf16_close(out, c["y"])


@pytest.mark.gpu
def test_kernels_contractions_match_the_reference_kernels(ops, ref) -> None:
    for name, atol in (("mid", 3e-2), ("tails", 3e-2), ("deep", 1.25e-1)):  # bf16 step at +-32 is 2^-3
        c = _case(ref, f"matmul_{name}")
        m, k = c["a"].shape
        n = c["w"].shape[1]
        out = torch.empty((m, n), dtype=BF16, device="cuda")
        ops.matmul(out, _bf(c["a"]), _bf(c["w"]), m, n, k)
        _bf16_close(out, c["y"], rtol=1.6e-2, atol=atol)
    c = _case(ref, "fused_qkv_projection")
    outs = [torch.empty(c[p].shape, dtype=BF16, device="cuda") for p in ("q", "k", "v")]
    ops.fused_qkv_projection(*outs, _bf(c["a"]), _bf(c["wq"]), _bf(c["wk"]), _bf(c["wv"]), 70, 11, 13, 9, 24)
    for got, part in zip(outs, ("q", "k", "v")):
        _bf16_close(got, c[part], rtol=1.6e-2, atol=3e-2)
    c = _case(ref, "body_qk")
    out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
    ops.batched_matmul(out, _bf(c["q"]), _bf(c["k"]), "body_qk", 12, 64, 64, 32, 4, scale=_bf(c["scale"]))
    _bf16_close(out, c["y"], rtol=1.6e-2, atol=1.6e-2)
    c = _case(ref, "body_attention_v")
    out = torch.empty(c["y"].shape, dtype=BF16, device="cuda")
    ops.batched_matmul(out, _bf(c["p"]), _bf(c["v"]), "body_attention_v", 12, 64, 32, 64, 4)
    _bf16_close(out, c["y"], rtol=1.6e-2, atol=1.6e-2)
    c = _case(ref, "policy_qk")
    records = torch.full((3, 4288), -123.0, dtype=BF16, device="cuda")
    ops.batched_matmul(records, _bf(c["q"]), _bf(c["k"]), "policy_qk", 3, 64, 64, 128, 1, scale=_bf(c["scale"]))
    _bf16_close(records, c["y"], rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.gpu
def test_kernels_softmax_layer_norm_and_promotion_match_the_reference_kernels(ops, ref) -> None:
    for name in ("softmax_random", "softmax_edges"):
        c = _case(ref, name)
        rows = c["qk"].shape[0]
        out = torch.empty((rows, 64), dtype=BF16, device="cuda")
        ops.softmax_64(out, _bf(c["qk"]), _bf(c["smolgen"]), rows)
        assert torch.equal(torch.isnan(out.float().cpu()), torch.isnan(c["y"].float()))
        _bf16_close(out, c["y"], atol=2e-3)
    for name, act in (("mish_noskip", "mish"), ("swish_noskip", "swish"), ("none_skip", "none"), ("swish_wide", "swish")):
        c = _case(ref, f"layer_norm_{name}")
        rows, width = c["x"].shape
        out = torch.empty((rows, width), dtype=BF16, device="cuda")
        ops.layer_norm(out, _bf(c["x"]), _bf(c["bias"]), _bf(c["gamma"]), _bf(c["beta"]), row_count=rows, width=width,
                       activation=act, epsilon=1e-3, skip=_bf(c["skip"]) if "skip" in c else None,
                       alpha=_bf(c["alpha"]) if "alpha" in c else None)
        _bf16_close(out, c["y"], rtol=1e-2, atol=1e-2)
    c = _case(ref, "promotion_logits")
    records = _bf(c["records"]).clone()
    ops.promotion_logits(records, _bf(c["keys"]), _bf(c["w"]), 3, 48)
    _bf16_close(records, c["y"], rtol=1.6e-2, atol=1.6e-2)
    assert torch.equal(records[:, :4096].float().cpu(), c["records"][:, :4096].float())
