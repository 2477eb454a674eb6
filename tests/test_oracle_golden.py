"""The CPU oracle against vectors produced by the reference's own test functions."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import bt4_oracle as O

# The reference functions return fp16; half an fp16 ulp at the magnitudes involved.
HALF_ATOL = 2e-3
HALF_RTOL = 1e-3


def _t(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(x))


@pytest.mark.parametrize(
    ("name", "activation"),
    [("ln_mish_noskip", "mish"), ("ln_swish_noskip", "swish"), ("ln_none_skip", "none"), ("ln_swish_wide", "swish")],
)
def test_layer_norm_matches_reference_function(golden, name, activation) -> None:
    skip = _t(golden[f"{name}/skip"]) if f"{name}/skip" in golden else None
    alpha = _t(golden[f"{name}/alpha"]) if f"{name}/alpha" in golden else None
    y = O.layer_norm(_t(golden[f"{name}/x"]), _t(golden[f"{name}/bias"]), _t(golden[f"{name}/gamma"]),
                     _t(golden[f"{name}/beta"]), activation, 1e-3, skip=skip, alpha=alpha)
    torch.testing.assert_close(y, _t(golden[f"{name}/y"]), rtol=HALF_RTOL, atol=HALF_ATOL)


@pytest.mark.parametrize("activation", ["mish", "swish", "none"])
def test_activations_match_reference_function(golden, activation) -> None:
    y = O.activate(_t(golden[f"act_{activation}/x"]), activation)
    torch.testing.assert_close(y, _t(golden[f"act_{activation}/y"]), rtol=0, atol=0)


def test_mish_branch_point_is_continuous() -> None:
    x = torch.tensor([-0.6001, -0.6, -0.5999])
    y = O.activate(x, "mish")
    expected = x * torch.tanh(torch.nn.functional.softplus(x))
    torch.testing.assert_close(y, expected, rtol=1e-5, atol=1e-6)


def test_softmax_random_rows(golden) -> None:
    y = O.softmax_64(_t(golden["softmax_random/qk"]), _t(golden["softmax_random/smolgen"]))
    torch.testing.assert_close(y, _t(golden["softmax_random/y"]), rtol=HALF_RTOL, atol=HALF_ATOL)
    torch.testing.assert_close(y.sum(dim=1), torch.ones(y.shape[0]), rtol=0, atol=1e-5)


def test_softmax_edge_rows(golden) -> None:
    y = O.softmax_64(_t(golden["softmax_edges/qk"]), _t(golden["softmax_edges/smolgen"]))
    torch.testing.assert_close(y, _t(golden["softmax_edges/y"]), rtol=HALF_RTOL, atol=HALF_ATOL, equal_nan=True)
    assert y[0, 0] == 1
    assert torch.equal(y[1, :2], torch.tensor([0.5, 0.5]))
    assert torch.equal(y[2], torch.full((64,), 1 / 64))
    assert torch.isnan(y[3]).all()
    assert torch.isnan(y[4]).all()
    assert torch.isfinite(y[5:]).all()


def test_softmax_shift_invariance() -> None:
    logits = (torch.arange(64, dtype=torch.float32) * 0.5).repeat(2, 1)
    zeros = torch.zeros_like(logits)
    torch.testing.assert_close(O.softmax_64(logits - 1024.0, zeros), O.softmax_64(logits, zeros), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["promo_random", "promo_exact"])
def test_promotion_logits(golden, name) -> None:
    y = O.promotion_logits(_t(golden[f"{name}/records"]), _t(golden[f"{name}/keys"]), _t(golden[f"{name}/w"]))
    exact = name == "promo_exact"
    if exact:  # the reference rounds its result to fp16; integers above 2048 are not all representable
        y = y.half().float()
    torch.testing.assert_close(y, _t(golden[f"{name}/y"]), rtol=0 if exact else 1e-3, atol=0 if exact else 4e-3)


def test_expand_planes_bit_order() -> None:
    masks = torch.tensor([[1, 1 << 62, -(1 << 63), 0, -1]], dtype=torch.int64)
    values = torch.tensor([[1.0, 0.5, 2.0, 3.0, 0.25]])
    planes = O.expand_planes(masks, values)
    assert planes.shape == (1, 5, 64)
    assert planes[0, 0, 0] == 1.0 and planes[0, 0, 1:].sum() == 0
    assert planes[0, 1, 62] == 0.5 and planes[0, 1].sum() == 0.5
    assert planes[0, 2, 63] == 2.0 and planes[0, 2].sum() == 2.0
    assert planes[0, 3].sum() == 0
    assert torch.equal(planes[0, 4], torch.full((64,), 0.25))


def test_policy_map_out_of_range_gives_zero() -> None:
    records = torch.arange(1, 11, dtype=torch.float32).reshape(2, 5)
    table = torch.tensor([4, -1, 0, 5, 2], dtype=torch.int32)
    out = O.policy_map(records, table)
    assert torch.equal(out, torch.tensor([[5.0, 0.0, 1.0, 0.0, 3.0], [10.0, 0.0, 6.0, 0.0, 8.0]]))


def test_policy_qk_leaves_promotion_slots_untouched() -> None:
    gen = torch.Generator().manual_seed(3)
    q, k = torch.randn((2, 64, 16), generator=gen), torch.randn((2, 64, 16), generator=gen)
    records = torch.full((2, 4288), -123.0)
    out = O.policy_qk(q, k, 0.25, records)
    assert torch.equal(out[:, 4096:], records[:, 4096:])
    torch.testing.assert_close(out[1, 5 * 64 + 9], 0.25 * (q[1, 5] * k[1, 9]).sum())


def test_body_qk_and_attention_v_head_interleave() -> None:
    gen = torch.Generator().manual_seed(4)
    b, h, d = 2, 3, 8
    q, k, v = (torch.randn((b, 64, h * d), generator=gen) for _ in range(3))
    s = O.body_qk(q, k, 0.5, h)
    torch.testing.assert_close(s[1, 2, 7, 9], 0.5 * (q[1, 7, 2 * d:3 * d] * k[1, 9, 2 * d:3 * d]).sum())
    p = torch.softmax(s, dim=-1)
    o = O.attention_v(p, v)
    torch.testing.assert_close(o[1, 7, 2 * d:3 * d], p[1, 2, 7] @ v[1, :, 2 * d:3 * d])
