"""GPU parity of every per-op entry point (through the C ABI) against the CPU oracle.

Inputs are bf16 values; the oracle evaluates in fp32 on the same values, and the result is
compared after the kernel's single rounding to bf16 (relative step 2^-8), so the tolerances
are one bf16 ulp plus a small absolute term, tighter than the reference's own fp16 test
tolerances scaled to bf16.  Layout / gather / convert ops are exact.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import bt4_oracle as O

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16
RTOL, ATOL = 8e-3, 4e-3  # one bf16 ulp is 2^-8 = 3.9e-3 relative


@pytest.fixture(scope="module")
def ops():
    from lczero_triton_b200 import build, ops as module

    build.build()
    return module


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(BF16)


def _dev(x: torch.Tensor) -> torch.Tensor:
    return x.cuda()


def _close(got: torch.Tensor, want: torch.Tensor, rtol: float = RTOL, atol: float = ATOL, **kw) -> None:
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=rtol, atol=atol, **kw)


def _masks(batch: int, seed: int):
    from lczero_triton_b200.synthetic import synthetic_planes

    return synthetic_planes(batch, seed)


# ------------------------------------------------------------------ layout ops (exact)

@pytest.mark.parametrize("batch", [1, 3, 32])
def test_expand_planes(ops, batch) -> None:
    masks, values = _masks(batch, 5)
    values[:, 3] = 0.3  # not representable in bf16: the cast happens before the select
    out = torch.empty((batch, 112, 64), dtype=BF16, device="cuda")
    ops.expand_planes(out, _dev(masks), _dev(values))
    want = O.expand_planes(masks, values, BF16)
    assert torch.equal(out.float().cpu(), want)


def test_expand_planes_bit_order(ops) -> None:
    masks = torch.tensor([[1, 1 << 62, -(1 << 63), 0, -1]], dtype=torch.int64)
    values = torch.tensor([[1.0, 0.5, 2.0, 3.0, 0.25]])
    out = torch.empty((1, 5, 64), dtype=BF16, device="cuda")
    ops.expand_planes(out, _dev(masks), _dev(values))
    got = out.float().cpu()
    assert got[0, 0, 0] == 1 and got[0, 0, 1:].sum() == 0
    assert got[0, 1, 62] == 0.5 and got[0, 2, 63] == 2.0 and got[0, 3].sum() == 0
    assert torch.equal(got[0, 4], torch.full((64,), 0.25))


def test_nchw_to_nhwc(ops) -> None:
    planes = _bf(torch.randn((5, 112, 64), generator=_gen(1)))
    out = torch.empty((5, 64, 12), dtype=BF16, device="cuda")
    ops.nchw_to_nhwc(out, _dev(planes), 5, 112, 12)
    assert torch.equal(out.cpu(), O.nchw_to_nhwc(planes, 12))


def test_preprocess_attention_body(ops) -> None:
    planes = _bf(torch.randn((3, 112, 64), generator=_gen(2)))
    enc = _bf(torch.randn((3, 64, 40), generator=_gen(3)))
    out = torch.empty((3, 64, 152), dtype=BF16, device="cuda")
    ops.preprocess_attention_body(out, _dev(planes), _dev(enc), 3, 112, 40)
    assert torch.equal(out.cpu(), O.preprocess_attention_body(planes, enc))


@pytest.mark.parametrize("enc", [64, 512, 20])
def test_fused_embedding_front_end(ops, enc) -> None:
    batch = 7
    masks, values = _masks(batch, 11)
    position = _bf(torch.randn((batch, 64, enc), generator=_gen(4)))
    planes = O.expand_planes(masks, values, BF16)
    pos_in = torch.empty((batch, 768), dtype=BF16, device="cuda")
    ops.embed_position_input(pos_in, _dev(masks), _dev(values), batch)
    assert torch.equal(pos_in.float().cpu(), O.nchw_to_nhwc(planes, 12).reshape(batch, 768))
    emb_in = torch.empty((batch * 64, 112 + enc), dtype=BF16, device="cuda")
    ops.embed_concat(emb_in, _dev(masks), _dev(values), _dev(position), batch, enc)
    want = O.preprocess_attention_body(planes, position.float()).reshape(batch * 64, 112 + enc)
    assert torch.equal(emb_in.float().cpu(), want)


def test_copy_type_converted(ops) -> None:
    x = _bf(torch.randn(1000, generator=_gen(5)))
    out = torch.empty(1000, dtype=torch.float32, device="cuda")
    ops.copy_type_converted(out, _dev(x))
    assert torch.equal(out.cpu(), x.float())


def test_policy_map_with_out_of_range_entries(ops) -> None:
    records = _bf(torch.randn((3, 4288), generator=_gen(6)))
    table = torch.randint(0, 4288, (1858,), generator=_gen(7), dtype=torch.int32)
    table[5], table[77], table[1857] = -1, 4288, 99999
    out = torch.empty((3, 1858), dtype=BF16, device="cuda")
    ops.policy_map(out, _dev(records), _dev(table), 3)
    want = O.policy_map(records.float(), table)
    assert torch.equal(out.float().cpu(), want)
    assert out[:, 5].abs().sum() == 0 and out[:, 77].abs().sum() == 0 and out[:, 1857].abs().sum() == 0


# ------------------------------------------------------------------ element-wise ops

def test_input_gating(ops) -> None:
    x = _bf(torch.randn((4, 64, 96), generator=_gen(8)))
    mult, add = _bf(torch.randn((64, 96), generator=_gen(9))), _bf(torch.randn((64, 96), generator=_gen(10)))
    out = _dev(x).clone()
    ops.input_gating(out, out, _dev(mult), _dev(add), 4, 64, 96)  # in place, as the graph does
    _close(out, O.input_gating(x, mult, add))


@pytest.mark.parametrize("activation", ["none", "mish", "relu"])
def test_add_vectors(ops, activation) -> None:
    x = _bf(torch.randn((6, 37), generator=_gen(11)) * 2)
    x[0, :3] = torch.tensor([-0.6001, -0.6, -0.5999]).to(BF16)
    bias = _bf(torch.randn(37, generator=_gen(12)))
    out = torch.empty_like(x, device="cuda")
    ops.add_vectors(out, _dev(x), _dev(bias), activation)
    _close(out, O.add_vectors(x, bias, activation))


@pytest.mark.parametrize("activation", ["none", "mish"])
def test_add_bias_batched(ops, activation) -> None:
    x = _bf(torch.randn((3, 5, 24), generator=_gen(13)))
    bias = _bf(torch.randn((3, 24), generator=_gen(14)))
    out = _dev(x).clone()
    ops.add_bias_batched(out, out, _dev(bias), 3, 5, 24, activation)
    _close(out, O.add_bias_batched(x, bias, activation))


@pytest.mark.parametrize(("m", "k", "widths"), [(5, 24, (11, 13, 9)), (70, 7, (11, 13, 9)), (300, 1024, (1024, 1024, 1024)),
                                               (8192, 1024, (1024, 1024, 1024))])
def test_fused_qkv_projection_matches_three_matmuls(ops, m, k, widths) -> None:
    """fused_qkv.py:30-123: three projections of one input with separate weights, widths and outputs
    (the reference's test uses widths 11 / 13 / 9, tests/test_fused_qkv.py:36-75)."""
    a = _bf(torch.randn((m, k), generator=_gen(140)) * 0.5)
    ws = [_bf(torch.randn((k, n), generator=_gen(141 + i)) * 0.5) for i, n in enumerate(widths)]
    outs = [torch.full((m, n), 7.0, dtype=BF16, device="cuda") for n in widths]
    ops.fused_qkv_projection(outs[0], outs[1], outs[2], _dev(a), *[_dev(w) for w in ws], m, *widths, k)
    atol = 0.25 * (k ** 0.5) * 2 ** -8 * 2 + 1e-3
    for out, w in zip(outs, ws):
        _close(out, O.matmul(a, w), rtol=8e-3, atol=atol)


def test_fused_qkv_bias_with_three_widths(ops) -> None:
    rows = 9
    tensors = [_bf(torch.randn((rows, w), generator=_gen(20 + i))) for i, w in enumerate((11, 13, 9))]
    biases = [_bf(torch.randn(w, generator=_gen(30 + i))) for i, w in enumerate((11, 13, 9))]
    dev = [_dev(t).clone() for t in tensors]
    ops.fused_qkv_bias(dev[0], _dev(biases[0]), dev[1], _dev(biases[1]), dev[2], _dev(biases[2]), rows)
    for got, x, b in zip(dev, tensors, biases):
        _close(got, x.float() + b.float())


# ------------------------------------------------------------------ layer norm

@pytest.mark.parametrize(
    ("name", "activation"),
    [("ln_mish_noskip", "mish"), ("ln_swish_noskip", "swish"), ("ln_none_skip", "none"), ("ln_swish_wide", "swish")],
)
def test_layer_norm_on_reference_vectors(ops, golden, name, activation) -> None:
    x, bias = _bf(torch.from_numpy(golden[f"{name}/x"])), _bf(torch.from_numpy(golden[f"{name}/bias"]))
    gamma, beta = _bf(torch.from_numpy(golden[f"{name}/gamma"])), _bf(torch.from_numpy(golden[f"{name}/beta"]))
    skip = _bf(torch.from_numpy(golden[f"{name}/skip"])) if f"{name}/skip" in golden else None
    alpha = _bf(torch.from_numpy(golden[f"{name}/alpha"])) if f"{name}/alpha" in golden else None
    rows, width = x.shape
    out = torch.empty_like(x, device="cuda")
    ops.layer_norm(out, _dev(x), _dev(bias), _dev(gamma), _dev(beta), row_count=rows, width=width,
                   activation=activation, skip=None if skip is None else _dev(skip),
                   alpha=None if alpha is None else _dev(alpha))
    want = O.layer_norm(x, bias, gamma, beta, activation, 1e-3, skip=skip, alpha=alpha)
    _close(out, want, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("width", [8, 128, 256, 768, 1024, 1536, 2048, 100, 8192])
@pytest.mark.parametrize("has_skip", [False, True])
def test_layer_norm_widths(ops, width, has_skip) -> None:
    rows = 19
    x = _bf(torch.randn((rows, width), generator=_gen(40)) * 1.5 + 0.5)
    bias, gamma = _bf(torch.randn(width, generator=_gen(41)) * 0.3), _bf(1 + 0.1 * torch.randn(width, generator=_gen(42)))
    beta = _bf(0.1 * torch.randn(width, generator=_gen(43)))
    skip = _bf(torch.randn((rows, width), generator=_gen(44))) if has_skip else None
    alpha = _bf(torch.tensor([0.4273])) if has_skip else None
    out = torch.empty_like(x, device="cuda")
    ops.layer_norm(out, _dev(x), _dev(bias), _dev(gamma), _dev(beta), row_count=rows, width=width,
                   activation="mish", skip=None if skip is None else _dev(skip),
                   alpha=None if alpha is None else _dev(alpha))
    _close(out, O.layer_norm(x, bias, gamma, beta, "mish", 1e-3, skip=skip, alpha=alpha), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("alias", ["input", "skip"])
def test_layer_norm_in_place(ops, alias) -> None:
    rows, width = 33, 1024
    x, skip = _bf(torch.randn((rows, width), generator=_gen(45))), _bf(torch.randn((rows, width), generator=_gen(46)))
    bias, gamma, beta = (_bf(torch.randn(width, generator=_gen(47 + i)) * 0.2) for i in range(3))
    alpha = _bf(torch.tensor([0.5]))
    dx, ds = _dev(x).clone(), _dev(skip).clone()
    out = dx if alias == "input" else ds
    ops.layer_norm(out, dx, _dev(bias), _dev(gamma), _dev(beta), row_count=rows, width=width, skip=ds,
                   alpha=_dev(alpha))
    _close(out, O.layer_norm(x, bias, gamma, beta, "none", 1e-3, skip=skip, alpha=alpha), rtol=1e-2, atol=1e-2)


def test_layer_norm_quantised_output_matches_quantiser(ops) -> None:
    from oracle import int8_oracle

    rows, width = 21, 1024
    x = _bf(torch.randn((rows, width), generator=_gen(50)))
    bias, gamma, beta = (_bf(torch.randn(width, generator=_gen(51 + i)) * 0.2) for i in range(3))
    out = torch.empty_like(x, device="cuda")
    q = torch.empty((rows, width), dtype=torch.int8, device="cuda")
    s = torch.empty((rows,), dtype=torch.float32, device="cuda")
    ops.layer_norm(out, _dev(x), _dev(bias), _dev(gamma), _dev(beta), row_count=rows, width=width, q_out=q, q_scale=s)
    want_q, want_s = int8_oracle.quantize_rows(out.cpu())  # the quantiser sees the stored bf16 rows
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu(), want_q)


@pytest.mark.parametrize(("rows", "width"), [(5, 1024), (3, 1536), (4, 40), (2, 8)])
def test_quantize_rows_is_bit_exact(ops, rows, width) -> None:
    from oracle import int8_oracle

    x = _bf(torch.randn((rows, width), generator=_gen(55)) * 3)
    x[0] = 0  # all-zero row: scale 1, zeros out
    q = torch.empty((rows, width), dtype=torch.int8, device="cuda")
    s = torch.empty((rows,), dtype=torch.float32, device="cuda")
    ops.quantize_rows(q, s, _dev(x), rows, width)
    want_q, want_s = int8_oracle.quantize_rows(x)
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu(), want_q)
    assert s[0] == 1 and q[0].abs().sum() == 0


@pytest.mark.parametrize(("rows", "width"), [(300, 1024), (77, 768), (9, 2048), (5, 64)])
def test_normalize_quantize_rows_from_partial_sums(ops, rows, width) -> None:
    """Deferred-LayerNorm rows to int8: mean / variance come from the 64-column partial sums a residual GEMM
    writes; the result must be the quantisation of the bf16-rounded LayerNorm (layer_norm.py:57-87 semantics)."""
    from oracle import int8_oracle

    z = _bf(torch.randn((rows, width), generator=_gen(56)) * 1.5 + 0.1)
    gamma = _bf(1.0 + 0.1 * torch.randn(width, generator=_gen(57)))
    beta = _bf(0.1 * torch.randn(width, generator=_gen(58)))
    groups = z.float().reshape(rows, width // 64, 64)
    stats = torch.stack((groups.sum(dim=2), (groups * groups).sum(dim=2)), dim=2).permute(1, 0, 2).contiguous()
    q = torch.empty((rows, width), dtype=torch.int8, device="cuda")
    s = torch.empty((rows,), dtype=torch.float32, device="cuda")
    ops.normalize_quantize_rows(q, s, _dev(z), stats.cuda(), _dev(gamma), _dev(beta), rows, width, 1e-3)
    zf = z.double()
    mean = zf.mean(dim=1, keepdim=True)
    var = (zf * zf).mean(dim=1, keepdim=True) - mean * mean
    y = ((zf - mean) / torch.sqrt(var + 1e-3) * gamma.double() + beta.double()).float().to(torch.bfloat16)
    want_q, want_s = int8_oracle.quantize_rows(y)
    # fp32 against fp64 statistics: a bf16 rounding may flip here and there, never more than one step
    torch.testing.assert_close(s.cpu(), want_s, rtol=1e-2, atol=0)
    diff = (q.cpu().int() - want_q.int()).abs()
    assert int(diff.max()) <= 1 and float((diff == 0).float().mean()) > 0.995


# ------------------------------------------------------------------ softmax and attention

def test_softmax_random_rows(ops, golden) -> None:
    qk, sg = _bf(torch.from_numpy(golden["softmax_random/qk"])), _bf(torch.from_numpy(golden["softmax_random/smolgen"]))
    out = torch.empty_like(qk, device="cuda")
    ops.softmax_64(out, _dev(qk), _dev(sg), qk.shape[0])
    _close(out, O.softmax_64(qk, sg), rtol=RTOL, atol=2e-3)
    torch.testing.assert_close(out.float().sum(dim=1).cpu(), torch.ones(qk.shape[0]), rtol=0, atol=1e-2)


def test_softmax_edge_rows(ops, golden) -> None:
    qk, sg = _bf(torch.from_numpy(golden["softmax_edges/qk"])), _bf(torch.from_numpy(golden["softmax_edges/smolgen"]))
    out = torch.empty_like(qk, device="cuda")
    ops.softmax_64(out, _dev(qk), _dev(sg), 8)
    got = out.float().cpu()
    _close(out, O.softmax_64(qk, sg), rtol=RTOL, atol=2e-3, equal_nan=True)
    assert got[0, 0] == 1
    assert torch.equal(got[1, :2], torch.tensor([0.5, 0.5]))
    assert torch.equal(got[2], torch.full((64,), 1 / 64))
    assert torch.isnan(got[3]).all() and torch.isnan(got[4]).all()
    assert torch.isfinite(got[5:]).all()


def test_softmax_in_place_and_shift_invariance(ops) -> None:
    """A large common offset does not destabilise the softmax (test_softmax_64.py:154-165); the offset
    comes in through the second operand so that both operands stay exactly representable in bf16."""
    logits = _bf((torch.arange(64, dtype=torch.float32) * 0.5).repeat(2, 1))
    zeros = torch.zeros_like(logits, device="cuda")
    offset = torch.full_like(logits, -1024.0, device="cuda")
    base, shifted = _dev(logits).clone(), _dev(logits).clone()
    ops.softmax_64(base, base, zeros, 2)  # in place, as the graph does
    ops.softmax_64(shifted, shifted, offset, 2)
    assert torch.equal(shifted, base)
    _close(base, torch.softmax(logits.float(), dim=1), rtol=RTOL, atol=2e-3)


# Even head counts run the tcgen05 kernel (pairs of heads); odd head counts run the mma.sync kernel,
# at each of its three heads-per-CTA settings (4, 8, 16: chosen from batch x heads against the SM count).
@pytest.mark.parametrize(("batch", "heads"), [(1, 4), (2, 32), (3, 24), (64, 32), (2, 3), (7, 5), (3, 31),
                                              (800, 31), (2600, 31)])
def test_fused_attention_matches_three_step_oracle(ops, batch, heads) -> None:
    d = heads * 32
    q, k, v = (_bf(torch.randn((batch, 64, d), generator=_gen(60 + i))) for i in range(3))
    bias = _bf(torch.randn((batch, heads, 64, 64), generator=_gen(63)) * 0.5)
    scale = 32 ** -0.5
    out = torch.empty((batch, 64, d), dtype=BF16, device="cuda")
    ops.attention(out, _dev(q), _dev(k), _dev(v), _dev(bias), scale, batch, heads)
    probs = O.softmax_64(O.body_qk(q, k, scale, heads), bias)
    want = O.attention_v(probs, v)
    _close(out, want, rtol=2e-2, atol=2e-2)  # P is rounded to bf16 before P.V, as the reference rounds it to fp16


def test_fused_attention_strided_operands_and_no_bias(ops) -> None:
    batch, heads, d = 5, 8, 256
    qkv = _bf(torch.randn((batch * 64, 3 * d), generator=_gen(64)))
    dq = _dev(qkv)
    out = torch.empty((batch * 64, d), dtype=BF16, device="cuda")
    ops.attention(out, dq[:, :d], dq[:, d:2 * d], dq[:, 2 * d:], None, 0.25, batch, heads,
                  ldq=3 * d, ldk=3 * d, ldv=3 * d, ldo=d)
    q, k, v = (qkv[:, i * d:(i + 1) * d].reshape(batch, 64, d) for i in range(3))
    probs = O.softmax_64(O.body_qk(q, k, 0.25, heads), torch.zeros((batch, heads, 64, 64)))
    _close(out.reshape(batch, 64, d), O.attention_v(probs, v), rtol=2e-2, atol=2e-2)


def test_fused_attention_nan_and_infinite_bias_rows(ops) -> None:
    batch, heads, d = 1, 4, 128
    q, k, v = (_bf(torch.randn((batch, 64, d), generator=_gen(65 + i))) for i in range(3))
    bias = torch.zeros((batch, heads, 64, 64))
    bias[0, 0, 3, 5] = float("inf")   # one +inf -> that key takes all the weight
    bias[0, 1, 7, :] = float("-inf")  # all -inf -> clamped, ordinary softmax of the scores
    bias[0, 2, 9, 1] = float("nan")   # NaN poisons the row
    bias = _bf(bias)
    out = torch.empty((batch, 64, d), dtype=BF16, device="cuda")
    ops.attention(out, _dev(q), _dev(k), _dev(v), _dev(bias), 0.2, batch, heads)
    want = O.attention_v(O.softmax_64(O.body_qk(q, k, 0.2, heads), bias), v)
    got = out.float().cpu()
    assert torch.isnan(got[0, 9, 64:96]).all() and torch.isnan(want[0, 9, 64:96]).all()
    finite = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), finite)
    torch.testing.assert_close(got[finite], want[finite], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got[0, 3, :32], v.float()[0, 5, :32], rtol=1e-2, atol=1e-2)


def test_fused_attention_rows_at_the_edges_of_the_clamp_range(ops) -> None:
    """softmax_64 clamps scores to +-131008 (softmax_64.py:45-71).  Rows far inside the range skip the
    clamp in the fused kernel; rows whose maximum sits at either end of the range must still agree with
    the oracle: a row pushed below the lower end flattens, a row with finite huge values saturates."""
    batch, heads, d = 1, 4, 128
    q, k, v = (_bf(torch.randn((batch, 64, d), generator=_gen(75 + i))) for i in range(3))
    bias = torch.zeros((batch, heads, 64, 64))
    bias[0, 0, 2, :] = -131072.0          # every score below the range: clamped to one value plus q.k
    bias[0, 0, 4, :] = -131072.0
    bias[0, 0, 4, 9] = -130048.0          # ... except one key just inside it, which takes all the weight
    bias[0, 1, 6, :] = -130944.0 + 0.0    # maximum within 256 of the lower end (rounds to a bf16 value)
    bias[0, 1, 6, 11] = -131072.0
    bias[0, 2, 8, 3] = 3.0e38             # finite, far above the range: clamped, the key still wins
    bias[0, 3, 10, :] = 65280.0           # large but inside: ordinary softmax of the scores
    bias = _bf(bias)
    out = torch.empty((batch, 64, d), dtype=BF16, device="cuda")
    ops.attention(out, _dev(q), _dev(k), _dev(v), _dev(bias), 0.2, batch, heads)
    want = O.attention_v(O.softmax_64(O.body_qk(q, k, 0.2, heads), bias), v)
    got = out.float().cpu()
    assert torch.isfinite(got).all() and torch.isfinite(want).all()
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got[0, 4, :32], v.float()[0, 9, :32], rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(got[0, 8, 64:96], v.float()[0, 3, 64:96], rtol=1e-2, atol=1e-2)


def test_fused_attention_non_finite_value_rows(ops) -> None:
    """A non-finite element of V.  The reference multiplies each head's probabilities by that head's V
    only (batched_matmul.py:150-210), so the damage stays inside the head: the mma.sync kernel (odd head
    count) must match the oracle exactly in where the NaNs are.  The tcgen05 kernel stacks two heads
    into one 128-row product with zero off-diagonal probability blocks, and 0 x inf = NaN also reaches
    the OTHER head of the pair (heads 2j and 2j+1) - the documented deviation; heads outside the pair
    stay clean."""
    batch, d_head = 2, 32
    for heads in (3, 4):
        d = heads * d_head
        q, k, v = (_bf(torch.randn((batch, 64, d), generator=_gen(85 + i))) for i in range(3))
        v[1, 17, 1 * d_head + 5] = float("inf")  # head 1 of position 1
        bias = _bf(torch.randn((batch, heads, 64, 64), generator=_gen(88)) * 0.5)
        out = torch.empty((batch, 64, d), dtype=BF16, device="cuda")
        ops.attention(out, _dev(q), _dev(k), _dev(v), _dev(bias), 0.2, batch, heads)
        want = O.attention_v(O.softmax_64(O.body_qk(q, k, 0.2, heads), bias), v)
        got = out.float().cpu()
        assert not torch.isfinite(want[1, :, d_head + 5]).any()      # the oracle: that output column of head 1
        assert torch.isfinite(want[1, :, :d_head]).all()
        clean = torch.ones_like(want, dtype=torch.bool)
        clean[1, :, d_head:2 * d_head] = False                         # head 1 itself
        if heads % 2 == 0:
            clean[1, :, :d_head] = False                               # its pair partner (tcgen05 kernel only)
            assert not torch.isfinite(got[1, :, d_head + 5]).any()
        else:
            assert torch.equal(torch.isfinite(got), torch.isfinite(want))
        assert torch.isfinite(got[clean]).all()
        torch.testing.assert_close(got[clean], want[clean], rtol=2e-2, atol=2e-2)


# ------------------------------------------------------------------ batched matmuls

def test_body_qk_matches_explicit_head_reshape(ops) -> None:
    samples, heads, depth = 9, 32, 32
    q = _bf(torch.randn((samples, 64, heads * depth), generator=_gen(70)) * 0.5)
    k = _bf(torch.randn((samples, 64, heads * depth), generator=_gen(71)) * 0.5)
    scale = _bf(torch.tensor([0.173]))
    out = torch.empty((samples, heads, 64, 64), dtype=BF16, device="cuda")
    ops.batched_matmul(out, _dev(q), _dev(k), "body_qk", samples * heads, 64, 64, depth, heads, scale=_dev(scale))
    _close(out, O.body_qk(q, k, float(scale.float()), heads), rtol=1e-2, atol=1e-2)


def test_body_qk_generic_shapes(ops) -> None:
    samples, heads, depth, m = 2, 3, 20, 10  # not the 64 x 64 x 32k fast path
    q = _bf(torch.randn((samples, m, heads * depth), generator=_gen(72)))
    k = _bf(torch.randn((samples, m, heads * depth), generator=_gen(73)))
    scale = _bf(torch.tensor([0.5]))
    out = torch.empty((samples, heads, m, m), dtype=BF16, device="cuda")
    ops.batched_matmul(out, _dev(q), _dev(k), "body_qk", samples * heads, m, m, depth, heads, scale=_dev(scale))
    qh = q.float().view(samples, m, heads, depth).permute(0, 2, 1, 3)
    kh = k.float().view(samples, m, heads, depth).permute(0, 2, 1, 3)
    _close(out, torch.matmul(qh, kh.transpose(-1, -2)) * 0.5, rtol=1e-2, atol=1e-2)


def test_attention_v_writes_merged_heads(ops) -> None:
    samples, heads, depth = 4, 6, 32
    p = _bf(torch.softmax(torch.randn((samples, heads, 64, 64), generator=_gen(74)), dim=-1))
    v = _bf(torch.randn((samples, 64, heads * depth), generator=_gen(75)))
    out = torch.empty((samples, 64, heads * depth), dtype=BF16, device="cuda")
    ops.batched_matmul(out, _dev(p), _dev(v), "body_attention_v", samples * heads, 64, depth, 64, heads)
    _close(out, O.attention_v(p, v), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("width", [128, 1024])
def test_policy_qk_leaves_promotion_slots_untouched(ops, width) -> None:
    batch = 5
    q = _bf(torch.randn((batch, 64, width), generator=_gen(76)) * 0.3)
    k = _bf(torch.randn((batch, 64, width), generator=_gen(77)) * 0.3)
    scale = _bf(torch.tensor([width ** -0.5]))
    records = torch.full((batch, 4288), -123.0, dtype=BF16, device="cuda")
    ops.batched_matmul(records, _dev(q), _dev(k), "policy_qk", batch, 64, 64, width, 1, scale=_dev(scale))
    want = O.policy_qk(q, k, float(scale.float()), torch.full((batch, 4288), -123.0))
    _close(records, want, rtol=1e-2, atol=1e-2)
    assert torch.equal(records[:, 4096:].float().cpu(), torch.full((batch, 192), -123.0))


# ------------------------------------------------------------------ policy tail

def test_promotion_logits_exact_integer_case(ops, golden) -> None:
    rec = _bf(torch.from_numpy(golden["promo_exact/records"]))
    keys, w = _bf(torch.from_numpy(golden["promo_exact/keys"])), _bf(torch.from_numpy(golden["promo_exact/w"]))
    dev = _dev(rec).clone()
    ops.promotion_logits(dev, _dev(keys), _dev(w), 2, 32)
    want = O.promotion_logits(rec, keys, w).to(BF16)
    assert torch.equal(dev[:, 4096:].cpu(), want)
    assert torch.equal(dev[:, :4096].cpu(), rec[:, :4096])
    assert dev[0, -1] != dev[1, 4096]


def test_promotion_logits_random(ops, golden) -> None:
    rec = _bf(torch.from_numpy(golden["promo_random/records"]))
    keys, w = _bf(torch.from_numpy(golden["promo_random/keys"])), _bf(torch.from_numpy(golden["promo_random/w"]))
    dev = _dev(rec).clone()
    ops.promotion_logits(dev, _dev(keys), _dev(w), 3, 48)
    _close(dev[:, 4096:], O.promotion_logits(rec, keys, w), rtol=1e-2, atol=1e-2)


def test_policy_tail_equals_promotion_plus_gather(ops) -> None:
    from lczero_triton_b200 import mapping_table

    batch, width = 6, 128
    rec = _bf(torch.randn((batch, 4288), generator=_gen(80)))
    keys, w = _bf(torch.randn((batch, 64, width), generator=_gen(81)) * 0.3), _bf(torch.randn((width, 4), generator=_gen(82)) * 0.3)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    out = torch.empty((batch, 1858), dtype=torch.float32, device="cuda")
    ops.policy_tail(out, _dev(rec), _dev(keys), _dev(w), _dev(table), batch, width)
    full = rec.float().clone()
    full[:, 4096:] = O.promotion_logits(rec, keys, w)
    _close(out, O.policy_map(full, table), rtol=1e-2, atol=1e-2)
    plain = table < 4096
    assert torch.equal(out.cpu()[:, plain], rec.float()[:, table[plain].long()])


def test_output_probabilities_over_legal_moves(ops) -> None:
    batch = 5
    logits = torch.randn((batch, 1858), generator=_gen(90)) * 2
    wdl = torch.randn((batch, 3), generator=_gen(91))
    legal = (torch.rand((batch, 1858), generator=_gen(92)) < 0.02).to(torch.uint8)
    legal[3] = 0  # a position without legal moves
    policy, wdl_probs, q_d = ops.output_probabilities(logits.cuda(), wdl.cuda(), legal.cuda())
    want_policy, want_wdl, want_q_d = O.output_probabilities(logits, wdl, legal)
    torch.testing.assert_close(policy.cpu(), want_policy, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(wdl_probs.cpu(), want_wdl, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(q_d.cpu(), want_q_d, rtol=1e-5, atol=1e-6)
    assert (q_d[:, 0].abs() <= 1).all() and torch.allclose(q_d[:, 1].cpu(), want_wdl[:, 1])
    assert policy[3].abs().sum() == 0 and (policy.cpu()[legal == 0] == 0).all()
    everything, _, _ = ops.output_probabilities(logits.cuda(), wdl.cuda(), None)
    torch.testing.assert_close(everything.cpu(), torch.softmax(logits, dim=-1), rtol=1e-5, atol=1e-7)
