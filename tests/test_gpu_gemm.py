"""GPU parity of the tensor-core GEMM (tcgen05 + TMA) through the C ABI.

bf16: compared with an fp32 matmul of the same bf16 values; the kernel accumulates in fp32
(TMEM) and rounds once to bf16, so the tolerance is one bf16 ulp of the result plus the fp32
accumulation-order noise.  int8: the s32 accumulators must equal the CPU integer product bit
for bit.  Every case is also run on the plain CUDA-core kernel as an independent cross-check.
"""

from __future__ import annotations

import pytest
import torch

from oracle import bt4_oracle as O
from oracle import int8_oracle

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    from lczero_triton_b200 import build, ops as module

    build.build()
    return module


@pytest.fixture(autouse=True)
def _no_device_timeouts():
    yield
    from lczero_triton_b200 import _lib

    status, detail = _lib.device_status()
    assert status == 0, f"a kernel's bounded wait ran out: {detail}"


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def _operands(m: int, n: int, k: int, seed: int):
    a = (torch.randn((m, k), generator=_gen(seed)) * 0.5).to(BF16)
    w = (torch.randn((k, n), generator=_gen(seed + 1)) * 0.5).to(BF16)
    return a, w


def _check(got: torch.Tensor, want: torch.Tensor, k: int) -> None:
    # |result| ~ 0.25 sqrt(k); one bf16 ulp of that plus a little.
    atol = 0.25 * (k ** 0.5) * 2 ** -8 * 2 + 1e-3
    torch.testing.assert_close(got.float().cpu(), want, rtol=8e-3, atol=atol)


SHAPES = [
    (128, 256, 64), (128, 256, 1024), (256, 1024, 1024), (1024, 1536, 1024), (640, 1024, 1536),
    (512, 3072, 1024), (300, 1000, 520), (64, 32768, 768), (4096, 32, 1024), (4096, 16, 128),
    (77, 64, 2048), (130, 128, 8192), (2048, 4096, 256), (33, 8192, 256), (1000, 1024, 624), (5, 128, 128),
    # many rows with a wide output: 256 x 256 tiles shared by CTA pairs (bf16: whenever the tile is 256 wide and
    # K > 512, so several of the smaller shapes above run on pairs too; int8: from 8192 rows)
    (8200, 1536, 1024), (16384, 3072, 1024), (8192, 1000, 520), (9000, 4096, 256),
    (900, 3104, 1024), (1300, 2048, 1024), (3000, 1024, 1024),  # few rows on pairs, the last pair half empty
    # a ragged last tile narrower than the tile: its MMAs cover 32 / 96 / 160 columns instead of 256
    (300, 800, 256), (8200, 1056, 1024), (8200, 1120, 1024), (700, 3232, 1024), (8192, 3104, 1024),
]


@pytest.mark.parametrize(("m", "n", "k"), SHAPES)
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_bf16_gemm_matches_fp32_matmul(ops, m, n, k, layout) -> None:
    from lczero_triton_b200 import _lib

    a, w = _operands(m, n, k, 100)
    want = O.matmul(a, w)
    out = torch.full((m, n), float("nan"), dtype=BF16, device="cuda")
    if layout == "nk":
        ops.gemm(out, a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, w_layout=_lib.W_NK)
    else:
        ops.gemm(out, a.cuda(), w.cuda(), m=m, n=n, k=k, w_layout=_lib.W_KN)
    _check(out, want, k)


@pytest.mark.parametrize("activation", ["none", "mish", "relu", "swish"])
def test_bf16_gemm_bias_activation_epilogue(ops, activation) -> None:
    from lczero_triton_b200 import _lib

    m, n, k = 384, 1536, 1024
    a, w = _operands(m, n, k, 110)
    a, w = (a.float() * 0.2).to(BF16), (w.float() * 0.2).to(BF16)
    bias = (torch.randn(n, generator=_gen(112)) * 0.5).to(BF16)
    want = O.activate(O.matmul(a, w) + bias.float(), activation)
    out = torch.empty((m, n), dtype=BF16, device="cuda")
    ops.gemm(out, a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, bias=bias.cuda(), activation=activation,
             w_layout=_lib.W_NK)
    torch.testing.assert_close(out.float().cpu(), want, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize(("m", "n", "k"), [(300, 400, 1600), (300, 408, 1600), (8300, 1040, 1536), (257, 272, 2048),
                                            (8300, 1040, 1024)])
def test_bf16_gemm_store_paths_at_matrix_edges(ops, m, n, k) -> None:
    """Long K takes the stores straight from registers (rows in whole 32-byte pieces), everything else
    the staged TMA store; both must respect a row pitch, ragged last tiles and leave neighbours alone."""
    from lczero_triton_b200 import _lib

    a, w = _operands(m, n, k, 125)
    a, w = (a.float() * 0.2).to(BF16), (w.float() * 0.2).to(BF16)
    bias = (torch.randn(n, generator=_gen(126)) * 0.5).to(BF16)
    want = O.activate(O.matmul(a, w) + bias.float(), "mish")
    pitch = n + 48
    wide = torch.full((m + 3, pitch), 7.0, dtype=BF16, device="cuda")
    ops.gemm(wide[:m, 16:16 + n], a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, bias=bias.cuda(), activation="mish",
             ldc=pitch, w_layout=_lib.W_NK)
    torch.testing.assert_close(wide[:m, 16:16 + n].float().cpu(), want, rtol=1e-2, atol=1e-2)
    assert (wide[:m, :16] == 7.0).all() and (wide[:m, 16 + n:] == 7.0).all() and (wide[m:] == 7.0).all()


def test_bf16_gemm_strided_output_and_f32_output(ops) -> None:
    from lczero_triton_b200 import _lib

    m, n, k = 200, 128, 256
    a, w = _operands(m, n, k, 120)
    want = O.matmul(a, w)
    wide = torch.zeros((m, 3 * n), dtype=BF16, device="cuda")
    ops.gemm(wide[:, n:2 * n], a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, ldc=3 * n, w_layout=_lib.W_NK)
    _check(wide[:, n:2 * n], want, k)
    assert wide[:, :n].abs().sum() == 0 and wide[:, 2 * n:].abs().sum() == 0
    f32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ops.gemm(f32, a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, w_layout=_lib.W_NK)
    torch.testing.assert_close(f32.cpu(), want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize(("m", "n", "k"), [(7, 37, 11), (64, 3, 128), (200, 1, 128), (33, 4, 100)])
def test_reference_layout_matmul_on_unaligned_shapes(ops, m, n, k) -> None:
    """Shapes TMA cannot address (the reference tests 7 x 37 x 11, test_matmul.py:115-138) take the
    CUDA-core kernel behind the same entry point."""
    a, w = _operands(m, n, k, 130)
    out = torch.empty((m, n), dtype=BF16, device="cuda")
    ops.matmul(out, a.cuda(), w.cuda(), m, n, k)
    _check(out, O.matmul(a, w), k)


@pytest.mark.parametrize(("m", "n", "k"), [(128, 256, 128), (300, 1000, 528), (1024, 3072, 1024), (512, 1024, 1536),
                                            (64, 128, 4096), (4096, 32, 1024), (8200, 1024, 1536), (16384, 1536, 1024)])
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_int8_gemm_accumulators_are_bit_exact(ops, m, n, k, layout) -> None:
    from lczero_triton_b200 import _lib

    aq = torch.randint(-127, 128, (m, k), generator=_gen(140), dtype=torch.int8)
    wq = torch.randint(-127, 128, (k, n), generator=_gen(141), dtype=torch.int8)
    want = int8_oracle.int_matmul(aq, wq)
    out = torch.full((m, n), -1, dtype=torch.int32, device="cuda")
    if layout == "nk":
        ops.gemm(out, aq.cuda(), wq.t().contiguous().cuda(), m=m, n=n, k=k, w_layout=_lib.W_NK)
    else:
        if n % 16 != 0:
            pytest.skip("TMA needs a 16-byte aligned row pitch for the [K,N] int8 layout")
        ops.gemm(out, aq.cuda(), wq.cuda(), m=m, n=n, k=k, w_layout=_lib.W_KN)
    assert torch.equal(out.cpu(), want)
    simt = torch.empty_like(out)
    ops.gemm(simt, aq.cuda(), wq.t().contiguous().cuda(), m=m, n=n, k=k, w_layout=_lib.W_NK, simt=True)
    assert torch.equal(simt.cpu(), want)


def test_int8_gemm_dequant_bias_mish_epilogue(ops) -> None:
    from lczero_triton_b200 import _lib

    m, n, k = 256, 1536, 1024
    a = (torch.randn((m, k), generator=_gen(150))).to(BF16)
    w = (torch.randn((k, n), generator=_gen(151)) * 0.02).to(BF16)
    bias = (torch.randn(n, generator=_gen(152)) * 0.1).to(BF16)
    aq, s_a = int8_oracle.quantize_rows(a)
    wq, s_w = int8_oracle.quantize_weight(w)
    want = O.activate(int8_oracle.dequant(int8_oracle.int_matmul(aq, wq), s_a, s_w, bias), "mish")
    out = torch.empty((m, n), dtype=BF16, device="cuda")
    ops.gemm(out, aq.cuda(), wq.t().contiguous().cuda(), m=m, n=n, k=k, bias=bias.cuda(), activation="mish",
             row_scale=s_a.cuda(), col_scale=s_w.cuda(), w_layout=_lib.W_NK)
    torch.testing.assert_close(out.float().cpu(), want, rtol=8e-3, atol=4e-3)


@pytest.mark.parametrize(("m", "n", "k"), [(256, 1536, 1024), (100, 1024, 1536), (33, 40, 24)])
def test_linear_int8_equals_quantise_then_gemm(ops, m, n, k) -> None:
    a = torch.randn((m, k), generator=_gen(160)).to(BF16)
    w = (torch.randn((k, n), generator=_gen(161)) * 0.02).to(BF16)
    bias = (torch.randn(n, generator=_gen(162)) * 0.1).to(BF16)
    wq, s_w = int8_oracle.quantize_weight(w)
    want = O.activate(int8_oracle.linear(a, w, bias), "mish")
    out = torch.empty((m, n), dtype=BF16, device="cuda")
    scratch_q = torch.empty((m, k), dtype=torch.int8, device="cuda")
    scratch_s = torch.empty((m,), dtype=torch.float32, device="cuda")
    ops.linear_int8(out, a.cuda(), wq.t().contiguous().cuda(), s_w.cuda(), bias.cuda(), scratch_q, scratch_s,
                    m=m, n=n, k=k, activation="mish")
    torch.testing.assert_close(out.float().cpu(), want, rtol=8e-3, atol=4e-3)
    want_q, want_s = int8_oracle.quantize_rows(a)
    assert torch.equal(scratch_q.cpu(), want_q) and torch.equal(scratch_s.cpu(), want_s)


def _partial_stats(z: torch.Tensor) -> torch.Tensor:
    """[parts, m, 2] partial (sum, sum of squares) over 64-column groups, as the GEMM epilogue emits them."""
    m, n = z.shape
    groups = z.float().reshape(m, n // 64, 64)
    return torch.stack((groups.sum(dim=2), (groups * groups).sum(dim=2)), dim=2).permute(1, 0, 2).contiguous()


@pytest.mark.parametrize("m", [1000, 9000])
def test_deferred_layer_norm_epilogues(ops, m) -> None:
    """Producer: z = alpha * (A W + b) + LN(z_prev) with partial row sums.  Consumer: LN(z) W' folded into
    the epilogue.  Both against the oracle's explicit LayerNorm (layer_norm.py:57-87 semantics)."""
    from lczero_triton_b200 import _lib

    d, f, eps, alpha = 1024, 1536, 1e-3, 0.4273
    g = _gen(170)
    z_prev = (torch.randn((m, d), generator=g) * 1.3 + 0.2).to(BF16)
    gamma, beta = (1 + 0.1 * torch.randn(d, generator=g)).to(BF16), (0.1 * torch.randn(d, generator=g)).to(BF16)
    a = (torch.randn((m, f), generator=g) * 0.5).to(BF16)
    w = (torch.randn((f, d), generator=g) * 0.05).to(BF16)
    bias = (torch.randn(d, generator=g) * 0.1).to(BF16)
    zero = torch.zeros(d)
    skip_ln = O.layer_norm(z_prev, zero, gamma, beta, "none", eps)
    want_z = alpha * (O.matmul(a, w) + bias.float()) + skip_ln
    stats_prev = _partial_stats(z_prev).cuda()
    z = torch.empty((m, d), dtype=BF16, device="cuda")
    stats = torch.full((d // 64, m, 2), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemm(z, a.cuda(), w.t().contiguous().cuda(), m=m, n=d, k=f, bias=bias.cuda(), w_layout=_lib.W_NK,
             res_skip=z_prev.cuda(), res_ln=(stats_prev, gamma.cuda(), beta.cuda()), res_alpha=alpha,
             stats_out=stats, ln_eps=eps)
    torch.testing.assert_close(z.float().cpu(), want_z, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(stats.cpu(), _partial_stats(z.cpu()), rtol=1e-4, atol=1e-3)

    # plain skip operand (the embedding's residual)
    z_plain = torch.empty((m, d), dtype=BF16, device="cuda")
    stats_plain = torch.empty_like(stats)
    ops.gemm(z_plain, a.cuda(), w.t().contiguous().cuda(), m=m, n=d, k=f, bias=bias.cuda(), w_layout=_lib.W_NK,
             res_skip=z_prev.cuda(), res_alpha=alpha, stats_out=stats_plain, ln_eps=eps)
    torch.testing.assert_close(z_plain.float().cpu(), alpha * (O.matmul(a, w) + bias.float()) + z_prev.float(),
                               rtol=1e-2, atol=2e-2)

    # consumer: mish(LN(z) W1 + b1) with gamma folded into the weight
    zc = z.cpu()
    w1 = (torch.randn((d, f), generator=g) * 0.03).to(BF16)
    b1 = (torch.randn(f, generator=g) * 0.1).to(BF16)
    scaled = (w1.float() * gamma.float()[:, None]).to(BF16)
    fold_c = scaled.float().sum(dim=0)
    fold_d = beta.float() @ w1.float() + b1.float()
    want_h = O.activate(O.matmul(O.layer_norm(zc, zero, gamma, beta, "none", eps), w1) + b1.float(), "mish")
    hidden = torch.empty((m, f), dtype=BF16, device="cuda")
    ops.gemm(hidden, z, scaled.t().contiguous().cuda(), m=m, n=f, k=d, activation="mish", w_layout=_lib.W_NK,
             ln_in=(stats, fold_c.cuda(), fold_d.cuda()), ln_eps=eps)
    torch.testing.assert_close(hidden.float().cpu(), want_h, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize(("m", "n_main", "n_tail", "k"), [(300, 256, 32, 512), (64, 256, 96, 256), (8300, 3072, 32, 1024),
                                                         (8200, 512, 200, 1024), (1, 256, 8, 64)])
def test_second_output_for_trailing_columns(ops, m, n_main, n_tail, k) -> None:
    """Two projections of the same rows as one product: columns [0, n_main) to one matrix, the rest to a
    second, narrower one (how smolgen's 32-wide compression rides on the QKV GEMM) - plain with bias and
    activation, and with the LayerNorm of the rows folded into the epilogue.  Neither output may be written
    outside its columns, and the pitch of each is its own."""
    from lczero_triton_b200 import _lib

    n = n_main + n_tail
    g = _gen(190)
    a = (torch.randn((m, k), generator=g) * 0.5).to(BF16)
    w = (torch.randn((k, n), generator=g) * 0.2).to(BF16)
    bias = (torch.randn(n, generator=g) * 0.5).to(BF16)
    want = O.activate(O.matmul(a, w) + bias.float(), "mish")
    main = torch.full((m + 1, n_main + 16), 7.0, dtype=BF16, device="cuda")
    tail = torch.full((m + 1, n_tail + 8), 7.0, dtype=BF16, device="cuda")
    ops.gemm(main[:m, :n_main], a.cuda(), w.t().contiguous().cuda(), m=m, n=n, k=k, bias=bias.cuda(), activation="mish",
             w_layout=_lib.W_NK, ldc=n_main + 16, out_tail=tail[:m, :n_tail], n_main=n_main)
    torch.testing.assert_close(main[:m, :n_main].float().cpu(), want[:, :n_main], rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(tail[:m, :n_tail].float().cpu(), want[:, n_main:], rtol=1e-2, atol=1e-2)
    assert (main[:m, n_main:] == 7.0).all() and (main[m:] == 7.0).all()
    assert (tail[:m, n_tail:] == 7.0).all() and (tail[m:] == 7.0).all()

    if n_tail % 8 == 0 and k % 64 == 0:
        # the reference's [K, N] weight layout takes the same second output (whole-tile MMAs there)
        main.fill_(7.0)
        tail.fill_(7.0)
        ops.gemm(main[:m, :n_main], a.cuda(), w.cuda(), m=m, n=n, k=k, bias=bias.cuda(), activation="mish",
                 w_layout=_lib.W_KN, ldc=n_main + 16, out_tail=tail[:m, :n_tail], n_main=n_main)
        torch.testing.assert_close(main[:m, :n_main].float().cpu(), want[:, :n_main], rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(tail[:m, :n_tail].float().cpu(), want[:, n_main:], rtol=1e-2, atol=1e-2)
        assert (main[:m, n_main:] == 7.0).all() and (tail[:m, n_tail:] == 7.0).all()

    # the same through the folded-LayerNorm epilogue (the form the forward pass uses)
    eps = 1e-3
    z = (torch.randn((m, k), generator=g) * 1.3 + 0.2).to(BF16)
    gamma, beta = (1 + 0.1 * torch.randn(k, generator=g)).to(BF16), (0.1 * torch.randn(k, generator=g)).to(BF16)
    w1 = (torch.randn((k, n), generator=g) * 0.05).to(BF16)
    scaled = (w1.float() * gamma.float()[:, None]).to(BF16)
    fold_c, fold_d = scaled.float().sum(dim=0), beta.float() @ w1.float() + bias.float()
    want = O.matmul(O.layer_norm(z, torch.zeros(k), gamma, beta, "none", eps), w1) + bias.float()
    stats = _partial_stats(z).cuda() if k % 64 == 0 else None
    if stats is not None:
        main.fill_(7.0)
        tail.fill_(7.0)
        ops.gemm(main[:m, :n_main], z.cuda(), scaled.t().contiguous().cuda(), m=m, n=n, k=k, w_layout=_lib.W_NK,
                 ldc=n_main + 16, ln_in=(stats, fold_c.cuda(), fold_d.cuda()), ln_eps=eps, out_tail=tail[:m, :n_tail],
                 n_main=n_main)
        torch.testing.assert_close(main[:m, :n_main].float().cpu(), want[:, :n_main], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(tail[:m, :n_tail].float().cpu(), want[:, n_main:], rtol=2e-2, atol=2e-2)
        assert (main[:m, n_main:] == 7.0).all() and (tail[:m, n_tail:] == 7.0).all()


def test_second_output_is_refused_where_it_cannot_be_honoured(ops) -> None:
    from lczero_triton_b200 import _lib

    a = torch.zeros((64, 64), dtype=BF16, device="cuda")
    w = torch.zeros((288, 64), dtype=BF16, device="cuda")
    main = torch.zeros((64, 256), dtype=BF16, device="cuda")
    tail = torch.zeros((64, 32), dtype=BF16, device="cuda")
    with pytest.raises(_lib.Lc0B200Error):  # n_main must be a multiple of 256
        ops.gemm(main[:, :128], a, w[:160], m=64, n=160, k=64, ldc=256, out_tail=tail, n_main=128)
    with pytest.raises(_lib.Lc0B200Error):  # not on the CUDA-core kernel
        ops.gemm(main, a, w, m=64, n=288, k=64, out_tail=tail, n_main=256, simt=True)
    with pytest.raises(_lib.Lc0B200Error):  # not with the residual epilogue
        ops.gemm(main, a, w, m=64, n=288, k=64, out_tail=tail, n_main=256, res_skip=main, res_alpha=1.0)


def test_int8_gemm_residual_epilogue(ops) -> None:
    """The residual form on the int8 GEMM: z = alpha * (dequant(Aq Wq) + b) + LN(z_prev), with row sums."""
    from lczero_triton_b200 import _lib

    m, d, f, eps, alpha = 8300, 1024, 1536, 1e-3, 0.4273
    g = _gen(180)
    z_prev = (torch.randn((m, d), generator=g) * 1.3 + 0.2).to(BF16)
    gamma, beta = (1 + 0.1 * torch.randn(d, generator=g)).to(BF16), (0.1 * torch.randn(d, generator=g)).to(BF16)
    a = torch.randn((m, f), generator=g).to(BF16)
    w = (torch.randn((f, d), generator=g) * 0.02).to(BF16)
    bias = (torch.randn(d, generator=g) * 0.1).to(BF16)
    aq, s_a = int8_oracle.quantize_rows(a)
    wq, s_w = int8_oracle.quantize_weight(w)
    branch = int8_oracle.dequant(int8_oracle.int_matmul(aq, wq), s_a, s_w, bias)
    want = alpha * branch + O.layer_norm(z_prev, torch.zeros(d), gamma, beta, "none", eps)
    z = torch.empty((m, d), dtype=BF16, device="cuda")
    stats = torch.empty((d // 64, m, 2), dtype=torch.float32, device="cuda")
    ops.gemm(z, aq.cuda(), wq.t().contiguous().cuda(), m=m, n=d, k=f, bias=bias.cuda(), w_layout=_lib.W_NK,
             row_scale=s_a.cuda(), col_scale=s_w.cuda(), res_skip=z_prev.cuda(),
             res_ln=(_partial_stats(z_prev).cuda(), gamma.cuda(), beta.cuda()), res_alpha=alpha, stats_out=stats,
             ln_eps=eps)
    torch.testing.assert_close(z.float().cpu(), want, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(stats.cpu(), _partial_stats(z.cpu()), rtol=1e-4, atol=1e-3)


def test_layer_norm_to_int8_only(ops) -> None:
    """LayerNorm straight to per-row int8, no bf16 copy stored (out == NULL)."""
    rows, width = 37, 1024
    x = torch.randn((rows, width), generator=_gen(181)).to(BF16)
    bias, gamma, beta = (torch.randn(width, generator=_gen(182 + i)).mul(0.2).to(BF16) for i in range(3))
    both = torch.empty_like(x, device="cuda")
    q1, s1 = torch.empty((rows, width), dtype=torch.int8, device="cuda"), torch.empty(rows, device="cuda")
    q2, s2 = torch.empty_like(q1), torch.empty_like(s1)
    ops.layer_norm(both, x.cuda(), bias.cuda(), gamma.cuda(), beta.cuda(), row_count=rows, width=width, q_out=q1, q_scale=s1)
    ops.layer_norm(None, x.cuda(), bias.cuda(), gamma.cuda(), beta.cuda(), row_count=rows, width=width, q_out=q2, q_scale=s2)
    assert torch.equal(q1, q2) and torch.equal(s1, s2)
    want_q, want_s = int8_oracle.quantize_rows(both.cpu())
    assert torch.equal(q2.cpu(), want_q) and torch.equal(s2.cpu(), want_s)


def test_gemm_linearity_at_full_size(ops) -> None:
    """Size-independent property at the benchmark's row count: GEMM(a1 + a2) = GEMM(a1) + GEMM(a2)
    when the sums are exact in bf16 (small integers), checked on sampled rows of a 262144-row problem."""
    from lczero_triton_b200 import _lib

    m, n, k = 262144, 1024, 1024
    gen = torch.Generator(device="cuda").manual_seed(7)
    a1 = torch.randint(-3, 4, (m, k), generator=gen, device="cuda").to(BF16)
    a2 = torch.randint(-3, 4, (m, k), generator=gen, device="cuda").to(BF16)
    w = torch.randint(-2, 3, (n, k), generator=gen, device="cuda").to(BF16)
    outs = []
    for a in (a1, a2, a1 + a2):
        out = torch.empty((m, n), dtype=torch.float32, device="cuda")
        ops.gemm(out, a, w, m=m, n=n, k=k, w_layout=_lib.W_NK)
        outs.append(out)
    assert torch.equal(outs[0] + outs[1], outs[2])  # integer-valued, exact in fp32
    rows = torch.tensor([0, 1, 127, 128, 131071, 200000, 262143], device="cuda")
    want = a1[rows].float() @ w.float().t()
    assert torch.equal(outs[0][rows], want)
