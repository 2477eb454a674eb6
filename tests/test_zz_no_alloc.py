"""The int8 dense layer that brings its own scratch (``lc0b200_linear_int8_static``).

It exists for callers that cannot get device memory at run time: an executor bound to a buffer
plan fixed at link time, or a search loop that must never hit cudaMalloc's device-wide stall.
Every case goes through the C ABI.  The first test calls it twice in a row, with different inputs
and a smaller second problem so that stale contents of the shared array would show, and requires
the very same bytes as the entry point that takes caller-provided scratch (both run the same two
kernels).  The limit cases sit exactly on the documented bounds, so the last row scale and the last
activation byte of the built-in array are written and read, and are held against the CPU int8
oracle as well; one step beyond either bound must be refused before anything is launched.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import bt4_oracle as O
from oracle import int8_oracle

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
MAX_ROWS = 16384
MAX_ACT_BYTES = 8 * 1024 * 1024


def _case(m: int, n: int, k: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=gen).to(BF16)
    wq = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8)
    col_scale = torch.rand(n, generator=gen) * 0.01 + 0.001
    bias = (torch.randn(n, generator=gen) * 0.1).to(BF16)
    return a, wq, col_scale, bias


def _oracle(a, wq, col_scale, bias, activation: str) -> torch.Tensor:
    aq, s_a = int8_oracle.quantize_rows(a)
    acc = int8_oracle.int_matmul(aq, wq.t().contiguous())
    return O.activate(int8_oracle.dequant(acc, s_a, col_scale, bias), activation)


def _both_entry_points(m: int, n: int, k: int, seed: int, activation: str):
    from lczero_triton_b200 import ops

    a, wq, col_scale, bias = _case(m, n, k, seed)
    dev = [t.cuda() for t in (a, wq, col_scale, bias)]
    want = torch.empty((m, n), dtype=BF16, device="cuda")
    scratch_q = torch.empty((m, k), dtype=torch.int8, device="cuda")
    scratch_s = torch.empty((m,), dtype=torch.float32, device="cuda")
    ops.linear_int8(want, *dev, scratch_q, scratch_s, m=m, n=n, k=k, activation=activation)
    got = torch.full((m, n), float("nan"), dtype=BF16, device="cuda")
    ops.linear_int8_static(got, *dev, m=m, n=n, k=k, activation=activation)
    torch.cuda.synchronize()
    return got, want, _oracle(a, wq, col_scale, bias, activation)


def test_static_scratch_variant_matches_caller_scratch_variant_twice() -> None:
    from lczero_triton_b200 import _lib, build

    build.build()
    for m, n, k, seed, activation in ((1000, 1536, 1024, 1, "mish"), (260, 1024, 1536, 2, "none")):
        got, want, oracle = _both_entry_points(m, n, k, seed, activation)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)
        torch.testing.assert_close(got.float().cpu(), oracle, rtol=8e-3, atol=4e-3)
    status, detail = _lib.device_status()
    assert status == 0, detail


@pytest.mark.parametrize(("m", "k"), [(MAX_ROWS, MAX_ACT_BYTES // MAX_ROWS), (MAX_ACT_BYTES // 1024, 1024)],
                         ids=["row-limit", "byte-limit"])
def test_static_scratch_variant_at_its_limits(m, k) -> None:
    """m = 16384 with m * k = 8 MiB uses every row scale and every activation byte of the array;
    m = 8192, k = 1024 reaches the byte bound with half the rows."""
    from lczero_triton_b200 import _lib, build

    build.build()
    assert m <= MAX_ROWS and m * k == MAX_ACT_BYTES
    got, want, oracle = _both_entry_points(m, 64, k, 3, "none")
    assert torch.equal(got, want)
    torch.testing.assert_close(got.float().cpu(), oracle, rtol=8e-3, atol=4e-3)
    # a following small call must not be disturbed by what the large one left behind
    got, want, oracle = _both_entry_points(33, 128, 96, 4, "relu")
    assert torch.equal(got, want)
    torch.testing.assert_close(got.float().cpu(), oracle, rtol=8e-3, atol=4e-3)
    status, detail = _lib.device_status()
    assert status == 0, detail


def test_static_scratch_variant_refuses_oversize_problems() -> None:
    from lczero_triton_b200 import _lib, build

    build.build()
    lib = _lib.load()
    fake = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    too_many_rows = lib.lc0b200_linear_int8_static(fake, fake, fake, fake, None, MAX_ROWS + 1, 64, 64, 0, None)
    too_many_bytes = lib.lc0b200_linear_int8_static(fake, fake, fake, fake, None, MAX_ROWS, 64, 528, 0, None)
    just_over = lib.lc0b200_linear_int8_static(fake, fake, fake, fake, None, 8193, 64, 1024, 0, None)
    assert too_many_rows == 7 and too_many_bytes == 7 and just_over == 7
    assert b"scratch" in lib.lc0b200_status_string(7)
