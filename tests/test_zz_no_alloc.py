"""The int8 dense layer that brings its own scratch (``lc0b200_linear_int8_static``).

It exists for callers that cannot get device memory at run time: an executor bound to a buffer
plan fixed at link time, or a search loop that must never hit cudaMalloc's device-wide stall.
The test calls it through the C ABI twice in a row, with different inputs and a smaller
second problem so that stale contents of the shared array would show, and requires the very
same result as the entry point that takes caller-provided scratch (both run the same two
kernels, so the comparison is exact).  This file sorts last on purpose: a run that stops at the
first failure has by then run everything else.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _case(m: int, n: int, k: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=gen).to(BF16).cuda()
    wq = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
    col_scale = (torch.rand(n, generator=gen) * 0.01 + 0.001).cuda()
    bias = (torch.randn(n, generator=gen) * 0.1).to(BF16).cuda()
    return a, wq, col_scale, bias


def test_static_scratch_variant_matches_caller_scratch_variant_twice() -> None:
    from lczero_triton_b200 import _lib, build, ops

    build.build()
    for m, n, k, seed, activation in ((1000, 1536, 1024, 1, "mish"), (260, 1024, 1536, 2, "none")):
        a, wq, col_scale, bias = _case(m, n, k, seed)
        want = torch.empty((m, n), dtype=BF16, device="cuda")
        scratch_q = torch.empty((m, k), dtype=torch.int8, device="cuda")
        scratch_s = torch.empty((m,), dtype=torch.float32, device="cuda")
        ops.linear_int8(want, a, wq, col_scale, bias, scratch_q, scratch_s, m=m, n=n, k=k, activation=activation)
        got = torch.full((m, n), float("nan"), dtype=BF16, device="cuda")
        ops.linear_int8_static(got, a, wq, col_scale, bias, m=m, n=n, k=k, activation=activation)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)
    status, detail = _lib.device_status()
    assert status == 0, detail


def test_static_scratch_variant_refuses_oversize_problems() -> None:
    from lczero_triton_b200 import _lib, build

    build.build()
    lib = _lib.load()
    fake = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    too_many_rows = lib.lc0b200_linear_int8_static(fake, fake, fake, fake, None, 16385, 64, 64, 0, None)
    too_many_bytes = lib.lc0b200_linear_int8_static(fake, fake, fake, fake, None, 8193, 64, 1024, 0, None)
    assert too_many_rows == 7 and too_many_bytes == 7
    assert b"scratch" in lib.lc0b200_status_string(7)
