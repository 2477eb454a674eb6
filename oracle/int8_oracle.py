"""CPU oracle for the int8 GEMM path.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference has no int8 code, test or document, so there is
nothing of the reference's to pin this against.  The quantiser below is this
project's own specification:

* weights, symmetric per output channel: ``s_w[n] = max_k |W[k,n]| / 127`` (1 if the
  column is all zero), ``Wq[k,n] = clamp(rint(W[k,n] / s_w[n]), -127, 127)``;
* activations, symmetric per token row, from the bf16 values the GPU stores:
  ``s_a[m] = max_k |A[m,k]| / 127`` (1 if the row is all zero),
  ``Aq[m,k] = clamp(rint(A[m,k] * (127 / max_k |A[m,k]|)), -127, 127)`` (one division per row; the
  factor is 1 for an all-zero row);
* ``rint`` is round-half-to-even, all arithmetic in IEEE fp32;
* ``acc[m,n] = sum_k int32(Aq[m,k]) * int32(Wq[k,n])`` exactly;
* ``y[m,n] = act((float(acc[m,n]) * s_a[m]) * s_w[n] + bias[n])``.

Integer accumulation has one right answer, so the int32 accumulators of any
correct kernel equal ``int_matmul`` bit for bit; that is what the tests check.
"""

from __future__ import annotations

import torch


def quantize_weight(w_kn: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Return ``(Wq int8 [K,N], s_w f32 [N])``."""
    w = w_kn.float()
    amax = w.abs().amax(dim=0)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    return torch.clamp(torch.round(w / scale), -127, 127).to(torch.int8), scale


def quantize_rows(a: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Return ``(Aq int8 [M,K], s_a f32 [M])``."""
    x = a.float()
    amax = x.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    # (torch evaluates ``127.0 / t`` as ``t.reciprocal() * 127.0``: divide two tensors for one rounding.)
    inv = torch.where(amax > 0, torch.full_like(amax, 127.0) / amax, torch.ones_like(amax))
    return torch.clamp(torch.round(x * inv[:, None]), -127, 127).to(torch.int8), scale


def int_matmul(aq: torch.Tensor, wq_kn: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulators of ``Aq[M,K] @ Wq[K,N]``."""
    return (aq.to(torch.int32) @ wq_kn.to(torch.int32)).to(torch.int32)


def dequant(acc: torch.Tensor, s_a: torch.Tensor, s_w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    y = (acc.float() * s_a[:, None]) * s_w[None, :]
    return y if bias is None else y + bias.float()[None, :]


def linear(a_bf16: torch.Tensor, w_kn: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Quantise activations and weights, multiply exactly, dequantise (fp32 result)."""
    aq, s_a = quantize_rows(a_bf16)
    wq, s_w = quantize_weight(w_kn)
    return dequant(int_matmul(aq, wq), s_a, s_w, bias)
