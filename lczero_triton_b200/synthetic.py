"""Seeded synthetic Lc0 input planes.

Stands in for lc0 ``backendbench`` positions, which the reference benchmarked
on (LC0EX_BACKEND_BENCHMARK.md:5-7) and which are not available offline.  The
packed layout is the reference's execution input: one u64 occupancy mask and
one f32 value per plane (network.py:328-340).
"""

from __future__ import annotations

import torch

from .config import INPUT_PLANES, SQUARES


def synthetic_planes(batch: int, seed: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Return ``(masks int64[B,112] holding u64 bit patterns, values f32[B,112])``.

    Planes 0..103 are 8 history steps x 13 planes: per step each square is
    occupied with p=0.40 by exactly one of 12 piece planes; the 13th plane
    (repetition) is all-ones with p=0.05.  Planes 104..107 castling (all-ones,
    p=0.5), 108 side to move (p=0.5), 109 rule50 scalar in [0,1] on an all-ones
    mask, 110 zero, 111 all-ones.
    """
    gen = torch.Generator().manual_seed(seed)
    occupied = torch.rand((batch, 8, SQUARES), generator=gen) < 0.40
    piece = torch.randint(0, 12, (batch, 8, SQUARES), generator=gen)
    bits = torch.zeros((batch, INPUT_PLANES, SQUARES), dtype=torch.bool)
    onehot = torch.nn.functional.one_hot(piece, 12).bool() & occupied[..., None]  # [B,8,64,12]
    steps = onehot.permute(0, 1, 3, 2)  # [B,8,12,64]
    for step in range(8):
        bits[:, step * 13: step * 13 + 12] = steps[:, step]
    repetition = torch.rand((batch, 8), generator=gen) < 0.05
    for step in range(8):
        bits[:, step * 13 + 12] = repetition[:, step, None]
    flags = torch.rand((batch, 5), generator=gen) < 0.5
    bits[:, 104:109] = flags[:, :, None]
    bits[:, 109] = True
    bits[:, 111] = True
    values = torch.ones((batch, INPUT_PLANES), dtype=torch.float32)
    values[:, 109] = torch.rand((batch,), generator=gen)
    weights = torch.ones(SQUARES, dtype=torch.int64) << torch.arange(SQUARES, dtype=torch.int64)
    masks = (bits.to(torch.int64) * weights).sum(dim=-1)  # wraps into the sign bit for square 63
    return masks.contiguous(), values.contiguous()
