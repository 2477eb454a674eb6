"""Attention-policy gather table: 1858 Lc0 move slots -> 4288-wide policy record.

The reference ships this table as an opaque compressed blob
(packages/lczero-triton/src/lczero_triton/bt4/kernels/mapping_table.py:15-65).
Here it is derived from chess move geometry instead:

* record slot ``from*64 + to`` holds the logit of a plain move (squares are
  ``rank*8 + file``); the 1792 plain moves are every queen-line or knight jump,
  ordered by from-square, then by to-square;
* record slots ``4096 + from_file*24 + to_file*3 + piece`` hold the 66
  under-promotion logits (rank 7 -> rank 8, file distance <= 1, piece in
  queen/rook/bishop order), ordered by from-file, to-file, piece.

``tests/test_mapping_table.py`` checks the derivation against the reference's
known-answer values and, when the reference tree is present, against its
decoded table entry by entry.
"""

from __future__ import annotations

from functools import lru_cache

from .config import POLICY_RECORD, POLICY_SIZE, PROMOTION_START


def _is_policy_move(src: int, dst: int) -> bool:
    if src == dst:
        return False
    dr = abs(dst // 8 - src // 8)
    df = abs(dst % 8 - src % 8)
    queen_line = dr == 0 or df == 0 or dr == df
    knight = (dr, df) in ((1, 2), (2, 1))
    return queen_line or knight


@lru_cache(maxsize=1)
def values() -> tuple[int, ...]:
    """Gather index into the policy record for each of the 1858 policy outputs."""
    table = [src * 64 + dst for src in range(64) for dst in range(64) if _is_policy_move(src, dst)]
    for src_file in range(8):
        for dst_file in range(8):
            if abs(src_file - dst_file) <= 1:
                for piece in range(3):
                    table.append(PROMOTION_START + src_file * 24 + dst_file * 3 + piece)
    if len(table) != POLICY_SIZE or len(set(table)) != POLICY_SIZE or max(table) >= POLICY_RECORD:
        raise RuntimeError("derived attention-policy mapping table is malformed")
    return tuple(table)
