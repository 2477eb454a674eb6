"""Known-answer checks for the derived attention-policy gather table
(reference: packages/lczero-triton/tests/test_mapping_table.py:9-18)."""

from __future__ import annotations

import numpy as np

from lczero_triton_b200 import mapping_table


def test_table_known_answers() -> None:
    table = mapping_table.values()
    assert len(table) == 1858
    assert len(set(table)) == 1858
    assert min(table) >= 0 and max(table) < 4288
    assert table[:10] == (1, 2, 3, 4, 5, 6, 7, 8, 9, 10)
    assert table[-10:] == (4260, 4261, 4262, 4263, 4282, 4283, 4284, 4285, 4286, 4287)


def test_table_equals_reference_decoded_table(golden) -> None:
    assert np.array_equal(np.asarray(mapping_table.values(), dtype=np.int32), golden["mapping_table"])
