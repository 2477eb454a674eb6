"""B200-native forward pass for Lc0 BT4-style transformer networks.

Public surface (names follow the reference package where it has a counterpart):

* ``load_network``, ``normalize_network``, ``validate_network_format``, ``NetworkFormatError``
  (``format.py``);
* ``Bt4Net`` — a network resident on one GPU with ``forward(plane_masks, plane_values)``
  (``net.py``);
* ``ops`` — one wrapper per C-ABI entry point, mirroring the reference's op functions.

Submodules are imported on first use so that ``import lczero_triton_b200`` stays cheap.
"""

from __future__ import annotations

import importlib

_LAZY = {
    "load_network": "format", "save_network": "format", "normalize_network": "format",
    "validate_network_format": "format", "NetworkFormatError": "format", "Network": "format",
    "Bt4Net": "net", "NativeNet": "native", "ShardedNet": "sharded", "NetConfig": "config", "CONFIGS": "config",
}


def __getattr__(name: str):
    if name in _LAZY:
        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    if name in ("ops", "net", "format", "config", "weights", "synthetic", "mapping_table", "sharded", "native", "build"):
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
