"""The weight table against the reference's own buffer declarations.

``tests/golden/reference_buffer_names.json`` lists every named buffer of the reference's graph builder
(``packages/lczero-triton/src/lczero_triton/bt4/network.py``), read from its source by
``tests/golden/make_golden.py``.  Expanding its templates over the encoder layers, the Q / K / V labels
and the two dense heads must give exactly the names ``weights.weight_shapes`` and the C network object
(``lc0b200_net_weight_info``) expect, matrices must be input-major ``[K, N]`` with the K the reference
passes as ``input_width``, and the graph's inputs and outputs must be the four buffers the forward
API takes and returns.  No GPU: the C object only plans its arena here.
"""

from __future__ import annotations

import ctypes
import json
import pathlib

import pytest

from lczero_triton_b200 import config
from lczero_triton_b200.weights import scalar_constants, weight_shapes

ROWS = json.loads((pathlib.Path(__file__).parent / "golden" / "reference_buffer_names.json").read_text())


def _expand(cfg) -> dict[str, dict]:
    """Reference templates -> concrete names for a network of ``cfg.layers`` encoder layers."""
    out: dict[str, dict] = {}
    for row in ROWS:
        name = row["name"]
        if row["function"] == "_dense_output_head":
            prefixes = ["/value", "/mlh"]
        elif "{prefix}" in name:
            prefixes = [f"/encoder{i}" for i in range(cfg.layers)]
        else:
            prefixes = [""]
        labels = ["Q", "K", "V"] if "{label}" in name else [""]
        for prefix in prefixes:
            for label in labels:
                out[name.replace("{prefix}", prefix).replace("{label}", label)] = row
    return out


def _input_width(cfg, name: str, expression: str) -> int:
    """The reference's ``input_width=`` expression evaluated for ``cfg`` (network.py:343-1466)."""
    if name.startswith(("/value", "/mlh")):
        embed, hidden = (cfg.value_embed, cfg.value_hidden) if name.startswith("/value") else (cfg.mlh_embed, cfg.mlh_hidden)
        return {"body_width": cfg.embedding, "flattened_width": 64 * embed, "hidden_width": hidden}[expression]
    if "/smolgen/" in name:
        return {"body_width": cfg.embedding, "_SQUARE_COUNT * compression_width": 64 * cfg.smolgen_compress,
                "hidden_width": cfg.smolgen_hidden}[expression]
    table = {"position_input_width": 64 * 12, "embedding_input_width": 112 + cfg.pos_enc, "_SQUARE_COUNT": 64,
             "body_width": cfg.embedding, "hidden_width": cfg.ffn, "generated_width": cfg.smolgen_gen,
             "model_width": cfg.policy_model if name.startswith("/policy") else cfg.embedding,
             "policy_width": cfg.policy}
    return table[expression]


@pytest.mark.parametrize("cfg_name", ["TINY", "BT3", "BT4"])
def test_weight_table_equals_the_reference_declarations(cfg_name) -> None:
    cfg = getattr(config, cfg_name)
    reference = _expand(cfg)
    learned = {k: v for k, v in reference.items() if v["kind"] in ("matrix", "vector")}
    constants = {k for k, v in reference.items() if v["kind"] == "constant"}
    shapes = weight_shapes(cfg)
    assert set(shapes) == set(learned)
    assert set(scalar_constants(cfg)) == constants
    for name, row in learned.items():
        if row["kind"] == "matrix":
            assert len(shapes[name]) == 2 and shapes[name][0] == _input_width(cfg, name, row["input_width"]), name
        else:
            assert len(shapes[name]) == 1, name
    io = sorted(k for k, v in reference.items() if v["kind"] == "io")
    assert io == ["/input/plane_masks", "/input/plane_values", "/output/mlh", "/output/policy", "/output/wdl"]


@pytest.mark.parametrize("cfg_name", ["TINY", "BT4"])
@pytest.mark.parametrize("mode", ["bf16", "int8"])
def test_c_network_object_expects_the_reference_names(cfg_name, mode) -> None:
    from lczero_triton_b200 import _lib, build
    from lczero_triton_b200.native import NetConfigC

    build.build()
    lib = _lib.load()
    cfg = getattr(config, cfg_name)
    cfg_c = NetConfigC.from_config(cfg, mode)
    nbytes = lib.lc0b200_net_arena_bytes(ctypes.byref(cfg_c), 2)
    assert nbytes > 0
    handle = ctypes.c_void_p()
    # Planning needs an address to lay buffers out from, never the memory behind it: no device call is made.
    assert lib.lc0b200_net_create(ctypes.byref(handle), ctypes.byref(cfg_c), 2, ctypes.c_void_p(1 << 20), nbytes) == 0
    name, count = ctypes.c_char_p(), ctypes.c_longlong()
    got: dict[str, int] = {}
    for index in range(lib.lc0b200_net_weight_count(handle)):
        assert lib.lc0b200_net_weight_info(handle, index, ctypes.byref(name), ctypes.byref(count)) == 0
        got[name.value.decode()] = count.value
    lib.lc0b200_net_destroy(handle)
    want = {k: 1 for k in scalar_constants(cfg)}
    for key, shape in weight_shapes(cfg).items():
        want[key] = 1
        for extent in shape:
            want[key] *= extent
    assert got == want
    reference = {k for k, v in _expand(cfg).items() if v["kind"] != "io"}
    assert set(got) == reference
