"""Network container: round trip, shape inference, and the error paths the reference tests for its
own loader (packages/lczero-triton/tests/test_bt4_format.py: bad files, missing weights, mismatched
layers)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from lczero_triton_b200 import format as fmt
from lczero_triton_b200.config import TINY
from lczero_triton_b200.weights import random_weights, scalar_constants


def test_round_trip_preserves_every_buffer(tmp_path) -> None:
    weights = random_weights(TINY, 5)
    path = tmp_path / "tiny.npz"
    fmt.save_network(path, weights, TINY)
    network = fmt.load_network(path)
    assert network.config == TINY
    assert set(network.weights) == set(weights)
    for key, value in weights.items():
        assert torch.equal(network.weights[key], value), key


def test_config_is_inferred_from_shapes_and_scalars_are_filled_in(tmp_path) -> None:
    weights = {k: v for k, v in random_weights(TINY, 6).items() if k not in scalar_constants(TINY)}
    path = tmp_path / "bare.npz"
    fmt.save_network(path, weights)  # no __config__, no scalar constants
    network = fmt.load_network(path)
    got, want = network.config, TINY
    assert (got.embedding, got.layers, got.heads, got.ffn, got.pos_enc) == (want.embedding, want.layers, want.heads, want.ffn, want.pos_enc)
    assert (got.smolgen_compress, got.smolgen_hidden, got.smolgen_gen) == (want.smolgen_compress, want.smolgen_hidden, want.smolgen_gen)
    for key, value in scalar_constants(TINY).items():
        assert float(network.weights[key].float()) == pytest.approx(value, rel=1e-2)


def test_unreadable_and_protobuf_files_are_rejected(tmp_path) -> None:
    bad = tmp_path / "garbage.npz"
    bad.write_bytes(b"not an archive")
    with pytest.raises(fmt.NetworkFormatError, match="invalid weights file"):
        fmt.load_network(bad)
    with pytest.raises(fmt.NetworkFormatError, match="net.proto"):
        fmt.load_network(tmp_path / "BT4.pb.gz")
    with pytest.raises(fmt.NetworkFormatError, match="invalid weights file"):
        fmt.load_network(tmp_path / "absent.npz")


def test_missing_and_misshapen_buffers_are_rejected() -> None:
    weights = random_weights(TINY, 7)
    network = fmt.Network(TINY, dict(weights))
    fmt.validate_network_format(network)
    del network.weights["/policy/promotion/matmul/w"]
    with pytest.raises(fmt.NetworkFormatError, match="missing /policy/promotion/matmul/w"):
        fmt.validate_network_format(network)
    network = fmt.Network(TINY, dict(weights))
    network.weights["/encoder1/ffn/dense1/w/w"] = torch.zeros((TINY.embedding, TINY.ffn + 8), dtype=torch.bfloat16)
    with pytest.raises(fmt.NetworkFormatError, match="/encoder1/ffn/dense1/w/w: expected shape"):
        fmt.validate_network_format(network)
    network = fmt.Network(TINY, dict(weights))
    network.weights[f"/encoder{TINY.layers}/mha/Q/w/w"] = weights["/encoder0/mha/Q/w/w"]
    with pytest.raises(fmt.NetworkFormatError, match="more encoder layers"):
        fmt.validate_network_format(network)


def test_normalisation_casts_to_storage_dtype() -> None:
    weights = {k: v.float().numpy().astype(np.float32) for k, v in random_weights(TINY, 8).items()}
    network = fmt.Network(TINY, {k: torch.from_numpy(v) for k, v in weights.items()})
    fmt.normalize_network(network)
    assert all(v.dtype == torch.bfloat16 and v.is_contiguous() for v in network.weights.values())
