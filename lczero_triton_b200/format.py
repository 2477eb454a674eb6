"""Network files: loading, normalisation and format validation.

Keeps the reference's entry points (``load_network``, ``normalize_network``,
``validate_network_format``, ``NetworkFormatError``;
packages/lczero-triton/src/lczero_triton/bt4/_format.py:12-114) for the container this
project can read offline: an ``.npz`` archive whose arrays are keyed by the reference's canonical
buffer names in its ``[K, N]`` layout (network.py:349-1466), plus an optional ``__config__``
JSON entry.  Lc0's own ``.pb.gz`` files need Python bindings generated from ``net.proto`` of
the lc0 source tree (the reference generates them at build time, justfile:11-18); without them a
``.pb.gz`` path is rejected with an explanation instead of being mis-parsed.
"""

from __future__ import annotations

import dataclasses
import json
import pathlib
from collections.abc import Mapping

import numpy as np
import torch

from .config import INPUT_PLANES, SQUARES, NetConfig
from .weights import scalar_constants, weight_shapes


class NetworkFormatError(ValueError):
    """The source network cannot be run by the BT4 forward pass."""


@dataclasses.dataclass
class Network:
    """A network in memory: its shape and its buffers under the reference's canonical names."""

    config: NetConfig
    weights: dict[str, torch.Tensor]


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise NetworkFormatError(message)


def infer_config(weights: Mapping[str, torch.Tensor], name: str = "inferred") -> NetConfig:
    """Derive every width from buffer shapes, the way the reference reads them off the protobuf
    layer sizes (network.py:349-372, :715-774, :877-936)."""
    def shape(key: str) -> tuple[int, ...]:
        _require(key in weights, f"weights: missing {key}")
        return tuple(weights[key].shape)

    emb = shape("/attn_body/matmul/w")
    _require(len(emb) == 2 and emb[0] > INPUT_PLANES, "/attn_body/matmul/w: expected [112 + E, D]")
    d, pos_enc = emb[1], emb[0] - INPUT_PLANES
    layers = 0
    while f"/encoder{layers}/mha/Q/w/w" in weights:
        layers += 1
    _require(layers > 0, "weights.encoder: no encoder layers")
    ffn = shape("/encoder0/ffn/dense1/w/w")[1]
    compress = shape("/encoder0/smolgen/compress/w")[1]
    hidden = shape("/encoder0/smolgen/dense1/w/w")[1]
    gen = shape("/const/smolgen_w")[0]
    total_gen = shape("/encoder0/smolgen/dense2/w/w")[1]
    _require(total_gen % gen == 0, "/encoder0/smolgen/dense2/w/w: width is not a multiple of the per-head width")
    heads = total_gen // gen
    _require(d % heads == 0 and d // heads == 32, "mha: only a per-head depth of 32 is supported")
    return NetConfig(name, embedding=d, layers=layers, heads=heads, ffn=ffn, pos_enc=pos_enc,
                     smolgen_compress=compress, smolgen_hidden=hidden, smolgen_gen=gen,
                     policy=shape("/policy/dense1/matmul/w")[1], policy_model=shape("/policy/Q/matmul/w")[1],
                     value_embed=shape("/value/embed/matmul/w")[1], value_hidden=shape("/value/dense1/matmul/w")[1],
                     mlh_embed=shape("/mlh/embed/matmul/w")[1], mlh_hidden=shape("/mlh/dense1/matmul/w")[1])


def normalize_network(network: Network) -> None:
    """In place: bf16 storage, contiguous buffers, and the one-element constants the reference only
    names (alpha, attention and policy scales; network.py:432-437, :925-936, :1246-1251) filled in
    when the file does not carry them."""
    for key, value in list(network.weights.items()):
        network.weights[key] = torch.as_tensor(value).to(torch.bfloat16).contiguous()
    for key, value in scalar_constants(network.config).items():
        if key not in network.weights:
            network.weights[key] = torch.tensor([value], dtype=torch.float32).to(torch.bfloat16)


def validate_network_format(network: Network) -> None:
    """Reject a network the forward pass cannot traverse: every buffer present, with the shape the
    graph expects (the reference rejects missing heads, missing encoders and mismatched layer sizes,
    _format.py:103-259)."""
    cfg = network.config
    _require(cfg.embedding % cfg.heads == 0 and cfg.head_depth == 32, "mha: only a per-head depth of 32 is supported")
    _require(cfg.layers > 0, "weights.encoder: no encoder layers")
    expected = weight_shapes(cfg)
    for key, shape in expected.items():
        _require(key in network.weights, f"weights: missing {key}")
        got = tuple(network.weights[key].shape)
        _require(got == tuple(shape), f"{key}: expected shape {tuple(shape)}, found {got}")
    for key in scalar_constants(cfg):
        _require(key in network.weights and network.weights[key].numel() == 1, f"weights: missing scalar {key}")
    extra = f"/encoder{cfg.layers}/mha/Q/w/w"
    _require(extra not in network.weights, f"weights.encoder: more encoder layers than the configuration ({cfg.layers})")
    _require(expected["/const/smolgen_w"][1] == SQUARES * SQUARES, "/const/smolgen_w: expected 4096 columns")


def save_network(path: str | pathlib.Path, weights: Mapping[str, torch.Tensor], config: NetConfig | None = None) -> None:
    """Write the ``.npz`` container (bf16 buffers are stored as their uint16 bit patterns)."""
    arrays = {}
    for key, value in weights.items():
        t = torch.as_tensor(value).detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            arrays["bf16:" + key] = t.view(torch.int16).numpy()
        else:
            arrays["f32:" + key] = t.float().numpy()
    if config is not None:
        arrays["__config__"] = np.frombuffer(json.dumps(dataclasses.asdict(config)).encode(), dtype=np.uint8)
    np.savez(path, **arrays)


def load_network(path: str | pathlib.Path) -> Network:
    """Read, normalise and validate one network file."""
    path = pathlib.Path(path)
    if path.name.endswith((".pb.gz", ".pb")):
        raise NetworkFormatError(
            f"invalid weights file {path}: Lc0 protobuf networks need bindings generated from lc0's net.proto, "
            "which are not available; export the buffers to the .npz container (format.save_network)")
    try:
        with np.load(path) as archive:
            entries = {key: archive[key] for key in archive.files}
    except (OSError, ValueError) as error:
        raise NetworkFormatError(f"invalid weights file {path}: {error}") from error
    config = None
    weights: dict[str, torch.Tensor] = {}
    for key, array in entries.items():
        if key == "__config__":
            try:
                config = NetConfig(**json.loads(bytes(array.tobytes()).decode()))
            except (TypeError, ValueError) as error:
                raise NetworkFormatError(f"invalid weights file {path}: bad __config__ ({error})") from error
        elif key.startswith("bf16:"):
            weights[key[5:]] = torch.from_numpy(np.ascontiguousarray(array)).view(torch.bfloat16)
        elif key.startswith("f32:"):
            weights[key[4:]] = torch.from_numpy(np.ascontiguousarray(array))
        else:
            weights[key] = torch.from_numpy(np.ascontiguousarray(array))
    _require(bool(weights), f"invalid weights file {path}: missing weights")
    network = Network(config if config is not None else infer_config(weights), weights)
    normalize_network(network)
    validate_network_format(network)
    return network
