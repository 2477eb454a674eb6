"""Canonical weight names, shapes and seeded random initialisation.

Names and the input-major ``[K, N]`` matrix layout are the ones the reference
declares for its persistent buffers
(packages/lczero-triton/src/lczero_triton/bt4/network.py:349-449 embedding,
:715-774 smolgen, :868-936 attention, :1089-1132 FFN, :1198-1251 policy,
:1427-1466 value / moves-left heads).
"""

from __future__ import annotations

import torch

from .config import INPUT_PLANES, POSITION_PLANES, SQUARES, NetConfig


def weight_shapes(cfg: NetConfig) -> dict[str, tuple[int, ...]]:
    """Every learned buffer the forward pass consumes, name -> shape."""
    d, f, e = cfg.embedding, cfg.ffn, cfg.pos_enc
    c, s1, g, h = cfg.smolgen_compress, cfg.smolgen_hidden, cfg.smolgen_gen, cfg.heads
    shapes: dict[str, tuple[int, ...]] = {
        "/attn_body/embedding/preprocess/matmul/w": (SQUARES * POSITION_PLANES, SQUARES * e),
        "/attn_body/embedding/preprocess/add/w": (SQUARES * e,),
        "/attn_body/matmul/w": (INPUT_PLANES + e, d),
        "/attn_body/add/w": (d,),
        "/attn_body/ln/w/scale": (d,),
        "/attn_body/ln/w/bias": (d,),
        "/ip_mul_gate/w": (SQUARES, d),
        "/ip_add_gate/w": (SQUARES, d),
        "/attn_body/ffn/dense1/w/w": (d, f),
        "/attn_body/ffn/dense1/b/w": (f,),
        "/attn_body/ffn/dense2/w/w": (f, d),
        "/attn_body/ffn/dense2/b/w": (d,),
        "/attn_body/ln2/w/scale": (d,),
        "/attn_body/ln2/w/bias": (d,),
        "/const/smolgen_w": (g, SQUARES * SQUARES),
    }
    for i in range(cfg.layers):
        p = f"/encoder{i}"
        shapes.update({
            f"{p}/smolgen/compress/w": (d, c),
            f"{p}/smolgen/dense1/w/w": (SQUARES * c, s1),
            f"{p}/smolgen/dense1/b/w": (s1,),
            f"{p}/smolgen/ln1/w/scale": (s1,),
            f"{p}/smolgen/ln1/w/bias": (s1,),
            f"{p}/smolgen/dense2/w/w": (s1, h * g),
            f"{p}/smolgen/dense2/b/w": (h * g,),
            f"{p}/smolgen/ln2/w/scale": (h * g,),
            f"{p}/smolgen/ln2/w/bias": (h * g,),
            f"{p}/mha/Q/w/w": (d, d),
            f"{p}/mha/Q/b/w": (d,),
            f"{p}/mha/K/w/w": (d, d),
            f"{p}/mha/K/b/w": (d,),
            f"{p}/mha/V/w/w": (d, d),
            f"{p}/mha/V/b/w": (d,),
            f"{p}/mha/out/dense/w/w": (d, d),
            f"{p}/mha/out/dense/b/w": (d,),
            f"{p}/ln1/w/scale": (d,),
            f"{p}/ln1/w/bias": (d,),
            f"{p}/ffn/dense1/w/w": (d, f),
            f"{p}/ffn/dense1/b/w": (f,),
            f"{p}/ffn/dense2/w/w": (f, d),
            f"{p}/ffn/dense2/b/w": (d,),
            f"{p}/ln2/w/scale": (d,),
            f"{p}/ln2/w/bias": (d,),
        })
    shapes.update({
        "/policy/dense1/matmul/w": (d, cfg.policy),
        "/policy/dense1/add/w": (cfg.policy,),
        "/policy/Q/matmul/w": (cfg.policy, cfg.policy_model),
        "/policy/Q/add/w": (cfg.policy_model,),
        "/policy/K/matmul/w": (cfg.policy, cfg.policy_model),
        "/policy/K/add/w": (cfg.policy_model,),
        "/policy/promotion/matmul/w": (cfg.policy_model, 4),
        "/value/embed/matmul/w": (d, cfg.value_embed),
        "/value/embed/add/w": (cfg.value_embed,),
        "/value/dense1/matmul/w": (SQUARES * cfg.value_embed, cfg.value_hidden),
        "/value/dense1/add/w": (cfg.value_hidden,),
        "/value/dense2/matmul/w": (cfg.value_hidden, 3),
        "/value/dense2/add/w": (3,),
        "/mlh/embed/matmul/w": (d, cfg.mlh_embed),
        "/mlh/embed/add/w": (cfg.mlh_embed,),
        "/mlh/dense1/matmul/w": (SQUARES * cfg.mlh_embed, cfg.mlh_hidden),
        "/mlh/dense1/add/w": (cfg.mlh_hidden,),
        "/mlh/dense2/matmul/w": (cfg.mlh_hidden, 1),
        "/mlh/dense2/add/w": (1,),
    })
    return shapes


def scalar_constants(cfg: NetConfig) -> dict[str, float]:
    """One-element constant buffers (the reference only names them,
    network.py:432-437, :925-936, :1246-1251; values come from the lc0 loader)."""
    out = {"/attn_body/ffn/alpha/w": cfg.alpha, "/policy/scale/w": cfg.policy_scale}
    for i in range(cfg.layers):
        out[f"/encoder{i}/mha/QK/scale/w"] = cfg.qk_scale
        out[f"/encoder{i}/alpha*input/w"] = cfg.alpha
        out[f"/encoder{i}/ffn/alpha/w"] = cfg.alpha
    return out


def random_weights(cfg: NetConfig, seed: int = 0, *, dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02) -> dict[str, torch.Tensor]:
    """Seeded N(0, std) weights rounded to the storage dtype (CPU tensors).

    LayerNorm scales are 1 + N(0, std): pure N(0, std) scales collapse every
    normalised activation to ~0 and make the network degenerate.
    """
    gen = torch.Generator().manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, shape in weight_shapes(cfg).items():
        w = torch.randn(shape, generator=gen, dtype=torch.float32) * std
        if name.endswith("/w/scale"):
            w = w + 1.0
        if name == "/ip_mul_gate/w":
            w = w + 1.0
        out[name] = w.to(dtype)
    for name, value in scalar_constants(cfg).items():
        out[name] = torch.tensor([value], dtype=torch.float32).to(dtype)
    return out
