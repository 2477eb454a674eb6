"""Static network shapes for the BT4-style forward pass.

The reference bakes every shape into its kernel specializations at graph-build
time (packages/lczero-triton/src/lczero_triton/bt4/network.py:343-1550 reads
them from the protobuf layer sizes).  Here they live in one dataclass.
"""

from __future__ import annotations

from dataclasses import dataclass

SQUARES = 64
INPUT_PLANES = 112
POSITION_PLANES = 12
POLICY_RECORD = 4288
POLICY_SIZE = 1858
PROMOTION_START = 4096


@dataclass(frozen=True)
class NetConfig:
    """Shape of one Lc0 attention-body network."""

    name: str
    embedding: int  # D, body width
    layers: int  # L, encoder count
    heads: int  # H
    ffn: int  # F, encoder and embedding FFN hidden width
    pos_enc: int  # E, positional-encoding channels per square
    smolgen_compress: int  # C, channels per token after compression
    smolgen_hidden: int  # S1, width after smolgen dense1
    smolgen_gen: int  # G, per-head generated width (rows of /const/smolgen_w)
    policy: int  # P, policy embedding width
    policy_model: int  # Pm, policy query/key width
    value_embed: int = 128
    value_hidden: int = 128
    mlh_embed: int = 32
    mlh_hidden: int = 128
    ln_eps: float = 1e-3

    @property
    def head_depth(self) -> int:
        return self.embedding // self.heads

    @property
    def alpha(self) -> float:
        """DeepNorm residual scale, (2 L)^(-1/4) (BT4_PLAN.md:70)."""
        return float((2.0 * self.layers) ** -0.25)

    @property
    def qk_scale(self) -> float:
        return float(self.head_depth ** -0.5)

    @property
    def policy_scale(self) -> float:
        return float(self.policy_model ** -0.5)

    def flops_per_position(self) -> float:
        """Algorithmic FLOPs (2 M N K over every GEMM and both attention matmuls)."""
        d, f, e, c = self.embedding, self.ffn, self.pos_enc, self.smolgen_compress
        s1, g, h = self.smolgen_hidden, self.smolgen_gen, self.heads
        t = SQUARES
        total = 0.0
        total += 2.0 * (SQUARES * POSITION_PLANES) * (SQUARES * e)  # positional dense
        total += 2.0 * t * (INPUT_PLANES + e) * d  # embedding
        total += 2.0 * t * d * f * 2  # embedding FFN
        per_layer = 0.0
        per_layer += 2.0 * t * d * c  # smolgen compress
        per_layer += 2.0 * (t * c) * s1  # smolgen dense1
        per_layer += 2.0 * s1 * (h * g)  # smolgen dense2
        per_layer += 2.0 * h * g * 4096  # shared 64x64 projection
        per_layer += 2.0 * t * d * d * 3  # Q, K, V
        per_layer += 2.0 * h * t * t * self.head_depth * 2  # QK^T and PV
        per_layer += 2.0 * t * d * d  # out projection
        per_layer += 2.0 * t * d * f * 2  # FFN
        total += self.layers * per_layer
        p, pm = self.policy, self.policy_model
        total += 2.0 * t * d * p + 2.0 * t * p * pm * 2  # policy dense + Q + K
        total += 2.0 * t * t * pm  # policy QK^T
        total += 2.0 * 8 * pm * 4  # promotion projection
        total += 2.0 * t * d * self.value_embed
        total += 2.0 * (t * self.value_embed) * self.value_hidden + 2.0 * self.value_hidden * 3
        total += 2.0 * t * d * self.mlh_embed
        total += 2.0 * (t * self.mlh_embed) * self.mlh_hidden + 2.0 * self.mlh_hidden * 1
        return total


TINY = NetConfig("tiny", embedding=128, layers=4, heads=4, ffn=256, pos_enc=64,
                 smolgen_compress=16, smolgen_hidden=64, smolgen_gen=64,
                 policy=128, policy_model=128)
BT3 = NetConfig("bt3", embedding=768, layers=15, heads=24, ffn=1024, pos_enc=512,
                smolgen_compress=32, smolgen_hidden=256, smolgen_gen=256,
                policy=768, policy_model=768)
BT4 = NetConfig("bt4", embedding=1024, layers=15, heads=32, ffn=1536, pos_enc=512,
                smolgen_compress=32, smolgen_hidden=256, smolgen_gen=256,
                policy=1024, policy_model=1024)

CONFIGS = {c.name: c for c in (TINY, BT3, BT4)}
