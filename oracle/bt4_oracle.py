"""CPU oracle for the BT4 forward pass.  TEST INFRASTRUCTURE ONLY.

This is a plain fp32 PyTorch restatement, on the CPU, of the math the reference
emits as a graph of Triton kernels.  Nothing in the product package imports it;
only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
legs may.  The reference has no forward function that runs on a CPU (it is a
graph compiler whose executor lives in an lc0 fork that is not part of its
tree), so the oracle is pinned three ways:

* every op below follows the PyTorch reference written in the matching
  reference test (cited per function as ``T/<file>:<lines>``, relative to
  ``packages/lczero-triton/tests/``) or, where the test computes the expected
  value inline, the kernel source (``K/<file>``, relative to
  ``packages/lczero-triton/src/lczero_triton/bt4/kernels/``);
  ``tests/golden/reference_vectors.npz`` holds vectors produced by importing
  those reference test functions (``tests/test_oracle_golden.py``);
* ``tests/golden/reference_kernel_outputs.npz`` holds the outputs of every
  Triton kernel of the reference launched on a B200, and
  ``tests/test_kernel_golden.py`` checks every op here against them;
* the op ORDER follows ``packages/lczero-triton/src/lczero_triton/bt4/network.py``
  (``N:<lines>``), and ``tests/golden/reference_network_outputs.npz`` holds the
  outputs of that graph itself (the reference's builder, kernels and allocation
  plan, launched node by node on a B200) for a 4-layer, the BT3 and the BT4
  shape; ``tests/test_network_golden.py`` checks ``forward`` here against them
  (fp16 rounding apart: 2e-3 on BT4 policy logits).

Parity status: pinned per op and end to end for the fp16 graph the reference
builds.  The lc0 runtime boundary itself (the fork that would load the
executable) does not exist to compare with.  The int8 path has no reference
counterpart at all; see ``oracle/int8_oracle.py``.

``round_to`` makes the oracle round every tensor the GPU path materialises in
HBM to that dtype (a "rounded" oracle) so that kernel bugs can be told apart
from accumulated bf16 drift.  With ``round_to=None`` everything stays fp32.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

SQUARES = 64
INPUT_PLANES = 112
POSITION_PLANES = 12
POLICY_RECORD = 4288
PROMOTION_START = 4096
SOFTMAX_CLAMP = 131008.0  # twice the fp16 maximum, K/softmax_64.py:62-65
MISH_BRANCH = -0.6


def _round(x: torch.Tensor, round_to: torch.dtype | None) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).float()


# --------------------------------------------------------------------------- activations

def activate(values: torch.Tensor, activation: str) -> torch.Tensor:
    """Lc0's activation formulas in fp32 (T/test_layer_norm.py:40-53,
    T/test_add_vectors.py:16-30).  Mish is Lc0's rational form, not softplus/tanh."""
    if activation == "mish":
        e = torch.exp(values)
        n = e * e + 2.0 * e
        q = values / (n + 2.0)
        return torch.where(values <= MISH_BRANCH, n * q, values - 2.0 * q)
    if activation == "swish":
        return values / (1.0 + torch.exp(-values))
    if activation == "relu":
        return torch.clamp_min(values, 0.0)
    if activation == "none":
        return values
    raise ValueError(f"unknown activation {activation!r}")


# --------------------------------------------------------------------------- per-op oracles

def expand_planes(masks: torch.Tensor, values: torch.Tensor, storage: torch.dtype | None = None) -> torch.Tensor:
    """``out[p, sq] = bit sq of mask[p] ? value[p] : 0`` (K/expand_planes.py:34-42,
    T/test_expand_planes.py:29-35).  The value is cast to the storage dtype before
    the select.  ``masks`` is int64 holding the u64 bit pattern."""
    shifts = torch.arange(SQUARES, dtype=torch.int64)
    bits = ((masks.reshape(-1, 1) >> shifts) & 1) != 0
    vals = _round(values.reshape(-1, 1).float(), storage)
    return torch.where(bits, vals, torch.zeros((), dtype=torch.float32)).reshape(*masks.shape, SQUARES)


def nchw_to_nhwc(planes: torch.Tensor, kept: int = POSITION_PLANES) -> torch.Tensor:
    """First ``kept`` planes, square-major: ``[B,C,64] -> [B,64,kept]``
    (K/nchw_to_nhwc.py:36-44, T/test_nchw_to_nhwc.py:43)."""
    return planes[:, :kept, :].permute(0, 2, 1).contiguous()


def preprocess_attention_body(planes: torch.Tensor, position: torch.Tensor) -> torch.Tensor:
    """Per token: 112 plane values then E positional channels
    (K/preprocess_attention_body.py:40-61, T/test_preprocess_attention_body.py:46)."""
    return torch.cat((planes.permute(0, 2, 1), position), dim=2)


def input_gating(x: torch.Tensor, mult: torch.Tensor, add: torch.Tensor) -> torch.Tensor:
    """``x * mult[sq, c] + add[sq, c]`` broadcast over the batch
    (K/input_gating.py:37-51, T/test_input_gating.py:34-36)."""
    return x.float() * mult.float() + add.float()


def add_vectors(x: torch.Tensor, bias: torch.Tensor, activation: str) -> torch.Tensor:
    """``act(x + bias[i mod n])`` over the flattened tensor
    (K/add_vectors.py:47-66, T/test_add_vectors.py:46)."""
    n = bias.numel()
    flat = x.float().reshape(-1, n) + bias.float().reshape(1, n)
    return activate(flat, activation).reshape(x.shape)


def add_bias_batched(x: torch.Tensor, bias: torch.Tensor, activation: str) -> torch.Tensor:
    """``act(x[bt, row, c] + bias[bt, c])`` (K/add_bias_batched.py:46-66,
    T/test_add_bias_batched.py:53)."""
    return activate(x.float() + bias.float()[:, None, :], activation)


def matmul(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Row-major ``A[M,K] @ W[K,N]`` with fp32 accumulation (T/test_matmul.py:106).
    The reference kernel may accumulate in fp16 (K/matmul.py:18); the oracle does not."""
    return a.float() @ w.float()


def layer_norm(x: torch.Tensor, bias: torch.Tensor, gammas: torch.Tensor, betas: torch.Tensor,
               activation: str, epsilon: float, *, skip: torch.Tensor | None = None,
               alpha: torch.Tensor | float | None = None) -> torch.Tensor:
    """bias -> activation -> alpha*branch + skip -> normalise (population variance,
    centred) -> gamma, beta (K/layer_norm.py:57-87, T/test_layer_norm.py:56-74)."""
    v = activate(x.float() + bias.float(), activation)
    if skip is not None:
        a = alpha.float() if isinstance(alpha, torch.Tensor) else float(alpha)
        v = a * v + skip.float()
    mean = v.mean(dim=-1, keepdim=True)
    var = ((v - mean) ** 2).mean(dim=-1, keepdim=True)
    return (v - mean) / torch.sqrt(var + epsilon) * gammas.float() + betas.float()


def body_qk(q: torch.Tensor, k: torch.Tensor, scale: float, heads: int) -> torch.Tensor:
    """``scale * Q_h K_h^T`` with heads interleaved in the channel dimension:
    ``[B,64,H*d] -> [B,H,64,64]`` (K/batched_matmul.py:95-99,140-141,
    T/test_batched_matmul.py:127-133)."""
    b, t, hd = q.shape
    qh = q.float().view(b, t, heads, hd // heads).permute(0, 2, 1, 3)
    kh = k.float().view(b, t, heads, hd // heads).permute(0, 2, 1, 3)
    return torch.matmul(qh, kh.transpose(-1, -2)) * scale


def softmax_64(scaled_qk: torch.Tensor, smolgen: torch.Tensor) -> torch.Tensor:
    """``softmax(clamp(qk + smolgen, +-131008))`` over rows of 64; NaN rows stay NaN
    (K/softmax_64.py:58-71, T/test_softmax_64.py:37-41)."""
    v = scaled_qk.float() + smolgen.float()
    v = torch.clamp(v, -SOFTMAX_CLAMP, SOFTMAX_CLAMP)
    return torch.softmax(v, dim=-1)


def attention_v(p: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``P[b,h] @ V[b,:,h]`` written merged ``[B,64,H*d]`` (K/batched_matmul.py:174-177,
    206-210, T/test_batched_matmul.py:167-170)."""
    b, h, t, _ = p.shape
    vh = v.float().view(b, t, h, -1).permute(0, 2, 1, 3)
    return torch.matmul(p.float(), vh).permute(0, 2, 1, 3).reshape(b, t, -1)


def policy_qk(q: torch.Tensor, k: torch.Tensor, scale: float, records: torch.Tensor | None = None) -> torch.Tensor:
    """``rec[b, i*64 + j] = scale * Qp[b,i] . Kp[b,j]`` into a record of stride 4288;
    the 192 promotion slots are left untouched (K/batched_matmul.py:100-105,
    T/test_batched_matmul.py:184-214)."""
    b = q.shape[0]
    if records is None:
        records = torch.zeros((b, POLICY_RECORD), dtype=torch.float32)
    qk = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    records = records.clone().float()
    records[:, :PROMOTION_START] = qk.reshape(b, PROMOTION_START)
    return records


def promotion_logits(records: torch.Tensor, keys: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """192 promotion logits per position (K/promotion_logits.py:118-145,
    T/test_promotion_logits.py:40-52): project key rows 56..63 with ``W[Pm,4]``, add
    channel 3 to channels 0..2, add to the QK block rows 48..55 x cols 56..63."""
    proj = torch.matmul(keys[:, 56:64].float(), w.float())  # [B, 8 to-files, 4]
    offsets = proj[:, :, :3] + proj[:, :, 3:4]
    qk = records[:, :PROMOTION_START].reshape(-1, 64, 64)[:, 48:56, 56:64].float()
    return (qk[:, :, :, None] + offsets[:, None, :, :]).reshape(-1, 192)


def policy_map(records: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Index gather with out-of-range indices producing 0 (K/policy_map.py:40-49,
    T/test_policy_map.py:38,42-61)."""
    table = table.long()
    valid = (table >= 0) & (table < records.shape[1])
    gathered = records[:, table.clamp(0, records.shape[1] - 1)]
    return torch.where(valid[None, :], gathered, torch.zeros((), dtype=records.dtype))


def output_probabilities(policy_logits: torch.Tensor, wdl_logits: torch.Tensor,
                         legal_mask: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """What lc0 does right after the graph (BT4_PLAN.md:42-43: the graph emits raw WDL logits, the
    softmax is applied on the host; BT4_PLAN.md:753 "Host WDL softmax and Q/D conversion"): WDL softmax,
    the policy softmax over the legal moves only, and ``(Q, D) = (W - L, D)``."""
    wdl = torch.softmax(wdl_logits.float(), dim=-1)
    logits = policy_logits.float()
    if legal_mask is not None:
        logits = torch.where(legal_mask != 0, logits, torch.full_like(logits, float("-inf")))
    policy = torch.softmax(logits, dim=-1)
    return torch.nan_to_num(policy, nan=0.0), wdl, torch.stack((wdl[:, 0] - wdl[:, 2], wdl[:, 1]), dim=1)


# --------------------------------------------------------------------------- whole network

def forward(weights: Mapping[str, torch.Tensor], cfg, masks: torch.Tensor, values: torch.Tensor, *,
            table: torch.Tensor, round_to: torch.dtype | None = None,
            taps: dict[str, torch.Tensor] | None = None, int8: bool = False):
    """fp32 forward in the reference's op order (N:343-643 embedding, N:705-850
    smolgen, N:853-1076 attention, N:1079-1186 FFN, N:1189-1356 policy,
    N:1409-1550 value / moves-left).

    Returns ``(policy f32[B,1858], wdl f32[B,3] raw logits, mlh f32[B,1])``.
    ``taps`` (optional dict) receives named intermediates for per-stage diffing.
    ``int8=True`` sends the four large GEMMs of every encoder layer (QKV, attention
    output, FFN dense1 and dense2) through ``oracle/int8_oracle.py`` on bf16-rounded
    activations; there is no reference counterpart for that mode.
    """
    if int8:
        from oracle import int8_oracle

        def big(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
            return int8_oracle.linear(a.to(torch.bfloat16), weight)
    else:
        big = matmul
    w = {k: v.float() for k, v in weights.items()}
    r = lambda x: _round(x, round_to)  # noqa: E731
    b = masks.shape[0]
    t = b * SQUARES
    d, h, e = cfg.embedding, cfg.heads, cfg.pos_enc
    eps = cfg.ln_eps

    def tap(name: str, x: torch.Tensor) -> None:
        if taps is not None:
            taps[name] = x.detach().clone()

    # ---- embedding
    planes = expand_planes(masks, values, round_to)  # [B,112,64]
    pos_in = nchw_to_nhwc(planes).reshape(b, SQUARES * POSITION_PLANES)
    position = r(add_vectors(matmul(pos_in, w["/attn_body/embedding/preprocess/matmul/w"]),
                             w["/attn_body/embedding/preprocess/add/w"], "none"))
    emb_in = preprocess_attention_body(planes, position.reshape(b, SQUARES, e)).reshape(t, INPUT_PLANES + e)
    projected = r(matmul(emb_in, w["/attn_body/matmul/w"]))
    skip = layer_norm(projected, w["/attn_body/add/w"], w["/attn_body/ln/w/scale"], w["/attn_body/ln/w/bias"],
                      "mish", eps)
    skip = r(input_gating(skip.reshape(b, SQUARES, d), w["/ip_mul_gate/w"], w["/ip_add_gate/w"]).reshape(t, d))
    hidden = r(add_bias_batched(matmul(skip, w["/attn_body/ffn/dense1/w/w"])[None],
                                w["/attn_body/ffn/dense1/b/w"][None], "mish")[0])
    branch = r(matmul(hidden, w["/attn_body/ffn/dense2/w/w"]))
    body = r(layer_norm(branch, w["/attn_body/ffn/dense2/b/w"], w["/attn_body/ln2/w/scale"],
                        w["/attn_body/ln2/w/bias"], "none", eps, skip=skip, alpha=w["/attn_body/ffn/alpha/w"]))
    tap("embedding", body)

    # ---- encoder tower
    for i in range(cfg.layers):
        p = f"/encoder{i}"
        compressed = r(matmul(body, w[f"{p}/smolgen/compress/w"]))  # [T, C]
        hid = r(matmul(compressed.reshape(b, -1), w[f"{p}/smolgen/dense1/w/w"]))
        hid = r(layer_norm(hid, w[f"{p}/smolgen/dense1/b/w"], w[f"{p}/smolgen/ln1/w/scale"],
                           w[f"{p}/smolgen/ln1/w/bias"], "swish", eps))
        gen = r(matmul(hid, w[f"{p}/smolgen/dense2/w/w"]))
        gen = r(layer_norm(gen, w[f"{p}/smolgen/dense2/b/w"], w[f"{p}/smolgen/ln2/w/scale"],
                           w[f"{p}/smolgen/ln2/w/bias"], "swish", eps))
        smolgen = r(matmul(gen.reshape(b * h, -1), w["/const/smolgen_w"])).reshape(b, h, SQUARES, SQUARES)

        q = r(big(body, w[f"{p}/mha/Q/w/w"]) + w[f"{p}/mha/Q/b/w"])
        k = r(big(body, w[f"{p}/mha/K/w/w"]) + w[f"{p}/mha/K/b/w"])
        v = r(big(body, w[f"{p}/mha/V/w/w"]) + w[f"{p}/mha/V/b/w"])
        scale = float(w[f"{p}/mha/QK/scale/w"])
        qk = body_qk(q.reshape(b, SQUARES, d), k.reshape(b, SQUARES, d), scale, h)
        probs = softmax_64(qk, smolgen)
        merged = r(attention_v(probs, v.reshape(b, SQUARES, d)).reshape(t, d))
        branch = r(big(merged, w[f"{p}/mha/out/dense/w/w"]))
        attended = r(layer_norm(branch, w[f"{p}/mha/out/dense/b/w"], w[f"{p}/ln1/w/scale"], w[f"{p}/ln1/w/bias"],
                                "none", eps, skip=body, alpha=w[f"{p}/alpha*input/w"]))
        hidden = r(add_bias_batched(big(attended, w[f"{p}/ffn/dense1/w/w"])[None],
                                    w[f"{p}/ffn/dense1/b/w"][None], "mish")[0])
        branch = r(big(hidden, w[f"{p}/ffn/dense2/w/w"]))
        body = r(layer_norm(branch, w[f"{p}/ffn/dense2/b/w"], w[f"{p}/ln2/w/scale"], w[f"{p}/ln2/w/bias"],
                            "none", eps, skip=attended, alpha=w[f"{p}/ffn/alpha/w"]))
        tap(f"encoder{i}", body)

    # ---- policy head
    emb = r(add_bias_batched(matmul(body, w["/policy/dense1/matmul/w"])[None],
                             w["/policy/dense1/add/w"][None], "mish")[0])
    qp = r(matmul(emb, w["/policy/Q/matmul/w"]) + w["/policy/Q/add/w"]).reshape(b, SQUARES, -1)
    kp = r(matmul(emb, w["/policy/K/matmul/w"]) + w["/policy/K/add/w"]).reshape(b, SQUARES, -1)
    records = r(policy_qk(qp, kp, float(w["/policy/scale/w"])))
    records[:, PROMOTION_START:] = r(promotion_logits(records, kp, w["/policy/promotion/matmul/w"]))
    tap("policy_records", records)
    policy = policy_map(records, table).float()

    # ---- value and moves-left heads
    def dense_head(prefix: str, final_activation: str) -> torch.Tensor:
        x = r(add_vectors(matmul(body, w[f"{prefix}/embed/matmul/w"]), w[f"{prefix}/embed/add/w"], "mish"))
        x = r(add_vectors(matmul(x.reshape(b, -1), w[f"{prefix}/dense1/matmul/w"]), w[f"{prefix}/dense1/add/w"], "mish"))
        x = r(add_vectors(matmul(x, w[f"{prefix}/dense2/matmul/w"]), w[f"{prefix}/dense2/add/w"], final_activation))
        return x.float()

    wdl = dense_head("/value", "none")
    mlh = dense_head("/mlh", "relu")
    return policy, wdl, mlh
