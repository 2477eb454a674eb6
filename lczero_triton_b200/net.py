"""Host-side forward pass: the reference's graph grammar executed on the sm_100a kernels.

``Bt4Net`` consumes a weight dictionary keyed by the reference's canonical buffer
names in its input-major ``[K, N]`` layout
(packages/lczero-triton/src/lczero_triton/bt4/network.py:343-1550) and exposes

    forward(plane_masks i64[B,112] (u64 bit patterns), plane_values f32[B,112])
        -> (policy f32[B,1858], wdl f32[B,3] raw logits, mlh f32[B,1])

which is the reference's execution I/O contract (network.py:328-340, :1252-1257,
:1467-1472; BT4_PLAN.md:83-89).  The op order follows ``_embedding`` (:343-643),
``_smolgen`` (:705-850), ``_attention`` (:853-1076), ``_ffn`` (:1079-1186),
``_policy_head`` (:1189-1356) and ``_dense_output_head`` (:1409-1550), with these
fusions: bias/activation live in GEMM epilogues, QK^T + smolgen bias + softmax + PV
is one kernel, Q/K/V (and, where 3 x embedding is a multiple of 256, smolgen's compression as trailing
columns with an output of their own) is one GEMM over a concatenated weight, plane expansion is
folded into the two embedding gather kernels, and promotion + gather + f32
widening is one kernel.

Everything runs through the C ABI (``include/lc0b200.h``); PyTorch only owns the
device memory and the stream.  There is no CPU path.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass

import torch

from . import _lib, mapping_table, ops
from .config import INPUT_PLANES, POLICY_RECORD, POLICY_SIZE, POSITION_PLANES, SQUARES, NetConfig


@dataclass
class _Dense:
    """One dense layer prepared for the GEMM kernel."""

    w: torch.Tensor  # bf16 or int8, layout per ``layout``
    layout: int  # _lib.W_NK or _lib.W_KN
    n: int
    k: int
    bias: torch.Tensor | None = None
    col_scale: torch.Tensor | None = None  # f32 [n] for int8 weights
    fold_c: torch.Tensor | None = None  # f32 [n]: column sums of the gamma-scaled weight (deferred LayerNorm)
    fold_d: torch.Tensor | None = None  # f32 [n]: beta^T W + bias


def quantize_weight_per_channel(w_kn: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-output-channel int8: ``s[n] = max_k |W[k,n]| / 127`` (1 for an all-zero
    column), ``Wq = clamp(rint(W / s), -127, 127)``.  Returns ``(Wq int8 [N,K], s f32 [N])``."""
    w = w_kn.float()
    amax = w.abs().amax(dim=0)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(w / scale), -127, 127).to(torch.int8)
    return q.t().contiguous(), scale.contiguous()


class Bt4Net:
    """A BT4-style network resident on one GPU."""

    def __init__(self, weights: Mapping[str, torch.Tensor], config: NetConfig, *, device: str | torch.device = "cuda",
                 mode: str = "bf16", weight_layout: str = "nk", deferred_layer_norm: bool | None = None) -> None:
        if mode not in ("bf16", "int8"):
            raise ValueError("mode must be 'bf16' or 'int8'")
        if weight_layout not in ("nk", "kn"):
            raise ValueError("weight_layout must be 'nk' (pre-transposed) or 'kn' (reference layout)")
        _lib.load()  # fail loudly now if the CUDA library is not built
        self.cfg = config
        self.mode = mode
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("Bt4Net needs a CUDA device; there is no CPU path")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        # The residual stream is kept un-normalised between GEMMs ("deferred LayerNorm"): the two
        # LayerNorm launches per encoder layer become epilogue arithmetic (see lc0b200_gemm_args).  In
        # int8 mode the GEMMs that read the stream need quantised rows, which one light kernel makes
        # from the un-normalised rows and the partial sums (ops.normalize_quantize_rows); measured 2 %
        # faster than stand-alone LayerNorm kernels that also emit the int8 rows.
        self.deferred = True if deferred_layer_norm is None else bool(deferred_layer_norm)
        self._layout = _lib.W_NK if weight_layout == "nk" else _lib.W_KN
        self._w = {k: v.to(device=self.device, dtype=torch.bfloat16).contiguous() for k, v in weights.items()}
        self._scalars = {k: float(v.float().reshape(-1)[0]) for k, v in weights.items() if v.numel() == 1}
        self.table = torch.tensor(mapping_table.values(), dtype=torch.int32, device=self.device)
        self._workspaces: dict[int, dict[str, torch.Tensor]] = {}
        self._prepare()

    # ------------------------------------------------------------------ weight preparation
    def _dense(self, name: str, bias: str | None = None, *, int8: bool = False) -> _Dense:
        w_kn = self._w[name]
        k, n = w_kn.shape
        b = self._w[bias] if bias is not None else None
        if int8:
            q, s = quantize_weight_per_channel(w_kn.cpu())
            return _Dense(q.to(self.device), _lib.W_NK, n, k, b, s.to(self.device))
        if self._layout == _lib.W_NK:
            packed = torch.empty((n, k), dtype=torch.bfloat16, device=self.device)
            ops.transpose(packed, w_kn, k, n)
            return _Dense(packed, _lib.W_NK, n, k, b)
        return _Dense(w_kn, _lib.W_KN, n, k, b)

    def _dense_cat(self, names: list[str], biases: list[str], *, int8: bool = False) -> _Dense:
        """Several projections of the same input as one GEMM: weights concatenated along N."""
        w_kn = torch.cat([self._w[n] for n in names], dim=1).contiguous()
        bias = torch.cat([self._w[b] for b in biases]).contiguous()
        k, n = w_kn.shape
        if int8:
            q, s = quantize_weight_per_channel(w_kn.cpu())
            return _Dense(q.to(self.device), _lib.W_NK, n, k, bias, s.to(self.device))
        if self._layout == _lib.W_NK:
            packed = torch.empty((n, k), dtype=torch.bfloat16, device=self.device)
            ops.transpose(packed, w_kn, k, n)
            return _Dense(packed, _lib.W_NK, n, k, bias)
        return _Dense(w_kn, _lib.W_KN, n, k, bias)

    def _dense_folded(self, names: list[str], biases: list[str | None] | None, gamma: str, beta: str) -> _Dense:
        """Dense layer(s) consuming a deferred-LayerNorm input: the weight is pre-scaled by the
        LayerNorm's gamma and two per-column vectors carry the mean and beta terms.  Several layers of the
        same input are concatenated along N; a ``None`` among ``biases`` is a layer without bias."""
        w = torch.cat([self._w[n] for n in names], dim=1).float()  # [K, N], bf16 values
        g, b = self._w[gamma].float(), self._w[beta].float()
        scaled = (w * g[:, None]).to(torch.bfloat16)
        fold_c = scaled.float().sum(dim=0).contiguous()
        fold_d = b @ w
        if biases is not None:
            parts = [self._w[x].float() if x is not None else
                     torch.zeros(self._w[n].shape[1], dtype=torch.float32, device=self.device)
                     for x, n in zip(biases, names)]
            fold_d = fold_d + torch.cat(parts)
        k, n = scaled.shape
        if self._layout == _lib.W_NK:
            packed = torch.empty((n, k), dtype=torch.bfloat16, device=self.device)
            ops.transpose(packed, scaled.contiguous(), k, n)
            return _Dense(packed, _lib.W_NK, n, k, None, None, fold_c, fold_d.contiguous())
        return _Dense(scaled.contiguous(), _lib.W_KN, n, k, None, None, fold_c, fold_d.contiguous())

    def _prepare(self) -> None:
        q8 = self.mode == "int8"
        d = self._dense
        self.pe = d("/attn_body/embedding/preprocess/matmul/w", "/attn_body/embedding/preprocess/add/w")
        self.emb = d("/attn_body/matmul/w")
        self.emb_ffn1 = d("/attn_body/ffn/dense1/w/w", "/attn_body/ffn/dense1/b/w")
        self.emb_ffn2 = d("/attn_body/ffn/dense2/w/w")
        self.smolgen_shared = d("/const/smolgen_w")
        self.layers = []
        for i in range(self.cfg.layers):
            p = f"/encoder{i}"
            self.layers.append({
                "compress": d(f"{p}/smolgen/compress/w"),
                "sg1": d(f"{p}/smolgen/dense1/w/w"),
                "sg2": d(f"{p}/smolgen/dense2/w/w"),
                "qkv": self._dense_cat([f"{p}/mha/Q/w/w", f"{p}/mha/K/w/w", f"{p}/mha/V/w/w"],
                                       [f"{p}/mha/Q/b/w", f"{p}/mha/K/b/w", f"{p}/mha/V/b/w"], int8=q8),
                "out": d(f"{p}/mha/out/dense/w/w", int8=q8),
                "ffn1": d(f"{p}/ffn/dense1/w/w", f"{p}/ffn/dense1/b/w", int8=q8),
                "ffn2": d(f"{p}/ffn/dense2/w/w", int8=q8),
            })
        # The second output of a GEMM starts at a multiple of 256 columns (lc0b200_gemm_args::n_main).
        self._fuse_compress = self._layout == _lib.W_NK and (3 * self.cfg.embedding) % 256 == 0
        if self.deferred:
            self.zero_bias = torch.zeros(self.cfg.embedding, dtype=torch.bfloat16, device=self.device)
            for i, layer in enumerate(self.layers):
                p = f"/encoder{i}"
                prev = "/attn_body/ln2" if i == 0 else f"/encoder{i - 1}/ln2"
                qkv_w = [f"{p}/mha/Q/w/w", f"{p}/mha/K/w/w", f"{p}/mha/V/w/w"]
                qkv_b = [f"{p}/mha/Q/b/w", f"{p}/mha/K/b/w", f"{p}/mha/V/b/w"]
                if not q8 and self._fuse_compress:
                    # Q, K, V and smolgen's compression all read the same rows: one GEMM, the compression as
                    # its trailing columns, written to a buffer of its own (lc0b200_gemm_args::out_tail_bf16).
                    layer["qkv_f"] = self._dense_folded([*qkv_w, f"{p}/smolgen/compress/w"], [*qkv_b, None],
                                                        f"{prev}/w/scale", f"{prev}/w/bias")
                else:
                    layer["compress_f"] = self._dense_folded([f"{p}/smolgen/compress/w"], None,
                                                             f"{prev}/w/scale", f"{prev}/w/bias")
                    if not q8:  # the int8 GEMMs read a quantised LayerNorm output instead of folding it
                        layer["qkv_f"] = self._dense_folded(qkv_w, qkv_b, f"{prev}/w/scale", f"{prev}/w/bias")
                if not q8:
                    layer["ffn1_f"] = self._dense_folded([f"{p}/ffn/dense1/w/w"], [f"{p}/ffn/dense1/b/w"],
                                                         f"{p}/ln1/w/scale", f"{p}/ln1/w/bias")
                layer["out_b"] = self._w[f"{p}/mha/out/dense/b/w"]
                layer["ffn2_b"] = self._w[f"{p}/ffn/dense2/b/w"]
        self.pol1 = d("/policy/dense1/matmul/w", "/policy/dense1/add/w")
        self.pol_q = d("/policy/Q/matmul/w", "/policy/Q/add/w")
        self.pol_k = d("/policy/K/matmul/w", "/policy/K/add/w")
        self.heads = {}
        for name in ("value", "mlh"):
            self.heads[name] = (d(f"/{name}/embed/matmul/w", f"/{name}/embed/add/w"),
                                d(f"/{name}/dense1/matmul/w", f"/{name}/dense1/add/w"),
                                d(f"/{name}/dense2/matmul/w", f"/{name}/dense2/add/w"))
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ workspace
    def _workspace(self, b: int) -> dict[str, torch.Tensor]:
        ws = self._workspaces.get(b)
        if ws is not None:
            return ws
        c = self.cfg
        t = b * SQUARES
        dev = self.device

        def bf(*shape: int) -> torch.Tensor:
            return torch.empty(shape, dtype=torch.bfloat16, device=dev)

        ws = {
            "pos_in": bf(b, SQUARES * POSITION_PLANES),
            "position": bf(b, SQUARES * c.pos_enc),
            "emb_in": bf(t, INPUT_PLANES + c.pos_enc),
            "x0": bf(t, c.embedding), "x1": bf(t, c.embedding), "x2": bf(t, c.embedding),
            "branch": bf(t, c.embedding),
            "hidden": bf(t, c.ffn),
            "qkv": bf(t, 3 * c.embedding),
            "merged": bf(t, c.embedding),
            "compressed": bf(t, c.smolgen_compress),
            "sg_hidden": bf(b, c.smolgen_hidden),
            "sg_gen": bf(b, c.heads * c.smolgen_gen),
            "sg_bias": bf(b * c.heads, SQUARES * SQUARES),
            "pol_emb": bf(t, c.policy), "pol_q": bf(t, c.policy_model), "pol_k": bf(t, c.policy_model),
            "records": bf(b, POLICY_RECORD),
            "val_emb": bf(t, c.value_embed), "val_hid": bf(b, c.value_hidden),
            "mlh_emb": bf(t, c.mlh_embed), "mlh_hid": bf(b, c.mlh_hidden),
            "policy": torch.empty((b, POLICY_SIZE), dtype=torch.float32, device=dev),
            "wdl": torch.empty((b, 3), dtype=torch.float32, device=dev),
            "mlh": torch.empty((b, 1), dtype=torch.float32, device=dev),
        }
        if self.deferred:
            parts = (c.embedding + 63) // 64
            for name in ("stats0", "stats1", "stats2"):
                ws[name] = torch.empty((parts, t, 2), dtype=torch.float32, device=dev)
            ws["ln_tap"] = bf(t, c.embedding)
        if self.mode == "int8":
            ws["q_d"] = torch.empty((t, c.embedding), dtype=torch.int8, device=dev)
            ws["q_f"] = torch.empty((t, c.ffn), dtype=torch.int8, device=dev)
            ws["q_scale"] = torch.empty((t,), dtype=torch.float32, device=dev)
        self._workspaces[b] = ws
        return ws

    # ------------------------------------------------------------------ building blocks
    def _gemm(self, out: torch.Tensor, a: torch.Tensor, layer: _Dense, m: int, *, activation: str = "none",
              use_bias: bool = True, row_scale: torch.Tensor | None = None, lda: int | None = None,
              ldc: int | None = None) -> torch.Tensor:
        return ops.gemm(out, a, layer.w, m=m, n=layer.n, k=layer.k, bias=layer.bias if use_bias else None,
                        activation=activation, w_layout=layer.layout, row_scale=row_scale,
                        col_scale=layer.col_scale, lda=lda, ldc=ldc)

    def _ln(self, out: torch.Tensor, x: torch.Tensor, bias: str, gamma: str, beta: str, rows: int, width: int, *,
            activation: str = "none", skip: torch.Tensor | None = None, alpha: str | None = None,
            q_out: torch.Tensor | None = None, q_scale: torch.Tensor | None = None) -> torch.Tensor:
        return ops.layer_norm(out, x, self._w[bias], self._w[gamma], self._w[beta], row_count=rows, width=width,
                              activation=activation, epsilon=self.cfg.ln_eps, skip=skip,
                              alpha=None if alpha is None else self._w[alpha], q_out=q_out, q_scale=q_scale)

    # ------------------------------------------------------------------ encoder tower
    def _smolgen_and_attention(self, ws, layer, i: int, b: int) -> None:
        """Per-position 64x64 logit bias for every head (network.py:778-849, 943-955), then the fused
        attention (network.py:1004-1047).  Expects ``ws["compressed"]`` and ``ws["qkv"]``."""
        c = self.cfg
        p = f"/encoder{i}"
        d, h = c.embedding, c.heads
        self._gemm(ws["sg_hidden"], ws["compressed"], layer["sg1"], b)
        self._ln(ws["sg_hidden"], ws["sg_hidden"], f"{p}/smolgen/dense1/b/w", f"{p}/smolgen/ln1/w/scale",
                 f"{p}/smolgen/ln1/w/bias", b, c.smolgen_hidden, activation="swish")
        self._gemm(ws["sg_gen"], ws["sg_hidden"], layer["sg2"], b)
        self._ln(ws["sg_gen"], ws["sg_gen"], f"{p}/smolgen/dense2/b/w", f"{p}/smolgen/ln2/w/scale",
                 f"{p}/smolgen/ln2/w/bias", b, h * c.smolgen_gen, activation="swish")
        self._gemm(ws["sg_bias"], ws["sg_gen"], self.smolgen_shared, b * h)
        qkv = ws["qkv"]
        ops.attention(ws["merged"], qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:], ws["sg_bias"],
                      self._scalars[f"{p}/mha/QK/scale/w"], b, h, c.head_depth, ldq=3 * d, ldk=3 * d, ldv=3 * d, ldo=d)

    def _tower(self, ws, skip: torch.Tensor, b: int, tap) -> torch.Tensor:
        """Embedding FFN tail and the encoder layers with stand-alone LayerNorm launches."""
        c = self.cfg
        t = b * SQUARES
        d = c.embedding
        q8 = self.mode == "int8"
        qd, qf, qs = (ws["q_d"], ws["q_f"], ws["q_scale"]) if q8 else (None, None, None)
        self._gemm(ws["branch"], ws["hidden"], self.emb_ffn2, t)
        body = self._ln(ws["x1"], ws["branch"], "/attn_body/ffn/dense2/b/w", "/attn_body/ln2/w/scale",
                        "/attn_body/ln2/w/bias", t, d, skip=skip, alpha="/attn_body/ffn/alpha/w",
                        q_out=qd, q_scale=qs)
        tap("embedding", body)
        free = [ws["x0"], ws["x2"]]  # residual-stream buffers not holding `body`
        for i, layer in enumerate(self.layers):
            p = f"/encoder{i}"
            # QKV first in int8 mode: it consumes the quantised copy of `body` before anything overwrites it.
            if q8:
                self._gemm(ws["qkv"], qd, layer["qkv"], t, row_scale=qs)
            else:
                self._gemm(ws["qkv"], body, layer["qkv"], t)
            self._gemm(ws["compressed"], body, layer["compress"], t)
            self._smolgen_and_attention(ws, layer, i, b)
            if q8:
                ops.quantize_rows(qd, qs, ws["merged"], t, d)
                self._gemm(ws["branch"], qd, layer["out"], t, row_scale=qs)
            else:
                self._gemm(ws["branch"], ws["merged"], layer["out"], t)
            attended = self._ln(free[0], ws["branch"], f"{p}/mha/out/dense/b/w", f"{p}/ln1/w/scale",
                                f"{p}/ln1/w/bias", t, d, skip=body, alpha=f"{p}/alpha*input/w",
                                q_out=qd, q_scale=qs)
            # FFN (network.py:1136-1185)
            if q8:
                self._gemm(ws["hidden"], qd, layer["ffn1"], t, activation="mish", row_scale=qs)
                ops.quantize_rows(qf, qs, ws["hidden"], t, c.ffn)
                self._gemm(ws["branch"], qf, layer["ffn2"], t, row_scale=qs)
            else:
                self._gemm(ws["hidden"], attended, layer["ffn1"], t, activation="mish")
                self._gemm(ws["branch"], ws["hidden"], layer["ffn2"], t)
            new_body = self._ln(free[1], ws["branch"], f"{p}/ffn/dense2/b/w", f"{p}/ln2/w/scale", f"{p}/ln2/w/bias",
                                t, d, skip=attended, alpha=f"{p}/ffn/alpha/w", q_out=qd, q_scale=qs)
            free = [body, attended]
            body = new_body
            tap(f"encoder{i}", body)
        return body

    def _gemm_folded(self, out: torch.Tensor, a: torch.Tensor, layer: _Dense, m: int, stats: torch.Tensor, *,
                     activation: str = "none") -> torch.Tensor:
        return ops.gemm(out, a, layer.w, m=m, n=layer.n, k=layer.k, activation=activation, w_layout=layer.layout,
                        ln_in=(stats, layer.fold_c, layer.fold_d), ln_eps=self.cfg.ln_eps)

    def _tower_deferred(self, ws, skip: torch.Tensor, b: int, tap) -> torch.Tensor:
        """The same layers with the residual stream kept un-normalised: every residual GEMM stores
        z = alpha * (branch + bias) + LN(previous z) with per-row partial sums, and every GEMM that
        reads the stream applies the pending LayerNorm in its epilogue.  No LayerNorm kernel runs
        inside the tower; one materialises the final body for the heads."""
        c = self.cfg
        t = b * SQUARES
        d = c.embedding
        eps = c.ln_eps
        w = self._w
        q8 = self.mode == "int8"
        qd, qf, qs = (ws["q_d"], ws["q_f"], ws["q_scale"]) if q8 else (None, None, None)

        def materialise(z: torch.Tensor, ln: str, out: torch.Tensor) -> torch.Tensor:
            return ops.layer_norm(out, z, self.zero_bias, w[f"{ln}/w/scale"], w[f"{ln}/w/bias"], row_count=t, width=d,
                                  epsilon=eps)

        def normalise_and_quantise(z: torch.Tensor, ln: str, row_stats: torch.Tensor) -> None:
            """int8 mode: LayerNorm(z) straight to per-row int8 (no bf16 copy is stored), mean and variance
            from the partial sums the producing GEMM wrote."""
            ops.normalize_quantize_rows(qd, qs, z, row_stats, w[f"{ln}/w/scale"], w[f"{ln}/w/bias"], t, d, eps)

        # embedding FFN tail: z = alpha * (hidden @ W2 + b2) + skip   (skip is a plain tensor here)
        z, stats, ln = ws["x1"], ws["stats0"], "/attn_body/ln2"
        ops.gemm(z, ws["hidden"], self.emb_ffn2.w, m=t, n=d, k=self.emb_ffn2.k, bias=w["/attn_body/ffn/dense2/b/w"],
                 w_layout=self.emb_ffn2.layout, res_skip=skip, res_alpha=self._scalars["/attn_body/ffn/alpha/w"],
                 stats_out=stats, ln_eps=eps)
        if tap is not None:
            tap("embedding", materialise(z, ln, ws["ln_tap"]))
        free_z = [ws["x0"], ws["x2"]]
        free_s = [ws["stats1"], ws["stats2"]]
        for i, layer in enumerate(self.layers):
            p = f"/encoder{i}"
            if q8:
                normalise_and_quantise(z, ln, stats)
                self._gemm(ws["qkv"], qd, layer["qkv"], t, row_scale=qs)
                self._gemm_folded(ws["compressed"], z, layer["compress_f"], t, stats)
            elif self._fuse_compress:
                f = layer["qkv_f"]
                ops.gemm(ws["qkv"], z, f.w, m=t, n=f.n, k=f.k, w_layout=f.layout, ln_in=(stats, f.fold_c, f.fold_d),
                         ln_eps=eps, out_tail=ws["compressed"], n_main=3 * d)
            else:
                self._gemm_folded(ws["qkv"], z, layer["qkv_f"], t, stats)
                self._gemm_folded(ws["compressed"], z, layer["compress_f"], t, stats)
            self._smolgen_and_attention(ws, layer, i, b)
            z1, stats1 = free_z[0], free_s[0]
            a_out, scale_out = ws["merged"], None
            if q8:
                ops.quantize_rows(qd, qs, ws["merged"], t, d)
                a_out, scale_out = qd, qs
            ops.gemm(z1, a_out, layer["out"].w, m=t, n=d, k=d, bias=layer["out_b"], w_layout=layer["out"].layout,
                     row_scale=scale_out, col_scale=layer["out"].col_scale,
                     res_skip=z, res_ln=(stats, w[f"{ln}/w/scale"], w[f"{ln}/w/bias"]),
                     res_alpha=self._scalars[f"{p}/alpha*input/w"], stats_out=stats1, ln_eps=eps)
            a_ffn2, scale_ffn2 = ws["hidden"], None
            if q8:
                normalise_and_quantise(z1, f"{p}/ln1", stats1)
                self._gemm(ws["hidden"], qd, layer["ffn1"], t, activation="mish", row_scale=qs)
                ops.quantize_rows(qf, qs, ws["hidden"], t, c.ffn)
                a_ffn2, scale_ffn2 = qf, qs
            else:
                self._gemm_folded(ws["hidden"], z1, layer["ffn1_f"], t, stats1, activation="mish")
            z2, stats2 = free_z[1], free_s[1]
            ops.gemm(z2, a_ffn2, layer["ffn2"].w, m=t, n=d, k=c.ffn, bias=layer["ffn2_b"],
                     w_layout=layer["ffn2"].layout, row_scale=scale_ffn2, col_scale=layer["ffn2"].col_scale,
                     res_skip=z1, res_ln=(stats1, w[f"{p}/ln1/w/scale"], w[f"{p}/ln1/w/bias"]),
                     res_alpha=self._scalars[f"{p}/ffn/alpha/w"], stats_out=stats2, ln_eps=eps)
            free_z, free_s = [z, z1], [stats, stats1]
            z, stats, ln = z2, stats2, f"{p}/ln2"
            if tap is not None:
                tap(f"encoder{i}", materialise(z, ln, ws["ln_tap"]))
        return materialise(z, ln, free_z[0])

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, plane_masks: torch.Tensor, plane_values: torch.Tensor,
                taps: dict[str, torch.Tensor] | None = None):
        """Run the network on device-resident packed planes.  The returned tensors are
        workspace buffers that the next call with the same batch size overwrites."""
        if plane_masks.dtype != torch.int64 or plane_values.dtype != torch.float32:
            raise ValueError("plane_masks must be int64 (u64 bit patterns) and plane_values float32")
        if plane_masks.shape != plane_values.shape or plane_masks.dim() != 2 or plane_masks.shape[1] != INPUT_PLANES:
            raise ValueError("inputs must both have shape [B, 112]")
        if plane_masks.device != self.device or plane_values.device != self.device:
            raise ValueError(f"inputs must live on {self.device}")
        plane_masks, plane_values = plane_masks.contiguous(), plane_values.contiguous()
        c = self.cfg
        b = plane_masks.shape[0]
        t = b * SQUARES
        d, h = c.embedding, c.heads
        ws = self._workspace(b)

        def tap(name: str, x: torch.Tensor) -> None:
            if taps is not None:
                taps[name] = x.detach().clone()

        # ---- input embedding (network.py:458-642)
        ops.embed_position_input(ws["pos_in"], plane_masks, plane_values, b)
        self._gemm(ws["position"], ws["pos_in"], self.pe, b)
        ops.embed_concat(ws["emb_in"], plane_masks, plane_values, ws["position"], b, c.pos_enc)
        self._gemm(ws["branch"], ws["emb_in"], self.emb, t)
        skip = self._ln(ws["x0"], ws["branch"], "/attn_body/add/w", "/attn_body/ln/w/scale", "/attn_body/ln/w/bias",
                        t, d, activation="mish")
        ops.input_gating(skip, skip, self._w["/ip_mul_gate/w"], self._w["/ip_add_gate/w"], b, SQUARES, d)
        self._gemm(ws["hidden"], skip, self.emb_ffn1, t, activation="mish")
        if self.deferred:
            body = self._tower_deferred(ws, skip, b, tap if taps is not None else None)
        else:
            body = self._tower(ws, skip, b, tap)

        # ---- policy head (network.py:1261-1356)
        self._gemm(ws["pol_emb"], body, self.pol1, t, activation="mish")
        self._gemm(ws["pol_q"], ws["pol_emb"], self.pol_q, t)
        self._gemm(ws["pol_k"], ws["pol_emb"], self.pol_k, t)
        ops.batched_matmul(ws["records"], ws["pol_q"], ws["pol_k"], "policy_qk", b, SQUARES, SQUARES,
                           c.policy_model, 1, scale=self._w["/policy/scale/w"])
        ops.policy_tail(ws["policy"], ws["records"], ws["pol_k"], self._w["/policy/promotion/matmul/w"], self.table,
                        b, c.policy_model)
        # ---- value and moves-left heads (network.py:1475-1550)
        for name, emb_buf, hid_buf, out_buf, final in (("value", "val_emb", "val_hid", "wdl", "none"),
                                                       ("mlh", "mlh_emb", "mlh_hid", "mlh", "relu")):
            embed, dense1, dense2 = self.heads[name]
            self._gemm(ws[emb_buf], body, embed, t, activation="mish")
            self._gemm(ws[hid_buf], ws[emb_buf], dense1, b, activation="mish")
            self._gemm(ws[out_buf], ws[hid_buf], dense2, b, activation=final)
        return ws["policy"], ws["wdl"], ws["mlh"]

    __call__ = forward
