"""Per-op Python wrappers over the C ABI, mirroring the reference's op functions
(``packages/lczero-triton/src/lczero_triton/bt4/kernels/*.py``): same op names and
argument meaning, tensors instead of graph buffers, launches on torch's current
CUDA stream.  Every wrapper raises on a non-zero status.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import ACTIVATIONS, BMM_OPERATIONS, GemmArgs, check


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def expand_planes(out: torch.Tensor, masks: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    _require(out, torch.bfloat16, "out"); _require(masks, torch.int64, "masks"); _require(values, torch.float32, "values")
    check(_lib.load().lc0b200_expand_planes(_p(out), _p(masks), _p(values), masks.numel(), _stream()), "expand_planes")
    return out


def nchw_to_nhwc(out: torch.Tensor, planes: torch.Tensor, batch_size: int, input_channels: int,
                 output_channels: int, height: int = 8, width: int = 8) -> torch.Tensor:
    _require(out, torch.bfloat16, "out"); _require(planes, torch.bfloat16, "planes")
    check(_lib.load().lc0b200_nchw_to_nhwc(_p(out), _p(planes), batch_size, input_channels, output_channels,
                                           height, width, _stream()), "nchw_to_nhwc")
    return out


def preprocess_attention_body(out: torch.Tensor, planes: torch.Tensor, encoding: torch.Tensor, batch_size: int,
                              input_channels: int, encoding_channels: int) -> torch.Tensor:
    check(_lib.load().lc0b200_preprocess_attention_body(_p(out), _p(planes), _p(encoding), batch_size,
                                                        input_channels, encoding_channels, _stream()),
          "preprocess_attention_body")
    return out


def input_gating(out: torch.Tensor, x: torch.Tensor, mult: torch.Tensor, add: torch.Tensor, batch_size: int,
                 square_count: int, channel_count: int) -> torch.Tensor:
    check(_lib.load().lc0b200_input_gating(_p(out), _p(x), _p(mult), _p(add), batch_size, square_count,
                                           channel_count, _stream()), "input_gating")
    return out


def add_vectors(out: torch.Tensor, x: torch.Tensor, bias: torch.Tensor, activation: str = "none") -> torch.Tensor:
    check(_lib.load().lc0b200_add_vectors(_p(out), _p(x), _p(bias), x.numel(), bias.numel(),
                                          ACTIVATIONS[activation], _stream()), "add_vectors")
    return out


def add_bias_batched(out: torch.Tensor, x: torch.Tensor, bias: torch.Tensor, batch_count: int, row_count: int,
                     channel_count: int, activation: str = "none") -> torch.Tensor:
    check(_lib.load().lc0b200_add_bias_batched(_p(out), _p(x), _p(bias), batch_count, row_count, channel_count,
                                               ACTIVATIONS[activation], _stream()), "add_bias_batched")
    return out


def copy_type_converted(out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    _require(out, torch.float32, "out"); _require(x, torch.bfloat16, "x")
    check(_lib.load().lc0b200_copy_type_converted(_p(out), _p(x), x.numel(), _stream()), "copy_type_converted")
    return out


def policy_map(out: torch.Tensor, records: torch.Tensor, table: torch.Tensor, batch_size: int,
               input_element_count: int = 4288, output_element_count: int = 1858) -> torch.Tensor:
    _require(table, torch.int32, "table")
    check(_lib.load().lc0b200_policy_map(_p(out), _p(records), _p(table), batch_size, input_element_count,
                                         output_element_count, _stream()), "policy_map")
    return out


def matmul(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, m: int, n: int, k: int) -> torch.Tensor:
    """``out[m,n] = a[m,k] @ w[k,n]`` with the reference's [K,N] weight layout."""
    _require(out, torch.bfloat16, "out"); _require(a, torch.bfloat16, "a"); _require(w, torch.bfloat16, "w")
    check(_lib.load().lc0b200_matmul(_p(out), _p(a), _p(w), m, n, k, _stream()), "matmul")
    return out


def fused_qkv_projection(q, k, v, a, wq, wk, wv, m: int, query_width: int, key_width: int, value_width: int,
                         depth: int):
    check(_lib.load().lc0b200_fused_qkv_projection(_p(q), _p(k), _p(v), _p(a), _p(wq), _p(wk), _p(wv), m,
                                                   query_width, key_width, value_width, depth, _stream()),
          "fused_qkv_projection", launches=3)
    return q, k, v


def fused_qkv_bias(q, qb, k, kb, v, vb, row_count: int):
    check(_lib.load().lc0b200_fused_qkv_bias(_p(q), _p(q), _p(qb), _p(k), _p(k), _p(kb), _p(v), _p(v), _p(vb),
                                             row_count, qb.numel(), kb.numel(), vb.numel(), _stream()),
          "fused_qkv_bias")
    return q, k, v


def batched_matmul(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, operation: str, batch_count: int, m: int,
                   n: int, k: int, heads_per_sample: int, scale: torch.Tensor | None = None) -> torch.Tensor:
    check(_lib.load().lc0b200_batched_matmul(_p(out), _p(a), _p(b), _p(scale), BMM_OPERATIONS[operation],
                                             batch_count, m, n, k, heads_per_sample, _stream()), "batched_matmul")
    return out


_OUT_KIND = {torch.bfloat16: _lib.OUT_BF16, torch.float32: _lib.OUT_F32, torch.int32: _lib.OUT_S32}


def gemm(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, *, m: int, n: int, k: int,
         bias: torch.Tensor | None = None, activation: str = "none", w_layout: int = _lib.W_NK,
         row_scale: torch.Tensor | None = None, col_scale: torch.Tensor | None = None,
         lda: int | None = None, ldw: int | None = None, ldc: int | None = None, simt: bool = False,
         ln_in: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None, ln_eps: float = 1e-3,
         res_skip: torch.Tensor | None = None, res_alpha: float = 1.0,
         res_ln: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
         stats_out: torch.Tensor | None = None, out_tail: torch.Tensor | None = None,
         n_main: int | None = None) -> torch.Tensor:
    """Tensor-core GEMM with fused epilogue (``include/lc0b200.h``: lc0b200_gemm).

    ``out_tail`` / ``n_main``: two projections of the same ``a`` as one product - columns ``[0, n_main)`` of
    the result go to ``out``, columns ``[n_main, n)`` to ``out_tail`` (bf16; ``n_main`` a multiple of 256).

    Deferred LayerNorm: ``ln_in=(stats [parts,m,2] f32, c [n] f32, d [n] f32)`` folds the LayerNorm of
    the rows of ``a`` into the epilogue; ``res_skip`` (+ ``res_ln=(stats, gamma, beta)`` when the skip
    operand is itself deferred) adds ``res_alpha * y`` to it; ``stats_out [ceil(n/64), m, 2]`` receives
    the partial sums of the stored rows."""
    if a.dtype not in (torch.bfloat16, torch.int8) or w.dtype != a.dtype:
        raise ValueError("a and w must both be bfloat16 or both int8")
    args = GemmArgs()
    args.out, args.a, args.w = _p(out), _p(a), _p(w)
    args.bias_bf16, args.row_scale, args.col_scale = _p(bias), _p(row_scale), _p(col_scale)
    args.m, args.n, args.k = m, n, k
    args.lda = k if lda is None else lda
    args.ldw = (n if w_layout == _lib.W_KN else k) if ldw is None else ldw
    args.ldc = (n if out_tail is None else n_main) if ldc is None else ldc
    if out_tail is not None:
        if n_main is None:
            raise ValueError("out_tail needs n_main")
        args.out_tail_bf16, args.ldc_tail, args.n_main = _p(out_tail), out_tail.stride(0), n_main
    args.in_type = _lib.IN_INT8 if a.dtype == torch.int8 else _lib.IN_BF16
    args.out_kind = _OUT_KIND[out.dtype]
    args.w_layout = w_layout
    args.activation = ACTIVATIONS[activation]
    args.ln_eps = ln_eps
    if ln_in is not None:
        stats, c, d = ln_in
        args.ln_in_stats, args.ln_in_c, args.ln_in_d, args.ln_in_parts = _p(stats), _p(c), _p(d), stats.shape[0]
    if res_skip is not None:
        args.res_skip_bf16, args.ld_skip, args.res_alpha = _p(res_skip), res_skip.stride(0), res_alpha
        if res_ln is not None:
            stats, gamma, beta = res_ln
            args.res_stats, args.res_gamma_bf16, args.res_beta_bf16 = _p(stats), _p(gamma), _p(beta)
            args.res_parts = stats.shape[0]
    args.stats_out = _p(stats_out)
    fn = _lib.load().lc0b200_gemm_simt if simt else _lib.load().lc0b200_gemm
    check(fn(ctypes.byref(args), _stream()), "gemm")
    return out


def transpose(dst: torch.Tensor, src: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    check(_lib.load().lc0b200_transpose(_p(dst), _p(src), rows, cols, src.element_size(), _stream()), "transpose")
    return dst


def layer_norm(out: torch.Tensor | None, x: torch.Tensor, bias: torch.Tensor, gammas: torch.Tensor, betas: torch.Tensor, *,
               row_count: int, width: int, activation: str = "none", epsilon: float = 1e-3,
               skip: torch.Tensor | None = None, alpha: torch.Tensor | None = None,
               q_out: torch.Tensor | None = None, q_scale: torch.Tensor | None = None) -> torch.Tensor:
    check(_lib.load().lc0b200_layer_norm(_p(out), _p(x), _p(bias), _p(skip), _p(gammas), _p(betas), _p(alpha),
                                         row_count, width, ACTIVATIONS[activation], 0 if skip is None else 1,
                                         epsilon, _p(q_out), _p(q_scale), _stream()), "layer_norm")
    return out


def softmax_64(out: torch.Tensor, scaled_qk: torch.Tensor, smolgen: torch.Tensor, row_count: int) -> torch.Tensor:
    check(_lib.load().lc0b200_softmax_64(_p(out), _p(scaled_qk), _p(smolgen), row_count, _stream()), "softmax_64")
    return out


def attention(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor | None,
              scale: float, batch_size: int, heads: int, depth: int = 32, *, ldq: int | None = None,
              ldk: int | None = None, ldv: int | None = None, ldo: int | None = None) -> torch.Tensor:
    """Fused QK^T + edge bias + softmax + PV for the 64-token board."""
    width = heads * depth
    check(_lib.load().lc0b200_attention(_p(out), _p(q), _p(k), _p(v), _p(bias), scale, batch_size, heads, depth,
                                        width if ldq is None else ldq, width if ldk is None else ldk,
                                        width if ldv is None else ldv, width if ldo is None else ldo, _stream()),
          "attention")
    return out


def quantize_rows(out: torch.Tensor, scale: torch.Tensor, x: torch.Tensor, row_count: int, width: int,
                  ld_in: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    _require(out, torch.int8, "out"); _require(scale, torch.float32, "scale"); _require(x, torch.bfloat16, "x")
    check(_lib.load().lc0b200_quantize_rows(_p(out), _p(scale), _p(x), row_count, width,
                                            width if ld_in is None else ld_in, _stream()), "quantize_rows")
    return out, scale


def normalize_quantize_rows(out: torch.Tensor, scale: torch.Tensor, z: torch.Tensor, stats: torch.Tensor,
                            gammas: torch.Tensor, betas: torch.Tensor, row_count: int, width: int,
                            epsilon: float = 1e-3) -> tuple[torch.Tensor, torch.Tensor]:
    """Deferred-LayerNorm rows (``z`` with the partial sums ``stats [parts, rows, 2]`` of a residual GEMM)
    normalised, rounded to bf16 and quantised per row to int8."""
    _require(out, torch.int8, "out"); _require(scale, torch.float32, "scale"); _require(z, torch.bfloat16, "z")
    check(_lib.load().lc0b200_normalize_quantize_rows(_p(out), _p(scale), _p(z), _p(stats), stats.shape[0], _p(gammas),
                                                      _p(betas), row_count, width, epsilon, _stream()),
          "normalize_quantize_rows")
    return out, scale


def linear_int8(out: torch.Tensor, a: torch.Tensor, w_nk: torch.Tensor, col_scale: torch.Tensor,
                bias: torch.Tensor | None, scratch_q: torch.Tensor, scratch_scale: torch.Tensor, *, m: int, n: int,
                k: int, activation: str = "none") -> torch.Tensor:
    """bf16 activations -> per-row int8 (into caller scratch) -> int8 GEMM -> dequant + bias + activation."""
    _require(a, torch.bfloat16, "a"); _require(w_nk, torch.int8, "w_nk"); _require(scratch_q, torch.int8, "scratch_q")
    check(_lib.load().lc0b200_linear_int8(_p(out), _p(a), _p(w_nk), _p(col_scale), _p(bias), _p(scratch_q),
                                          _p(scratch_scale), m, n, k, ACTIVATIONS[activation], _stream()),
          "linear_int8", launches=2)
    return out


def linear_int8_static(out: torch.Tensor, a: torch.Tensor, w_nk: torch.Tensor, col_scale: torch.Tensor,
                       bias: torch.Tensor | None, *, m: int, n: int, k: int, activation: str = "none") -> torch.Tensor:
    """``linear_int8`` for callers that cannot allocate: the quantised activations and row scales
    go to an array built into the library (limits in ``include/lc0b200.h``), so only the input,
    the weights and the output are passed.  Calls share that array; keep them on one stream."""
    _require(a, torch.bfloat16, "a"); _require(w_nk, torch.int8, "w_nk")
    check(_lib.load().lc0b200_linear_int8_static(_p(out), _p(a), _p(w_nk), _p(col_scale), _p(bias), m, n, k,
                                                 ACTIVATIONS[activation], _stream()),
          "linear_int8_static", launches=2)
    return out


def promotion_logits(records: torch.Tensor, keys: torch.Tensor, w: torch.Tensor, batch_size: int,
                     width: int) -> torch.Tensor:
    check(_lib.load().lc0b200_promotion_logits(_p(records), _p(keys), _p(w), batch_size, width, _stream()),
          "promotion_logits")
    return records


def embed_position_input(out: torch.Tensor, masks: torch.Tensor, values: torch.Tensor, batch_size: int) -> torch.Tensor:
    check(_lib.load().lc0b200_embed_position_input(_p(out), _p(masks), _p(values), batch_size, _stream()),
          "embed_position_input")
    return out


def embed_concat(out: torch.Tensor, masks: torch.Tensor, values: torch.Tensor, position: torch.Tensor,
                 batch_size: int, encoding_channels: int) -> torch.Tensor:
    check(_lib.load().lc0b200_embed_concat(_p(out), _p(masks), _p(values), _p(position), batch_size,
                                           encoding_channels, _stream()), "embed_concat")
    return out


def policy_tail(out: torch.Tensor, records: torch.Tensor, keys: torch.Tensor, w: torch.Tensor, table: torch.Tensor,
                batch_size: int, width: int) -> torch.Tensor:
    _require(out, torch.float32, "out")
    check(_lib.load().lc0b200_policy_tail(_p(out), _p(records), _p(keys), _p(w), _p(table), batch_size, width,
                                          _stream()), "policy_tail")
    return out


def output_probabilities(policy_logits: torch.Tensor, wdl_logits: torch.Tensor,
                         legal_mask: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """WDL softmax, policy softmax over the legal moves (``legal_mask`` uint8 [B,1858], None = all) and the
    search's value pair ``q_d[b] = (W - L, D)``.  Returns ``(policy_probs, wdl_probs, q_d)``."""
    _require(policy_logits, torch.float32, "policy_logits"); _require(wdl_logits, torch.float32, "wdl_logits")
    if legal_mask is not None:
        _require(legal_mask, torch.uint8, "legal_mask")
    batch, size = policy_logits.shape
    policy, wdl = torch.empty_like(policy_logits), torch.empty_like(wdl_logits)
    q_d = torch.empty((batch, 2), dtype=torch.float32, device=wdl_logits.device)
    check(_lib.load().lc0b200_output_probabilities(_p(policy), _p(wdl), _p(q_d), _p(policy_logits), _p(wdl_logits),
                                                   _p(legal_mask), batch, size, _stream()), "output_probabilities")
    return policy, wdl, q_d
