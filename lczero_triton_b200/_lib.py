"""ctypes binding of ``liblc0b200.so`` (the C ABI declared in ``include/lc0b200.h``).

There is no fallback: if the library is missing or a call returns a non-zero
status the caller gets an exception.
"""

from __future__ import annotations

import ctypes
import pathlib
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_uint, c_void_p

LIBRARY_PATH = pathlib.Path(__file__).resolve().parent / "liblc0b200.so"

OK = 0
ACTIVATIONS = {"none": 0, "mish": 1, "relu": 2, "swish": 3}
BMM_OPERATIONS = {"body_qk": 0, "body_attention_v": 1, "policy_qk": 2}
IN_BF16, IN_INT8 = 0, 1
OUT_BF16, OUT_F32, OUT_S32 = 0, 1, 2
W_KN, W_NK = 0, 1


class Lc0B200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("out", c_void_p), ("a", c_void_p), ("w", c_void_p), ("bias_bf16", c_void_p),
        ("row_scale", c_void_p), ("col_scale", c_void_p),
        ("m", c_longlong), ("n", c_int), ("k", c_int),
        ("lda", c_longlong), ("ldw", c_longlong), ("ldc", c_longlong),
        ("in_type", c_int), ("out_kind", c_int), ("w_layout", c_int), ("activation", c_int),
        ("ln_in_stats", c_void_p), ("ln_in_c", c_void_p), ("ln_in_d", c_void_p),
        ("ln_in_parts", c_int), ("ln_eps", c_float),
        ("res_skip_bf16", c_void_p), ("ld_skip", c_longlong), ("res_stats", c_void_p),
        ("res_gamma_bf16", c_void_p), ("res_beta_bf16", c_void_p), ("res_parts", c_int), ("res_alpha", c_float),
        ("stats_out", c_void_p),
        ("out_tail_bf16", c_void_p), ("ldc_tail", c_longlong), ("n_main", c_int),
    ]


_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float

# name -> argument types (every function returns int except the two string getters).
SIGNATURES: dict[str, tuple] = {
    "lc0b200_device_status": (POINTER(c_uint),),
    "lc0b200_expand_planes": (_P, _P, _P, _L, _P),
    "lc0b200_nchw_to_nhwc": (_P, _P, _I, _I, _I, _I, _I, _P),
    "lc0b200_preprocess_attention_body": (_P, _P, _P, _I, _I, _I, _P),
    "lc0b200_input_gating": (_P, _P, _P, _P, _I, _I, _I, _P),
    "lc0b200_add_vectors": (_P, _P, _P, _L, _I, _I, _P),
    "lc0b200_add_bias_batched": (_P, _P, _P, _I, _L, _I, _I, _P),
    "lc0b200_copy_type_converted": (_P, _P, _L, _P),
    "lc0b200_policy_map": (_P, _P, _P, _I, _I, _I, _P),
    "lc0b200_matmul": (_P, _P, _P, _L, _I, _I, _P),
    "lc0b200_fused_qkv_projection": (_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P),
    "lc0b200_fused_qkv_bias": (_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _P),
    "lc0b200_batched_matmul": (_P, _P, _P, _P, _I, _L, _I, _I, _I, _I, _P),
    "lc0b200_gemm": (POINTER(GemmArgs), _P),
    "lc0b200_gemm_simt": (POINTER(GemmArgs), _P),
    "lc0b200_transpose": (_P, _P, _I, _I, _I, _P),
    "lc0b200_layer_norm": (_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _F, _P, _P, _P),
    "lc0b200_softmax_64": (_P, _P, _P, _L, _P),
    "lc0b200_attention": (_P, _P, _P, _P, _P, _F, _L, _I, _I, _L, _L, _L, _L, _P),
    "lc0b200_quantize_rows": (_P, _P, _P, _L, _I, _L, _P),
    "lc0b200_normalize_quantize_rows": (_P, _P, _P, _P, _I, _P, _P, _L, _I, _F, _P),
    "lc0b200_linear_int8": (_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _P),
    "lc0b200_linear_int8_static": (_P, _P, _P, _P, _P, _L, _I, _I, _I, _P),
    "lc0b200_promotion_logits": (_P, _P, _P, _I, _I, _P),
    "lc0b200_embed_position_input": (_P, _P, _P, _I, _P),
    "lc0b200_embed_concat": (_P, _P, _P, _P, _I, _I, _P),
    "lc0b200_policy_tail": (_P, _P, _P, _P, _P, _I, _I, _P),
    "lc0b200_output_probabilities": (_P, _P, _P, _P, _P, _P, _I, _I, _P),
    "lc0b200_net_arena_bytes": (_P, _I),
    "lc0b200_net_create": (POINTER(c_void_p), _P, _I, _P, ctypes.c_size_t),
    "lc0b200_net_destroy": (_P,),
    "lc0b200_net_weight_count": (_P,),
    "lc0b200_net_weight_info": (_P, _I, POINTER(c_char_p), POINTER(c_longlong)),
    "lc0b200_net_set_weight": (_P, c_char_p, _P, _L, _P),
    "lc0b200_net_finalize": (_P, _P),
    "lc0b200_net_forward": (_P, _P, _P, _I, _P, _P, _P, _P),
}
# Return types other than the int status.
RESTYPES = {"lc0b200_net_arena_bytes": ctypes.c_size_t, "lc0b200_net_destroy": None}
STRING_GETTERS = ("lc0b200_version", "lc0b200_status_string")

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load the library once and declare every prototype; raise if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIBRARY_PATH.exists():
        raise Lc0B200Error(
            f"{LIBRARY_PATH} is missing: build it with `python -m lczero_triton_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = list(argtypes)
        fn.restype = RESTYPES.get(name, c_int)
    lib.lc0b200_version.argtypes = []
    lib.lc0b200_version.restype = c_char_p
    lib.lc0b200_status_string.argtypes = [c_int]
    lib.lc0b200_status_string.restype = c_char_p
    _lib = lib
    return lib


_launches = 0


def launch_count() -> int:
    """Kernels launched through this binding so far (successful C-ABI compute calls)."""
    return _launches


def check(status: int, what: str, launches: int = 1) -> None:
    global _launches
    _launches += launches
    if status != OK:
        text = load().lc0b200_status_string(status).decode()
        raise Lc0B200Error(f"{what} failed with status {status} ({text})")


def device_status() -> tuple[int, tuple[int, int, int, int]]:
    """Synchronise and return (status, detail words) of the device-side wait flag."""
    words = (c_uint * 4)()
    status = load().lc0b200_device_status(words)
    return status, tuple(int(w) for w in words)
