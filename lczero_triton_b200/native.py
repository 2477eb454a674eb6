"""The whole forward pass through the C ABI's network object (``lc0b200_net_*``).

``NativeNet`` is what a C or C++ engine would do with ``include/lc0b200.h``, written in Python:
size the arena, create the network, hand the weights over under the reference's canonical names
(packages/lczero-triton/src/lczero_triton/bt4/network.py:343-1466), finalise, run.  PyTorch only
provides the device memory and the stream.  ``net.Bt4Net`` is the same graph driven operator by
operator from Python; the tests hold the two against each other.
"""

from __future__ import annotations

import ctypes
from collections.abc import Mapping

import torch

from . import _lib
from .config import INPUT_PLANES, POLICY_SIZE, NetConfig


class NetConfigC(ctypes.Structure):
    """``lc0b200_net_config``."""

    _fields_ = [(name, ctypes.c_int) for name in (
        "embedding", "layers", "heads", "ffn", "pos_enc", "smolgen_compress", "smolgen_hidden", "smolgen_gen",
        "policy", "policy_model", "value_embed", "value_hidden", "mlh_embed", "mlh_hidden")] + [
            ("ln_eps", ctypes.c_float), ("int8_gemms", ctypes.c_int)]

    @classmethod
    def from_config(cls, cfg: NetConfig, mode: str = "bf16") -> "NetConfigC":
        return cls(cfg.embedding, cfg.layers, cfg.heads, cfg.ffn, cfg.pos_enc, cfg.smolgen_compress, cfg.smolgen_hidden,
                   cfg.smolgen_gen, cfg.policy, cfg.policy_model, cfg.value_embed, cfg.value_hidden, cfg.mlh_embed,
                   cfg.mlh_hidden, cfg.ln_eps, 1 if mode == "int8" else 0)


class NativeNet:
    """A BT4-style network held by the C library: bf16 with the LayerNorms folded into the GEMMs, or
    (``mode="int8"``) int8 GEMMs with stand-alone LayerNorm kernels."""

    def __init__(self, weights: Mapping[str, torch.Tensor], config: NetConfig, max_batch: int, *,
                 device: str | torch.device = "cuda", mode: str = "bf16") -> None:
        if mode not in ("bf16", "int8"):
            raise ValueError("mode must be 'bf16' or 'int8'")
        self._lib = _lib.load()
        self._handle = ctypes.c_void_p()
        self.cfg = config
        self.max_batch = max_batch
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("NativeNet needs a CUDA device; there is no CPU path")
        cfg_c = NetConfigC.from_config(config, mode)
        nbytes = self._lib.lc0b200_net_arena_bytes(ctypes.byref(cfg_c), max_batch)
        if nbytes == 0:
            raise ValueError("the C library rejects this network shape (head depth must be 32)")
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        _lib.check(self._lib.lc0b200_net_create(ctypes.byref(self._handle), ctypes.byref(cfg_c), max_batch,
                                                self.arena.data_ptr(), nbytes), "net_create", launches=0)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        name, count = ctypes.c_char_p(), ctypes.c_longlong()
        for index in range(self._lib.lc0b200_net_weight_count(self._handle)):
            _lib.check(self._lib.lc0b200_net_weight_info(self._handle, index, ctypes.byref(name), ctypes.byref(count)),
                       "net_weight_info", launches=0)
            key = name.value.decode()
            if key not in weights:
                raise KeyError(f"weights lack {key}")
            host = weights[key].detach().to(device="cpu", dtype=torch.bfloat16).contiguous()
            if host.numel() != count.value:
                raise ValueError(f"{key}: {host.numel()} elements, the network expects {count.value}")
            _lib.check(self._lib.lc0b200_net_set_weight(self._handle, name.value, host.data_ptr(), count.value, stream),
                       "net_set_weight", launches=0)
        _lib.check(self._lib.lc0b200_net_finalize(self._handle, stream), "net_finalize", launches=0)

    def forward(self, plane_masks: torch.Tensor, plane_values: torch.Tensor):
        """``(masks int64 [B,112], values f32 [B,112])`` on the device -> ``(policy, wdl logits, mlh)`` f32."""
        if plane_masks.dtype != torch.int64 or plane_values.dtype != torch.float32:
            raise ValueError("plane_masks must be int64 (u64 bit patterns) and plane_values float32")
        if plane_masks.shape != plane_values.shape or plane_masks.dim() != 2 or plane_masks.shape[1] != INPUT_PLANES:
            raise ValueError("inputs must both have shape [B, 112]")
        b = plane_masks.shape[0]
        masks, values = plane_masks.contiguous(), plane_values.contiguous()
        policy = torch.empty((b, POLICY_SIZE), dtype=torch.float32, device=self.device)
        wdl = torch.empty((b, 3), dtype=torch.float32, device=self.device)
        mlh = torch.empty((b, 1), dtype=torch.float32, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(self._lib.lc0b200_net_forward(self._handle, masks.data_ptr(), values.data_ptr(), b, policy.data_ptr(),
                                                 wdl.data_ptr(), mlh.data_ptr(), stream), "net_forward", launches=0)
        return policy, wdl, mlh

    __call__ = forward

    def close(self) -> None:
        if self._handle:
            self._lib.lc0b200_net_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass
