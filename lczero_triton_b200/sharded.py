"""Several GPUs, one process: a batch of positions split across replicas of the network.

Positions are independent (the batch is the leading dimension of every buffer of the reference
graph, network.py:328-340), so each GPU holds a full copy of the weights, takes one contiguous range
of positions and there is nothing to exchange: no collective, no peer access.  ``ShardedNet`` keeps
one replica (``native.NativeNet``: the whole forward behind the C ABI) and one worker thread per
device; ``forward`` copies each range to its device, runs the replicas concurrently (the C calls
release the interpreter lock) and stitches the results back in position order.

``shard_range`` is also what a process-per-GPU launcher uses to pick its range (``bench.py``).
"""

from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from concurrent.futures import ThreadPoolExecutor

import torch

from .config import INPUT_PLANES, POLICY_SIZE, NetConfig


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of positions for ``rank`` of ``world``; sizes differ by at most one."""
    if total < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad shard request: total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _native_replica(weights, cfg: NetConfig, max_batch: int, device: torch.device, mode: str):
    from .native import NativeNet

    with torch.cuda.device(device):
        return NativeNet(weights, cfg, max_batch, device=device, mode=mode)


class ShardedNet:
    """``forward(plane_masks, plane_values)`` over every device in ``devices``.

    Inputs may live on the host (pinned memory makes the copies asynchronous) or on any device; the
    outputs ``(policy f32[B,1858], wdl f32[B,3], mlh f32[B,1])`` are host tensors (pinned when CUDA is
    in use), overwritten by the next call.  ``max_batch`` is the largest batch ``forward`` accepts; each
    replica is sized for its share of it.  ``replica_factory(weights, cfg, max_batch, device, mode)``
    builds one replica (anything with ``forward(masks, values)`` on ``device``); the default builds a
    ``NativeNet``.
    """

    def __init__(self, weights: Mapping[str, torch.Tensor], cfg: NetConfig, max_batch: int, *,
                 devices: Sequence[str | torch.device | int] | None = None, mode: str = "bf16",
                 replica_factory: Callable | None = None) -> None:
        if devices is None:
            devices = list(range(torch.cuda.device_count()))
        if len(devices) == 0:
            raise ValueError("ShardedNet needs at least one device; there is no CPU path")
        if max_batch < 1:
            raise ValueError("max_batch must be positive")
        self.devices = [torch.device("cuda", d) if isinstance(d, int) else torch.device(d) for d in devices]
        self.cfg = cfg
        self.max_batch = max_batch
        self._world = len(self.devices)
        factory = replica_factory or _native_replica
        per_replica = shard_range(max_batch, 0, self._world)[1]  # rank 0 holds the largest share
        self._pool = ThreadPoolExecutor(max_workers=self._world, thread_name_prefix="lc0b200-shard")
        self._replicas = list(self._pool.map(
            lambda dev: factory(weights, cfg, max(1, per_replica), dev, mode), self.devices))
        pin = any(d.type == "cuda" for d in self.devices)
        self._out = (torch.empty((max_batch, POLICY_SIZE), dtype=torch.float32, pin_memory=pin),
                     torch.empty((max_batch, 3), dtype=torch.float32, pin_memory=pin),
                     torch.empty((max_batch, 1), dtype=torch.float32, pin_memory=pin))

    def _run_shard(self, rank: int, masks: torch.Tensor, values: torch.Tensor, lo: int, hi: int) -> None:
        if hi == lo:
            return
        device = self.devices[rank]
        on_gpu = device.type == "cuda"
        if on_gpu:
            torch.cuda.set_device(device)  # per thread: the C library works on the thread's current device
        part_masks = masks[lo:hi].to(device, non_blocking=True)
        part_values = values[lo:hi].to(device, non_blocking=True)
        outs = self._replicas[rank].forward(part_masks, part_values)
        for dst, src in zip(self._out, outs):
            dst[lo:hi].copy_(src, non_blocking=True)
        if on_gpu:
            torch.cuda.current_stream(device).synchronize()

    def forward(self, plane_masks: torch.Tensor, plane_values: torch.Tensor):
        if plane_masks.dtype != torch.int64 or plane_values.dtype != torch.float32:
            raise ValueError("plane_masks must be int64 (u64 bit patterns) and plane_values float32")
        if plane_masks.shape != plane_values.shape or plane_masks.dim() != 2 or plane_masks.shape[1] != INPUT_PLANES:
            raise ValueError("inputs must both have shape [B, 112]")
        batch = plane_masks.shape[0]
        if batch > self.max_batch:
            raise ValueError(f"batch {batch} exceeds max_batch {self.max_batch}")
        ranges = [shard_range(batch, r, self._world) for r in range(self._world)]
        jobs = [self._pool.submit(self._run_shard, r, plane_masks, plane_values, lo, hi)
                for r, (lo, hi) in enumerate(ranges)]
        for job in jobs:
            job.result()  # re-raises a replica's exception here
        return tuple(t[:batch] for t in self._out)

    __call__ = forward

    def close(self) -> None:
        for replica in self._replicas:
            closer = getattr(replica, "close", None)
            if closer is not None:
                closer()
        self._replicas = []
        self._pool.shutdown(wait=True)
