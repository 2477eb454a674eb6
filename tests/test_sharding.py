"""Host-side logic of the multi-GPU path on CPU: positions shard into disjoint contiguous ranges,
ranks agree on a max-over-ranks time through a gloo group, and stitching the shards back gives
the unsharded result (positions are independent).  World size 2, spawned as child processes."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lczero_triton_b200.sharding import shard_range
from oracle import bt4_oracle as O


def test_shard_ranges_cover_the_batch_exactly_once() -> None:
    for total in (0, 1, 7, 64, 4096, 4099):
        for world in (1, 2, 3, 8):
            ranges = [shard_range(total, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1


def test_shard_range_rejects_bad_arguments() -> None:
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
    with pytest.raises(ValueError):
        shard_range(-1, 0, 1)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lczero_triton_b200 import mapping_table
    from lczero_triton_b200.config import TINY
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    torch.set_num_threads(1)
    weights = random_weights(TINY, 0)
    masks, values = synthetic_planes(6, 0)
    lo, hi = shard_range(6, rank, world)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    policy, wdl, mlh = O.forward(weights, TINY, masks[lo:hi], values[lo:hi], table=table)
    elapsed = torch.tensor([1.0 + rank], dtype=torch.float64)  # stand-in for a device-side time
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    torch.save({"lo": lo, "hi": hi, "policy": policy, "wdl": wdl, "max_time": float(elapsed)}, f"{out_dir}/r{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_result(tmp_path) -> None:
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    from lczero_triton_b200 import mapping_table
    from lczero_triton_b200.config import TINY
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert [(p["lo"], p["hi"]) for p in parts] == [(0, 3), (3, 6)]
    assert all(p["max_time"] == 2.0 for p in parts)
    masks, values = synthetic_planes(6, 0)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    torch.set_num_threads(1)
    policy, wdl, _ = O.forward(random_weights(TINY, 0), TINY, masks, values, table=table)
    torch.testing.assert_close(torch.cat([p["policy"] for p in parts]), policy, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.cat([p["wdl"] for p in parts]), wdl, rtol=1e-5, atol=1e-6)
