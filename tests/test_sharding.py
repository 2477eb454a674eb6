"""The multi-GPU path.  On CPU: positions shard into disjoint contiguous ranges; ``ShardedNet`` (one
process, one replica and one thread per device) splits a batch, runs its replicas and stitches the
results in position order, shown with stand-in replicas; two gloo ranks (child processes) agree on a
max-over-ranks time and reproduce the unsharded result.  On two GPUs: ``ShardedNet`` over both devices
gives, bit for bit, what one GPU gives for the whole batch."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lczero_triton_b200.sharded import ShardedNet, shard_range
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


class _FakeReplica:
    """Stands in for a network replica on the CPU: every output row is a function of its own input row."""

    calls: list[tuple[str, int]] = []

    def __init__(self, weights, cfg, max_batch, device, mode) -> None:
        self.max_batch, self.device = max_batch, device

    def forward(self, masks: torch.Tensor, values: torch.Tensor):
        assert masks.shape[0] <= self.max_batch
        _FakeReplica.calls.append((str(self.device), masks.shape[0]))
        key = (masks.sum(dim=1) % 1000).float()[:, None] + values.sum(dim=1, keepdim=True)
        return key.expand(-1, 1858).contiguous(), key.expand(-1, 3) * 2.0, key * 3.0


@pytest.mark.parametrize(("batch", "world"), [(7, 2), (64, 3), (2, 4), (1, 1)])
def test_sharded_net_splits_and_stitches_in_position_order(batch, world) -> None:
    from lczero_triton_b200.config import TINY
    from lczero_triton_b200.synthetic import synthetic_planes

    _FakeReplica.calls = []
    net = ShardedNet({}, TINY, max_batch=64, devices=["cpu"] * world, replica_factory=_FakeReplica)
    masks, values = synthetic_planes(batch, 5)
    policy, wdl, mlh = net.forward(masks, values)
    want = _FakeReplica({}, TINY, 64, "cpu", "bf16").forward(masks, values)
    assert torch.equal(policy, want[0]) and torch.equal(wdl, want[1]) and torch.equal(mlh, want[2])
    sizes = sorted(n for _, n in _FakeReplica.calls[:-1])
    assert sum(sizes) == batch and len(sizes) == min(batch, world)  # empty shards launch nothing
    assert max(sizes) - min(sizes) <= 1 or len(sizes) < world
    net.close()


def test_sharded_net_reports_a_failing_replica_and_bad_inputs() -> None:
    from lczero_triton_b200.config import TINY
    from lczero_triton_b200.synthetic import synthetic_planes

    class Failing(_FakeReplica):
        def forward(self, masks, values):
            raise RuntimeError("replica lost")

    masks, values = synthetic_planes(4, 0)
    net = ShardedNet({}, TINY, max_batch=4, devices=["cpu", "cpu"], replica_factory=Failing)
    with pytest.raises(RuntimeError, match="replica lost"):
        net.forward(masks, values)
    net.close()
    net = ShardedNet({}, TINY, max_batch=2, devices=["cpu"], replica_factory=_FakeReplica)
    with pytest.raises(ValueError):
        net.forward(masks, values)            # batch above max_batch
    with pytest.raises(ValueError):
        net.forward(masks[:2].int(), values[:2])
    net.close()
    with pytest.raises(ValueError):
        ShardedNet({}, TINY, max_batch=2, devices=[], replica_factory=_FakeReplica)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["bf16", "int8"])
def test_two_gpus_in_one_process_equal_one_gpu(mode) -> None:
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from lczero_triton_b200 import _lib, build
    from lczero_triton_b200.config import TINY
    from lczero_triton_b200.native import NativeNet
    from lczero_triton_b200.synthetic import synthetic_planes
    from lczero_triton_b200.weights import random_weights

    build.build()
    weights = random_weights(TINY, 4)
    masks, values = synthetic_planes(37, 4)
    both = ShardedNet(weights, TINY, max_batch=64, devices=[0, 1], mode=mode)
    got = [x.clone() for x in both.forward(masks.pin_memory(), values.pin_memory())]
    again = [x.clone() for x in both.forward(masks, values)]
    both.close()
    with torch.cuda.device(0):
        one = NativeNet(weights, TINY, 64, device="cuda:0", mode=mode)
        want = [x.cpu() for x in one.forward(masks.cuda(0), values.cuda(0))]
        one.close()
    for g, a, w in zip(got, again, want):
        assert torch.equal(g, a) and torch.equal(g, w)
    for device in (0, 1):  # the status words are per device: neither GPU saw a wait run out
        with torch.cuda.device(device):
            status, detail = _lib.device_status()
            assert status == 0, (device, detail)
