"""Whole-network parity at the benchmark's own sizes: BT3 shape at batch 256, BT4 shape at batches
1024 and 4096, bf16 and int8, through the Python-driven network (both towers) and the C network object.

Positions are independent, so a batch of 4096 run on the GPU is checked against the fp32 CPU oracle on
a handful of SAMPLED positions: the first and last, both sides of a 256-row output-tile edge (positions
3 | 4), of a 128-position boundary, of the wave edge of the persistent GEMMs (148 CTAs x 128 rows =
74 CTA pairs x 256 rows = 296 positions) and of the middle of the batch.  At these sizes the GEMMs run
as 256 x 256 tiles on CTA pairs, which small batches never reach.

Tolerance.  The stated target is "policy logits and WDL within 1e-2 absolute or 1 % relative of the fp32
forward".  That is a statement about bf16 rounding through fifteen layers, not a hard bound: an fp32
oracle that merely ROUNDS every stored tensor to bf16 already lands at 0.007-0.009 worst error over
15 k logits of N(0, 0.02) networks, so over millions of logits some element must cross 1e-2 whatever
the kernels do.  The tests therefore hold the GPU path to the target on the sampled positions with a
small allowance for such elements, and - the discriminating check - to the error of that rounded oracle
on the very same positions: the GPU path may not be worse than bf16 storage makes unavoidable by more
than a factor.
"""

from __future__ import annotations

import functools

import pytest
import torch

from oracle import bt4_oracle as O

WAVE_POSITIONS = 296  # 148 CTAs x 128 token rows / 64 tokens per position


def sample_positions(batch: int, seed: int = 0) -> list[int]:
    """At least sixteen positions of a batch: the edges named in the module docstring plus seeded picks."""
    half = batch // 2
    picks = {0, 1, 3, 4, 127, 128, WAVE_POSITIONS - 1, WAVE_POSITIONS, 2 * WAVE_POSITIONS - 1, 2 * WAVE_POSITIONS,
             half - 1, half, batch - 5, batch - 4, batch - 2, batch - 1}
    picks = {p for p in picks if 0 <= p < batch}
    gen = torch.Generator().manual_seed(1000 + seed)
    while len(picks) < min(batch, 20):
        picks.add(int(torch.randint(0, batch, (1,), generator=gen)))
    return sorted(picks)


def misses(got: torch.Tensor, want: torch.Tensor) -> int:
    """Elements outside "1e-2 absolute or 1 % relative"."""
    err = (got - want).abs()
    return int((~((err <= 1e-2) | (err <= 1e-2 * want.abs()))).sum())


@functools.lru_cache(maxsize=2)
def _weights(cfg_name: str, seed: int):
    from lczero_triton_b200 import config, weights

    return weights.random_weights(getattr(config, cfg_name), seed)


@functools.lru_cache(maxsize=1)
def _table() -> torch.Tensor:
    from lczero_triton_b200 import mapping_table

    return torch.tensor(mapping_table.values(), dtype=torch.int32)


def run_case(cfg_name: str, batch: int, driver: str, mode: str, seed: int) -> dict:
    """One GPU forward at (shape, batch) and the CPU oracles on the sampled positions.

    driver: "deferred" / "standalone" (net.Bt4Net with the LayerNorms folded into the GEMM epilogues or
    as kernels of their own) or "native" (the C network object).  Returns the outputs on the sampled
    positions, the oracles' outputs and, for the Python-driven network, the sampled tap rows."""
    from lczero_triton_b200 import _lib, build, config, native, net, synthetic

    build.build()
    cfg = getattr(config, cfg_name)
    weights = _weights(cfg_name, seed)
    masks, values = synthetic.synthetic_planes(batch, seed)
    picks = sample_positions(batch, seed)
    index = torch.tensor(picks)
    taps: dict[str, torch.Tensor] = {}
    if driver == "native":
        runner = native.NativeNet(weights, cfg, max_batch=batch, mode=mode)
        outs = runner.forward(masks.cuda(), values.cuda())
    else:
        runner = net.Bt4Net(weights, cfg, mode=mode, deferred_layer_norm=(driver == "deferred"))
        outs = runner.forward(masks.cuda(), values.cuda(), taps=taps)
    got = [x[index.cuda()].float().cpu() for x in outs]
    rows = (index[:, None] * 64 + torch.arange(64)[None, :]).reshape(-1)
    got_taps = {k: v[rows.cuda()].float().cpu() for k, v in taps.items()
                if k in ("embedding", "encoder0", f"encoder{cfg.layers - 1}")}
    status, detail = _lib.device_status()
    assert status == 0, f"a kernel's bounded wait ran out: {detail}"
    if driver == "native":
        runner.close()
    del runner, outs, taps
    torch.cuda.empty_cache()

    want_taps: dict[str, torch.Tensor] = {}
    sub_masks, sub_values = masks[index], values[index]
    want = O.forward(weights, cfg, sub_masks, sub_values, table=_table(), taps=want_taps)
    rounded = O.forward(weights, cfg, sub_masks, sub_values, table=_table(), round_to=torch.bfloat16)
    result = {"picks": picks, "got": got, "want": want, "rounded": rounded, "got_taps": got_taps,
              "want_taps": {k: want_taps[k] for k in got_taps}, "cfg": cfg}
    if mode == "int8":
        result["want_int8"] = O.forward(weights, cfg, sub_masks, sub_values, table=_table(), int8=True,
                                        round_to=torch.bfloat16)
    return result


def summarise(result: dict) -> dict:
    """Error figures of one case (what the assertions below and the design notes quote)."""
    out = {}
    for name, g, w, r in zip(("policy", "wdl", "mlh"), result["got"], result["want"], result["rounded"]):
        err, err_r = (g - w).abs(), (r - w).abs()
        out[name] = {"max": float(err.max()), "mean": float(err.mean()), "misses": misses(g, w), "count": g.numel(),
                     "spread": float(w.std()), "rounded_max": float(err_r.max()), "rounded_mean": float(err_r.mean()),
                     "rounded_misses": misses(r, w)}
    return out


def assert_bf16_case(result: dict) -> None:
    stats = summarise(result)
    for stage, got in result["got_taps"].items():
        err = (got - result["want_taps"][stage]).abs()
        assert float(err.max()) < 0.25 and float(err.mean()) < 1.2e-2, (stage, float(err.max()), float(err.mean()))
    for name in ("policy", "wdl", "mlh"):
        s = stats[name]
        # the stated target, with an allowance of one element in 5000 for what bf16 storage itself costs
        assert s["misses"] <= s["rounded_misses"] + max(1, s["count"] // 5000), (name, s)
        # never far from the target, and never much worse than an fp32 forward that only rounds to bf16
        assert s["max"] <= 1.5e-2, (name, s)
        assert s["max"] <= 2.0 * s["rounded_max"] + 2e-3, (name, s)
        assert s["mean"] <= 2.0 * s["rounded_mean"] + 2e-4, (name, s)
    assert stats["policy"]["max"] < 0.3 * stats["policy"]["spread"]


def assert_int8_case(result: dict) -> None:
    """No tolerance is promised end to end for int8 (one rounding flip in a quantised activation moves
    the result by a quantisation step; bit-exactness is checked at the GEMM boundary).  The outputs must
    track the int8 oracle within a fraction of their spread, and stay near the fp32 forward."""
    for g, w, f in zip(result["got"][:2], result["want_int8"][:2], result["want"][:2]):
        spread = float(f.std())
        assert float((g - w).abs().mean()) < 0.05 * spread
        assert float((g - w).abs().max()) < 0.5 * spread
        assert float((g - f).abs().max()) < 0.75 * spread


CASES = [
    ("BT3", 256, "deferred", "bf16"), ("BT3", 256, "standalone", "bf16"), ("BT3", 256, "native", "bf16"),
    ("BT3", 256, "deferred", "int8"),
    ("BT4", 1024, "deferred", "bf16"), ("BT4", 1024, "native", "bf16"), ("BT4", 1024, "native", "int8"),
    ("BT4", 4096, "deferred", "bf16"), ("BT4", 4096, "standalone", "bf16"), ("BT4", 4096, "native", "bf16"),
    ("BT4", 4096, "deferred", "int8"), ("BT4", 4096, "native", "int8"),
]


@pytest.mark.gpu
@pytest.mark.parametrize(("cfg_name", "batch", "driver", "mode"), CASES,
                         ids=[f"{c}-b{b}-{d}-{m}" for c, b, d, m in CASES])
def test_sampled_positions_at_benchmark_sizes(cfg_name, batch, driver, mode) -> None:
    result = run_case(cfg_name, batch, driver, mode, seed=0)
    assert len(result["picks"]) >= 16
    if mode == "bf16":
        assert_bf16_case(result)
    else:
        assert_int8_case(result)


@pytest.mark.gpu
@pytest.mark.parametrize("driver", ["deferred", "standalone"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_tolerance_holds_on_every_seed(driver, seed) -> None:
    """Seeds 1-4 for weights and planes (seed 0 is covered above), BT4 shape at batch 1024, both towers."""
    assert_bf16_case(run_case("BT4", 1024, driver, "bf16", seed))


def test_sampled_positions_cover_the_tile_and_wave_edges() -> None:
    picks = sample_positions(4096)
    for p in (0, 3, 4, 127, 128, 295, 296, 591, 592, 2047, 2048, 4092, 4095):
        assert p in picks
    assert len(sample_positions(256)) >= 16 and max(sample_positions(256)) == 255
