"""The benchmark's output contract, checked without a GPU: the reference arm's JSON line and the clock sampler."""

from __future__ import annotations

import argparse
import json
import pathlib
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_reference_arm_prints_the_contract_line(monkeypatch, capsys) -> None:
    monkeypatch.setattr(bench, "_cpu_forward_rate", lambda cfg, batch, repeats, warmup: (70.0, 1800.0))
    monkeypatch.delenv("RANK", raising=False)
    args = argparse.Namespace(gpus=1, steps=2, warmup=1, batch=4096, mode="bf16")
    bench.run_reference(args)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == "positions/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["n_gpus"] == 1
    assert line["value"] == 70.0 and line["e2e"] == {"value": 70.0, "unit": "positions/s", "h2d_bytes_per_step": 0,
                                                      "d2h_bytes_per_step": 0}
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == 70.0
    assert str(bench.CPU_SAMPLE_BATCH) in baseline["sample"] and "workload" in line["config"]


def test_other_ranks_of_the_reference_arm_stay_silent(monkeypatch, capsys) -> None:
    monkeypatch.setenv("RANK", "3")
    bench.run_reference(argparse.Namespace(gpus=8, steps=1, warmup=1, batch=4096, mode="bf16"))
    assert capsys.readouterr().out == ""


def test_clock_sampler_summarises_nvidia_smi_lines() -> None:
    sampler = bench.ClockSampler(0)
    sampler.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0,
                                  "poll": lambda self: None})()
    sampler.lines = [
        "0, 1335, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "0, 1290, 1965, 998.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "0, 1400, 1965, 950.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
        "garbage",
    ]
    summary = sampler.stop()
    assert summary["sm_mhz"] == 1335.0 and summary["sm_max_mhz"] == 1965.0 and summary["samples"] == 3
    assert summary["reasons"] == ["sw_power_cap"]


def test_clock_sampler_runs_only_around_warm_up_and_timed_steps(monkeypatch) -> None:
    """The sampler is started by the timing loop itself and halted before the closing barrier, so that what it
    reports is the clock under the measured load, not the idle clock during set-up or while other ranks finish."""
    events: list[str] = []
    sampler = bench.ClockSampler(0)
    monkeypatch.setattr(sampler, "start", lambda: events.append("start"))
    monkeypatch.setattr(sampler, "halt", lambda: events.append("halt"))
    monkeypatch.setattr(bench, "_barrier", lambda dist: events.append("barrier"))
    monkeypatch.setattr(bench, "_max_over_ranks", lambda value, dist: value)

    class _Event:
        def __init__(self, enable_timing=True): pass
        def record(self): events.append("record")
        def elapsed_time(self, other): return 1.0

    monkeypatch.setattr(bench.torch.cuda, "Event", _Event)
    monkeypatch.setattr(bench.torch.cuda, "synchronize", lambda: events.append("sync"))
    bench._timed_steps(lambda: events.append("step"), 3, 2, None, sampler)
    assert events == ["start", "step", "step", "step", "barrier", "record", "step", "step", "record", "sync", "halt", "barrier"]


def test_reference_gpu_arm_says_unavailable_without_a_device(monkeypatch, capsys) -> None:
    """The extra arm (the reference's own program on the GPU) never falls back to anything: without a CUDA
    device, Triton or the reference install it prints one line saying which is missing."""
    monkeypatch.delenv("RANK", raising=False)
    monkeypatch.setattr(bench.torch.cuda, "is_available", lambda: False)
    bench.run_reference_gpu(type("A", (), {"batch": 4096, "steps": 2, "warmup": 1})())
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference-gpu" and "unavailable" in line
