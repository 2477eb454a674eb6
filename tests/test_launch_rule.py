"""Source-level check of the programmatic-dependent-launch rule (no GPU needed).

A kernel launched through ``launch_dependent`` (or with ``dependent_launch_attribute`` in its launch
configuration) may start while the kernel before it on the stream is still running.  It is only correct if it
executes ``grid_dependency_wait()`` before its first access to global memory; a kernel that lacks the wait
would race silently and, most of the time, still pass numerical tests.  This test reads ``csrc/*.cu`` and
requires the wait in the body of every kernel that is launched that way.
"""

from __future__ import annotations

import pathlib
import re

CSRC = pathlib.Path(__file__).resolve().parents[1] / "lczero_triton_b200" / "csrc"


def _kernel_bodies(text: str) -> dict[str, str]:
    """name -> body text of every ``__global__`` function in a translation unit."""
    bodies: dict[str, str] = {}
    for match in re.finditer(r"__global__", text):
        k, depth = match.end(), 0
        while not (text[k] == "{" and depth == 0):
            depth += {"(": 1, ")": -1}.get(text[k], 0)
            k += 1
        header = text[match.end():k]
        names = re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*\(", re.sub(r"__launch_bounds__\s*\([^)]*(\([^)]*\))*[^)]*\)", "", header))
        if not names:
            continue
        end, depth = k, 0
        while True:
            depth += {"{": 1, "}": -1}.get(text[end], 0)
            if depth == 0:
                break
            end += 1
        bodies[names[0]] = text[k:end + 1]
    return bodies


def _dependently_launched(text: str) -> set[str]:
    names = set(re.findall(r"launch_dependent\(\s*([A-Za-z_][A-Za-z0-9_]*)", text))
    names.discard("kernel")  # a function-pointer variable; resolved below
    return names


def test_every_dependently_launched_kernel_waits_for_its_predecessor() -> None:
    checked = 0
    for path in sorted(CSRC.glob("*.cu")):
        text = path.read_text()
        bodies = _kernel_bodies(text)
        launched = _dependently_launched(text)
        if "dependent_launch_attribute(" in text or re.search(r"launch_dependent\(\s*kernel\b", text):
            # launches through a kernel pointer: every kernel of the file is a candidate
            launched |= set(bodies)
        for name in sorted(launched):
            assert name in bodies, f"{path.name}: {name} is launched dependently but not defined in this file"
            body = bodies[name]
            assert "grid_dependency_wait()" in body, f"{path.name}: {name} never waits for the kernel before it"
            wait = body.index("grid_dependency_wait()")
            # nothing that dereferences a kernel argument may come before the wait (the library's own status
            # words, written only when a kernel gives up, are not data of the stream)
            before = body[:wait].replace("p.status[", "")
            assert not re.search(r"__ldg\(|\bp\.[a-z_]+\[|tma_load_2d|tma_store_2d|\bout\[|\bin\[", before), \
                f"{path.name}: {name} touches global memory before grid_dependency_wait()"
            assert "grid_dependency_release()" in before, f"{path.name}: {name} should release its dependents first"
            checked += 1
    assert checked >= 25


def test_kernel_parser_sees_the_kernels() -> None:
    bodies = _kernel_bodies((CSRC / "layernorm.cu").read_text())
    assert {"layer_norm_warp_kernel", "layer_norm_wide_kernel", "layer_norm_block_kernel", "normalize_quantize_kernel"} <= set(bodies)
    assert "gemm_tcgen05_kernel" in _kernel_bodies((CSRC / "gemm_tcgen05.cu").read_text())
    assert "attention_tc_kernel" in _kernel_bodies((CSRC / "attention_tc.cu").read_text())
