"""This library's lc0ex linker against the reference linker's own result on the reference's own graph.

``tests/golden/reference_program_plan.json`` is written by ``tests/golden/make_network_golden.py --dry``: the
reference's graph builder walks a 4-layer network and the BT4 network, and the reference's
``ExecutableBuilder._analyze_invocations`` and ``BufferBuilder.plan`` produce the reduced dependencies of all
104 / 291 calls and the offsets of every buffer.  Here the same buffers are declared and the same calls made,
in the same order, through ``lc0ex_bridge``; its executable must carry the same dependency lists, the same
offsets and the same allocation sizes.
"""

from __future__ import annotations

import functools
import json
import pathlib

import numpy as np
import pytest

from lczero_triton_b200 import lc0ex_bridge as B

GOLDEN = pathlib.Path(__file__).parent / "golden"


@functools.lru_cache(maxsize=1)
def _plans() -> dict:
    return json.loads((GOLDEN / "reference_program_plan.json").read_text())


def _replay(plan: dict):
    builder = B.ExecutableBuilder()
    program = builder.program(name="main")
    buffers = []
    for b in plan["buffers"]:
        if b["name"] is None:
            assert not b["persistent"]
            buffers.append(program.temporary_buffer(size_bytes=b["size_bytes"], alignment_bytes=b["alignment_bytes"]))
        else:
            declare = builder.persistent_buffer if b["persistent"] else program.buffer
            buffers.append(declare(name=b["name"], shape=b["shape"], dtype=getattr(B.DataType, b["dtype"]),
                                   writable=b["writable"], alignment_bytes=b["alignment_bytes"]))
    symbol = builder.add_symbol(B.SymbolArtifact(B.BinaryFormat.CUBIN, b"table", "table"))
    kernels: dict[str, B.KernelHandle] = {}
    for call in plan["calls"]:
        if call["kernel"] not in kernels:
            parameters = (B.ParameterType.POINTER,) * len(call["arguments"]) + (B.ParameterType.NULL_POINTER,) * 2
            kernels[call["kernel"]] = builder.add_kernel(B.KernelArtifact(
                B.BinaryFormat.CUBIN, call["kernel"].encode(), call["kernel"], parameters, (1, 1, 1), (32, 1, 1), 0))
        arguments = [symbol if a < 0 else buffers[a] for a in call["arguments"]]
        program.call(kernels[call["kernel"]], *arguments, readonly=[buffers[i] for i in call["readonly"]])
    return builder.build(), buffers


@pytest.mark.parametrize("case", ["tiny_b5", "bt4_b2"])
def test_linker_reproduces_the_reference_linker_on_the_reference_graph(case) -> None:
    plan = _plans()[case]
    executable, buffers = _replay(plan)
    program = executable.programs[0]
    assert [node.dependencies for node in program.nodes] == plan["dependencies"]
    want = plan["plans"]
    assert executable.persistent_allocation.size_bytes == want["persistent"]["size_bytes"]
    assert executable.persistent_allocation.alignment_bytes == want["persistent"]["alignment_bytes"]
    assert program.execution_allocation.size_bytes == want["execution"]["size_bytes"]
    assert program.execution_allocation.alignment_bytes == want["execution"]["alignment_bytes"]
    offsets = {int(k): v for kind in ("persistent", "execution") for k, v in want[kind]["offsets"].items()}
    checked = 0
    for node, call in zip(program.nodes, plan["calls"]):
        assert len(node.arguments) == len(call["arguments"])
        for argument, index in zip(node.arguments, call["arguments"]):
            if index < 0:
                assert argument.kind == "symbol"
                continue
            assert argument.kind == ("persistent" if plan["buffers"][index]["persistent"] else "execution")
            assert argument.offset == offsets[index], (call["kernel"], index)
            checked += 1
    assert checked > 3 * len(plan["calls"])
    named = {b.name: b.offset for b in executable.buffers + program.buffers}
    for index, b in enumerate(plan["buffers"]):
        if b["name"] is not None:
            assert named[b["name"]] == offsets[index]


def test_plan_of_the_dry_walk_is_the_plan_of_the_program_that_ran() -> None:
    """The execution allocation the CPU-only walk plans is byte for byte the size of the one the compiled
    program ran in on the GPU (stored beside its outputs), node counts included."""
    with np.load(GOLDEN / "reference_network_outputs.npz") as ran:
        for case, key in (("tiny_b5", "tiny_b5_s11"), ("bt4_b2", "bt4_b2_s14")):
            nodes, _kernels, execution_bytes, temporaries_bytes = (int(x) for x in ran[f"{key}/nodes"])
            plan = _plans()[case]
            assert len(plan["calls"]) == nodes
            assert plan["plans"]["execution"]["size_bytes"] == execution_bytes
            assert sum(b["size_bytes"] for b in plan["buffers"] if b["name"] is None) == temporaries_bytes
