"""The lc0ex bridge: the linker's plan (dependencies, buffer packing) and the kernel artifacts.

The linker cases restate the behaviours the reference pins for its own linker
(packages/lc0ex/tests/test_builder.py:42-192, packages/lc0ex/tests/test_kernel_builder.py:59-197) against
``lczero_triton_b200.lc0ex_bridge``: same declarations in, same sizes, offsets and dependency lists out.
The artifact cases compile real pointer-only entry points for sm_100a (nvcc needs no GPU) and, on a GPU,
launch them the way an lc0ex runtime does - module load, symbol lookup, a static grid and nothing but
pointers - and check the results against the CPU oracle.
"""

from __future__ import annotations

import json

import pytest
import torch

from lczero_triton_b200 import lc0ex_bridge as B
from oracle import bt4_oracle as O

F16, F32, U8, U64, BF16 = B.DataType.F16, B.DataType.F32, B.DataType.U8, B.DataType.U64, B.DataType.BF16
POINTER, NULL_POINTER = B.ParameterType.POINTER, B.ParameterType.NULL_POINTER


def _builder() -> B.ExecutableBuilder:
    return B.ExecutableBuilder().set_target(B.Vendor.NVIDIA, "sm_100a")


def _artifact(*, function: str = "kernel", parameters=(POINTER,)) -> B.KernelArtifact:
    return B.KernelArtifact(B.BinaryFormat.CUBIN, b"fake cubin", function, tuple(parameters), (2, 3, 1), (128, 1, 1), 256)


def _external(builder: B.ExecutableBuilder, name: str, *, writable: bool = False) -> B.Buffer:
    return builder.persistent_buffer(name=name, shape=(1,), dtype=F16, writable=writable)


# ------------------------------------------------------------------ buffers and packing

def test_buffer_is_an_opaque_storage_identity() -> None:
    buffer = B.Buffer()
    assert not hasattr(buffer, "shape") and not hasattr(buffer, "dtype") and not hasattr(buffer, "reshape")


def test_persistent_buffer_is_packed_into_the_executable_allocation() -> None:
    builder = _builder()
    result = builder.persistent_buffer(name="weights", shape=(2, 3), dtype=F16, alignment_bytes=16)
    executable = builder.build()
    assert isinstance(result, B.Buffer)
    assert (executable.persistent_allocation.size_bytes, executable.persistent_allocation.alignment_bytes) == (12, 16)
    first = executable.buffers[0]
    assert (first.name, first.offset, first.shape, first.data_type) == ("weights", 0, (2, 3), F16)


def test_a_name_is_one_buffer_within_its_scope_and_private_to_programs() -> None:
    builder = _builder()
    assert builder.persistent_buffer(name="w", shape=(2, 3), dtype=F16) is builder.persistent_buffer(name="w", shape=(2, 3), dtype=F16)
    first, second = builder.program(name="batch-1"), builder.program(name="batch-2")
    first.buffer(name="input", shape=(1,), dtype=F16)
    second.buffer(name="input", shape=(2,), dtype=F16)
    executable = builder.build()
    assert [p.name for p in executable.programs] == ["batch-1", "batch-2"]
    assert executable.programs[0].buffers[0].shape == (1,) and executable.programs[1].buffers[0].shape == (2,)


def test_unused_temporaries_do_not_force_an_allocation_and_used_ones_are_packed() -> None:
    builder = _builder()
    program = builder.program(name="main")
    program.temporary_buffer(size_bytes=128, alignment_bytes=64)
    assert builder.build().programs[0].execution_allocation is None
    first = program.temporary_buffer(size_bytes=64, alignment_bytes=32)
    second = program.temporary_buffer(size_bytes=64, alignment_bytes=32)
    kernel = builder.add_kernel(_artifact())
    program.call(kernel, first)
    program.call(kernel, second)
    assert builder.build().programs[0].execution_allocation.size_bytes == 128  # unordered: no sharing


def test_named_execution_buffers_keep_their_order_and_alignment() -> None:
    builder = _builder()
    program = builder.program(name="main")
    program.buffer(name="input", shape=(2,), dtype=F16, alignment_bytes=16)
    program.buffer(name="output", shape=(2,), dtype=F16, writable=True, alignment_bytes=16)
    main = builder.build().programs[0]
    assert main.execution_allocation.size_bytes == 20
    assert [(b.name, b.offset) for b in main.buffers] == [("input", 0), ("output", 16)]


@pytest.mark.parametrize(("dtype", "size"), [(F32, 4), (U8, 1), (F16, 2), (U64, 8), (BF16, 2)])
def test_data_type_sizes(dtype, size) -> None:
    assert B.data_type_size_bytes(dtype) == size


def test_unknown_dtype_is_rejected_at_declaration() -> None:
    with pytest.raises(KeyError):
        _builder().persistent_buffer(name="unknown", shape=(1,), dtype=B.DataType.UNKNOWN)


def test_metadata_and_target_survive_the_written_form(tmp_path) -> None:
    builder = _builder().set_metadata(b"fingerprint")
    builder.build_and_write(tmp_path / "net.lc0ex.json")
    restored = json.loads((tmp_path / "net.lc0ex.json").read_text())
    assert restored["metadata"] == "ZmluZ2VycHJpbnQ=" and restored["target"] == ["NVIDIA", "sm_100a"]
    assert restored["magic"] == 0x1C0E and restored["format"] == 1
    with pytest.raises(ValueError):
        B.ExecutableBuilder().build_and_write(tmp_path / "incomplete.lc0ex.json")


# ------------------------------------------------------------------ calls and dependencies

def test_call_serializes_kernel_metadata_and_argument_offsets() -> None:
    builder = _builder()
    program = builder.program(name="main")
    kernel = builder.add_kernel(_artifact(parameters=(POINTER, POINTER, POINTER)))
    program.call(kernel, _external(builder, "first"), _external(builder, "second"), _external(builder, "third"))
    executable = builder.build()
    node = executable.programs[0].nodes[0]
    assert executable.kernels[0].function == "kernel" and node.grid == (2, 3, 1) and node.block == (128, 1, 1)
    assert node.dynamic_shared_memory_bytes == 256
    assert [(a.kind, a.offset) for a in node.arguments] == [("persistent", 0), ("persistent", 2), ("persistent", 4)]


def test_null_pointer_slots_belong_to_the_runtime_and_the_count_is_checked() -> None:
    builder = _builder()
    program = builder.program(name="main")
    kernel = builder.add_kernel(_artifact(parameters=(POINTER, NULL_POINTER, POINTER)))
    first, second = _external(builder, "first"), _external(builder, "second")
    program.call(kernel, first, second)
    executable = builder.build()
    assert list(executable.kernels[0].parameters) == [POINTER, NULL_POINTER, POINTER]
    assert [a.offset for a in executable.programs[0].nodes[0].arguments] == [0, 2]
    with pytest.raises(ValueError, match="Kernel call has 3 arguments; expected 2."):
        program.call(kernel, first, second, first)


def test_readonly_weights_order_nothing_and_writers_order_readers_and_writers() -> None:
    builder = _builder()
    program = builder.program(name="main")
    kernel = builder.add_kernel(_artifact())
    weights = _external(builder, "weights")
    program.call(kernel, weights)
    program.call(kernel, weights)
    output = _external(builder, "output", writable=True)
    program.call(kernel, output)                       # 2: write
    program.call(kernel, output, readonly=(output,))   # 3: read  -> after 2
    program.call(kernel, output)                       # 4: write -> after 3 (and 2, implied)
    nodes = builder.build().programs[0].nodes
    assert [n.dependencies for n in nodes] == [[], [], [], [2], [3]]


def test_dependencies_are_transitively_reduced_but_keep_independent_readers() -> None:
    builder = _builder()
    program = builder.program(name="main")
    one = builder.add_kernel(_artifact())
    two = builder.add_kernel(_artifact(function="two", parameters=(POINTER, POINTER)))
    x, y = _external(builder, "x", writable=True), _external(builder, "y", writable=True)
    program.call(one, x)                          # 0: write x
    program.call(two, x, y, readonly=(x,))        # 1: read x, write y   -> [0]
    program.call(two, x, y, readonly=(x, y))      # 2: read x, read y    -> [1]      (0 is implied by 1)
    program.call(one, x, readonly=(x,))           # 3: read x            -> [0]
    program.call(one, x)                          # 4: write x           -> [2, 3]   (readers 1, 2, 3; 1 implied by 2)
    nodes = builder.build().programs[0].nodes
    assert [n.dependencies for n in nodes] == [[], [0], [1], [0], [2, 3]]


def test_ordered_temporaries_share_one_range_and_prefer_a_slot_of_their_own_size() -> None:
    builder = _builder()
    program = builder.program(name="main")
    kernel = builder.add_kernel(_artifact(parameters=(POINTER, POINTER)))
    first = program.temporary_buffer(size_bytes=64, alignment_bytes=32)
    second = program.temporary_buffer(size_bytes=64, alignment_bytes=32)
    bridge = _external(builder, "bridge", writable=True)
    program.call(kernel, first, bridge)
    program.call(kernel, bridge, second, readonly=(bridge,))
    main = builder.build().programs[0]
    assert main.execution_allocation.size_bytes == 64
    assert main.nodes[0].arguments[0].offset == main.nodes[1].arguments[1].offset
    assert main.nodes[1].dependencies == [0]
    # a chain 256 -> 64 -> 256 -> 64 bytes: each range is dead two steps later, and a slot of the same size is preferred
    builder = _builder()
    program = builder.program(name="chain")
    kernel = builder.add_kernel(_artifact(parameters=(POINTER, POINTER)))
    sizes = [256, 64, 256, 64]
    temps = [program.temporary_buffer(size_bytes=s, alignment_bytes=64) for s in sizes]
    for src, dst in zip(temps, temps[1:]):
        program.call(kernel, dst, src, readonly=(src,))
    chain = builder.build().programs[0]
    offsets = {}
    for node, (src, dst) in zip(chain.nodes, zip(range(3), range(1, 4))):
        offsets[dst], offsets[src] = node.arguments[0].offset, node.arguments[1].offset
    assert offsets[2] == offsets[0] and offsets[3] == offsets[1] and offsets[0] != offsets[1]
    assert chain.execution_allocation.size_bytes == 256 + 64


def test_equal_artifacts_are_one_kernel_and_symbols_are_pointer_arguments() -> None:
    builder = _builder()
    assert builder.add_kernel(_artifact()) is builder.add_kernel(_artifact())
    program = builder.program(name="main")
    kernel = builder.add_kernel(_artifact(parameters=(POINTER, POINTER)))
    output = _external(builder, "output", writable=True)
    symbol = builder.add_symbol(B.SymbolArtifact(B.BinaryFormat.CUBIN, b"fake cubin", "mapping_table"))
    program.call(kernel, output, symbol)
    executable = builder.build()
    argument = executable.programs[0].nodes[0].arguments[1]
    assert isinstance(symbol, B.SymbolHandle) and len(executable.binaries) == 1
    assert (argument.kind, argument.binary_idx, argument.symbol_name, argument.offset) == ("symbol", 0, "mapping_table", None)


# ------------------------------------------------------------------ kernel artifacts of this library

def test_compiled_artifacts_are_pointer_only_with_static_launch_metadata() -> None:
    ln = B.compile_kernel("layer_norm_skip", {"ROWS": 640, "WIDTH": 1024, "ACTIVATION": 0, "EPSILON": "1e-3f"})
    assert ln.binary_data[:4] == b"\x7fELF" and ln.function.encode() in ln.binary_data
    assert ln.parameters == (POINTER,) * 7 and ln.grid == (320, 1, 1) and ln.block == (64, 1, 1)
    assert ln.dynamic_shared_memory_bytes == 0
    assert set(B.adapters()) >= {"layer_norm", "layer_norm_skip", "softmax_64", "qk_64", "expand_planes", "nchw_to_nhwc",
                                 "preprocess_attention_body", "input_gating", "add_vectors", "add_bias_batched",
                                 "copy_type_converted", "policy_map", "promotion_logits", "fused_qkv_bias", "matmul_simt"}
    with pytest.raises(ValueError):
        B.compile_kernel("softmax_64", {})
    # and it links: weights persistent, activations temporaries, one program
    builder = _builder()
    program = builder.program(name="batch-10")
    kernel = builder.add_kernel(ln)
    names = ("/encoder0/mha/out/dense/b/w", "/encoder0/ln1/w/scale", "/encoder0/ln1/w/bias")
    bias, gamma, beta = (builder.persistent_buffer(name=n, shape=(1024,), dtype=BF16, alignment_bytes=16) for n in names)
    alpha = builder.persistent_buffer(name="/encoder0/alpha*input/w", shape=(1,), dtype=BF16, alignment_bytes=16)
    rows = [program.temporary_buffer(size_bytes=640 * 1024 * 2, alignment_bytes=256) for _ in range(3)]
    program.call(kernel, rows[2], rows[0], bias, rows[1], gamma, beta, alpha, readonly=(rows[0], rows[1]))
    executable = builder.build()
    assert executable.programs[0].execution_allocation.size_bytes == 3 * 640 * 1024 * 2
    assert len(executable.binaries) == 1 and executable.kernels[0].function == ln.function


def _launch(artifact: B.KernelArtifact, tensors: list[torch.Tensor]) -> None:
    """What an lc0ex runtime does with a node: load the binary, look the entry point up, launch it with its
    static grid and block and the pointer arguments.  (``tensors`` are device tensors; holding them here keeps
    their memory from being handed out again before the kernel has run.)"""
    import ctypes

    assert all(t.is_cuda for t in tensors)
    pointers = [t.data_ptr() for t in tensors]

    from cuda.bindings import driver

    def ok(result):
        assert result[0] == driver.CUresult.CUDA_SUCCESS, result[0]
        return result[1] if len(result) == 2 else result[1:]

    module = ok(driver.cuModuleLoadData(artifact.binary_data))
    function = ok(driver.cuModuleGetFunction(module, artifact.function.encode()))
    values = (ctypes.c_void_p * len(pointers))(*pointers)
    slots = (ctypes.c_void_p * len(pointers))(*[ctypes.addressof(values) + i * ctypes.sizeof(ctypes.c_void_p)
                                                for i in range(len(pointers))])
    stream = torch.cuda.current_stream().cuda_stream
    result = driver.cuLaunchKernel(function, *artifact.grid, *artifact.block, artifact.dynamic_shared_memory_bytes,
                                   stream, ctypes.addressof(slots), 0)
    assert result[0] == driver.CUresult.CUDA_SUCCESS, result[0]
    torch.cuda.synchronize()
    ok(driver.cuModuleUnload(module))


@pytest.mark.gpu
def test_artifacts_run_as_an_lc0ex_runtime_would_launch_them() -> None:
    torch.cuda.init()
    torch.zeros(1, device="cuda")
    gen = torch.Generator().manual_seed(11)
    rows, width = 333, 1024
    x, skip = (torch.randn((rows, width), generator=gen).to(torch.bfloat16) for _ in range(2))
    bias, beta = (torch.randn(width, generator=gen).mul(0.3).to(torch.bfloat16) for _ in range(2))
    gamma = (1 + 0.1 * torch.randn(width, generator=gen)).to(torch.bfloat16)
    alpha = torch.tensor([0.43]).to(torch.bfloat16)
    ln = B.compile_kernel("layer_norm_skip", {"ROWS": rows, "WIDTH": width, "ACTIVATION": 1, "EPSILON": "1e-3f"})
    dev = [t.cuda() for t in (x, bias, skip, gamma, beta, alpha)]
    out = torch.empty((rows, width), dtype=torch.bfloat16, device="cuda")
    _launch(ln, [out, *dev])
    want = O.layer_norm(x.float(), bias.float(), gamma.float(), beta.float(), "mish", 1e-3, skip=skip.float(), alpha=alpha.float())
    torch.testing.assert_close(out.float().cpu(), want, rtol=8e-3, atol=8e-3)

    rows = 5000
    qk = (torch.randn((rows, 64), generator=gen) * 3).to(torch.bfloat16)
    smolgen = (torch.randn((rows, 64), generator=gen) * 2).to(torch.bfloat16)
    sm = B.compile_kernel("softmax_64", {"ROWS": rows})
    probs = torch.empty((rows, 64), dtype=torch.bfloat16, device="cuda")
    _launch(sm, [probs, qk.cuda(), smolgen.cuda()])
    torch.testing.assert_close(probs.float().cpu(), O.softmax_64(qk, smolgen).float(), rtol=8e-3, atol=2e-3)


@pytest.mark.gpu
def test_element_wise_and_gather_artifacts_match_the_oracle() -> None:
    from lczero_triton_b200 import mapping_table
    from lczero_triton_b200.synthetic import synthetic_planes

    torch.zeros(1, device="cuda")
    gen = torch.Generator().manual_seed(12)
    bf = torch.bfloat16
    batch = 5
    # expand_planes (exact)
    masks, values = synthetic_planes(batch, 3)
    planes = torch.empty((batch, 112, 64), dtype=bf, device="cuda")
    _launch(B.compile_kernel("expand_planes", {"PLANE_COUNT": batch * 112}),
            [planes, masks.cuda(), values.cuda()])
    assert torch.equal(planes.float().cpu(), O.expand_planes(masks, values, bf).float())
    # add_vectors with mish, input_gating
    x = torch.randn((batch * 64, 128), generator=gen).to(bf)
    bias = torch.randn(128, generator=gen).to(bf)
    out = torch.empty_like(x, device="cuda")
    _launch(B.compile_kernel("add_vectors", {"ELEMENTS": x.numel(), "BIAS_ELEMENTS": 128, "ACTIVATION": 1}),
            [out, x.cuda(), bias.cuda()])
    torch.testing.assert_close(out.float().cpu(), O.add_vectors(x.float(), bias.float(), "mish"), rtol=8e-3, atol=4e-3)
    mult, add = (torch.randn((64, 128), generator=gen).to(bf) for _ in range(2))
    _launch(B.compile_kernel("input_gating", {"BATCH": batch, "SQUARES": 64, "CHANNELS": 128}),
            [out, x.cuda(), mult.cuda(), add.cuda()])
    want = O.input_gating(x.float().reshape(batch, 64, 128), mult.float(), add.float()).reshape(-1, 128)
    torch.testing.assert_close(out.float().cpu(), want, rtol=8e-3, atol=4e-3)
    # three bias adds of different widths in one launch, in place (the reference's own widths 11 / 13 / 9)
    widths = (11, 13, 9)
    parts = [torch.randn((9, w), generator=gen).to(bf) for w in widths]
    biases = [torch.randn(w, generator=gen).to(bf) for w in widths]
    dev_parts, dev_biases = [t.cuda() for t in parts], [t.cuda() for t in biases]
    _launch(B.compile_kernel("fused_qkv_bias", {"ROWS": 9, "QUERY_WIDTH": 11, "KEY_WIDTH": 13, "VALUE_WIDTH": 9}),
            [t for trio in zip(dev_parts, dev_parts, dev_biases) for t in trio])
    for got, x_, b_ in zip(dev_parts, parts, biases):
        torch.testing.assert_close(got.float().cpu(), (x_.float() + b_.float()).to(bf).float(), rtol=0, atol=0)
    # the CUDA-core matmul on the value head's last layer shape and on the reference's tail case 7 x 37 x 11
    for m, k, n in ((batch, 128, 3), (7, 37, 11)):
        a_, w_ = (torch.randn(shape, generator=gen).mul(0.3).to(bf) for shape in ((m, k), (k, n)))
        product = torch.empty((m, n), dtype=bf, device="cuda")
        _launch(B.compile_kernel("matmul_simt", {"M": m, "N": n, "K": k}), [product, a_.cuda(), w_.cuda()])
        torch.testing.assert_close(product.float().cpu(), O.matmul(a_, w_), rtol=8e-3, atol=8e-3)
    # body_qk on the tensor cores, policy_map and the f32 widening (exact)
    heads = 4
    q, k = (torch.randn((batch, 64, heads * 32), generator=gen).mul(0.5).to(bf) for _ in range(2))
    scale = torch.tensor([0.173]).to(bf)
    scores = torch.empty((batch, heads, 64, 64), dtype=bf, device="cuda")
    _launch(B.compile_kernel("qk_64", {"BATCH_COUNT": batch * heads, "DEPTH": 32, "HEADS": heads, "INTERLEAVED": 1,
                                       "OUT_STRIDE": 4096}),
            [scores, q.cuda(), k.cuda(), scale.cuda()])
    torch.testing.assert_close(scores.float().cpu(), O.body_qk(q, k, float(scale.float()), heads), rtol=1e-2, atol=1e-2)
    records = torch.randn((batch, 4288), generator=gen).to(bf)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)
    gathered = torch.empty((batch, 1858), dtype=bf, device="cuda")
    _launch(B.compile_kernel("policy_map", {"BATCH": batch, "IN_COUNT": 4288, "OUT_COUNT": 1858}),
            [gathered, records.cuda(), table.cuda()])
    assert torch.equal(gathered.float().cpu(), O.policy_map(records, table).float())
    wide = torch.empty((batch, 1858), dtype=torch.float32, device="cuda")
    _launch(B.compile_kernel("copy_type_converted", {"ELEMENTS": batch * 1858}), [wide, gathered])
    assert torch.equal(wide.cpu(), gathered.float().cpu())


def _execute(executable: B.Executable, program_index: int, persistent: dict[str, torch.Tensor],
             inputs: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """A minimal lc0ex runtime for the tests: one allocation for the persistent buffers, one for the program,
    named buffers filled by name, nodes launched in an order that respects their dependency lists (here: index
    order, checked), every argument resolved to allocation base + offset.  Returns the program's named buffers."""
    program = executable.programs[program_index]
    element = {B.DataType.F32: torch.float32, B.DataType.BF16: torch.bfloat16, B.DataType.F16: torch.float16,
               B.DataType.U8: torch.uint8, B.DataType.U64: torch.int64}
    arenas = {"persistent": torch.zeros(executable.persistent_allocation.size_bytes + 256, dtype=torch.uint8, device="cuda"),
              "execution": torch.zeros(program.execution_allocation.size_bytes + 256, dtype=torch.uint8, device="cuda")}

    def view(kind: str, buffer: B.NamedBuffer) -> torch.Tensor:
        count = 1
        for extent in buffer.shape:
            count *= extent
        nbytes = count * B.data_type_size_bytes(buffer.data_type)
        return arenas[kind][buffer.offset:buffer.offset + nbytes].view(element[buffer.data_type]).reshape(buffer.shape)

    for buffer in executable.buffers:
        view("persistent", buffer).copy_(persistent[buffer.name])
    named = {buffer.name: view("execution", buffer) for buffer in program.buffers}
    for name, value in inputs.items():
        named[name].copy_(value)
    done: set[int] = set()
    for index, node in enumerate(program.nodes):
        assert all(dep in done for dep in node.dependencies), (index, node.dependencies)
        kernel = executable.kernels[node.kernel_idx]
        artifact = B.KernelArtifact(*executable.binaries[kernel.binary_idx], kernel.function, kernel.parameters,
                                    node.grid, node.block, node.dynamic_shared_memory_bytes)
        pointers = [arenas[a.kind][a.offset:] for a in node.arguments]
        _launch(artifact, pointers)
        done.add(index)
    return named


@pytest.mark.gpu
def test_a_linked_program_runs_the_policy_tail_of_the_graph() -> None:
    """network.py:1261-1356 as an lc0ex program of pointer-only kernels: policy QK into the 4288-slot record,
    promotion logits in place, gather through the table, widening to f32.  Weights and the table are named
    persistent buffers, Q / K the program's named inputs, the record and the gathered logits temporaries that
    the linker places, the f32 logits the named output; the run is checked against the oracle's policy head."""
    from lczero_triton_b200 import mapping_table

    torch.zeros(1, device="cuda")
    gen = torch.Generator().manual_seed(21)
    batch, width = 6, 128
    bf = torch.bfloat16
    q, k = (torch.randn((batch, 64, width), generator=gen).mul(0.4).to(bf) for _ in range(2))
    promotion_w = torch.randn((width, 4), generator=gen).mul(0.3).to(bf)
    scale = torch.tensor([width ** -0.5]).to(bf)
    table = torch.tensor(mapping_table.values(), dtype=torch.int32)

    builder = B.ExecutableBuilder().set_target(B.Vendor.NVIDIA, "sm_100a")
    program = builder.program(name=f"batch-{batch}")
    qk = builder.add_kernel(B.compile_kernel("qk_64", {"BATCH_COUNT": batch, "DEPTH": width, "HEADS": 1, "INTERLEAVED": 0,
                                                       "OUT_STRIDE": 4288}))
    promo = builder.add_kernel(B.compile_kernel("promotion_logits", {"BATCH": batch, "WIDTH": width}))
    gather = builder.add_kernel(B.compile_kernel("policy_map", {"BATCH": batch, "IN_COUNT": 4288, "OUT_COUNT": 1858}))
    widen = builder.add_kernel(B.compile_kernel("copy_type_converted", {"ELEMENTS": batch * 1858}))
    w_scale = builder.persistent_buffer(name="/policy/scale/w", shape=(1,), dtype=BF16, alignment_bytes=256)
    w_promo = builder.persistent_buffer(name="/policy/promotion/matmul/w", shape=(width, 4), dtype=BF16, alignment_bytes=256)
    # the reference exports the table as a module symbol; a named persistent buffer of raw bytes serves here
    w_table = builder.persistent_buffer(name="/policy/mapping_table", shape=(1858 * 4,), dtype=U8, alignment_bytes=256)
    in_q = program.buffer(name="/policy/Q", shape=(batch, 64, width), dtype=BF16, alignment_bytes=256)
    in_k = program.buffer(name="/policy/K", shape=(batch, 64, width), dtype=BF16, alignment_bytes=256)
    out = program.buffer(name="/output/policy", shape=(batch, 1858), dtype=F32, writable=True, alignment_bytes=256)
    records = program.temporary_buffer(size_bytes=batch * 4288 * 2, alignment_bytes=256)
    gathered = program.temporary_buffer(size_bytes=batch * 1858 * 2, alignment_bytes=256)
    program.call(qk, records, in_q, in_k, w_scale)
    program.call(promo, records, in_k, w_promo)
    program.call(gather, gathered, records, w_table, readonly=(records,))
    program.call(widen, out, gathered, readonly=(gathered,))
    executable = builder.build()
    nodes = executable.programs[0].nodes
    assert [n.dependencies for n in nodes] == [[], [0], [1], [2]]
    assert executable.programs[0].execution_allocation.size_bytes >= batch * (2 * 64 * width * 2 + 1858 * 4 + 4288 * 2)

    named = _execute(executable, 0,
                     {"/policy/scale/w": scale.cuda(), "/policy/promotion/matmul/w": promotion_w.cuda(),
                      "/policy/mapping_table": table.cuda().view(torch.uint8)},
                     {"/policy/Q": q.cuda(), "/policy/K": k.cuda()})
    want_records = O.policy_qk(q, k, float(scale.float()))
    want_records = want_records.to(bf).float()
    want_records[:, 4096:] = O.promotion_logits(want_records, k, promotion_w).to(bf).float()
    want = O.policy_map(want_records, table).float()
    torch.testing.assert_close(named["/output/policy"].cpu(), want, rtol=1.6e-2, atol=1.6e-2)
