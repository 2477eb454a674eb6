"""Bridge to the lc0ex executable format: kernels of this library as lc0ex kernel artifacts, and a linker
that records calls, orders them and plans the buffers the way the reference's linker does.

The reference packs its Triton CUBINs, a buffer allocation plan and a node list into one ``.lc0ex`` file
that an lc0 backend executes (packages/lc0ex/src/lc0ex/builder.py:232-286).  The contract a kernel has to
meet there is narrow (packages/lc0ex/src/lc0ex/kernel_builder.py:9-19,
packages/lc0ex/src/lc0ex/triton_module_compiler.py:13-16,60): a CUBIN, an entry symbol, a parameter list
made of device POINTERS only (plus slots the runtime fills with a null pointer), and a grid, block and
dynamic shared-memory size fixed at link time.  This module provides, for this library's kernels,

* ``KernelArtifact`` / ``SymbolArtifact`` with the reference's fields, and ``compile_kernel``: one
  ``nvcc -cubin`` run for sm_100a over a generated translation unit that wraps a kernel body of
  ``csrc/`` in an ``extern "C"`` entry point whose parameters are pointers only, every shape baked in as a
  compile-time constant (``adapters()`` lists the ops that have such a wrapper);
* ``ExecutableBuilder`` / ``ProgramBuilder`` with the reference's surface: named persistent buffers
  (weights), per-program named buffers (inputs / outputs) and anonymous temporaries, ``call`` with the
  reference's argument-count check (builder.py:123-132), and ``build`` which derives for every node its
  REDUCED dependency list from the read / write hazards on the opaque buffers (builder.py:325-499) and
  packs each allocation, letting temporaries share a range only when every access of one is ordered
  before every access of the other (buffer_builder.py:183-277).  The result is the same plan the
  reference computes - same dependency lists, same offsets - as a tree of plain dataclasses.

Not provided: the protobuf wire format.  ``lc0ex.proto`` lives in the lc0 fork that the reference
includes as an un-vendored submodule, so ``Executable.to_dict`` / ``build_and_write`` emit a JSON document
with the same fields instead of ``NeuralExecutable.SerializeToString()``.

The tensor-core GEMM and the fused attention read their operands through TMA descriptors, which hold
absolute addresses and therefore cannot be link-time constants; how they fit the pointer-only contract is
set out beside ``TENSORMAP_NOTE`` below.
"""

from __future__ import annotations

import base64
import enum
import json
import math
import pathlib
import shutil
import subprocess
import tempfile
from collections.abc import Sequence
from dataclasses import asdict, dataclass, field

CSRC = pathlib.Path(__file__).resolve().parent / "csrc"

TENSORMAP_NOTE = """\
A CUtensorMap encodes the tensor's absolute base address, so it can be neither a link-time constant nor a
kernel parameter of a pointer-only ABI.  The plan for the TMA kernels (tensor-core GEMM, fused attention):
each compiled module exports, as an immutable module symbol (a SymbolArtifact), one descriptor TEMPLATE per
operand - encoded for the static shape, box and swizzle with a placeholder address; every program starts
with one small node that receives the templates and the operand buffers as pointers, copies each template
into a descriptor table (an ordinary temporary of the execution allocation) and patches its address field
on the device (tensormap.replace.tile.global_address, then the tensormap proxy fence); the TMA kernels
then take a pointer to their slice of that table as one more pointer parameter and read the descriptors
from global memory instead of from __grid_constant__ parameters.  Nothing but pointers crosses the ABI and
the grid stays static."""


class ParameterType(enum.IntEnum):
    """Kernel parameter kinds of the lc0ex ABI (``PARAMETER_TYPE_*`` of the reference's protobuf)."""

    POINTER = 1
    NULL_POINTER = 2


class BinaryFormat(enum.IntEnum):
    CUBIN = 1


class Vendor(enum.IntEnum):
    NVIDIA = 1


class DataType(enum.IntEnum):
    """Element types a named buffer may declare (buffer_builder.py:70-85)."""

    UNKNOWN = 0
    F32 = 1
    U8 = 2
    F16 = 3
    U64 = 4
    BF16 = 5


_ELEMENT_BYTES = {DataType.F32: 4, DataType.U8: 1, DataType.F16: 2, DataType.U64: 8, DataType.BF16: 2}


def data_type_size_bytes(dtype: DataType) -> int:
    """Bytes per element; ``KeyError`` for anything that is not a concrete type."""
    return _ELEMENT_BYTES[DataType(dtype)]


@dataclass(frozen=True)
class KernelArtifact:
    """One exported entry point and its launch metadata (kernel_builder.py:9-19)."""

    binary_format: BinaryFormat
    binary_data: bytes
    function: str
    parameters: tuple[ParameterType, ...]
    grid: tuple[int, int, int]
    block: tuple[int, int, int]
    dynamic_shared_memory_bytes: int


@dataclass(frozen=True)
class SymbolArtifact:
    """One immutable pointer symbol exported by a compiled module (kernel_builder.py:27-33)."""

    binary_format: BinaryFormat
    binary_data: bytes
    symbol_name: str


class KernelHandle:
    """Opaque linker-side reference to a registered kernel."""


class SymbolHandle:
    """Opaque linker-side reference to a registered module symbol."""


class Buffer:
    """Opaque identity of one logical device-memory range: no shape, no dtype, no views."""

    __slots__ = ()


# --------------------------------------------------------------------------- the linked result

@dataclass
class AllocationInfo:
    size_bytes: int
    alignment_bytes: int


@dataclass
class NamedBuffer:
    name: str
    offset: int
    data_type: DataType
    shape: tuple[int, ...]


@dataclass
class Argument:
    """Either a range of an allocation (``kind`` "persistent" / "execution" and a byte offset) or a module symbol."""

    kind: str
    offset: int | None = None
    binary_idx: int | None = None
    symbol_name: str | None = None


@dataclass
class Node:
    kernel_idx: int
    dependencies: list[int]
    grid: tuple[int, int, int]
    block: tuple[int, int, int]
    dynamic_shared_memory_bytes: int
    arguments: list[Argument]


@dataclass
class Program:
    name: str
    metadata: bytes | None
    execution_allocation: AllocationInfo | None
    buffers: list[NamedBuffer]
    nodes: list[Node]


@dataclass
class KernelEntry:
    binary_idx: int
    function: str
    parameters: tuple[ParameterType, ...]


@dataclass
class Executable:
    magic: int
    format: int
    target: tuple[Vendor, str] | None
    metadata: bytes | None
    persistent_allocation: AllocationInfo | None
    buffers: list[NamedBuffer]
    binaries: list[tuple[BinaryFormat, bytes]]
    kernels: list[KernelEntry]
    programs: list[Program] = field(default_factory=list)

    def to_dict(self) -> dict:
        def clean(value):
            if isinstance(value, bytes):
                return base64.b64encode(value).decode()
            if isinstance(value, enum.Enum):
                return value.name
            if isinstance(value, dict):
                return {k: clean(v) for k, v in value.items()}
            if isinstance(value, (list, tuple)):
                return [clean(v) for v in value]
            return value

        return clean(asdict(self))


# --------------------------------------------------------------------------- buffers and their packing

@dataclass
class _Range:
    allocation: object          # identity token of the allocation
    size_bytes: int
    alignment_bytes: int
    writable: bool
    name: str | None = None     # None: an anonymous temporary, free to share storage
    shape: tuple[int, ...] = ()
    dtype: DataType | None = None


def _round_up(value: int, alignment: int) -> int:
    return -(-value // alignment) * alignment


class _Storage:
    """Every logical range of an executable, grouped by allocation (one persistent, one per program)."""

    def __init__(self) -> None:
        self.persistent = object()
        self.ranges: dict[Buffer, _Range] = {}
        self.members: dict[object, list[Buffer]] = {self.persistent: []}
        self.named: dict[tuple[object, str], Buffer] = {}

    def new_allocation(self) -> object:
        token = object()
        self.members[token] = []
        return token

    def declare(self, allocation: object, *, name: str, shape: Sequence[int], dtype: DataType, writable: bool,
                alignment_bytes: int | None) -> Buffer:
        known = self.named.get((allocation, name))
        if known is not None:  # a name is ONE buffer within its scope
            return known
        element = data_type_size_bytes(dtype)
        shape = tuple(int(s) for s in shape)
        buffer = Buffer()
        self.ranges[buffer] = _Range(allocation, math.prod(shape) * element,
                                     element if alignment_bytes is None else alignment_bytes, writable, name, shape,
                                     DataType(dtype))
        self.members[allocation].append(buffer)
        self.named[(allocation, name)] = buffer
        return buffer

    def temporary(self, allocation: object, size_bytes: int, alignment_bytes: int) -> Buffer:
        buffer = Buffer()
        self.ranges[buffer] = _Range(allocation, size_bytes, alignment_bytes, True)
        self.members[allocation].append(buffer)
        return buffer

    def pack(self, allocation: object, overlap: dict[Buffer, set[Buffer]]):
        """Lay out one allocation: named buffers first, in declaration order, each at its alignment; then the
        temporaries that some node uses (the keys of ``overlap``), grouped into shared slots.  A temporary
        joins an existing slot only if it overlaps in time with none of the slot's members; among such slots
        it prefers one of exactly its size, then the smallest resulting slot, then the smallest resulting
        alignment (buffer_builder.py:236-277).  Returns ``(AllocationInfo, {buffer: offset})`` or ``None``
        for an allocation nothing lives in."""
        named = [b for b in self.members[allocation] if self.ranges[b].name is not None]
        used = [b for b in self.members[allocation] if self.ranges[b].name is None and b in overlap]
        if not named and not used:
            return None
        offsets: dict[Buffer, int] = {}
        size, alignment = 0, 1
        for buffer in named:
            r = self.ranges[buffer]
            alignment = max(alignment, r.alignment_bytes)
            size = _round_up(size, r.alignment_bytes)
            offsets[buffer] = size
            size += r.size_bytes
        slots: list[dict] = []
        for buffer in used:
            r = self.ranges[buffer]
            free = [s for s in slots if not (overlap[buffer] & s["members"])]
            if free:
                slot = min(free, key=lambda s: (s["size"] != r.size_bytes, max(s["size"], r.size_bytes),
                                                max(s["alignment"], r.alignment_bytes)))
                slot["size"] = max(slot["size"], r.size_bytes)
                slot["alignment"] = max(slot["alignment"], r.alignment_bytes)
                slot["members"].add(buffer)
            else:
                slots.append({"size": r.size_bytes, "alignment": r.alignment_bytes, "members": {buffer}})
        for slot in slots:
            alignment = max(alignment, slot["alignment"])
            size = _round_up(size, slot["alignment"])
            for buffer in slot["members"]:
                offsets[buffer] = size
            size += slot["size"]
        return AllocationInfo(size, alignment), offsets

    def named_buffers(self, allocation: object, offsets: dict[Buffer, int]) -> list[NamedBuffer]:
        return [NamedBuffer(self.ranges[b].name, offsets[b], self.ranges[b].dtype, self.ranges[b].shape)
                for b in self.members[allocation] if self.ranges[b].name is not None]


# --------------------------------------------------------------------------- programs

@dataclass
class _Call:
    kernel: KernelHandle
    arguments: tuple[Buffer | SymbolHandle, ...]
    reads_only: frozenset[Buffer]


def order_calls(calls: Sequence[_Call]) -> tuple[list[list[int]], list[int]]:
    """Dependencies of every call on earlier calls, transitively reduced, and every call's ancestor set.

    Hazards on the opaque buffer identities: a read depends on the last write (RAW); a write depends on the
    last write (WAW) and on every read since it (WAR).  A dependency already implied by another one (it is
    an ancestor of a later direct dependency) is dropped, so the lists stay short while the partial order is
    unchanged (builder.py:447-484).  Ancestor sets are integers used as bit sets, bit i = call i."""
    last_write: dict[Buffer, int] = {}
    reads_since: dict[Buffer, list[int]] = {}
    ancestors: list[int] = []
    reduced: list[list[int]] = []
    for index, call in enumerate(calls):
        direct: set[int] = set()
        for buffer in {a for a in call.arguments if isinstance(a, Buffer)}:
            if buffer in last_write:
                direct.add(last_write[buffer])
            if buffer in call.reads_only:
                reads_since.setdefault(buffer, []).append(index)
            else:
                direct.update(reads_since.get(buffer, ()))
                last_write[buffer] = index
                reads_since[buffer] = []
        kept: list[int] = []
        reach = 0
        for dep in sorted(direct, reverse=True):  # latest first: it is the most likely to imply the others
            if not (reach >> dep) & 1:
                kept.append(dep)
                reach |= ancestors[dep] | (1 << dep)
        reduced.append(kept[::-1])
        ancestors.append(reach)
    return reduced, ancestors


def overlapping_temporaries(calls: Sequence[_Call], ancestors: Sequence[int], storage: _Storage) -> dict[Buffer, set[Buffer]]:
    """For every temporary some call touches, the temporaries of the same allocation it may be live together
    with: two ranges may share storage only if EVERY access of one is an ancestor of every access of the
    other (builder.py:486-499)."""
    touched: dict[Buffer, list[int]] = {}
    for index, call in enumerate(calls):
        for buffer in {a for a in call.arguments if isinstance(a, Buffer)}:
            if storage.ranges[buffer].name is None:
                touched.setdefault(buffer, []).append(index)
    overlap: dict[Buffer, set[Buffer]] = {b: set() for b in touched}
    items = list(touched.items())

    def all_before(first: list[int], second: list[int]) -> bool:
        return all((ancestors[s] >> f) & 1 for f in first for s in second)

    for i, (a, a_calls) in enumerate(items):
        for b, b_calls in items[i + 1:]:
            if storage.ranges[a].allocation is not storage.ranges[b].allocation:
                continue
            if not (all_before(a_calls, b_calls) or all_before(b_calls, a_calls)):
                overlap[a].add(b)
                overlap[b].add(a)
    return overlap


class ProgramBuilder:
    """One program (one batch size of the network) and its private execution allocation."""

    def __init__(self, owner: "ExecutableBuilder", name: str, metadata: bytes | None) -> None:
        self._owner = owner
        self._name = name
        self.metadata = metadata
        self._allocation = owner._storage.new_allocation()
        self._calls: list[_Call] = []

    @property
    def name(self) -> str:
        return self._name

    def buffer(self, *, name: str, shape: Sequence[int], dtype: DataType, writable: bool = False,
               alignment_bytes: int | None = None) -> Buffer:
        """A named input / output of this program."""
        return self._owner._storage.declare(self._allocation, name=name, shape=shape, dtype=dtype, writable=writable,
                                            alignment_bytes=alignment_bytes)

    def temporary_buffer(self, *, size_bytes: int, alignment_bytes: int) -> Buffer:
        """An anonymous scratch range; it exists in the plan only if some call uses it."""
        return self._owner._storage.temporary(self._allocation, size_bytes, alignment_bytes)

    def persistent_buffer(self, **kwargs) -> Buffer:
        return self._owner.persistent_buffer(**kwargs)

    def set_target(self, vendor: Vendor, architecture: str) -> "ProgramBuilder":
        self._owner.set_target(vendor, architecture)
        return self

    def add_kernel(self, kernel: KernelArtifact) -> KernelHandle:
        return self._owner.add_kernel(kernel)

    def add_symbol(self, symbol: SymbolArtifact) -> SymbolHandle:
        return self._owner.add_symbol(symbol)

    def call(self, kernel: KernelHandle, *arguments: Buffer | SymbolHandle, readonly: Sequence[Buffer] = ()) -> None:
        """Append one launch.  ``arguments`` fill the kernel's POINTER parameters in order (null-pointer slots
        are the runtime's).  Named buffers that were not declared writable are read-only accesses by
        default; ``readonly`` marks further read-only accesses."""
        artifact = self._owner._kernels[kernel]
        expected = sum(p != ParameterType.NULL_POINTER for p in artifact.parameters)
        if len(arguments) != expected:
            raise ValueError(f"Kernel call has {len(arguments)} arguments; expected {expected}.")
        ranges = self._owner._storage.ranges
        implicit = {a for a in arguments if isinstance(a, Buffer) and ranges[a].name is not None and not ranges[a].writable}
        self._calls.append(_Call(kernel, tuple(arguments), frozenset(set(readonly) | implicit)))


class ExecutableBuilder:
    """An executable: shared persistent storage (weights), kernels, and one program per batch size."""

    MAGIC = 0x1C0E
    FORMAT = 1

    def __init__(self) -> None:
        self._target: tuple[Vendor, str] | None = None
        self._metadata: bytes | None = None
        self._storage = _Storage()
        self._kernels: dict[KernelHandle, KernelArtifact] = {}
        self._kernel_by_value: dict[KernelArtifact, KernelHandle] = {}
        self._symbols: dict[SymbolHandle, SymbolArtifact] = {}
        self._symbol_by_value: dict[SymbolArtifact, SymbolHandle] = {}
        self._programs: list[ProgramBuilder] = []

    def persistent_buffer(self, *, name: str, shape: Sequence[int], dtype: DataType, writable: bool = False,
                          alignment_bytes: int | None = None) -> Buffer:
        return self._storage.declare(self._storage.persistent, name=name, shape=shape, dtype=dtype, writable=writable,
                                     alignment_bytes=alignment_bytes)

    def program(self, *, name: str, metadata: bytes | None = None) -> ProgramBuilder:
        program = ProgramBuilder(self, name, None if metadata is None else bytes(metadata))
        self._programs.append(program)
        return program

    def set_target(self, vendor: Vendor, architecture: str) -> "ExecutableBuilder":
        self._target = (Vendor(vendor), architecture)
        return self

    def set_metadata(self, metadata: bytes) -> "ExecutableBuilder":
        self._metadata = bytes(metadata)
        return self

    def add_kernel(self, kernel: KernelArtifact) -> KernelHandle:
        """Equal artifacts are one kernel: the same handle comes back."""
        handle = self._kernel_by_value.get(kernel)
        if handle is None:
            handle = KernelHandle()
            self._kernels[handle] = kernel
            self._kernel_by_value[kernel] = handle
        return handle

    def add_symbol(self, symbol: SymbolArtifact) -> SymbolHandle:
        handle = self._symbol_by_value.get(symbol)
        if handle is None:
            handle = SymbolHandle()
            self._symbols[handle] = symbol
            self._symbol_by_value[symbol] = handle
        return handle

    def build(self) -> Executable:
        storage = self._storage
        packed = storage.pack(storage.persistent, {})
        persistent_info, persistent_offsets = packed if packed is not None else (None, {})
        executable = Executable(self.MAGIC, self.FORMAT, self._target, self._metadata, persistent_info,
                                storage.named_buffers(storage.persistent, persistent_offsets), [], [])
        binary_index: dict[tuple[BinaryFormat, bytes], int] = {}

        def binary(fmt: BinaryFormat, data: bytes) -> int:
            key = (fmt, data)
            if key not in binary_index:
                binary_index[key] = len(executable.binaries)
                executable.binaries.append(key)
            return binary_index[key]

        kernel_index: dict[KernelHandle, int] = {}
        for handle, artifact in self._kernels.items():
            kernel_index[handle] = len(executable.kernels)
            executable.kernels.append(KernelEntry(binary(artifact.binary_format, artifact.binary_data),
                                                  artifact.function, tuple(artifact.parameters)))
        symbol_place = {h: (binary(s.binary_format, s.binary_data), s.symbol_name) for h, s in self._symbols.items()}
        for program in self._programs:
            dependencies, ancestors = order_calls(program._calls)
            overlap = overlapping_temporaries(program._calls, ancestors, storage)
            packed = storage.pack(program._allocation, overlap)
            info, offsets = packed if packed is not None else (None, {})
            nodes = []
            for call, deps in zip(program._calls, dependencies):
                artifact = self._kernels[call.kernel]
                arguments = []
                for argument in call.arguments:
                    if isinstance(argument, Buffer):
                        if storage.ranges[argument].allocation is storage.persistent:
                            arguments.append(Argument("persistent", persistent_offsets[argument]))
                        else:
                            arguments.append(Argument("execution", offsets[argument]))
                    else:
                        index, symbol_name = symbol_place[argument]
                        arguments.append(Argument("symbol", None, index, symbol_name))
                nodes.append(Node(kernel_index[call.kernel], deps, tuple(artifact.grid), tuple(artifact.block),
                                  artifact.dynamic_shared_memory_bytes, arguments))
            executable.programs.append(Program(program.name, program.metadata, info,
                                               storage.named_buffers(program._allocation, offsets), nodes))
        return executable

    def build_and_write(self, path: str | pathlib.Path) -> Executable:
        """Build and write the JSON form of the executable (not the reference's protobuf wire format, whose
        schema is not available).  Like the reference's serialiser, refuses an executable without a target."""
        executable = self.build()
        if executable.target is None:
            raise ValueError("the executable has no target: call set_target(vendor, architecture) first")
        target = pathlib.Path(path)
        target.parent.mkdir(parents=True, exist_ok=True)
        target.write_text(json.dumps(executable.to_dict()))
        return executable


# --------------------------------------------------------------------------- kernels of this library as artifacts

@dataclass(frozen=True)
class Adapter:
    """How one op of ``csrc/`` becomes a pointer-only entry point.

    ``source`` is the ``csrc`` file that holds the kernel body, ``pointers`` the entry point's parameters in
    the reference's ABI order (outputs, inputs, weights), ``constants`` the names of the integers / floats
    baked in per specialization, ``body`` the C++ statements of the entry point (they see the pointers by
    name and the constants as macros), and ``launch`` maps the constants to ``(grid, block, smem)``."""

    source: str
    pointers: tuple[tuple[str, str], ...]  # (C type, name)
    constants: tuple[str, ...]
    body: str
    launch: object


_LN_WARPS_PER_BLOCK = 2  # kWarpsPerBlock of csrc/layernorm.cu: one warp per row, this many rows per CTA


def _ln_launch(c: dict) -> tuple[tuple[int, int, int], tuple[int, int, int], int]:
    return ((-(-c["ROWS"] // _LN_WARPS_PER_BLOCK), 1, 1), (32 * _LN_WARPS_PER_BLOCK, 1, 1), 0)


def _stream_launch(total_of):
    """Grid of the grid-stride element-wise kernels: one thread per element up to 32 CTAs per SM of a B200."""
    def launch(c: dict) -> tuple[tuple[int, int, int], tuple[int, int, int], int]:
        return ((max(1, min(-(-total_of(c) // 256), 148 * 32)), 1, 1), (256, 1, 1), 0)
    return launch


_BF, _CBF = "bf16*", "const bf16*"

# Entry-point parameters follow the reference's kernel ABI: outputs, then inputs, then weights; the integers
# each reference specialization bakes in are the constants here.  (K/ = bt4/kernels/ of the reference.)
_ADAPTERS: dict[str, Adapter] = {
    # K/layer_norm.py:37-161, the variant with a skip operand; ABI order of T/test_layer_norm.py:412-415.
    "layer_norm_skip": Adapter(
        "layernorm.cu",
        ((_BF, "out"), (_CBF, "in"), (_CBF, "bias"), (_CBF, "skip"), (_CBF, "gamma"), (_CBF, "beta"), (_CBF, "alpha")),
        ("ROWS", "WIDTH", "ACTIVATION", "EPSILON"),
        "LnParams p = {out, in, bias, skip, gamma, beta, alpha, nullptr, nullptr, ROWS, WIDTH, ACTIVATION, 1, EPSILON};\n"
        "  layer_norm_warp_body<(WIDTH + 255) / 256, ACTIVATION, 1, 0>(p);",
        _ln_launch),
    "layer_norm": Adapter(
        "layernorm.cu",
        ((_BF, "out"), (_CBF, "in"), (_CBF, "bias"), (_CBF, "gamma"), (_CBF, "beta")),
        ("ROWS", "WIDTH", "ACTIVATION", "EPSILON"),
        "LnParams p = {out, in, bias, nullptr, gamma, beta, nullptr, nullptr, nullptr, ROWS, WIDTH, ACTIVATION, 0, EPSILON};\n"
        "  layer_norm_warp_body<(WIDTH + 255) / 256, ACTIVATION, 0, 0>(p);",
        _ln_launch),
    # K/softmax_64.py:45-71
    "softmax_64": Adapter(
        "attention.cu", ((_BF, "out"), (_CBF, "scaled_qk"), (_CBF, "smolgen")), ("ROWS",),
        "softmax_64_body(out, scaled_qk, smolgen, ROWS);",
        lambda c: ((-(-c["ROWS"] // 8), 1, 1), (256, 1, 1), 0)),
    # K/batched_matmul.py:68-141, 64 x 64 outputs: body_qk (INTERLEAVED 1, OUT_STRIDE 4096) and policy_qk (0, 4288)
    "qk_64": Adapter(
        "attention.cu", ((_BF, "out"), (_CBF, "q"), (_CBF, "k"), (_CBF, "scale")),
        ("BATCH_COUNT", "DEPTH", "HEADS", "INTERLEAVED", "OUT_STRIDE"),
        "QkParams p = {out, q, k, scale, OUT_STRIDE, DEPTH, HEADS, INTERLEAVED};\n  qk_mma_body(p);",
        lambda c: ((c["BATCH_COUNT"], 1, 1), (128, 1, 1), 0)),
    # K/expand_planes.py:26-42
    "expand_planes": Adapter(
        "elementwise.cu", ((_BF, "out"), ("const uint64_t*", "masks"), ("const float*", "values")), ("PLANE_COUNT",),
        "expand_planes_body(out, masks, values, PLANE_COUNT);", _stream_launch(lambda c: c["PLANE_COUNT"] * 64)),
    # K/nchw_to_nhwc.py:26-44
    "nchw_to_nhwc": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "in")), ("BATCH", "INPUT_CHANNELS", "OUTPUT_CHANNELS", "HW"),
        "nchw_to_nhwc_body(out, in, (long long)BATCH * HW * OUTPUT_CHANNELS, INPUT_CHANNELS, OUTPUT_CHANNELS, HW);",
        _stream_launch(lambda c: c["BATCH"] * c["HW"] * c["OUTPUT_CHANNELS"])),
    # K/preprocess_attention_body.py:26-61
    "preprocess_attention_body": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "planes"), (_CBF, "encoding")),
        ("BATCH", "INPUT_CHANNELS", "ENCODING_CHANNELS"),
        "preprocess_attention_body_body(out, planes, encoding, (long long)BATCH * 64 * (INPUT_CHANNELS + ENCODING_CHANNELS),"
        " INPUT_CHANNELS, ENCODING_CHANNELS);",
        _stream_launch(lambda c: c["BATCH"] * 64 * (c["INPUT_CHANNELS"] + c["ENCODING_CHANNELS"]))),
    # K/input_gating.py:26-51
    "input_gating": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "in"), (_CBF, "mult"), (_CBF, "add")), ("BATCH", "SQUARES", "CHANNELS"),
        "input_gating_body(out, in, mult, add, (long long)BATCH * SQUARES * CHANNELS, (long long)SQUARES * CHANNELS);",
        _stream_launch(lambda c: c["BATCH"] * c["SQUARES"] * c["CHANNELS"])),
    # K/add_vectors.py:37-66: out[i] = act(in[i] + bias[i mod BIAS_ELEMENTS])
    "add_vectors": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "in"), (_CBF, "bias")), ("ELEMENTS", "BIAS_ELEMENTS", "ACTIVATION"),
        "add_bias_body(out, in, bias, ELEMENTS, BIAS_ELEMENTS, ELEMENTS, ACTIVATION);",
        _stream_launch(lambda c: c["ELEMENTS"])),
    # K/add_bias_batched.py:35-66: out[bt,row,c] = act(in[bt,row,c] + bias[bt,c])
    "add_bias_batched": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "in"), (_CBF, "bias")), ("BATCH_COUNT", "ROWS", "CHANNELS", "ACTIVATION"),
        "add_bias_body(out, in, bias, (long long)BATCH_COUNT * ROWS * CHANNELS, CHANNELS, (long long)ROWS * CHANNELS, ACTIVATION);",
        _stream_launch(lambda c: c["BATCH_COUNT"] * c["ROWS"] * c["CHANNELS"])),
    # K/matmul.py:57-116 on the CUDA cores (ABI order out, a, w of T/test_matmul.py:204-208; [K,N] weights): the
    # form for the small and odd-shaped layers (output widths 1, 3, 4; rows that TMA cannot address).  The large
    # layers belong on the tensor-core kernel, whose descriptors need the plan in TENSORMAP_NOTE.
    "matmul_simt": Adapter(
        "gemm_simt.cu", ((_BF, "out"), (_CBF, "a"), (_CBF, "w")), ("M", "N", "K"),
        "SimtParams p = {out, a, w, nullptr, nullptr, nullptr, M, K, N, N, N, K, LC0B200_OUT_BF16, LC0B200_ACT_NONE, 1};\n"
        "  gemm_simt_body<false>(p);",
        lambda c: ((-(-c["N"] // 64), -(-c["M"] // 64), 1), (256, 1, 1), 0)),
    # K/fused_qkv.py:132-183: three row-broadcast bias adds in one launch (ABI order of T/test_fused_qkv.py:95-109)
    "fused_qkv_bias": Adapter(
        "elementwise.cu",
        ((_BF, "q_out"), (_CBF, "q_in"), (_CBF, "q_bias"), (_BF, "k_out"), (_CBF, "k_in"), (_CBF, "k_bias"),
         (_BF, "v_out"), (_CBF, "v_in"), (_CBF, "v_bias")),
        ("ROWS", "QUERY_WIDTH", "KEY_WIDTH", "VALUE_WIDTH"),
        "QkvBiasParams p = {{q_out, k_out, v_out}, {q_in, k_in, v_in}, {q_bias, k_bias, v_bias},"
        " {QUERY_WIDTH, KEY_WIDTH, VALUE_WIDTH}, ROWS};\n  fused_qkv_bias_body(p);",
        lambda c: ((max(1, min(-(-c["ROWS"] * max(c["QUERY_WIDTH"], c["KEY_WIDTH"], c["VALUE_WIDTH"]) // 256), 148 * 32)),
                    3, 1), (256, 1, 1), 0)),
    # K/copy_type_converted.py:26-34
    "copy_type_converted": Adapter(
        "elementwise.cu", (("float*", "out"), (_CBF, "in")), ("ELEMENTS",),
        "widen_body(out, in, ELEMENTS);", _stream_launch(lambda c: c["ELEMENTS"])),
    # K/policy_map.py:28-49 (the table is the module symbol the reference exports, K/mapping_table.py:68-89: a pointer)
    "policy_map": Adapter(
        "elementwise.cu", ((_BF, "out"), (_CBF, "in"), ("const int32_t*", "table")), ("BATCH", "IN_COUNT", "OUT_COUNT"),
        "policy_map_body(out, in, table, (long long)BATCH * OUT_COUNT, IN_COUNT, OUT_COUNT);",
        _stream_launch(lambda c: c["BATCH"] * c["OUT_COUNT"])),
    # K/promotion_logits.py:67-145 (ABI order records, keys, weights)
    "promotion_logits": Adapter(
        "policy.cu", ((_BF, "records"), (_CBF, "keys"), (_CBF, "w")), ("BATCH", "WIDTH"),
        "promotion_logits_body(records, keys, w, WIDTH);", lambda c: ((c["BATCH"], 1, 1), (256, 1, 1), 0)),
}


def adapters() -> tuple[str, ...]:
    """Ops of this library that have a pointer-only entry point for lc0ex."""
    return tuple(_ADAPTERS)


def adapter_source(op: str, function: str, constants: dict) -> str:
    """The generated translation unit of one specialization."""
    adapter = _ADAPTERS[op]
    missing = [c for c in adapter.constants if c not in constants]
    if missing:
        raise ValueError(f"{op}: missing constants {missing}")
    defines = "\n".join(f"#define {name} {constants[name]}" for name in adapter.constants)
    params = ", ".join(f"{ctype} {name}" for ctype, name in adapter.pointers)
    _, block, _ = adapter.launch(constants)
    return (f'#include "{CSRC / adapter.source}"\n{defines}\nusing namespace lc0b200;\n'
            f'extern "C" __global__ void __launch_bounds__({block[0]}) {function}({params}) {{\n  {adapter.body}\n}}\n')


def compile_kernel(op: str, constants: dict, *, nvcc: str | None = None) -> KernelArtifact:
    """Compile one specialization of ``op`` into a CUBIN for sm_100a and describe it as a kernel artifact."""
    adapter = _ADAPTERS[op]
    missing = [c for c in adapter.constants if c not in constants]
    if missing:
        raise ValueError(f"{op}: missing constants {missing}")
    suffix = "_".join(f"{name.lower()}{str(constants[name]).replace('.', 'p').replace('-', 'm')}" for name in adapter.constants)
    function = f"lc0b200_{op}_{suffix}"
    compiler = nvcc or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    with tempfile.TemporaryDirectory() as scratch:
        source = pathlib.Path(scratch) / f"{function}.cu"
        source.write_text(adapter_source(op, function, constants))
        target = pathlib.Path(scratch) / f"{function}.cubin"
        done = subprocess.run([compiler, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                               "-o", str(target), str(source)], capture_output=True, text=True, check=False)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed for {function}:\n{done.stdout}\n{done.stderr}")
        data = target.read_bytes()
    grid, block, smem = adapter.launch(constants)
    return KernelArtifact(BinaryFormat.CUBIN, data, function, (ParameterType.POINTER,) * len(adapter.pointers), grid, block, smem)
