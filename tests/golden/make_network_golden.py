"""Generate ``tests/golden/reference_network_outputs.npz``: the reference's OWN graph run end to end.

Run on a machine with a GPU and the unmodified reference package installed under ``baseline/_ref``:

    python tests/golden/make_network_golden.py [output.npz]        # needs a GPU
    python tests/golden/make_network_golden.py [output.npz] --only bt4_b64   # one case, merged into the file
    python tests/golden/make_network_golden.py --dry               # no GPU: walks the graph, launches nothing,
                                                                   # writes reference_program_plan.json

The reference has no runtime of its own: ``lczero_triton.bt4.network`` appends kernel invocations to an
``lc0ex`` program and the lc0 fork that would run it is not in its tree.  This script is the missing forty
lines of runtime.  It calls the reference's graph builder (``network._network``, the function its ``build``
calls per batch size) with the reference's ``ExecutableBuilder`` / ``KernelCache``, so every node is the
reference's Triton kernel, autotuned and compiled to a CUBIN by the reference's own compile functions, and
the temporaries live where the reference linker's allocation plan (``BufferBuilder.plan`` over the conflicts
of ``ExecutableBuilder._analyze_invocations``) puts them.  It then does what the executable format says a
runtime does: load each CUBIN, and launch the nodes in program order on one stream with their static grids
and the planned addresses (NULL for the two Triton scratch parameters, the module global for symbols).

What is NOT the reference here, and why it does not matter for the numbers:

* the three generated protobuf modules (``lc0ex_pb2``, ``lc0ex_metadata_pb2``, ``net_pb2``) do not exist
  offline (they are generated from an un-vendored submodule).  They are replaced by stubs whose enum
  constants are distinct integers; graph construction only compares them and uses them as dict keys.
  ``ExecutableBuilder.build`` (serialisation) is never called;
* ``build``'s front half (normalise / validate / fingerprint a ``net_pb2.Net``) is skipped: ``_network`` reads
  only ``len(layer.params)`` of each weight field, ``len(weights.encoder)`` and ``weights.headcount``, which a
  small attribute tree supplies from the shapes in ``lczero_triton_b200.weights``;
* weight VALUES never pass through the graph builder: the program only names persistent buffers, which this
  script fills by name, as the lc0 loader would.

Weights are ``random_weights(cfg, seed)`` made exact in fp16 (``exact_in_both``), inputs
``synthetic_planes(batch, seed)``; the test regenerates both from the seeds, so only the three outputs per case
are stored.  ``tests/test_network_golden.py`` holds the CPU oracle (no GPU needed) and, on a GPU, this library's
forward to them.
"""

from __future__ import annotations

import collections
import ctypes
import json
import pathlib
import sys
import time
import types

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path[:0] = [str(ROOT / "baseline" / "_ref"), str(ROOT)]

# (config name, batch, seed).  Batches are small: the reference autotunes every kernel specialisation.
CASES = (("tiny", 5, 11), ("tiny", 64, 12), ("bt3", 3, 13), ("bt4", 2, 14), ("bt4", 64, 15))

TOP_LEVEL = {
    "weights.ip_emb_preproc_w": "/attn_body/embedding/preprocess/matmul/w",
    "weights.ip_emb_preproc_b": "/attn_body/embedding/preprocess/add/w",
    "weights.ip_emb_w": "/attn_body/matmul/w",
    "weights.ip_emb_b": "/attn_body/add/w",
    "weights.ip_emb_ln_gammas": "/attn_body/ln/w/scale",
    "weights.ip_emb_ln_betas": "/attn_body/ln/w/bias",
    "weights.ip_mult_gate": "/ip_mul_gate/w",
    "weights.ip_add_gate": "/ip_add_gate/w",
    "weights.ip_emb_ffn.dense1_w": "/attn_body/ffn/dense1/w/w",
    "weights.ip_emb_ffn.dense1_b": "/attn_body/ffn/dense1/b/w",
    "weights.ip_emb_ffn.dense2_w": "/attn_body/ffn/dense2/w/w",
    "weights.ip_emb_ffn.dense2_b": "/attn_body/ffn/dense2/b/w",
    "weights.ip_emb_ffn_ln_gammas": "/attn_body/ln2/w/scale",
    "weights.ip_emb_ffn_ln_betas": "/attn_body/ln2/w/bias",
    "weights.smolgen_w": "/const/smolgen_w",
    "weights.policy_heads.vanilla.ip_pol_w": "/policy/dense1/matmul/w",
    "weights.policy_heads.vanilla.ip_pol_b": "/policy/dense1/add/w",
    "weights.policy_heads.vanilla.ip2_pol_w": "/policy/Q/matmul/w",
    "weights.policy_heads.vanilla.ip2_pol_b": "/policy/Q/add/w",
    "weights.policy_heads.vanilla.ip3_pol_w": "/policy/K/matmul/w",
    "weights.policy_heads.vanilla.ip3_pol_b": "/policy/K/add/w",
    "weights.policy_heads.vanilla.ip4_pol_w": "/policy/promotion/matmul/w",
    "weights.value_heads.winner.ip_val_w": "/value/embed/matmul/w",
    "weights.value_heads.winner.ip_val_b": "/value/embed/add/w",
    "weights.value_heads.winner.ip1_val_w": "/value/dense1/matmul/w",
    "weights.value_heads.winner.ip1_val_b": "/value/dense1/add/w",
    "weights.value_heads.winner.ip2_val_w": "/value/dense2/matmul/w",
    "weights.value_heads.winner.ip2_val_b": "/value/dense2/add/w",
    "weights.ip_mov_w": "/mlh/embed/matmul/w",
    "weights.ip_mov_b": "/mlh/embed/add/w",
    "weights.ip1_mov_w": "/mlh/dense1/matmul/w",
    "weights.ip1_mov_b": "/mlh/dense1/add/w",
    "weights.ip2_mov_w": "/mlh/dense2/matmul/w",
    "weights.ip2_mov_b": "/mlh/dense2/add/w",
}
PER_ENCODER = {
    "mha.smolgen.compress": "smolgen/compress/w",
    "mha.smolgen.dense1_w": "smolgen/dense1/w/w",
    "mha.smolgen.dense1_b": "smolgen/dense1/b/w",
    "mha.smolgen.ln1_gammas": "smolgen/ln1/w/scale",
    "mha.smolgen.ln1_betas": "smolgen/ln1/w/bias",
    "mha.smolgen.dense2_w": "smolgen/dense2/w/w",
    "mha.smolgen.dense2_b": "smolgen/dense2/b/w",
    "mha.smolgen.ln2_gammas": "smolgen/ln2/w/scale",
    "mha.smolgen.ln2_betas": "smolgen/ln2/w/bias",
    "mha.q_w": "mha/Q/w/w", "mha.q_b": "mha/Q/b/w",
    "mha.k_w": "mha/K/w/w", "mha.k_b": "mha/K/b/w",
    "mha.v_w": "mha/V/w/w", "mha.v_b": "mha/V/b/w",
    "mha.dense_w": "mha/out/dense/w/w", "mha.dense_b": "mha/out/dense/b/w",
    "ln1_gammas": "ln1/w/scale", "ln1_betas": "ln1/w/bias",
    "ffn.dense1_w": "ffn/dense1/w/w", "ffn.dense1_b": "ffn/dense1/b/w",
    "ffn.dense2_w": "ffn/dense2/w/w", "ffn.dense2_b": "ffn/dense2/b/w",
    "ln2_gammas": "ln2/w/scale", "ln2_betas": "ln2/w/bias",
}


def buffer_name(path: str) -> str | None:
    """Protobuf field path of a weight (as the reference's graph builder spells it in its ``path=`` arguments)
    -> the persistent buffer name it declares for it (bt4/network.py:349-449, 715-774, 868-936, 1089-1132,
    1198-1251, 1427-1466)."""
    if path in TOP_LEVEL:
        return TOP_LEVEL[path]
    head, _, rest = path.partition(".")[2].partition(".")
    if head.startswith("encoder") and rest in PER_ENCODER:
        return f"/{head}/{PER_ENCODER[rest]}"
    return None


def exact_in_both(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """bf16 weights whose values are also exact in fp16 (magnitudes below fp16's normal range become zero)."""
    out = {}
    for name, w in weights.items():
        f = w.float()
        out[name] = torch.where(f.abs() < 2.0 ** -14, torch.zeros_like(f), f).to(torch.bfloat16)
        assert torch.equal(out[name].float().half().float(), out[name].float()), name
    return out


def stub_generated_protobuf_modules() -> None:
    """Stand-ins for the generated ``*_pb2`` modules: every UPPER_CASE attribute is a distinct integer (the
    same name always the same integer), every other attribute a nested namespace."""
    numbers: dict[str, int] = {}

    class _Namespace(type):
        def __getattr__(cls, key):
            if key.startswith("__"):
                raise AttributeError(key)
            if key.isupper() or key.split("_")[0].isupper():
                return numbers.setdefault(key, len(numbers) + 1)
            return _Namespace(key, (), {})

        def __or__(cls, other):
            return cls

        def __ror__(cls, other):
            return cls

    for name in ("lc0ex_pb2", "lc0ex_metadata_pb2", "net_pb2"):
        module = types.ModuleType("lc0ex.proto." + name)
        module.__getattr__ = lambda key, _root=_Namespace("root", (), {}): getattr(_root, key)
        sys.modules["lc0ex.proto." + name] = module


class _Field:
    """The part of a ``net_pb2.Weights`` tree the graph builder reads: attribute paths, ``len(params)``,
    ``encoder``, ``headcount`` and ``HasField``."""

    def __init__(self, path: str, cfg, shapes: dict[str, tuple[int, ...]]):
        self._path, self._cfg, self._shapes = path, cfg, shapes

    def __getattr__(self, key: str):
        if key.startswith("__"):
            raise AttributeError(key)
        return _Field(f"{self._path}.{key}", self._cfg, self._shapes)

    @property
    def params(self) -> bytes:
        name = buffer_name(self._path)
        return b"" if name is None else bytes(2 * int(np.prod(self._shapes[name])))

    @property
    def encoder(self) -> list["_Field"]:
        return [_Field(f"{self._path}.encoder{i}", self._cfg, self._shapes) for i in range(self._cfg.layers)]

    @property
    def headcount(self) -> int:
        return self._cfg.heads

    def HasField(self, name: str) -> bool:  # noqa: N802 (protobuf's spelling)
        return False


def build_program(cfg, batch: int, *, dry: bool):
    """The reference's graph for one batch size: ``(executable builder, program builder, consumed paths)``."""
    import lc0ex
    from lczero_triton.bt4 import network
    from lczero_triton.bt4.kernels._cache import KernelCache
    from lczero_triton_b200 import weights as W

    shapes = W.weight_shapes(cfg)
    builder = lc0ex.ExecutableBuilder()
    program = builder.program(name="main")
    consumed: list[str] = []

    class _Marks(dict):
        def __missing__(self, path):
            consumed.append(path)
            return types.SimpleNamespace(SetInParent=lambda: None)

    if dry:
        # No GPU: nothing is compiled.  A kernel is a placeholder artifact named after its compile function,
        # with as many pointer parameters as its first call passes; everything else (buffers, calls, read-only
        # sets, dependency analysis, allocation plan) is the reference's code on the reference's graph.
        from lc0ex.kernel_builder import KernelArtifact, KernelHandle
        from lc0ex.proto import lc0ex_pb2

        handles: dict[tuple, KernelHandle] = {}
        names: dict[KernelHandle, str] = {}

        def get(compiler, specialization):
            handle = handles.setdefault((compiler, specialization), KernelHandle())
            names[handle] = f"{compiler.__name__}#{list(handles).index((compiler, specialization))}"
            return handle

        recorded_call = program.call

        def call(kernel, *arguments, readonly=()):
            if kernel not in builder._kernels:
                builder._kernels[kernel] = KernelArtifact(
                    binary_format=lc0ex_pb2.Binary.FORMAT_CUBIN, binary_data=b"", function=names[kernel],
                    parameters=(lc0ex_pb2.PARAMETER_TYPE_POINTER,) * len(arguments)
                    + (lc0ex_pb2.PARAMETER_TYPE_NULL_POINTER,) * 2,
                    grid=(1, 1, 1), block=(1, 1, 1), dynamic_shared_memory_bytes=0)
            recorded_call(kernel, *arguments, readonly=readonly)

        program.call = call  # type: ignore[method-assign]
        kernels = types.SimpleNamespace(get=get)
        architecture = 100
    else:
        from lczero_triton.bt4.kernels._autotune import active_architecture

        kernels = KernelCache(builder)
        architecture = active_architecture()
    context = network._BuildContext(builder=program, kernels=kernels, batch_size=batch, architecture=architecture,
                                    fingerprint=None, fingerprint_layers=_Marks())
    network._network(context, _Field("weights", cfg, shapes))
    unknown = [p for p in consumed if buffer_name(p) is None]
    assert not unknown, unknown
    return builder, program, consumed


def dump_plan(builder, program) -> dict:
    """The reference linker's view of one program, as plain data: every buffer in creation order, every call
    with its buffer arguments and read-only set, the reduced dependencies (``_analyze_invocations``) and both
    allocation plans (``BufferBuilder.plan``)."""
    from lc0ex.buffer_builder import Buffer
    from lc0ex.proto import lc0ex_pb2

    buffers = builder._buffers
    records = buffers._records
    ids = {buffer: index for index, buffer in enumerate(records)}
    dtype_names = {getattr(lc0ex_pb2.Buffer, "DATA_TYPE_" + n): n for n in ("F32", "F16", "U64", "U8", "BF16")}
    dependencies, conflicts = builder._analyze_invocations(program)
    plans = {"persistent": buffers.plan(buffers.persistent_allocation(), {}),
             "execution": buffers.plan(program._allocation, conflicts)}
    return {
        "buffers": [{"persistent": r.allocation.is_persistent(), "size_bytes": r.size_bytes,
                     "alignment_bytes": r.alignment_bytes, "writable": r.writable,
                     "name": None if r.external is None else r.external.name,
                     "shape": None if r.external is None else list(r.external.shape),
                     "dtype": None if r.external is None else dtype_names[r.external.dtype]} for r in records.values()],
        "calls": [{"kernel": builder._kernels[i.kernel].function,
                   "arguments": [ids[a] if isinstance(a, Buffer) else -1 for a in i.arguments],
                   "readonly": sorted(ids[b] for b in i.readonly)} for i in program._invocations],
        "dependencies": [list(d) for d in dependencies],
        "plans": {kind: {"size_bytes": plan.size_bytes, "alignment_bytes": plan.alignment_bytes,
                         "offsets": {str(ids[b]): loc.offset for b, loc in plan.locations.items()}}
                  for kind, plan in plans.items()},
    }


class LoadedProgram:
    """One program of the reference's executable on the current device: allocations made and filled, CUBINs
    loaded, every node's launch arguments resolved to the reference linker's planned addresses."""

    def __init__(self, builder, program, persistent: dict[str, torch.Tensor], inputs: dict[str, torch.Tensor], *,
                 fill: int) -> None:
        from cuda.bindings import driver
        from lc0ex.buffer_builder import Buffer
        from lc0ex.proto import lc0ex_pb2

        self._driver = driver
        ok = self._ok
        buffers = builder._buffers
        records = buffers._records
        _, conflicts = builder._analyze_invocations(program)
        plans = {True: buffers.plan(buffers.persistent_allocation(), {}), False: buffers.plan(program._allocation, conflicts)}
        self._blobs = {kind: torch.full((plan.size_bytes + 256,), fill, dtype=torch.uint8, device="cuda")
                       for kind, plan in plans.items()}

        def view(buffer) -> torch.Tensor:
            record = records[buffer]
            kind = record.allocation.is_persistent()
            offset = plans[kind].locations[buffer].offset
            assert offset % record.alignment_bytes == 0 and offset + record.size_bytes <= plans[kind].size_bytes
            return self._blobs[kind][offset:offset + record.size_bytes]

        dtypes = {lc0ex_pb2.Buffer.DATA_TYPE_F32: torch.float32, lc0ex_pb2.Buffer.DATA_TYPE_F16: torch.float16,
                  lc0ex_pb2.Buffer.DATA_TYPE_U64: torch.int64}
        self.named: dict[str, torch.Tensor] = {}
        for kind, source in ((True, persistent), (False, inputs)):
            for buffer, external in plans[kind].external_buffers:
                target = view(buffer).view(dtypes[external.dtype]).reshape(external.shape)
                self.named[external.name] = target
                if external.name in source:
                    target.copy_(source[external.name].to(dtypes[external.dtype]).reshape(external.shape))
                else:
                    assert not kind and external.name.startswith("/output/"), external.name
        missing = set(persistent) - set(self.named)
        assert not missing, missing

        self._modules: dict[bytes, object] = {}

        def module_of(binary: bytes):
            if binary not in self._modules:
                self._modules[binary] = ok(driver.cuModuleLoadData(binary))
            return self._modules[binary]

        self._nodes = []
        for invocation in program._invocations:
            artifact = builder._kernels[invocation.kernel]
            function = ok(driver.cuModuleGetFunction(module_of(artifact.binary_data), artifact.function.encode()))
            if artifact.dynamic_shared_memory_bytes > 48 * 1024:
                ok(driver.cuFuncSetAttribute(function,
                                             driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                             artifact.dynamic_shared_memory_bytes))
            arguments = iter(invocation.arguments)
            pointers = []
            for parameter in artifact.parameters:
                if parameter == lc0ex_pb2.PARAMETER_TYPE_NULL_POINTER:
                    pointers.append(0)
                    continue
                argument = next(arguments)
                if isinstance(argument, Buffer):
                    pointers.append(view(argument).data_ptr())
                else:
                    symbol = builder._symbols[argument]
                    address, _size = ok(driver.cuModuleGetGlobal(module_of(symbol.binary_data), symbol.symbol_name.encode()))
                    pointers.append(int(address))
            assert next(arguments, None) is None
            values = (ctypes.c_void_p * len(pointers))(*pointers)
            slots = (ctypes.c_void_p * len(pointers))(*[ctypes.addressof(values) + i * ctypes.sizeof(ctypes.c_void_p)
                                                        for i in range(len(pointers))])
            self._nodes.append((function, artifact, values, slots))
        counts = collections.Counter(node[1].function for node in self._nodes)
        self.info = {"nodes": len(self._nodes), "kernels": len(builder._kernels),
                     "execution_bytes": plans[False].size_bytes, "persistent_bytes": plans[True].size_bytes,
                     "temporaries_bytes": sum(r.size_bytes for r in records.values() if r.external is None),
                     "functions": dict(counts)}

    def _ok(self, result):
        assert result[0] == self._driver.CUresult.CUDA_SUCCESS, result[0]
        return result[1] if len(result) == 2 else result[1:]

    def launch(self) -> None:
        """Every node in program order on torch's current stream (a valid order of the dependency graph)."""
        stream = torch.cuda.current_stream().cuda_stream
        for function, artifact, _values, slots in self._nodes:
            self._ok(self._driver.cuLaunchKernel(function, *artifact.grid, *artifact.block,
                                                 artifact.dynamic_shared_memory_bytes, stream, ctypes.addressof(slots), 0))

    def outputs(self) -> dict[str, torch.Tensor]:
        torch.cuda.synchronize()
        return {name: tensor.clone().cpu() for name, tensor in self.named.items() if name.startswith("/output/")}

    def close(self) -> None:
        torch.cuda.synchronize()
        for module in self._modules.values():
            self._ok(self._driver.cuModuleUnload(module))
        self._modules, self._nodes = {}, []


def run_program(builder, program, persistent: dict[str, torch.Tensor], inputs: dict[str, torch.Tensor], *,
                fill: int) -> tuple[dict[str, torch.Tensor], dict]:
    """Launch the program's nodes in order at the reference linker's planned addresses."""
    loaded = LoadedProgram(builder, program, persistent, inputs, fill=fill)
    loaded.launch()
    outputs = loaded.outputs()
    loaded.close()
    return outputs, loaded.info


def main(argv: list[str]) -> None:
    dry = "--dry" in argv
    only = argv[argv.index("--only") + 1] if "--only" in argv else None
    positional = [a for i, a in enumerate(argv) if not a.startswith("--") and (i == 0 or argv[i - 1] != "--only")]
    target = pathlib.Path(positional[0]) if positional else pathlib.Path(__file__).with_name("reference_network_outputs.npz")
    stub_generated_protobuf_modules()
    from lczero_triton_b200 import config as C
    from lczero_triton_b200 import synthetic
    from lczero_triton_b200 import weights as W

    out: dict[str, np.ndarray] = {}
    if only is not None and not dry and target.exists():
        with np.load(target) as existing:
            out.update({key: existing[key] for key in existing.files})
    plans: dict[str, dict] = {}
    for cfg_name, batch, seed in CASES:
        if only is not None and f"{cfg_name}_b{batch}" != only:
            continue
        cfg = C.CONFIGS[cfg_name]
        started = time.time()
        builder, program, consumed = build_program(cfg, batch, dry=dry)
        if dry:
            declared = {e.name for _, e in builder._buffers.plan(builder._buffers.persistent_allocation(), {}).external_buffers}
            expected = set(W.weight_shapes(cfg)) | set(W.scalar_constants(cfg))
            print(f"{cfg_name} batch {batch}: {len(program._invocations)} nodes, {len(consumed)} weight fields, "
                  f"persistent names equal: {declared == expected}")
            assert declared == expected, (sorted(declared - expected), sorted(expected - declared))
            plans[f"{cfg_name}_b{batch}"] = dump_plan(builder, program)
            continue
        built = time.time() - started
        weights = exact_in_both(W.random_weights(cfg, seed))
        masks, values = synthetic.synthetic_planes(batch, seed)
        inputs = {"/input/plane_masks": masks.cuda(), "/input/plane_values": values.cuda()}
        persistent = {name: w.float().half().cuda() for name, w in weights.items()}
        key = f"{cfg_name}_b{batch}_s{seed}"
        results = {}
        for fill in (0xFF, 0x00):  # temporaries start as fp16 NaN, then as zeros: a node that read before a write shows
            outputs, info = run_program(builder, program, persistent, inputs, fill=fill)
            results[fill] = outputs
        same = all(torch.equal(results[0xFF][n], results[0x00][n]) for n in results[0x00])
        finite = all(bool(torch.isfinite(t).all()) for t in results[0xFF].values())
        print(f"{key}: graph built in {built:.0f} s, {info['nodes']} nodes over {info['kernels']} kernels, execution "
              f"allocation {info['execution_bytes']} B for {info['temporaries_bytes']} B of temporaries, outputs finite "
              f"{finite}, independent of the initial contents of the allocation {same}", flush=True)
        assert finite and same
        for name, tensor in results[0x00].items():
            out[f"{key}{name}"] = tensor.float().numpy()
        out[f"{key}/nodes"] = np.array([info["nodes"], info["kernels"], info["execution_bytes"], info["temporaries_bytes"]])
        out[f"{key}/functions"] = np.array(sorted(f"{k} x{v}" for k, v in info["functions"].items()))
        np.savez_compressed(target, **out)  # after every case: a later case that fails keeps the earlier ones
    if dry:
        plan_target = pathlib.Path(__file__).with_name("reference_program_plan.json")
        keep = {key: plans[key] for key in ("tiny_b5", "bt4_b2") if key in plans}
        plan_target.write_text(json.dumps(keep, separators=(",", ":")))
        print(f"wrote {plan_target} ({plan_target.stat().st_size} bytes)")
    else:
        print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main(sys.argv[1:])
