"""Generate ``tests/golden/reference_vectors.npz`` from the reference's own code.

Run once, in a container that has the reference tree, as
``python tests/golden/make_golden.py <path-to-reference>``.  It imports the
PyTorch reference functions that the reference's GPU tests compare their
kernels with (``packages/lczero-triton/tests/test_layer_norm.py:40-74``,
``test_softmax_64.py:37-41``, ``test_promotion_logits.py:40-52``) and its
decoded policy gather table (``bt4/kernels/mapping_table.py:53-65``), evaluates
them on seeded CPU inputs and stores inputs and outputs.  The reference's
generated protobuf bindings do not exist offline, so the three ``*_pb2``
modules are replaced by attribute stubs; none of the imported functions uses
them.  The reference functions round their result to fp16; the stored
expectation is that fp16 tensor widened to fp32.

It also writes ``tests/golden/reference_buffer_names.json``: every named buffer the reference's graph
builder declares (``bt4/network.py``), taken from the source by an ``ast`` walk of the calls that carry
a ``name=`` / ``output_name=`` argument - the name template as written (``{prefix}`` and ``{label}``
left in place), the declaring helper, the expression given as the matrix's input width, and the line.
``tests/test_buffer_names.py`` holds this package's weight table and the C network object to it.
"""

from __future__ import annotations

import pathlib
import sys
import types

import numpy as np
import torch


def _stub_generated_protobuf_modules() -> None:
    class _Stub(type):
        def __getattr__(cls, key):
            if key.startswith("__"):
                raise AttributeError(key)
            return _Stub(key, (), {})

        def __or__(cls, other):
            return cls

        def __ror__(cls, other):
            return cls

    for name in ("lc0ex_pb2", "lc0ex_metadata_pb2", "net_pb2"):
        module = types.ModuleType("lc0ex.proto." + name)

        def _getattr(key, _Stub=_Stub):
            if key.startswith("__"):
                raise AttributeError(key)
            if key.isupper() or key.split("_")[0].isupper():
                return 0
            return _Stub(key, (), {})

        module.__getattr__ = _getattr
        sys.modules["lc0ex.proto." + name] = module


def buffer_names(root: pathlib.Path) -> list[dict]:
    """Named buffers of the reference graph builder, read from its source text."""
    import ast

    source = root / "packages/lczero-triton/src/lczero_triton/bt4/network.py"
    tree = ast.parse(source.read_text())
    rows: list[dict] = []

    def template(node: ast.expr) -> str | None:
        if isinstance(node, ast.Constant) and isinstance(node.value, str):
            return node.value
        if isinstance(node, ast.JoinedStr):
            return "".join(v.value if isinstance(v, ast.Constant) else "{" + ast.unparse(v.value) + "}"
                           for v in node.values)
        return None  # a variable: the helper that forwards a caller's name

    class Walk(ast.NodeVisitor):
        function = None

        def visit_FunctionDef(self, node: ast.FunctionDef) -> None:
            outer, self.function = self.function, node.name
            self.generic_visit(node)
            self.function = outer

        def visit_Call(self, node: ast.Call) -> None:
            keywords = {k.arg: k.value for k in node.keywords if k.arg}
            named = keywords.get("name", keywords.get("output_name"))
            text = template(named) if named is not None else None
            if text is not None:
                helper = ast.unparse(node.func)
                kind = {"_matrix_f16": "matrix", "_vector_f16": "vector",
                        "context.builder.persistent_buffer": "constant"}.get(helper, "io")
                rows.append({"name": text, "kind": kind, "function": self.function, "line": node.lineno,
                             "input_width": ast.unparse(keywords["input_width"]) if "input_width" in keywords else None})
            self.generic_visit(node)

    Walk().visit(tree)
    return rows


def main(reference_root: str) -> None:
    root = pathlib.Path(reference_root)
    import json

    names = buffer_names(root)
    names_target = pathlib.Path(__file__).with_name("reference_buffer_names.json")
    names_target.write_text(json.dumps(names, indent=1) + "\n")
    print(f"wrote {names_target} ({len(names)} named buffers)")
    _stub_generated_protobuf_modules()
    sys.path[:0] = [
        str(root / "packages/lc0ex/src"),
        str(root / "packages/lczero-triton/src"),
        str(root / "packages/lczero-triton/tests"),
    ]
    import test_layer_norm
    import test_promotion_logits
    import test_softmax_64
    from lczero_triton.bt4.kernels import mapping_table

    out: dict[str, np.ndarray] = {}
    gen = torch.Generator().manual_seed(1234)

    def rnd(*shape, scale=1.0):
        return (torch.randn(shape, generator=gen) * scale).half()

    # --- layer norm: the four variants the network uses (BT4_PLAN.md:479-484)
    cases = [
        ("ln_mish_noskip", 6, 128, "mish", False),
        ("ln_swish_noskip", 5, 256, "swish", False),
        ("ln_none_skip", 7, 96, "none", True),
        ("ln_swish_wide", 2, 8192, "swish", False),
    ]
    for name, rows, width, act, has_skip in cases:
        x, bias = rnd(rows, width), rnd(width, scale=0.5)
        gam, bet = (1.0 + rnd(width, scale=0.1).float()).half(), rnd(width, scale=0.1)
        skip = rnd(rows, width) if has_skip else None
        alpha = torch.tensor([0.4272], dtype=torch.float16) if has_skip else None
        if name == "ln_swish_wide":
            x = (x.float() + 8.0).half()  # population variance with a large mean, test_layer_norm.py:186-215
        y = test_layer_norm._reference(x, bias, gam, bet, act, 1e-3, skip=skip, alpha=alpha)
        out[f"{name}/x"], out[f"{name}/bias"] = x.numpy(), bias.numpy()
        out[f"{name}/gamma"], out[f"{name}/beta"] = gam.numpy(), bet.numpy()
        if has_skip:
            out[f"{name}/skip"], out[f"{name}/alpha"] = skip.numpy(), alpha.numpy()
        out[f"{name}/y"] = y.float().numpy()

    # --- activations around the mish branch point (test_add_vectors.py:39-42)
    pts = torch.tensor([-8.0, -2.0, -0.6001, -0.6, -0.5999, -0.1, 0.0, 0.3, 1.0, 4.0, 11.0])
    for act in ("mish", "swish", "none"):
        out[f"act_{act}/x"] = pts.numpy()
        out[f"act_{act}/y"] = test_layer_norm._activate(pts.clone(), act).numpy()

    # --- softmax: random rows and the edge rows of test_softmax_64.py:112-149
    qk, sg = rnd(48, 64, scale=3.0), rnd(48, 64, scale=2.0)
    out["softmax_random/qk"], out["softmax_random/smolgen"] = qk.numpy(), sg.numpy()
    out["softmax_random/y"] = test_softmax_64._reference(qk, sg).float().numpy()
    qk = torch.zeros((8, 64), dtype=torch.float16)
    sg = torch.zeros_like(qk)
    qk[0, 0] = torch.inf
    qk[1, :2] = torch.inf
    qk[2] = -torch.inf
    qk[3, 0] = torch.inf
    sg[3, 0] = -torch.inf
    qk[4, 7] = torch.nan
    qk[5, 0] = 65504.0
    sg[5, 0] = 65504.0
    qk[6, 0] = -65504.0
    sg[6, 0] = -65504.0
    qk[7] = torch.linspace(-20.0, 20.0, 64).half()
    sg[7] = torch.linspace(3.0, -4.0, 64).half()
    out["softmax_edges/qk"], out["softmax_edges/smolgen"] = qk.numpy(), sg.numpy()
    out["softmax_edges/y"] = test_softmax_64._reference(qk, sg).float().numpy()

    # --- promotion logits: random and the exact-integer case of test_promotion_logits.py:147-187
    rec, keys, w = rnd(3, 4288), rnd(3, 64, 48, scale=0.5), rnd(48, 4, scale=0.5)
    out["promo_random/records"], out["promo_random/keys"], out["promo_random/w"] = rec.numpy(), keys.numpy(), w.numpy()
    out["promo_random/y"] = test_promotion_logits._reference(rec, keys, w).float().numpy()
    rec = torch.full((2, 4288), -123.0, dtype=torch.float16)
    keys = torch.zeros((2, 64, 32), dtype=torch.float16)
    w = torch.zeros((32, 4), dtype=torch.float16)
    w[0] = torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float16)
    for b in range(2):
        for s in range(8):
            for t in range(8):
                rec[b, (48 + s) * 64 + 56 + t] = b * 100 + s * 10 + t
        for t in range(8):
            keys[b, 56 + t, 0] = b * 10 + t + 1
    out["promo_exact/records"], out["promo_exact/keys"], out["promo_exact/w"] = rec.numpy(), keys.numpy(), w.numpy()
    out["promo_exact/y"] = test_promotion_logits._reference(rec, keys, w).float().numpy()

    # --- policy gather table
    out["mapping_table"] = np.asarray(mapping_table.values(), dtype=np.int32)

    target = pathlib.Path(__file__).with_name("reference_vectors.npz")
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path-to-reference>")
    main(sys.argv[1])
