"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the public
header declares, and rejects bad arguments with status codes before touching a device."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest

from lczero_triton_b200 import _lib, build

ROOT = pathlib.Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared_symbols() -> set[str]:
    text = (ROOT / "include" / "lc0b200.h").read_text()
    return set(re.findall(r"LC0B200_API\s+[\w\s\*]*?\b(lc0b200_\w+)\s*\(", text))


def test_header_symbols_are_exported(lib) -> None:
    declared = _declared_symbols()
    assert len(declared) >= 25
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared in include/lc0b200.h but not exported: {missing}"


def test_binding_covers_every_declared_symbol() -> None:
    bound = set(_lib.SIGNATURES) | set(_lib.STRING_GETTERS)
    assert _declared_symbols() == bound


def test_status_strings(lib) -> None:
    assert lib.lc0b200_status_string(0) == b"ok"
    assert b"null" in lib.lc0b200_status_string(1)
    assert lib.lc0b200_version().startswith(b"lc0b200")


def test_null_pointers_are_rejected(lib) -> None:
    assert lib.lc0b200_expand_planes(None, None, None, 4, None) == 1
    assert lib.lc0b200_matmul(None, None, None, 4, 4, 4, None) == 1
    assert lib.lc0b200_layer_norm(None, None, None, None, None, None, None, 1, 8, 0, 0, 1e-3, None, None, None) == 1
    assert lib.lc0b200_gemm(None, None) == 1


def test_bad_shapes_and_codes_are_rejected(lib) -> None:
    fake = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    assert lib.lc0b200_expand_planes(fake, fake, fake, -1, None) == 2
    assert lib.lc0b200_add_vectors(fake, fake, fake, 8, 0, 0, None) == 2
    assert lib.lc0b200_add_vectors(fake, fake, fake, 8, 4, 7, None) == 2
    assert lib.lc0b200_layer_norm(fake, fake, fake, None, fake, fake, None, 1, 8, 2, 0, 1e-3, None, None, None) == 3
    assert lib.lc0b200_layer_norm(fake, fake, fake, None, fake, fake, None, 1, 8, 0, 1, 1e-3, None, None, None) == 1
    assert lib.lc0b200_attention(fake, fake, fake, fake, None, 1.0, 1, 4, 16, 128, 128, 128, 128, None) == 3
    assert lib.lc0b200_attention(fake, fake, fake, fake, None, 1.0, 1, 4, 32, 64, 128, 128, 128, None) == 2
    assert lib.lc0b200_attention(ctypes.c_void_p(258), fake, fake, fake, None, 1.0, 1, 4, 32, 128, 128, 128, 128,
                                 None) == 4
    assert lib.lc0b200_batched_matmul(fake, fake, fake, fake, 9, 1, 64, 64, 32, 1, None) == 3
    args = _lib.GemmArgs()
    args.out = args.a = args.w = 256
    args.m, args.n, args.k = 4, 4, 4
    args.lda = args.ldw = args.ldc = 2  # pitches shorter than the rows
    assert lib.lc0b200_gemm(ctypes.byref(args), None) == 2
    args.lda = args.ldw = args.ldc = 4
    args.out_kind = _lib.OUT_S32  # raw accumulators only exist for int8 inputs
    assert lib.lc0b200_gemm(ctypes.byref(args), None) == 3


def test_missing_library_fails_loudly(monkeypatch, tmp_path) -> None:
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIBRARY_PATH", tmp_path / "absent.so")
    with pytest.raises(_lib.Lc0B200Error, match="no CPU or PyTorch fallback"):
        _lib.load()


C_CALLER = r"""
#include <stdio.h>
#include "lc0b200.h"
int main(void) {
  lc0b200_net_config cfg = {128, 4, 4, 256, 64, 16, 64, 64, 128, 128, 128, 128, 32, 128, 1e-3f, 0};
  size_t bytes = lc0b200_net_arena_bytes(&cfg, 32);
  lc0b200_gemm_args args = {0};
  printf("%zu %d %d %s\n", bytes, lc0b200_gemm(&args, NULL),
         lc0b200_net_forward(NULL, NULL, NULL, 1, NULL, NULL, NULL, NULL), lc0b200_version());
  return bytes > 0 ? 0 : 1;
}
"""


def test_header_is_plain_c_and_links_from_a_c_program(lib, tmp_path) -> None:
    """The boundary is a C ABI: a C11 translation unit includes the header, links against the
    library and calls it (no device needed for what it calls)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    source = tmp_path / "caller.c"
    source.write_text(C_CALLER)
    exe = tmp_path / "caller"
    libdir = _lib.LIBRARY_PATH.parent
    subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(source), "-o", str(exe),
                    "-L", str(libdir), "-l:liblc0b200.so", f"-Wl,-rpath,{libdir}"], check=True)
    done = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
    fields = done.stdout.split()
    assert int(fields[0]) > 1_000_000 and fields[3].startswith("lc0b200")
    assert fields[1] == "1" and fields[2] == "1"  # null pointers are refused with a status, not a crash
