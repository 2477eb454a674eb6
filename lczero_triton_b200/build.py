"""Build recipe for the in-tree CUDA library (nvcc, sm_100a only).

``python -m lczero_triton_b200.build`` compiles ``csrc/*.cu`` into
``lczero_triton_b200/liblc0b200.so``.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import fcntl
import os
import pathlib
import shutil
import subprocess
import sys

PACKAGE_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIBRARY = PACKAGE_DIR / "liblc0b200.so"
SOURCES = ("api.cu", "gemm_tcgen05.cu", "gemm_simt.cu", "elementwise.cu", "layernorm.cu", "attention.cu", "attention_tc.cu", "policy.cu",
           "no_alloc.cu", "net_runtime.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--threads", "0",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def needs_build() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    inputs.append(PACKAGE_DIR.parent / "include" / "lc0b200.h")
    return any(p.stat().st_mtime > built for p in inputs)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile the library if any source is newer than it; return its path."""
    if not force and not needs_build():
        return LIBRARY
    # Several ranks of one job may get here together: one builds (into a temporary file that is
    # renamed into place), the others wait on the lock and then find the library up to date.
    with open(PACKAGE_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():
                return LIBRARY
            scratch = LIBRARY.with_suffix(f".so.tmp{os.getpid()}")
            cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", str(scratch), *[str(CSRC / s) for s in SOURCES]]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            result = subprocess.run(cmd, capture_output=True, text=True, check=False)
            if result.returncode != 0:
                scratch.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
            os.replace(scratch, LIBRARY)
            if verbose:
                print(result.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
