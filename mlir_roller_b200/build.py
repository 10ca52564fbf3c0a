"""Builds libroller_b200.so (the sm_100a kernels + C ABI) in-tree with nvcc.

Run as `python -m mlir_roller_b200.build`; `build()` is also what the repository's build check
calls. nvcc cross-compiles for sm_100a without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libroller_b200.so"

SOURCES = ["gemm_variants.cu", "gemm_variants_16.cu", "capi.cu", "noalloc.cu", "peer_flags.cu", "skinny_simt.cu"]
HEADERS = ["ptx_sm100.cuh", "gemm_tf32_sm100.cuh", "gemm_launch.h", "gemm_variant_make.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--use_fast_math",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libroller_b200.so cannot be built")
    return exe


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / f for f in SOURCES + HEADERS] + [PKG_DIR.parent / "include" / "roller_b200.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), lib_path: Path | None = None) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library. `defines` (e.g.
    ["RB200_SMALL_STAGES=4"]) and `lib_path` build a variant of the library somewhere else, for
    comparing build-time tunables; the package itself always loads the default one."""
    out = LIB_PATH if lib_path is None else Path(lib_path)
    if not force and not defines and lib_path is None and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    build_dir = PKG_DIR / "build" if lib_path is None else out.parent / (out.stem + "_build")
    build_dir.mkdir(parents=True, exist_ok=True)
    procs = []
    for src in SOURCES:      # the translation units are independent: compile them side by side
        obj = build_dir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(str(obj))
    failed = [cmd for cmd, pr in procs if pr.wait() != 0]
    if failed:
        raise subprocess.CalledProcessError(1, failed[0])
    subprocess.run([nvcc, "-shared", "-o", str(out), *objs, "-gencode",
                    "arch=compute_100a,code=sm_100a"], check=True)
    return out


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
