"""Builds libb200w4a4.so in-tree with plain nvcc for sm_100a (seconds, no torch headers).

Plays the role of the JIT build in the reference wrapper
(vdm_infer/kernels/vdm_w4a4.py:130-167: torch.utils.cpp_extension.load with
-O3 --use_fast_math -lineinfo).  Differences: the target is always sm_100a, the
product is a C-ABI shared library instead of a pybind module, and fast-math is
off because the quantiser's codes are pinned to IEEE division and rounding.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ROOT = CSRC.parent.parent
LIB_NAME = "libb200w4a4.so"
SOURCES = ["b200w4a4_api.cu"]
HEADERS = ["gemm_w4a4.cuh", "quant_act.cuh", "weight_pack.cuh", "ptx.cuh", "attn_glue.cuh"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def nvcc_path() -> str | None:
    home = os.environ.get("CUDA_HOME")
    if home and (Path(home) / "bin" / "nvcc").exists():
        return str(Path(home) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    default = Path("/usr/local/cuda/bin/nvcc")
    return str(default) if default.exists() else None


def lib_path() -> Path:
    return Path(os.environ.get("VDM_W4A4_EXTENSIONS_DIR", str(CSRC))) / LIB_NAME


def is_stale(lib: Path) -> bool:
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [ROOT / "include" / "b200w4a4.h"]
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library unless it is newer than its sources.  Several processes may call this
    at once (one rank per GPU): a file lock lets one of them compile while the others wait, and
    the result is moved into place atomically so nobody maps a half-written file."""
    import fcntl

    lib = lib_path()
    if not force and not is_stale(lib):
        return lib
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libb200w4a4.so (set CUDA_HOME)")
    lib.parent.mkdir(parents=True, exist_ok=True)
    with open(lib.with_suffix(".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale(lib):   # another process built it while this one waited
                return lib
            tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
            cmd = [nvcc, *NVCC_FLAGS]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-o", str(tmp), *[str(CSRC / s) for s in SOURCES]]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp, lib)
            if verbose:
                print(proc.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


if __name__ == "__main__":
    print(build(force=True, verbose=bool(int(os.environ.get("VDM_W4A4_VERBOSE", "0")))))
