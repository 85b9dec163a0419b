"""Builds the REFERENCE's own CUDA extension for sm_100a as a checker / same-box GPU baseline.

TEST / BASELINE INFRASTRUCTURE.  Compiles vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu from the
reference checkout where it lies (DSAQUANT_REFERENCE, or a `reference` directory beside this repository)
with the reference's own flags (-O3 --use_fast_math -lineinfo, vdm_w4a4.py:151-162) into
oracle/_ref/vdm_w4a4_ref_ext.so (git-ignored; no reference source is copied).  The module is a
pybind11 torch extension: import it with oracle._ref_loader.load().  It is used only by tests
(byte-for-byte check of the vdm_w4a4_packed_v1 layout against the reference packer, statistics
of the reference kernel's output against the oracle) and by the GPU-baseline leg of the
benchmark notes; nothing in the product path touches it.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "vdm_w4a4_ref_ext.so"
NAME = "vdm_w4a4_ref_ext"


def reference_checkout() -> Path | None:
    """The DSAQuant checkout: the directory DSAQUANT_REFERENCE names, else a directory called
    `reference` next to this repository; None when neither holds the kernel source."""
    cands = [os.environ.get("DSAQUANT_REFERENCE"), str(HERE.parent.parent / "reference")]
    for c in cands:
        if c and (Path(c) / "vdm_infer" / "kernels" / "csrc" / "vdm_w4a4_kernel.cu").exists():
            return Path(c)
    return None


def build(force: bool = False) -> Path | None:
    ref = reference_checkout()
    if ref is None:
        return OUT if OUT.exists() else None
    src = ref / "vdm_infer" / "kernels" / "csrc" / "vdm_w4a4_kernel.cu"
    if not src.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime > src.stat().st_mtime:
        return OUT
    import torch
    from torch.utils import cpp_extension as ce

    OUT.parent.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    lib_dir = Path(torch.__file__).parent / "lib"
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-lineinfo",
           "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
           f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
           *inc, str(src), "-o", str(OUT), f"-L{lib_dir}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
           "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-Xlinker", f"-rpath={lib_dir}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("building the reference extension failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
