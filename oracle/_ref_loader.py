"""Imports oracle/_ref/vdm_w4a4_ref_ext.so (the reference's own CUDA extension built by
oracle/build_ref_ext.py).  TEST / BASELINE INFRASTRUCTURE only.  Returns None when the
library has not been built."""
from __future__ import annotations

import importlib.util
from pathlib import Path

_PATH = Path(__file__).resolve().parent / "_ref" / "vdm_w4a4_ref_ext.so"
_MOD = None


def load():
    global _MOD
    if _MOD is not None:
        return _MOD
    if not _PATH.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location("vdm_w4a4_ref_ext", str(_PATH))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _MOD = mod
    return mod
