"""B200-native W4A4 linear-layer hot path behind DSAQuant's module API.

    dsaquant_b200.kernels.vdm_w4a4            <-> vdm_infer.kernels.vdm_w4a4
    dsaquant_b200.quantization.quant_linear   <-> vdm_infer.quantization.quant_linear
    dsaquant_b200.checkpoints.packed_checkpoint <-> vdm_infer.checkpoints.packed_checkpoint
    dsaquant_b200.attention_qkv.get_qkv_projections <-> modules.attention._get_qkv_projections

`install_as_vdm_infer()` registers these modules under the reference's import paths so
existing callers pick them up without edits.
"""
from __future__ import annotations

import sys
import types

__version__ = "0.1.0"


def install_as_vdm_infer(override: bool = False) -> None:
    """Alias this package's modules as vdm_infer.kernels.vdm_w4a4, vdm_infer.quantization.quant_linear
    and vdm_infer.checkpoints.packed_checkpoint in sys.modules."""
    from .checkpoints import packed_checkpoint
    from .kernels import vdm_w4a4
    from .quantization import quant_linear

    mapping = {
        "vdm_infer.kernels.vdm_w4a4": vdm_w4a4,
        "vdm_infer.quantization.quant_linear": quant_linear,
        "vdm_infer.checkpoints.packed_checkpoint": packed_checkpoint,
    }
    for name, mod in mapping.items():
        parts = name.split(".")
        for i in range(1, len(parts)):
            pkg = ".".join(parts[:i])
            if pkg not in sys.modules:
                sys.modules[pkg] = types.ModuleType(pkg)
                sys.modules[pkg].__path__ = []  # mark as package
        if override or name not in sys.modules:
            sys.modules[name] = mod
            setattr(sys.modules[".".join(parts[:-1])], parts[-1], mod)
