"""Exporter: full (legacy) quantised state -> `vdm_w4a4_packed_v1` file.

Does what the reference's scripts/export_packed_checkpoint.py:49-87 does after it has built the
model through its evaluation module (scripts/eval_quant_vdm_single.py:299-345): initialise the
weight quantisers, load the full quantised state dict (fp weights plus `wquantizer.scale`
entries, optionally nested under "model"), switch every QuantLinear to kernel mode -- which packs
the int4 codes and per-channel steps on the GPU through b200w4a4_pack_weight -- and write the
inference-only file with the reference's metadata keys.  Building the model itself (diffusers
classes, pretrained weights) stays with the caller: pass a model whose Linear layers have already
been replaced by QuantLinear.

    python -m dsaquant_b200.checkpoints.export --builder pkg.module:function \
           --quant-checkpoint-path full.pt --output packed.pt [--float-dtype float16]

`--builder` names a zero-argument callable that returns that model.
"""
from __future__ import annotations

import argparse
import gc
import importlib
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from .packed_checkpoint import (PACKED_CHECKPOINT_FORMAT, enable_quant_kernels, is_packed_checkpoint,
                                load_quant_checkpoint, save_packed_checkpoint)


def export_packed_checkpoint(
    model: nn.Module,
    quant_state: Optional[Dict[str, Any]],
    output_path: str,
    *,
    quant_linear_cls: Optional[type] = None,
    device: torch.device | str = "cuda",
    dtype: torch.dtype = torch.float16,
    float_dtype: torch.dtype = torch.float16,
    metadata: Optional[Dict[str, Any]] = None,
) -> Dict[str, Any]:
    """Packs every QuantLinear of `model` and writes `output_path`.  `quant_state` is the full
    quantised checkpoint (a state dict, or {"model": state dict}); None keeps the weights and
    quantiser scales the model already has.  Returns {"layers", "bytes", "path"}."""
    if quant_linear_cls is None:
        from ..quantization.quant_linear import QuantLinear as quant_linear_cls
    if quant_state is not None and is_packed_checkpoint(quant_state):
        raise ValueError("the source checkpoint is already packed")
    device = torch.device(device)
    model = model.to(device)
    layers = [(n, m) for n, m in model.named_modules() if isinstance(m, quant_linear_cls)]
    if not layers:
        raise RuntimeError("the model has no QuantLinear layers to export")
    # Quantiser scales exist (and have their final shapes) before the state dict is applied.
    with torch.no_grad():
        for _, layer in layers:
            if layer.wquantizer is not None and layer.weight is not None:
                layer.wquantizer(layer.weight.detach())
                layer.wquantizer.build()
            if layer.aquantizer is not None:
                layer.aquantizer.build()
            layer.set_quant_state(use_wq=True, use_aq=False)
    model = model.to(dtype)
    if quant_state is not None:
        state = quant_state["model"] if "model" in quant_state else quant_state
        missing, unexpected = model.load_state_dict(state, strict=False, assign=True)
        if missing:
            print(f"  Missing keys: {len(missing)}")
        if unexpected:
            print(f"  Unexpected keys: {len(unexpected)}")
        del state
        gc.collect()
    model = model.to(dtype).to(device)
    enable_quant_kernels(model, quant_linear_cls=quant_linear_cls)
    not_packed = [n for n, m in layers if not getattr(m, "use_vdm_kernel", False)]
    if not_packed:
        raise RuntimeError(f"{len(not_packed)} layers could not be packed, e.g. {', '.join(not_packed[:4])}")
    meta = {"format": PACKED_CHECKPOINT_FORMAT}
    meta.update(metadata or {})
    out = Path(output_path)
    out.parent.mkdir(parents=True, exist_ok=True)
    save_packed_checkpoint(model, str(out), metadata=meta, float_dtype=float_dtype)
    size = out.stat().st_size
    print(f"Packed checkpoint size: {size / 1024 ** 3:.3f} GiB")
    return {"layers": len(layers), "bytes": size, "path": str(out)}


def main() -> None:
    ap = argparse.ArgumentParser(description="Export a packed DSAQuant W4A4 checkpoint (vdm_w4a4_packed_v1)")
    ap.add_argument("--builder", required=True, help="module:function returning the model with QuantLinear layers")
    ap.add_argument("--quant-checkpoint-path", required=True, help="full quantised checkpoint (.pt/.pth) to pack")
    ap.add_argument("--output", required=True, help="output packed .pt path")
    ap.add_argument("--float-dtype", choices=("float16", "bfloat16"), default="float16")
    ap.add_argument("--model", default=None, help="model name recorded in the metadata")
    args = ap.parse_args()
    mod_name, _, fn_name = args.builder.partition(":")
    builder = getattr(importlib.import_module(mod_name), fn_name)

    def no_dcp(path):
        raise ValueError(f"{path}: only .pt / .pth checkpoints can be read here (no distributed-checkpoint reader)")

    state = load_quant_checkpoint(args.quant_checkpoint_path, no_dcp)
    print(f"Exporting {args.model or args.builder} as {PACKED_CHECKPOINT_FORMAT}")
    export_packed_checkpoint(
        builder(), state, args.output,
        float_dtype=torch.float16 if args.float_dtype == "float16" else torch.bfloat16,
        metadata={"model": args.model, "source_quant_checkpoint": args.quant_checkpoint_path})


if __name__ == "__main__":
    main()
