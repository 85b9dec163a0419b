"""vdm_w4a4_packed_v1 checkpoint helpers with the API of the reference module
vdm_infer/checkpoints/packed_checkpoint.py (format tags :18-25, is_packed_checkpoint :28,
load_quant_checkpoint :32-37, load_packed_quantized_model :52-148, enable_quant_kernels
:151-164, enable_fused_qkv :167-188, packed_state_dict_from_model :190-199,
save_packed_checkpoint :202-215).

A packed checkpoint is `{"format": "vdm_w4a4_packed_v1", "metadata": {...}, "model": state_dict}`
where every QuantLinear contributes `<name>.vdm_weight_packed` (u8 [N,K/2]),
`<name>.vdm_weight_scale_packed` (f16 [N,K/64]), `<name>.vdm_weight_scale` (f16 [N]) and
`<name>.bias`, and no fp `weight`.  The only addition here is the load-time repack: after the
model has moved to its device each layer's v1 buffers are converted once into the layout the
tcgen05 GEMM stages with TMA (`repack_for_b200=True`).
"""
from __future__ import annotations

import gc
from typing import Any

import torch
import torch.nn as nn

PACKED_CHECKPOINT_FORMAT = "vdm_w4a4_packed_v1"
_LEGACY_PACKED_CHECKPOINT_FORMAT = "vdm_" + "diy" + "_w4a4_packed_v1"
VDM_BUFFER_SUFFIXES = ("vdm_weight_packed", "vdm_weight_scale_packed", "vdm_weight_scale")
_LEGACY_BUFFER_SUFFIXES = tuple("diy_" + s[len("vdm_"):] for s in VDM_BUFFER_SUFFIXES)
_QUANTIZER_MARKS = (".wquantizer.", ".aquantizer.")


def is_packed_checkpoint(ckpt: Any) -> bool:
    if not isinstance(ckpt, dict) or "model" not in ckpt:
        return False
    return ckpt.get("format") in (PACKED_CHECKPOINT_FORMAT, _LEGACY_PACKED_CHECKPOINT_FORMAT)


def load_quant_checkpoint(path: str, dcp_loader) -> dict:
    """A `.pt`/`.pth` file is read with torch.load (CPU, weights only); anything else goes
    through `dcp_loader` (distributed-checkpoint directory)."""
    if path.endswith((".pt", ".pth")):
        print(f"Loading torch checkpoint from {path}")
        return torch.load(path, map_location="cpu", weights_only=True)
    return dcp_loader(path)


def _key(module_name: str, suffix: str) -> str:
    return f"{module_name}.{suffix}" if module_name else suffix


def _set_buffer(module: nn.Module, name: str, tensor: torch.Tensor) -> None:
    module._buffers.pop(name, None)
    if hasattr(module, name):
        delattr(module, name)
    module.register_buffer(name, tensor.detach().contiguous())


def _is_quant_state(key: str) -> bool:
    return any(mark in key for mark in _QUANTIZER_MARKS)


def load_packed_quantized_model(
    model: nn.Module,
    packed_ckpt: dict,
    *,
    quant_linear_cls: type[nn.Module],
    dtype: torch.dtype,
    device: torch.device,
    require_vdm_kernel: bool = True,
    repack_for_b200: bool = True,
) -> tuple[list[str], list[str]]:
    """Populate a freshly built model (its Linear layers already swapped for QuantLinear) from
    a packed checkpoint; returns (missing, unexpected) keys of the non-quantised part."""
    if not is_packed_checkpoint(packed_ckpt):
        found = packed_ckpt.get("format") if isinstance(packed_ckpt, dict) else type(packed_ckpt)
        raise ValueError(f"Unsupported checkpoint format: {found}")
    if require_vdm_kernel:
        from dsaquant_b200.kernels.vdm_w4a4 import is_available, load_error

        assert is_available(), f"DSAQuant W4A4 kernel not compiled/available: {load_error()}"

    state = packed_ckpt["model"]
    qlayers = {name: mod for name, mod in model.named_modules() if isinstance(mod, quant_linear_cls)}
    fp_weight_keys = {_key(name, "weight") for name in qlayers}
    all_suffixes = VDM_BUFFER_SUFFIXES + _LEGACY_BUFFER_SUFFIXES

    plain = {k: v for k, v in state.items()
             if not k.endswith(all_suffixes) and not _is_quant_state(k)
             and not k.endswith("._bias_half") and k not in fp_weight_keys}
    missing, unexpected = model.load_state_dict(plain, strict=False, assign=True)
    missing = [k for k in missing if k not in fp_weight_keys and not _is_quant_state(k)]

    absent: list[str] = []
    loaded = 0
    for name, mod in qlayers.items():
        chosen = {}
        for suffix, legacy in zip(VDM_BUFFER_SUFFIXES, _LEGACY_BUFFER_SUFFIXES):
            k_new, k_old = _key(name, suffix), _key(name, legacy)
            chosen[suffix] = k_new if k_new in state else k_old
        lacking = [k for k in chosen.values() if k not in state]
        if lacking:
            absent.extend(lacking)
            continue
        for suffix, k in chosen.items():
            _set_buffer(mod, suffix, state[k])
        mod.use_vdm_kernel, mod.use_kernel, mod.use_kernel_fused = True, False, False
        mod.set_quant_state(use_wq=True, use_aq=True)
        if getattr(mod, "weight", None) is not None:
            mod.register_parameter("weight", None)
        for qname in ("wquantizer", "aquantizer"):
            if hasattr(mod, qname):
                delattr(mod, qname)
                setattr(mod, qname, None)
        loaded += 1

    if absent:
        raise KeyError(f"Packed checkpoint is missing {len(absent)} VDM buffers, e.g. {', '.join(absent[:8])}")
    if loaded == 0:
        raise RuntimeError("No QuantLinear layers were populated from the packed checkpoint")

    del state, plain
    gc.collect()

    model = model.to(dtype).to(device)
    for mod in model.modules():
        if isinstance(mod, quant_linear_cls):
            if mod.bias is not None:
                mod._bias_half = mod.bias.half().contiguous()
            if repack_for_b200 and torch.device(device).type == "cuda":
                mod.prepare_b200_weights()
    print(f"Loaded packed DSAQuant W4A4 checkpoint: {loaded} QuantLinear layers")
    return list(missing), list(unexpected)


def enable_quant_kernels(model: nn.Module, *, quant_linear_cls: type[nn.Module]) -> None:
    print("Enabling DSAQuant W4A4 kernel mode...")
    for name, mod in model.named_modules():
        if not isinstance(mod, quant_linear_cls):
            continue
        mod.set_quant_state(use_wq=True, use_aq=True)
        try:
            mod.enable_vdm_kernel_mode()
        except Exception as exc:
            print(f"  Failed to enable VDM kernel for {name}: {exc}")


def enable_fused_qkv(model: nn.Module, *, quant_linear_cls: type[nn.Module],
                     attention_cls: type[nn.Module], use_fused_qkv: bool) -> None:
    if not use_fused_qkv:
        return
    print("Enabling fused QKV kernel (vdm)...")
    for mod in model.modules():
        if not isinstance(mod, attention_cls):
            continue
        projs = (mod.to_q, mod.to_k, mod.to_v)
        if all(isinstance(p, quant_linear_cls) and p.use_vdm_kernel for p in projs):
            mod.use_fused_qkv_kernel = True
            mod.qkv_kernel_backend = "vdm"


def packed_state_dict_from_model(model: nn.Module, *, float_dtype: torch.dtype = torch.float16) -> dict[str, torch.Tensor]:
    packed: dict[str, torch.Tensor] = {}
    for key, value in model.state_dict().items():
        if _is_quant_state(key) or key.endswith("._bias_half"):
            continue
        t = value.detach().cpu().contiguous()
        packed[key] = t.to(float_dtype) if t.is_floating_point() else t
    return packed


def save_packed_checkpoint(model: nn.Module, output_path: str, *, metadata: dict[str, Any] | None = None,
                           float_dtype: torch.dtype = torch.float16) -> None:
    torch.save({"format": PACKED_CHECKPOINT_FORMAT, "metadata": metadata or {},
                "model": packed_state_dict_from_model(model, float_dtype=float_dtype)}, output_path)
    print(f"Saved packed checkpoint to {output_path}")
