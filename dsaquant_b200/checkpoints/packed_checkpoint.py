"""Reader / writer for `vdm_w4a4_packed_v1` checkpoints behind the function names of the reference
module vdm_infer/checkpoints/packed_checkpoint.py (format tags :18-25, is_packed_checkpoint :28,
load_quant_checkpoint :32-37, load_packed_quantized_model :52-148, enable_quant_kernels :151-164,
enable_fused_qkv :167-188, packed_state_dict_from_model :190-199, save_packed_checkpoint :202-215).

File layout: `{"format": "vdm_w4a4_packed_v1", "metadata": {...}, "model": state_dict}`.  Each
QuantLinear appears in the state dict as
    <name>.vdm_weight_packed        u8  [N, K/2]    int4 codes in the v1 tile order
    <name>.vdm_weight_scale_packed  f16 [N, K/64]   per-channel steps in the v1 lane order
    <name>.vdm_weight_scale         f16 [N]         the same steps, plain
    <name>.bias                     optional
and has no floating-point `weight`.  An older export spells the buffers `diy_*`; both are read.

What this module adds to the reference behaviour is one step at the end of loading: once the model
sits on its CUDA device every layer's v1 buffers are repacked into the layout the tcgen05 GEMM
stages with TMA (`repack_for_b200=True`), so the first forward does not pay for it.
"""
from __future__ import annotations

import gc
from typing import Any, Dict, Iterable, List, Tuple

import torch
import torch.nn as nn

PACKED_CHECKPOINT_FORMAT = "vdm_w4a4_packed_v1"
VDM_BUFFER_SUFFIXES = ("vdm_weight_packed", "vdm_weight_scale_packed", "vdm_weight_scale")
_LEGACY_PACKED_CHECKPOINT_FORMAT = PACKED_CHECKPOINT_FORMAT.replace("vdm_", "vdm_diy_", 1)
_LEGACY_BUFFER_SUFFIXES = tuple(s.replace("vdm_", "diy_", 1) for s in VDM_BUFFER_SUFFIXES)
_KNOWN_FORMATS = frozenset((PACKED_CHECKPOINT_FORMAT, _LEGACY_PACKED_CHECKPOINT_FORMAT))
_BUFFER_ENDINGS = VDM_BUFFER_SUFFIXES + _LEGACY_BUFFER_SUFFIXES


def is_packed_checkpoint(ckpt: Any) -> bool:
    return isinstance(ckpt, dict) and "model" in ckpt and ckpt.get("format") in _KNOWN_FORMATS


def load_quant_checkpoint(path: str, dcp_loader) -> dict:
    """`.pt` / `.pth`: torch.load on the CPU, tensors only.  Any other path is a distributed
    checkpoint directory and goes to `dcp_loader`."""
    if not path.endswith((".pt", ".pth")):
        return dcp_loader(path)
    print(f"Loading torch checkpoint from {path}")
    return torch.load(path, map_location="cpu", weights_only=True)


# ----------------------------------------------------------------------------- key handling
def _belongs_to_quantizer(key: str) -> bool:
    return ".wquantizer." in key or ".aquantizer." in key


def _join(prefix: str, leaf: str) -> str:
    return leaf if not prefix else prefix + "." + leaf


def _layer_buffers(state: Dict[str, torch.Tensor], layer_name: str) -> Tuple[Dict[str, torch.Tensor], List[str]]:
    """The three buffers of one layer (current spelling preferred, legacy accepted) and the keys
    that the checkpoint lacks."""
    found: Dict[str, torch.Tensor] = {}
    lacking: List[str] = []
    for current, legacy in zip(VDM_BUFFER_SUFFIXES, _LEGACY_BUFFER_SUFFIXES):
        for key in (_join(layer_name, current), _join(layer_name, legacy)):
            if key in state:
                found[current] = state[key]
                break
        else:
            lacking.append(_join(layer_name, legacy))
    return found, lacking


def _replace_buffer(module: nn.Module, name: str, tensor: torch.Tensor) -> None:
    module._buffers.pop(name, None)
    if hasattr(module, name):
        delattr(module, name)
    module.register_buffer(name, tensor.detach().contiguous())


def _switch_layer_to_packed(layer: nn.Module, buffers: Dict[str, torch.Tensor]) -> None:
    """Attach the packed buffers and drop what they replace (fp weight, both fake quantisers)."""
    for name, tensor in buffers.items():
        _replace_buffer(layer, name, tensor)
    layer.use_vdm_kernel = True
    layer.use_kernel = layer.use_kernel_fused = False
    layer.set_quant_state(use_wq=True, use_aq=True)
    if getattr(layer, "weight", None) is not None:
        layer.register_parameter("weight", None)
    for attr in ("wquantizer", "aquantizer"):
        if hasattr(layer, attr):
            delattr(layer, attr)
            setattr(layer, attr, None)


def _quant_layers(model: nn.Module, cls: type) -> Iterable[Tuple[str, nn.Module]]:
    return ((n, m) for n, m in model.named_modules() if isinstance(m, cls))


# ----------------------------------------------------------------------------- loader
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
    """Fills a freshly built model, whose Linear layers are already QuantLinear, from a packed
    checkpoint.  Returns the (missing, unexpected) keys of the part that is not quantised."""
    if not is_packed_checkpoint(packed_ckpt):
        got = packed_ckpt.get("format") if isinstance(packed_ckpt, dict) else type(packed_ckpt)
        raise ValueError(f"Unsupported checkpoint format: {got}")
    if require_vdm_kernel:
        from dsaquant_b200.kernels import vdm_w4a4

        assert vdm_w4a4.is_available(), f"DSAQuant W4A4 kernel not compiled/available: {vdm_w4a4.load_error()}"

    state = packed_ckpt["model"]
    layers = dict(_quant_layers(model, quant_linear_cls))
    fp_weights = {_join(name, "weight") for name in layers}

    # 1. everything that is not part of a quantised layer goes through load_state_dict
    ordinary = {key: value for key, value in state.items()
                if key not in fp_weights and not key.endswith(_BUFFER_ENDINGS)
                and not key.endswith("._bias_half") and not _belongs_to_quantizer(key)}
    missing, unexpected = model.load_state_dict(ordinary, strict=False, assign=True)
    missing = [key for key in missing if key not in fp_weights and not _belongs_to_quantizer(key)]

    # 2. the quantised layers take their three buffers
    absent: List[str] = []
    attached = 0
    for name, layer in layers.items():
        buffers, lacking = _layer_buffers(state, name)
        if lacking:
            absent += lacking
            continue
        _switch_layer_to_packed(layer, buffers)
        attached += 1
    if absent:
        raise KeyError(f"Packed checkpoint is missing {len(absent)} VDM buffers, e.g. {', '.join(absent[:8])}")
    if attached == 0:
        raise RuntimeError("No QuantLinear layers were populated from the packed checkpoint")
    del state, ordinary
    gc.collect()

    # 3. move, then per-layer device-side preparation
    model = model.to(dtype).to(device)
    on_gpu = torch.device(device).type == "cuda"
    for _, layer in _quant_layers(model, quant_linear_cls):
        if layer.bias is not None:
            layer._bias_half = layer.bias.half().contiguous()
        if repack_for_b200 and on_gpu:
            layer.prepare_b200_weights()
    print(f"Loaded packed DSAQuant W4A4 checkpoint: {attached} QuantLinear layers")
    return list(missing), list(unexpected)


# ----------------------------------------------------------------------------- switches on a live model
def enable_quant_kernels(model: nn.Module, *, quant_linear_cls: type[nn.Module]) -> None:
    print("Enabling DSAQuant W4A4 kernel mode...")
    for name, layer in _quant_layers(model, quant_linear_cls):
        layer.set_quant_state(use_wq=True, use_aq=True)
        try:
            layer.enable_vdm_kernel_mode()
        except Exception as exc:  # keep going: the reference reports and continues (:161-164)
            print(f"  Failed to enable VDM kernel for {name}: {exc}")


def enable_fused_qkv(model: nn.Module, *, quant_linear_cls: type[nn.Module],
                     attention_cls: type[nn.Module], use_fused_qkv: bool) -> None:
    if not use_fused_qkv:
        return
    print("Enabling fused QKV kernel (vdm)...")

    def ready(proj) -> bool:
        return isinstance(proj, quant_linear_cls) and bool(proj.use_vdm_kernel)

    for attn in model.modules():
        if isinstance(attn, attention_cls) and ready(attn.to_q) and ready(attn.to_k) and ready(attn.to_v):
            attn.use_fused_qkv_kernel = True
            attn.qkv_kernel_backend = "vdm"
            if hasattr(attn, "cross_attention_dim_head"):
                # Build the concatenated buffers now, so that the member layers' own copies and
                # per-layer repacks are released at load time instead of at the first forward.
                from dsaquant_b200.attention_qkv import prepare_fused_projections

                prepare_fused_projections(attn)


# ----------------------------------------------------------------------------- writer
def packed_state_dict_from_model(model: nn.Module, *, float_dtype: torch.dtype = torch.float16) -> dict[str, torch.Tensor]:
    """State dict as the packed format stores it: CPU tensors, floating point cast to
    `float_dtype`, without fake-quantiser state and without the derived fp16 bias copies."""
    out: dict[str, torch.Tensor] = {}
    for key, value in model.state_dict().items():
        if key.endswith("._bias_half") or _belongs_to_quantizer(key):
            continue
        host = value.detach().cpu().contiguous()
        out[key] = host.to(float_dtype) if host.is_floating_point() else host
    return out


def save_packed_checkpoint(model: nn.Module, output_path: str, *, metadata: dict[str, Any] | None = None,
                           float_dtype: torch.dtype = torch.float16) -> None:
    state = packed_state_dict_from_model(model, float_dtype=float_dtype)
    torch.save({"format": PACKED_CHECKPOINT_FORMAT, "metadata": dict(metadata or {}), "model": state}, output_path)
    print(f"Saved packed checkpoint to {output_path}")
