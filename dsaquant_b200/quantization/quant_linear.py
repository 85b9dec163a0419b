"""QuantLinear / UniformQuantizer with the module API of the reference
(vdm_infer/quantization/quant_linear.py:6-86 UniformQuantizer, :98-181 QuantLinear).

Same constructor arguments, attributes, buffers (vdm_weight_packed,
vdm_weight_scale_packed, vdm_weight_scale), methods and forward dispatch, so a
model whose nn.Linear layers were swapped for the reference class can use this
one unchanged.  The kernel branch calls the sm_100a library through
dsaquant_b200.kernels.vdm_w4a4; the fake-quant branch is plain PyTorch and is
what calibration / CPU code paths of the reference use.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class UniformQuantizer(nn.Module):
    """Uniform fake-quantiser. Scale (and zero point) are fixed by the first forward and kept
    until `init` is cleared, exactly like the reference (:76-78)."""

    _GROUPINGS = ("per_tensor", "per_channel", "per_token", "per_group")

    def __init__(self, bit: int = 4, sym: bool = True, granularity: str = "per_channel",
                 group_size: int = -1, round_zero: bool = True, cali: str = "mse",
                 clip_ratio: float = 1.0, **kwargs) -> None:
        super().__init__()
        self.bit, self.sym = bit, sym
        self.granularity, self.group_size = granularity, group_size
        self.round_zero, self.cali, self.clip_ratio = round_zero, cali, clip_ratio
        levels = 2 ** bit
        self.P = levels // 2 - 1 if sym else levels - 1   # largest code
        self.N = -(levels // 2) if sym else 0             # smallest code
        self.scale = None
        self.zero_point = None
        self.init = False

    def reshape(self, x: torch.Tensor) -> torch.Tensor:
        g = self.granularity
        if g not in self._GROUPINGS:
            raise ValueError(f"Unsupported granularity: {g}")
        if g == "per_tensor":
            return x.reshape(1, -1)
        if g == "per_channel":
            return x.reshape(x.shape[0], -1)
        if g == "per_token":
            return x.reshape(-1, x.shape[-1])
        return x.reshape(-1, self.group_size)

    def _set_buffer(self, name: str, value: Optional[torch.Tensor]) -> None:
        if hasattr(self, name):
            delattr(self, name)
        if value is None:
            setattr(self, name, None)
        else:
            self.register_buffer(name, value)

    def init_qparams(self, x: torch.Tensor) -> None:
        rows = self.reshape(x.float())
        lo = rows.amin(dim=-1, keepdim=True) * self.clip_ratio
        hi = rows.amax(dim=-1, keepdim=True) * self.clip_ratio
        if self.sym:
            scale = torch.maximum(lo.abs(), hi.abs()).clamp(min=1e-5) / self.P
            zero = None
        else:
            scale = ((hi - lo) / self.P).clamp_min(1e-9)
            zero = (-torch.round(lo / scale)).clamp(self.N, self.P)
        self._set_buffer("scale", scale.to(dtype=x.dtype))
        self._set_buffer("zero_point", None if zero is None else zero.to(dtype=x.dtype))
        self.init = True

    def quant(self, x: torch.Tensor, scale: torch.Tensor, zero_point):
        if zero_point is None:
            q = torch.round(x / scale)
        elif self.round_zero:
            q = torch.round(x / scale) + zero_point
        else:
            q = torch.round(x / scale + zero_point)
        return torch.clamp(q, self.N, self.P)

    def dequant(self, x: torch.Tensor, scale: torch.Tensor, zero_point):
        return x * scale if zero_point is None else scale * (x - zero_point)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.init or self.scale is None:
            self.init_qparams(x)
        rows = self.reshape(x)
        codes = self.quant(rows, self.scale, self.zero_point)
        return self.dequant(codes, self.scale, self.zero_point).reshape(x.shape)

    def build(self) -> None:
        if self.scale is not None:
            self.init = True


QuantizerMap = {name: UniformQuantizer
                for name in ("uniform", "lsq", "lsq+", "dynamic", "learnable_clipped_dynamic")}


class QuantLinear(nn.Module):
    def __init__(self, layer: nn.Linear,
                 quantizer_type: dict = {"w": "uniform", "act": "uniform"},
                 q_params: dict = {"w": {}, "act": {}}) -> None:
        super().__init__()
        self.kwd_func = F.linear
        self.weight = nn.Parameter(layer.weight.detach().clone())
        self.out_features, self.in_features = self.weight.shape
        self.bias = None if layer.bias is None else nn.Parameter(layer.bias.detach().clone())
        self.use_wq = False
        self.use_aq = False
        self.wquantizer = QuantizerMap[quantizer_type["w"]](**q_params["w"])
        self.aquantizer = QuantizerMap[quantizer_type["act"]](**q_params["act"])
        self.extra_repr_prefix = layer.extra_repr()
        self.use_hadamard = False
        self.use_timestep_scaling = False
        self.use_kernel = False
        self.use_kernel_fused = False
        self.use_vdm_kernel = False
        self.kernel_clip_ratio = 0.95
        self._bias_half = None

    # ---- state switches (names as in the reference) ----
    def set_quant_state(self, use_wq: bool = False, use_aq: bool = False) -> None:
        self.use_wq, self.use_aq = use_wq, use_aq

    def set_cur_timestep(self, t) -> None:
        self.cur_timestep = t

    def set_hadamard(self, use_hadamard: bool = False) -> None:
        if use_hadamard:
            raise NotImplementedError("Hadamard rotation is not included in the inference-only release.")
        self.use_hadamard = False

    # ---- kernel mode ----
    def prepare_vdm_kernel_weights(self):
        """fp weight + learned per-channel scale -> the three vdm_w4a4_packed_v1 buffers (:136-144)."""
        from dsaquant_b200.kernels.vdm_w4a4 import pack_weight_with_scale

        assert self.wquantizer is not None and self.wquantizer.scale is not None, \
            "Weight quantizer scale is missing"
        assert self.wquantizer.sym, "Only symmetric quantization supported for VDM kernel"
        scale = self.wquantizer.scale.detach().view(-1)
        qweight, packed_scales, channel_scales = pack_weight_with_scale(self.weight.detach(), scale)
        self.register_buffer("vdm_weight_packed", qweight)
        self.register_buffer("vdm_weight_scale_packed", packed_scales)
        self.register_buffer("vdm_weight_scale", channel_scales.half())

    def prepare_b200_weights(self):
        """Load-time repack of this layer's v1 buffers into the tcgen05 staging layout
        (done lazily by the first forward otherwise)."""
        from dsaquant_b200.kernels.vdm_w4a4 import prepare_b200_weight

        return prepare_b200_weight(self.vdm_weight_packed, self.vdm_weight_scale_packed)

    def enable_vdm_kernel_mode(self):
        from dsaquant_b200.kernels.vdm_w4a4 import is_available, load_error

        assert is_available(), f"DSAQuant W4A4 kernel not compiled/available: {load_error()}"
        if not hasattr(self, "vdm_weight_packed"):
            self.prepare_vdm_kernel_weights()
        self.use_vdm_kernel = True
        self.use_kernel = False
        self.use_kernel_fused = False
        if self.bias is not None:
            self._bias_half = self.bias.half().contiguous()
        if getattr(self, "weight", None) is not None:
            self.register_parameter("weight", None)
        if getattr(self, "wquantizer", None) is not None:
            del self.wquantizer
            self.wquantizer = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.use_vdm_kernel:
            from dsaquant_b200.kernels.vdm_w4a4 import linear_vdm_w4a4

            return linear_vdm_w4a4(x, self.vdm_weight_packed, self.vdm_weight_scale_packed,
                                   self.bias, self.kernel_clip_ratio, bias_half=self._bias_half)
        w = self.weight
        if self.use_wq and self.wquantizer is not None:
            w = self.wquantizer(w)
        if self.use_aq and self.aquantizer is not None:
            x = self.aquantizer(x)
        return self.kwd_func(x, w, self.bias)

    def extra_repr(self) -> str:
        return (f"{self.extra_repr_prefix}, use_aq={self.use_aq}, use_wq={self.use_wq}, "
                f"use_vdm_kernel={self.use_vdm_kernel}")
