"""`QuantLinear` with the module interface of the reference
(vdm_infer/quantization/quant_linear.py:98-181): constructor arguments, attributes, the three
`vdm_*` buffers, method names and the forward dispatch are the reference's, so a model whose
nn.Linear layers were swapped for the reference class can use this one unchanged.

Two ways to evaluate the layer:
  kernel mode   (`use_vdm_kernel`)  per-token int4 activations x packed int4 weights on the
                                    sm_100a library (dsaquant_b200.kernels.vdm_w4a4); no CPU route
  fake-quant    (`use_wq`/`use_aq`) quantise-dequantise in PyTorch around F.linear, what calibration
                                    and the reference's CPU paths use
The quantiser itself is in uniform_quantizer.py and re-exported here under the reference's names.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .uniform_quantizer import QuantizerMap, UniformQuantizer  # noqa: F401  (reference import path)

_DEFAULT_KINDS = {"w": "uniform", "act": "uniform"}
_NO_PARAMS = {"w": {}, "act": {}}


def _kernels():
    from dsaquant_b200.kernels import vdm_w4a4

    return vdm_w4a4


class QuantLinear(nn.Module):
    def __init__(self, layer: nn.Linear, quantizer_type: dict = _DEFAULT_KINDS, q_params: dict = _NO_PARAMS) -> None:
        super().__init__()
        self.weight = nn.Parameter(layer.weight.detach().clone())
        self.bias = nn.Parameter(layer.bias.detach().clone()) if layer.bias is not None else None
        self.out_features, self.in_features = self.weight.shape
        self.extra_repr_prefix = layer.extra_repr()
        self.kwd_func = F.linear
        # fake-quant state
        self.wquantizer = QuantizerMap[quantizer_type["w"]](**q_params["w"])
        self.aquantizer = QuantizerMap[quantizer_type["act"]](**q_params["act"])
        self.use_wq = self.use_aq = False
        self.use_hadamard = self.use_timestep_scaling = False
        # kernel state (use_kernel / use_kernel_fused are the reference's other back-ends: never set here)
        self.use_kernel = self.use_kernel_fused = self.use_vdm_kernel = False
        self.kernel_clip_ratio = 0.95
        self._bias_half = None

    # ------------------------------------------------------------------ switches
    def set_quant_state(self, use_wq: bool = False, use_aq: bool = False) -> None:
        self.use_wq = use_wq
        self.use_aq = use_aq

    def set_cur_timestep(self, t) -> None:
        self.cur_timestep = t

    def set_hadamard(self, use_hadamard: bool = False) -> None:
        if use_hadamard:
            raise NotImplementedError("Hadamard rotation is not included in the inference-only release.")
        self.use_hadamard = False

    # ------------------------------------------------------------------ kernel mode
    def prepare_vdm_kernel_weights(self):
        """fp weight + the weight quantiser's per-channel step -> the three vdm_w4a4_packed_v1
        buffers (reference :136-144)."""
        wq = self.wquantizer
        assert wq is not None and wq.scale is not None, "Weight quantizer scale is missing"
        assert wq.sym, "Only symmetric quantization supported for VDM kernel"
        packed, scales_v1, scales = _kernels().pack_weight_with_scale(self.weight.detach(), wq.scale.detach().view(-1))
        for name, value in (("vdm_weight_packed", packed), ("vdm_weight_scale_packed", scales_v1),
                            ("vdm_weight_scale", scales.half())):
            self.register_buffer(name, value)

    def prepare_b200_weights(self):
        """Converts this layer's v1 buffers into the layout the tcgen05 GEMM stages (once, cached;
        the first forward does it otherwise)."""
        return _kernels().prepare_b200_weight(self.vdm_weight_packed, self.vdm_weight_scale_packed)

    def enable_vdm_kernel_mode(self):
        k = _kernels()
        assert k.is_available(), f"DSAQuant W4A4 kernel not compiled/available: {k.load_error()}"
        if not hasattr(self, "vdm_weight_packed"):
            self.prepare_vdm_kernel_weights()
        self.use_vdm_kernel, self.use_kernel, self.use_kernel_fused = True, False, False
        self._bias_half = None if self.bias is None else self.bias.half().contiguous()
        # the packed buffers replace the fp weight and its quantiser
        if getattr(self, "weight", None) is not None:
            self.register_parameter("weight", None)
        if getattr(self, "wquantizer", None) is not None:
            del self.wquantizer
            self.wquantizer = None

    # ------------------------------------------------------------------ forward
    def _forward_fake_quant(self, x: torch.Tensor) -> torch.Tensor:
        weight = self.wquantizer(self.weight) if (self.use_wq and self.wquantizer is not None) else self.weight
        if self.use_aq and self.aquantizer is not None:
            x = self.aquantizer(x)
        return self.kwd_func(x, weight, self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.use_vdm_kernel:
            return self._forward_fake_quant(x)
        return _kernels().linear_vdm_w4a4(x, self.vdm_weight_packed, self.vdm_weight_scale_packed, self.bias,
                                          self.kernel_clip_ratio, bias_half=self._bias_half)

    def extra_repr(self) -> str:
        state = f"use_aq={self.use_aq}, use_wq={self.use_wq}, use_vdm_kernel={self.use_vdm_kernel}"
        return f"{self.extra_repr_prefix}, {state}"
