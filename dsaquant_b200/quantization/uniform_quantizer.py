"""Uniform fake-quantiser behind the reference's `UniformQuantizer` interface
(vdm_infer/quantization/quant_linear.py:6-86): same constructor keywords, attributes (`bit`, `sym`,
`granularity`, `P`, `N`, `scale`, `zero_point`, `init`) and methods, so calibration code and
checkpoints written against the reference class keep working.

The arithmetic lives in three free functions so it can be read (and tested) without the module
state: how a tensor is grouped, how the step size is derived from a group's range, and the
round / clamp / rescale itself.  Scale and zero point are frozen by the first call and reused
until `init` is cleared, which is the reference's behaviour (:76-78) and the reason parity tests
reset `init` before every dynamic per-token call.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

GRANULARITIES = ("per_tensor", "per_channel", "per_token", "per_group")


def group_rows(x: torch.Tensor, granularity: str, group_size: int) -> torch.Tensor:
    """2-D view whose rows share one step size."""
    if granularity == "per_tensor":
        return x.reshape(1, -1)
    if granularity == "per_channel":
        return x.reshape(x.shape[0], -1)
    if granularity == "per_token":
        return x.reshape(-1, x.shape[-1])
    if granularity == "per_group":
        return x.reshape(-1, group_size)
    raise ValueError(f"Unsupported granularity: {granularity}")


def range_to_qparams(rows: torch.Tensor, symmetric: bool, lowest: int, highest: int,
                     clip_ratio: float) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Step size (and zero point for the asymmetric case) of every row, computed in fp32."""
    r = rows.float()
    small = r.amin(dim=-1, keepdim=True) * clip_ratio
    large = r.amax(dim=-1, keepdim=True) * clip_ratio
    if symmetric:
        return torch.maximum(small.abs(), large.abs()).clamp(min=1e-5) / highest, None
    step = ((large - small) / highest).clamp_min(1e-9)
    return step, (-torch.round(small / step)).clamp(lowest, highest)


def to_codes(rows: torch.Tensor, step: torch.Tensor, zero: Optional[torch.Tensor], lowest: int,
             highest: int, round_zero: bool) -> torch.Tensor:
    if zero is None:
        q = torch.round(rows / step)
    elif round_zero:
        q = torch.round(rows / step) + zero
    else:
        q = torch.round(rows / step + zero)
    return torch.clamp(q, lowest, highest)


def from_codes(codes: torch.Tensor, step: torch.Tensor, zero: Optional[torch.Tensor]) -> torch.Tensor:
    return codes * step if zero is None else step * (codes - zero)


class UniformQuantizer(nn.Module):
    def __init__(self, bit: int = 4, sym: bool = True, granularity: str = "per_channel",
                 group_size: int = -1, round_zero: bool = True, cali: str = "mse",
                 clip_ratio: float = 1.0, **kwargs) -> None:
        super().__init__()
        self.bit = bit
        self.sym = sym
        self.granularity = granularity
        self.group_size = group_size
        self.round_zero = round_zero
        self.cali = cali
        self.clip_ratio = clip_ratio
        span = 1 << bit
        # P / N: largest / smallest integer code (names of the reference)
        self.P, self.N = (span // 2 - 1, -(span // 2)) if sym else (span - 1, 0)
        self.scale: Optional[torch.Tensor] = None
        self.zero_point: Optional[torch.Tensor] = None
        self.init = False

    # -- state ---------------------------------------------------------------------------------
    def _store(self, name: str, value: Optional[torch.Tensor]) -> None:
        """`scale` / `zero_point` are buffers when set (they travel with state_dict) and plain None
        attributes otherwise."""
        if hasattr(self, name):
            delattr(self, name)
        if value is None:
            setattr(self, name, None)
        else:
            self.register_buffer(name, value)

    def build(self) -> None:
        if self.scale is not None:
            self.init = True

    # -- reference method names ----------------------------------------------------------------
    def reshape(self, x: torch.Tensor) -> torch.Tensor:
        return group_rows(x, self.granularity, self.group_size)

    def init_qparams(self, x: torch.Tensor) -> None:
        step, zero = range_to_qparams(self.reshape(x), self.sym, self.N, self.P, self.clip_ratio)
        self._store("scale", step.to(dtype=x.dtype))
        self._store("zero_point", None if zero is None else zero.to(dtype=x.dtype))
        self.init = True

    def quant(self, x: torch.Tensor, scale: torch.Tensor, zero_point) -> torch.Tensor:
        return to_codes(x, scale, zero_point, self.N, self.P, self.round_zero)

    def dequant(self, x: torch.Tensor, scale: torch.Tensor, zero_point) -> torch.Tensor:
        return from_codes(x, scale, zero_point)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.scale is None or not self.init:
            self.init_qparams(x)
        grouped = self.reshape(x)
        restored = self.dequant(self.quant(grouped, self.scale, self.zero_point), self.scale, self.zero_point)
        return restored.reshape(x.shape)


# The inference release maps every quantiser name of the training code onto the uniform one.
QuantizerMap = dict.fromkeys(("uniform", "lsq", "lsq+", "dynamic", "learnable_clipped_dynamic"), UniformQuantizer)
