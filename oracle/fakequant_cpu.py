"""CPU restatement of the reference's PyTorch fake-quant W4A4 forward, for timing only
(TEST / BASELINE INFRASTRUCTURE, not product code).

Follows QuantLinear.forward with use_wq = use_aq = True
(vdm_infer/quantization/quant_linear.py:173-178) and UniformQuantizer.forward on a 2-D input
with a fresh scale per call (:43-48, :64-66, :76-82): quantise-dequantise the activations per
token and the weights per output channel, then F.linear in fp32.  The weight fake-quant runs
every forward in the reference too (the quantizer is applied to self.weight on each call).
bench.py times this on the host cores as the CPU baseline; results are checked against
oracle/w4a4_oracle.py in tests/test_oracle.py.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def fake_quant_rows(t: torch.Tensor, scale: torch.Tensor | None = None, clip: float = 1.0):
    """Symmetric 4-bit per-row quantise-dequantise. Returns (dequantised, scale [rows,1])."""
    if scale is None:
        amax = t.abs().amax(dim=-1, keepdim=True)
        scale = amax.clamp(min=1e-5) / 7 * clip
    q = torch.clamp(torch.round(t / scale), -8, 7)
    return q * scale, scale


@torch.no_grad()
def fakequant_linear(x: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor,
                     bias: torch.Tensor | None, clip: float = 1.0) -> torch.Tensor:
    """x [M,K] fp32, w [N,K] fp32, w_scale [N] -> [M,N] fp32."""
    w_dq, _ = fake_quant_rows(w, w_scale.reshape(-1, 1).float())
    x_dq, _ = fake_quant_rows(x, None, clip)
    return F.linear(x_dq, w_dq, bias)
