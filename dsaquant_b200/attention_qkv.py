"""Fused QKV / KV projection call site, mirroring `_get_qkv_projections` of the reference
(vdm_infer/models/wan_vdm/modules/attention.py:35-121).

Contract of `attn` (the reference's WanAttention): attributes to_q / to_k / to_v (QuantLinear in
kernel mode), cross_attention_dim_head (None for self-attention), use_fused_qkv_kernel,
qkv_kernel_backend == "vdm"; the concatenated packed weights, packed scales and fp16 bias are
cached on the module under the same attribute names the reference uses (_vdm_qkv_* / _vdm_kv_*).
Self-attention: one activation quantisation + one GEMM with N = 3*D.  Cross-attention: Q on the
M video tokens, fused K/V (N = 2*D) on the text tokens.
"""
from __future__ import annotations

import torch

from .kernels.vdm_w4a4 import linear_vdm_w4a4, linear_vdm_w4a4_qkv


def _cat_cached(attn, prefix: str, layers) -> None:
    if getattr(attn, f"{prefix}_weight_packed", None) is None:
        setattr(attn, f"{prefix}_weight_packed",
                torch.cat([l.vdm_weight_packed for l in layers], dim=0).contiguous())
        setattr(attn, f"{prefix}_weight_scale",
                torch.cat([l.vdm_weight_scale_packed for l in layers], dim=0).contiguous())
    if not hasattr(attn, f"{prefix}_bias_half") or getattr(attn, f"{prefix}_bias_half") is None:
        n = layers[0].vdm_weight_packed.shape[0]
        if any(l._bias_half is not None for l in layers):
            dev = layers[0].vdm_weight_packed.device
            parts = [l._bias_half if l._bias_half is not None
                     else torch.zeros(n, dtype=torch.float16, device=dev) for l in layers]
            setattr(attn, f"{prefix}_bias_half", torch.cat(parts, dim=0).contiguous())
        else:
            setattr(attn, f"{prefix}_bias_half", None)


def get_qkv_projections(attn, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor):
    if encoder_hidden_states is None:
        encoder_hidden_states = hidden_states
    fused = getattr(attn, "use_fused_qkv_kernel", False) and getattr(attn, "qkv_kernel_backend", None) == "vdm"
    if not fused:
        return attn.to_q(hidden_states), attn.to_k(encoder_hidden_states), attn.to_v(encoder_hidden_states)

    if attn.cross_attention_dim_head is None:
        _cat_cached(attn, "_vdm_qkv", (attn.to_q, attn.to_k, attn.to_v))
        return linear_vdm_w4a4_qkv(
            hidden_states,
            attn.to_q.vdm_weight_packed, attn.to_q.vdm_weight_scale_packed,
            attn.to_k.vdm_weight_packed, attn.to_k.vdm_weight_scale_packed,
            attn.to_v.vdm_weight_packed, attn.to_v.vdm_weight_scale_packed,
            clip_ratio=attn.to_q.kernel_clip_ratio,
            w_qkv_packed=attn._vdm_qkv_weight_packed,
            w_qkv_scale=attn._vdm_qkv_weight_scale,
            qkv_bias_half=attn._vdm_qkv_bias_half,
        )

    query = attn.to_q(hidden_states)
    _cat_cached(attn, "_vdm_kv", (attn.to_k, attn.to_v))
    kv = linear_vdm_w4a4(encoder_hidden_states, attn._vdm_kv_weight_packed, attn._vdm_kv_weight_scale,
                         bias=None, clip_ratio=attn.to_k.kernel_clip_ratio,
                         bias_half=attn._vdm_kv_bias_half)
    key, value = kv.split(attn.to_k.vdm_weight_packed.shape[0], dim=-1)
    return query, key, value


_get_qkv_projections = get_qkv_projections  # the reference's (private) name
