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

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from .kernels.vdm_w4a4 import linear_vdm_w4a4, linear_vdm_w4a4_qkv


def _cat_cached(attn, prefix: str, layers) -> None:
    """Builds (once) the concatenated v1 weight / scale / bias caches of a fused projection under
    the attribute names the reference uses.  The member layers then stop holding copies of their
    own: their `vdm_weight_packed` / `vdm_weight_scale_packed` buffers become row views of the
    concatenated tensors (same bytes, still saved per layer by a state dict), and the per-layer
    repacked weights, which the fused path never reads, are dropped from the repack table."""
    if getattr(attn, f"{prefix}_weight_packed", None) is None:
        from .kernels.vdm_w4a4 import release_b200_weight

        packed = torch.cat([l.vdm_weight_packed for l in layers], dim=0).contiguous()
        scale = torch.cat([l.vdm_weight_scale_packed for l in layers], dim=0).contiguous()
        setattr(attn, f"{prefix}_weight_packed", packed)
        setattr(attn, f"{prefix}_weight_scale", scale)
        row = 0
        for l in layers:
            n = l.vdm_weight_packed.shape[0]
            release_b200_weight(l.vdm_weight_packed)
            l._buffers["vdm_weight_packed"] = packed[row:row + n]
            l._buffers["vdm_weight_scale_packed"] = scale[row:row + n]
            row += n
    if not hasattr(attn, f"{prefix}_bias_half") or getattr(attn, f"{prefix}_bias_half") is None:
        n = layers[0].vdm_weight_packed.shape[0]
        if any(l._bias_half is not None for l in layers):
            dev = layers[0].vdm_weight_packed.device
            parts = [l._bias_half if l._bias_half is not None
                     else torch.zeros(n, dtype=torch.float16, device=dev) for l in layers]
            setattr(attn, f"{prefix}_bias_half", torch.cat(parts, dim=0).contiguous())
        else:
            setattr(attn, f"{prefix}_bias_half", None)


def prepare_fused_projections(attn) -> None:
    """What the first fused forward would do, done ahead of time: concatenate the members'
    buffers and (on a CUDA device) repack the concatenated weight for the GEMM."""
    from .kernels.vdm_w4a4 import prepare_b200_weight

    if attn.cross_attention_dim_head is None:
        prefix, layers = "_vdm_qkv", (attn.to_q, attn.to_k, attn.to_v)
    else:
        prefix, layers = "_vdm_kv", (attn.to_k, attn.to_v)
    _cat_cached(attn, prefix, layers)
    packed = getattr(attn, f"{prefix}_weight_packed")
    if packed.is_cuda:
        prepare_b200_weight(packed, getattr(attn, f"{prefix}_weight_scale"))


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


def rope_cos_sin(freqs: torch.Tensor) -> torch.Tensor:
    """complex [L, 1, head_dim/2] (or [L, head_dim/2]) rotation factors as the reference builds them
    (modules/embedding.py:103-156) -> fp32 [L, head_dim/2, 2] = (cos, sin), what qk_norm_rope reads."""
    f = freqs.reshape(freqs.shape[0], -1)
    return torch.view_as_real(f.to(torch.complex64)).contiguous()


def qk_norm_rope(x: torch.Tensor, norm_weight: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                 eps: float, head_dim: int, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """One pass over q or k ([..., L, D] fp16, rows may be strided): RMSNorm across heads with an
    fp16 weight, rotary embedding, cast to the attention dtype; what the reference's processor does
    with norm_q / norm_k, apply_rotary_emb and the attention op's casts (attention.py:167-177).
    norm_weight None: no norm; cos_sin None: no rotation.  Returns a contiguous [..., L, D] tensor."""
    lib = _lib.load()
    if not x.is_cuda:
        raise RuntimeError("qk_norm_rope needs CUDA tensors")
    if x.dtype != torch.float16:
        raise RuntimeError("qk_norm_rope takes fp16 input")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("out_dtype must be float16 or bfloat16")
    d = x.shape[-1]
    lead = tuple(x.shape[:-1])
    x2 = x.reshape(-1, d)
    if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8) or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
    if rows == 0:
        return out.view(*lead, d)
    w = None
    if norm_weight is not None:
        w = norm_weight.detach().reshape(-1)
        if w.dtype != torch.float16 or not w.is_contiguous() or w.data_ptr() % 16:
            w = w.half().contiguous().clone()
        if w.numel() != d:
            raise ValueError("norm_weight must have D elements")
    cs = None
    if cos_sin is not None:
        cs = cos_sin
        if cs.dtype != torch.float32 or not cs.is_contiguous() or cs.data_ptr() % 16:
            cs = cs.float().contiguous().clone()
        if cs.numel() != rows * head_dim:
            raise ValueError("cos_sin must be [L, head_dim/2, 2] for the L rows of x")
    with torch.cuda.device(x.device):
        rc = lib.b200w4a4_qk_norm_rope(
            x2.data_ptr(), x2.stride(0) if rows > 1 else d, w.data_ptr() if w is not None else None,
            cs.data_ptr() if cs is not None else None, float(eps), int(head_dim), out.data_ptr(),
            0 if out_dtype == torch.float16 else 1, d, rows, d,
            torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "qk_norm_rope")
    return out.view(*lead, d)


def qk_norm_rope_push(x: torch.Tensor, norm_weight: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                      eps: float, head_dim: int, dest_ptrs: Sequence[int], dest_ld: int, row0: int,
                      out_dtype: torch.dtype = torch.bfloat16, *, flag_ptrs: Optional[Sequence[int]] = None,
                      flag_index: int = 0, epoch: int = 0, ticket: Optional[torch.Tensor] = None) -> None:
    """qk_norm_rope whose rows go to every destination in `dest_ptrs` (device addresses of
    [>= row0 + L, D] matrices with row pitch dest_ld: this GPU's gather buffer and the peer-mapped
    buffers of the other GPUs of the group) at row offset row0.  With flag_ptrs / ticket the kernel
    then writes `epoch` to flag_ptrs[d] + 4 * flag_index on every destination (see wait_flags).
    Addresses are plain integers because peer memory has no torch tensor on this rank."""
    lib = _lib.load()
    if not x.is_cuda or x.dtype != torch.float16:
        raise RuntimeError("qk_norm_rope_push takes fp16 CUDA tensors")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("out_dtype must be float16 or bfloat16")
    if (flag_ptrs is None) != (ticket is None):
        raise ValueError("flag_ptrs and ticket go together")
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8) or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    if rows == 0:
        return
    n = len(dest_ptrs)
    w = None
    if norm_weight is not None:
        w = norm_weight.detach().reshape(-1)
        if w.dtype != torch.float16 or not w.is_contiguous() or w.data_ptr() % 16:
            w = w.half().contiguous().clone()
    cs = None
    if cos_sin is not None:
        cs = cos_sin if (cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
                         and cos_sin.data_ptr() % 16 == 0) else cos_sin.float().contiguous().clone()
        if cs.numel() != rows * head_dim:
            raise ValueError("cos_sin must be [L, head_dim/2, 2] for the L rows of x")
    outs = (ctypes.c_void_p * n)(*[int(p) for p in dest_ptrs])
    flags = None
    if flag_ptrs is not None:
        if len(flag_ptrs) != n:
            raise ValueError("one flag array per destination")
        if ticket.dtype != torch.int32 or ticket.numel() < 1 or ticket.device != x.device:
            raise ValueError("ticket must be an int32 tensor on x's device")
        flags = (ctypes.c_void_p * n)(*[int(p) if p else None for p in flag_ptrs])
    with torch.cuda.device(x.device):
        rc = lib.b200w4a4_qk_norm_rope_push(
            x2.data_ptr(), x2.stride(0) if rows > 1 else d, w.data_ptr() if w is not None else None,
            cs.data_ptr() if cs is not None else None, float(eps), int(head_dim), outs, n,
            0 if out_dtype == torch.float16 else 1, int(dest_ld), int(row0), flags, int(flag_index),
            int(epoch) & 0xFFFFFFFF, ticket.data_ptr() if ticket is not None else None, rows, d,
            torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "qk_norm_rope_push")


def merge_attention(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor) -> torch.Tensor:
    """Attention over the union of two disjoint key sets from its two partial results.
    o1, o2: bf16 [1, H, L, hd] as attention kernels return them (memory order [L, H, hd], i.e. a
    transposed view of an [L, H*hd] matrix); lse1, lse2: fp32 [1, H, L] (or [1, H, L, 1]).
    Returns bf16 [L, H*hd] (contiguous):  o1 * w1 + o2 * w2 with w_i = exp(lse_i - logaddexp(lse1, lse2))."""
    lib = _lib.load()
    if o1.dtype != torch.bfloat16 or o2.dtype != torch.bfloat16 or not o1.is_cuda:
        raise RuntimeError("merge_attention takes bf16 CUDA tensors")
    _, h, l, hd = o1.shape
    rows = []
    for o in (o1, o2):
        m = o.transpose(1, 2).reshape(l, h * hd)        # a view when the memory order is [L, H, hd]
        if m.stride(1) != 1 or m.stride(0) % 8 or m.data_ptr() % 16:
            m = m.contiguous()
        rows.append(m)
    ls = [t.reshape(h, l).float().contiguous() for t in (lse1, lse2)]
    out = torch.empty((l, h * hd), dtype=torch.bfloat16, device=o1.device)
    with torch.cuda.device(o1.device):
        rc = lib.b200w4a4_attn_merge(rows[0].data_ptr(), rows[0].stride(0), rows[1].data_ptr(), rows[1].stride(0),
                                     ls[0].data_ptr(), ls[1].data_ptr(), out.data_ptr(), l, h, hd,
                                     torch.cuda.current_stream(o1.device).cuda_stream)
    _lib.check(rc, "attn_merge")
    return out


def wait_flags(flags: torch.Tensor, epoch: int, timeout_ms: int = 1000) -> None:
    """Enqueues the bounded wait for `flags` (int32 [n <= 32], this GPU's memory) to reach `epoch`.
    A wait that runs out is reported by vdm_w4a4.last_device_status() == 105, not by a hang."""
    lib = _lib.load()
    if not flags.is_cuda or flags.dtype != torch.int32 or not flags.is_contiguous():
        raise RuntimeError("flags must be a contiguous int32 CUDA tensor")
    with torch.cuda.device(flags.device):
        rc = lib.b200w4a4_wait_flags(flags.data_ptr(), flags.numel(), int(epoch) & 0xFFFFFFFF, int(timeout_ms),
                                     torch.cuda.current_stream(flags.device).cuda_stream)
    _lib.check(rc, "wait_flags")
