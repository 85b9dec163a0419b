"""Benchmark harness: a diffusers-free restatement of the Wan DiT denoising forward, used only to
time and parity-check the full-step configurations (Wan 2.1 1.3B / 14B, Wan 2.2 5B) around the
W4A4 linear path.  It is NOT part of the product: the product is the linear layer.

Follows, by file:line of the reference,
  model forward            vdm_infer/models/wan_vdm/modules/model.py:172-360
  transformer block        vdm_infer/models/wan_vdm/modules/dit_block.py:15-117
  attention processor      vdm_infer/models/wan_vdm/modules/attention.py:133-216 (RMSNorm across heads,
                           3-D RoPE, SDPA), fused QKV call site :35-121
  embeddings / RoPE table  vdm_infer/models/wan_vdm/modules/embedding.py:7-156
  SDPA op                  vdm_infer/models/base/vdm_attn.py:241-259
  model shapes             vdm_infer/models/wan_vdm/__init__.py:13-112
and, for the two diffusers classes whose arithmetic matters (not in the reference tree):
FP32LayerNorm = LayerNorm evaluated in fp32 and cast back; FeedForward(gelu-approximate) =
Linear -> tanh-GELU -> Linear.  Weights are random (std 0.02, biases 0, scale/shift tables
std 0.02, norm weights 1) as the reference's init_weights does; every nn.Linear inside the
blocks is a W4A4 QuantLinear (10 per block), the patch / condition / output projections stay fp16.
Attention runs as bf16 SDPA (the benchmark definition; the reference pipeline runs it in fp16).

Two linear back-ends share the same int4 weight codes:
  "kernel"  dsaquant_b200 QuantLinear in kernel mode (sm_100a library), fused QKV / KV
  "oracle"  PyTorch fake-quant with per-token dynamic activation scales in fp32 (test reference)

`set_fused(True)` (kernel back-end only) routes a block through the library's fused entry points:
layer norm + modulation and GELU inside the quantiser, GELU / gated skip / split q-k-v outputs in
the GEMM epilogue, RMSNorm across heads + RoPE + bf16 cast of q and k in one pass (qk_norm_rope).

Row sharding (multi-GPU inside one CFG branch): every per-token op runs on this rank's rows;
self-attention all-gathers K and V of the branch group after RMSNorm + RoPE.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from dsaquant_b200 import sharding
from dsaquant_b200.attention_qkv import get_qkv_projections
from dsaquant_b200.quantization.quant_linear import QuantLinear

class PhaseTimer:
    """Attributes GPU time of one stream to named phases: mark(name) records a CUDA event; the
    time from one mark to the next belongs to the earlier mark's name.  Used by the benchmark
    for one extra, untimed step; None otherwise."""

    def __init__(self):
        self.marks = []

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, ev))

    def totals_ms(self) -> dict:
        out = {}
        for (name, a), (_, b) in zip(self.marks, self.marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


PHASES: Optional[PhaseTimer] = None


def set_phase_timer(timer: Optional[PhaseTimer]) -> None:
    """Installs (or removes) the phase timer here and as the library wrapper's quant/gemm hook."""
    global PHASES
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    PHASES = timer
    vdm.set_phase_hook(None if timer is None else timer.mark)


def _mark(name: str) -> None:
    if PHASES is not None:
        PHASES.mark(name)


QPARAMS = {"w": {"bit": 4, "sym": True, "granularity": "per_channel"}, "act": {"bit": 4, "sym": True}}
KERNEL_CLIP = 0.95


@dataclass(frozen=True)
class WanConfig:
    name: str
    dim: int
    heads: int
    ffn: int
    layers: int
    in_ch: int
    out_ch: int
    latent: Tuple[int, int, int, int]          # C, F, H, W of the latent video
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    patch: Tuple[int, int, int] = (1, 2, 2)
    eps: float = 1e-6

    @property
    def tokens(self) -> int:
        _, f, h, w = self.latent
        return (f // self.patch[0]) * (h // self.patch[1]) * (w // self.patch[2])


CONFIGS = {
    # Wan 2.1 T2V 1.3B: 81 frames at 480x832 -> latent 16x21x60x104 -> 32760 tokens
    "wan21_1.3b": WanConfig("wan21_1.3b", 1536, 12, 8960, 30, 16, 16, (16, 21, 60, 104)),
    # Wan 2.2 TI2V 5B: 121 frames at 704x1280 -> latent 48x31x44x80 -> 27280 tokens
    "wan22_5b": WanConfig("wan22_5b", 3072, 24, 14336, 30, 48, 48, (48, 31, 44, 80)),
    # Wan 2.1 T2V 14B
    "wan21_14b": WanConfig("wan21_14b", 5120, 40, 13824, 40, 16, 16, (16, 21, 60, 104)),
}


def tiny_config(dim=256, heads=2, ffn=512, layers=2, latent=(16, 3, 8, 12)) -> WanConfig:
    return WanConfig("tiny", dim, heads, ffn, layers, latent[0], latent[0], latent, text_dim=128, text_len=64)


# --------------------------------------------------------------------------- linear back-ends
class OracleW4A4Linear(nn.Module):
    """PyTorch fake-quant W4A4 linear on the SAME weight codes as a kernel-mode QuantLinear:
    per-token dynamic activation scale (max(absmax,1e-5)/7*clip, fp32), codes by true division,
    fp32 matmul of the integer codes, dequant, bias, fp16."""

    def __init__(self, ql: QuantLinear, codes: torch.Tensor):
        super().__init__()
        self.register_buffer("codes", codes.float())
        self.register_buffer("w_scale", ql.vdm_weight_scale.float())
        self.bias_half = ql._bias_half
        self.clip = ql.kernel_clip_ratio
        self.vdm_weight_packed = ql.vdm_weight_packed

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).float()
        # tensor / tensor: torch turns division by a python scalar on CUDA into a multiplication
        # by its reciprocal, which is not the pinned IEEE division.
        seven = torch.full((), 7.0, dtype=torch.float32, device=x2.device)
        s = (x2.abs().amax(dim=1, keepdim=True).clamp(min=1e-5) / seven) * self.clip
        q = torch.clamp(torch.round(x2 / s), -8, 7)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            acc = q @ self.codes.t()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        y = acc * (s * self.w_scale[None, :])
        if self.bias_half is not None:
            y = y + self.bias_half.float()[None, :]
        return y.half().reshape(*shape, -1)


def _quantize_linear(lin: nn.Linear) -> QuantLinear:
    """nn.Linear -> kernel-mode QuantLinear (abs-max/7 weight scales, packed on the GPU), the
    reference's legacy build path (quant_linear.py:136-160)."""
    ql = QuantLinear(lin, {"w": "lsq", "act": "dynamic"}, QPARAMS).to(lin.weight.device).half()
    ql.wquantizer(ql.weight.detach())
    ql.set_quant_state(True, True)
    ql.enable_vdm_kernel_mode()
    ql.prepare_b200_weights()
    return ql


# --------------------------------------------------------------------------- model pieces
def fp32_layer_norm(x: torch.Tensor, eps: float, weight=None, bias=None) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), None if weight is None else weight.float(),
                        None if bias is None else bias.float(), eps)


class RMSNormAcrossHeads(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_table(head_dim: int, f: int, h: int, w: int, device) -> torch.Tensor:
    """Complex rotation factors [f*h*w, 1, head_dim/2] (embedding.py:103-156)."""
    def table(dim, end=1024, theta=10000.0):
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].double() / dim))
        ang = torch.outer(torch.arange(end).double(), freqs)
        return torch.polar(torch.ones_like(ang), ang)
    d = head_dim
    ft, ht, wt = table(d - 2 * (d // 3)), table(d // 3), table(d // 3)
    out = torch.cat([ft[:f].view(f, 1, 1, -1).expand(f, h, w, -1),
                     ht[:h].view(1, h, 1, -1).expand(f, h, w, -1),
                     wt[:w].view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1)
    return out.reshape(f * h * w, 1, -1).to(torch.complex64).to(device)


def apply_rope(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [1, L, H, D]; freqs [L, 1, D/2] complex64 (attention.py:133-137, fp32 variant)."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * freqs[None]).flatten(3).to(x.dtype)


class WanAttention(nn.Module):
    def __init__(self, cfg: WanConfig, cross: bool):
        super().__init__()
        d = cfg.dim
        self.heads = cfg.heads
        self.cross_attention_dim_head = d // cfg.heads if cross else None
        self.to_q, self.to_k, self.to_v, self.to_out = (nn.Linear(d, d) for _ in range(4))
        self.norm_q = RMSNormAcrossHeads(d, cfg.eps)
        self.norm_k = RMSNormAcrossHeads(d, cfg.eps)
        self.use_fused_qkv_kernel = False
        self.qkv_kernel_backend = None

    def forward(self, x, ctx, freqs, group=None, m_total=None):
        q, k, v = get_qkv_projections(self, x, ctx)
        return self.to_out(self.core(q, k, v, ctx is None, freqs, group, m_total))

    def core(self, q, k, v, is_self, freqs, group=None, m_total=None):
        """RMSNorm across heads, RoPE, (K/V all-gather under row sharding), bf16 SDPA."""
        dtype = q.dtype
        gather = group is not None and is_self
        if gather:
            # Row-sharded self-attention: every rank needs all keys and values of its branch.
            # V needs no further processing, so its all-gather starts now and overlaps the
            # RMSNorm / RoPE of q and k.
            v_work, v_full = sharding.all_gather_rows(v.reshape(v.shape[1], -1).to(torch.bfloat16), m_total, group,
                                                      async_op=True)
        q, k = self.norm_q(q), self.norm_k(k)
        q, k, v = (t.unflatten(2, (self.heads, -1)) for t in (q, k, v))
        if freqs is not None:
            q, k = apply_rope(q, freqs), apply_rope(k, freqs)
        if gather:
            k = sharding.all_gather_rows(k.reshape(k.shape[1], -1).to(torch.bfloat16), m_total, group)
            k = k.view(1, m_total, self.heads, -1)
            v_work.wait()
            v = v_full.view(1, m_total, self.heads, -1)
        o = F.scaled_dot_product_attention(q.transpose(1, 2).bfloat16(), k.transpose(1, 2).bfloat16(),
                                           v.transpose(1, 2).bfloat16(), dropout_p=0.0, is_causal=False)
        return o.transpose(1, 2).flatten(2, 3).to(dtype)


_LSE_BACKEND = None


def sdpa_with_lse(q, k, v):
    """Library attention that also returns the log-sum-exp of every query row, [1,H,Lq] fp32 (what
    merging attention over two disjoint key ranges needs).  q, k, v: [1,H,L,hd] bf16.  Uses the
    cuDNN attention op when it accepts the call, else the flash op; both are torch library kernels."""
    global _LSE_BACKEND
    order = [_LSE_BACKEND] if _LSE_BACKEND else ["cudnn", "flash"]
    err = None
    for name in order:
        try:
            if name == "cudnn":
                out = torch.ops.aten._scaled_dot_product_cudnn_attention(q, k, v, None, True, 0.0, False, False)
            else:
                out = torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.0, False, False)
            _LSE_BACKEND = name
            return out[0], out[1].reshape(q.shape[0], q.shape[1], q.shape[2]).float()
        except Exception as exc:  # try the next library kernel
            err = exc
    raise RuntimeError(f"no library attention kernel returned a log-sum-exp: {err}")


def merge_attention(o1, l1, o2, l2):
    """Attention over the union of two disjoint key sets from the two partial results:
    out = o1 * exp(l1 - l) + o2 * exp(l2 - l) with l = logaddexp(l1, l2).  o: [1,H,L,hd], l: [1,H,L]."""
    l = torch.logaddexp(l1, l2)
    w1, w2 = torch.exp(l1 - l)[..., None], torch.exp(l2 - l)[..., None]
    return (o1.float() * w1 + o2.float() * w2).to(o1.dtype)


def _core_fused(attn, q, k, v, is_self, freqs, group=None, m_total=None):
    """`WanAttention.core` with the per-token glue in the library: RMSNorm across heads, RoPE and the
    bf16 cast of q and k run as one pass each (dsaquant_b200.attention_qkv.qk_norm_rope), v is cast
    in one pass, and the attention output stays bf16 (the output projection quantises it directly).
    q, k, v: [1, L, D] fp16 as written by the split QKV epilogue."""
    from dsaquant_b200.attention_qkv import qk_norm_rope

    heads = attn.heads
    d = q.shape[-1]
    hd = d // heads
    eps = attn.norm_q.eps
    cs = None if freqs is None else torch.view_as_real(freqs).reshape(freqs.shape[0], -1)
    gather = group is not None and is_self
    exchange = getattr(attn, "kv_exchange", None) if gather else None
    _mark("glue")
    if exchange is not None and exchange.rotated:
        # Own rows first, peers after them: attention over the local keys runs while the peers'
        # rows are still on their way, and the two partial results are merged by log-sum-exp.
        exchange.begin_block()
        exchange.push("v", v[0], None, None, eps, hd)
        exchange.push("k", k[0], attn.norm_k.weight, cs, eps, hd)
        qn = qk_norm_rope(q[0], attn.norm_q.weight, cs, eps, hd)
        lq = qn.shape[0]
        qh = qn.view(1, lq, heads, hd).transpose(1, 2)
        _mark("sdpa")
        k_loc, v_loc = exchange.local_rows()
        o1, l1 = sdpa_with_lse(qh, k_loc.view(1, -1, heads, hd).transpose(1, 2), v_loc.view(1, -1, heads, hd).transpose(1, 2))
        _mark("exchange_wait")
        k_rem, v_rem = exchange.remote_rows()
        _mark("sdpa")
        o2, l2 = sdpa_with_lse(qh, k_rem.view(1, -1, heads, hd).transpose(1, 2), v_rem.view(1, -1, heads, hd).transpose(1, 2))
        from dsaquant_b200.attention_qkv import merge_attention as merge_fused

        o = merge_fused(o1, l1, o2, l2)                 # [Lq, D] bf16, one pass
        exchange.end_block()
        _mark("other")
        return o.view(1, lq, d)
    if exchange is not None:
        # The kernels that produce K and V store their rows into every rank's gather buffer.
        exchange.begin_block()
        exchange.push("v", v[0], None, None, eps, hd)
        exchange.push("k", k[0], attn.norm_k.weight, cs, eps, hd)
        qn = qk_norm_rope(q[0], attn.norm_q.weight, cs, eps, hd)
        _mark("exchange_wait")
        kn, vb = exchange.gathered(m_total, attn.kv_senders)
    else:
        vb = qk_norm_rope(v[0], None, None, eps, hd)
        if gather:
            v_work, v_full = sharding.all_gather_rows(vb, m_total, group, async_op=True)
        # K before Q: its all-gather is asynchronous too and overlaps Q's pass.
        kn = qk_norm_rope(k[0], attn.norm_k.weight, cs, eps, hd)
        if gather:
            k_work, k_full = sharding.all_gather_rows(kn, m_total, group, async_op=True)
        qn = qk_norm_rope(q[0], attn.norm_q.weight, cs, eps, hd)
        if gather:
            _mark("exchange_wait")
            k_work.wait()
            v_work.wait()
            kn, vb = k_full, v_full
    _mark("sdpa")
    lq, lk = qn.shape[0], kn.shape[0]
    o = F.scaled_dot_product_attention(qn.view(1, lq, heads, hd).transpose(1, 2),
                                       kn.view(1, lk, heads, hd).transpose(1, 2),
                                       vb.view(1, lk, heads, hd).transpose(1, 2), dropout_p=0.0, is_causal=False)
    if exchange is not None:
        exchange.end_block()
    _mark("other")
    return o.transpose(1, 2).reshape(1, lq, d)


class WanBlock(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        d = cfg.dim
        self.eps = cfg.eps
        self.attn1 = WanAttention(cfg, cross=False)
        self.attn2 = WanAttention(cfg, cross=True)
        self.norm2 = nn.LayerNorm(d, cfg.eps, elementwise_affine=True)
        self.ffn_up = nn.Linear(d, cfg.ffn)
        self.ffn_down = nn.Linear(cfg.ffn, d)
        self.scale_shift_table = nn.Parameter(torch.randn(1, 6, d) * 0.02)

    fused = False   # kernel back-end only: fold norms / modulation / GELU / gated skips into the linears

    def forward_fused(self, x, ctx, temb6, freqs, group=None, m_total=None):
        """Same block with the elementwise work folded into the W4A4 library calls: layer norm +
        modulation run inside the quantiser, GELU and `skip + out * gate` inside the GEMM epilogue."""
        from dsaquant_b200.attention_qkv import _cat_cached
        from dsaquant_b200.kernels.vdm_w4a4 import linear_vdm_w4a4_fused as fused, linear_vdm_w4a4_split as split

        mod = (self.scale_shift_table.float() + temb6.float())          # [1 or L, 6, D]
        shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (mod[:, i] for i in range(6))
        a1, a2 = self.attn1, self.attn2
        d = x.shape[-1]
        clip = a1.to_q.kernel_clip_ratio
        # 1. self-attention
        _cat_cached(a1, "_vdm_qkv", (a1.to_q, a1.to_k, a1.to_v))
        q, k, v = split(x, a1._vdm_qkv_weight_packed, a1._vdm_qkv_weight_scale, 3, a1._vdm_qkv_bias_half, clip,
                        prologue="layernorm_mod", mod_scale=scale_msa, mod_shift=shift_msa, ln_eps=self.eps)
        o = _core_fused(a1, q, k, v, True, freqs, group, m_total)
        x = fused(o, a1.to_out.vdm_weight_packed, a1.to_out.vdm_weight_scale_packed, a1.to_out._bias_half, clip,
                  epilogue="gate_residual", residual=x, gate=gate_msa)
        # 2. cross-attention (affine layer norm = modulation with scale = weight - 1, shift = bias)
        q = fused(x, a2.to_q.vdm_weight_packed, a2.to_q.vdm_weight_scale_packed, a2.to_q._bias_half, clip,
                  prologue="layernorm_mod", mod_scale=self.norm2.weight.float() - 1.0,
                  mod_shift=self.norm2.bias.float(), ln_eps=self.eps)
        _cat_cached(a2, "_vdm_kv", (a2.to_k, a2.to_v))
        k, v = split(ctx, a2._vdm_kv_weight_packed, a2._vdm_kv_weight_scale, 2, a2._vdm_kv_bias_half, clip)
        o = _core_fused(a2, q, k, v, False, None)
        if not hasattr(self, "_ones"):
            self._ones = torch.ones(d, dtype=torch.float32, device=x.device)
        x = fused(o, a2.to_out.vdm_weight_packed, a2.to_out.vdm_weight_scale_packed, a2.to_out._bias_half, clip,
                  epilogue="gate_residual", residual=x, gate=self._ones)
        # 3. feed-forward
        h = fused(x, self.ffn_up.vdm_weight_packed, self.ffn_up.vdm_weight_scale_packed, self.ffn_up._bias_half, clip,
                  prologue="layernorm_mod", mod_scale=c_scale, mod_shift=c_shift, ln_eps=self.eps,
                  epilogue="gelu_tanh")
        return fused(h, self.ffn_down.vdm_weight_packed, self.ffn_down.vdm_weight_scale_packed,
                     self.ffn_down._bias_half, clip, epilogue="gate_residual", residual=x, gate=c_gate)

    def forward(self, x, ctx, temb6, freqs, group=None, m_total=None):
        if self.fused:
            return self.forward_fused(x, ctx, temb6, freqs, group, m_total)
        # temb6 [1 or L, 6, D] fp32; the reference materialises it per token (model.py:220-231).
        mod = self.scale_shift_table.float() + temb6.float()
        shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (mod[:, i][None] for i in range(6))
        h = (fp32_layer_norm(x, self.eps) * (1 + scale_msa) + shift_msa).to(x.dtype)
        x = (x.float() + self.attn1(h, None, freqs, group, m_total).float() * gate_msa).to(x.dtype)
        h = fp32_layer_norm(x, self.eps, self.norm2.weight, self.norm2.bias).to(x.dtype)
        x = x + self.attn2(h, ctx, None)
        h = (fp32_layer_norm(x, self.eps) * (1 + c_scale) + c_shift).to(x.dtype)
        h = self.ffn_down(F.gelu(self.ffn_up(h), approximate="tanh"))
        return (x.float() + h.float() * c_gate).to(x.dtype)


class WanDiT(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        p = math.prod(cfg.patch)
        self.patch_embedding_mlp = nn.Linear(cfg.in_ch * p, d)
        self.time_embedder = nn.Sequential(nn.Linear(cfg.freq_dim, d), nn.SiLU(), nn.Linear(d, d))
        self.time_proj = nn.Linear(d, 6 * d)
        self.text_embedder = nn.Sequential(nn.Linear(cfg.text_dim, d), nn.GELU(approximate="tanh"), nn.Linear(d, d))
        self.blocks = nn.ModuleList([WanBlock(cfg) for _ in range(cfg.layers)])
        self.proj_out = nn.Linear(d, cfg.out_ch * p)
        self.scale_shift_table = nn.Parameter(torch.randn(1, 2, d) * 0.02)
        self.backend = "fp16"

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        g = torch.Generator(device=self.proj_out.weight.device).manual_seed(seed)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=g, device=m.weight.device) * 0.02)
                m.bias.zero_()
        for name, prm in self.named_parameters():
            if name.endswith("scale_shift_table"):
                prm.copy_(torch.randn(prm.shape, generator=g, device=prm.device) * 0.02)

    # ---- W4A4 conversion --------------------------------------------------------------
    _QUANT_NAMES = ("to_q", "to_k", "to_v", "to_out")

    @torch.no_grad()
    def quantize_blocks(self, backend: str = "kernel", keep_oracle: bool = False):
        """Swap the 10 linears of every block for kernel-mode QuantLinears (and enable fused
        QKV / KV).  With keep_oracle=True also builds OracleW4A4Linear twins on the same codes,
        selectable with set_backend("oracle")."""
        from dsaquant_b200.kernels import vdm_w4a4 as vdm

        for blk in self.blocks:
            holders = [(blk.attn1, n) for n in self._QUANT_NAMES] + [(blk.attn2, n) for n in self._QUANT_NAMES] + \
                      [(blk, "ffn_up"), (blk, "ffn_down")]
            for owner, name in holders:
                ql = _quantize_linear(getattr(owner, name))
                setattr(owner, name, ql)
                if keep_oracle:
                    n, k = ql.out_features, ql.in_features
                    codes = vdm.unpack_codes(ql.vdm_weight_packed, n, k, 2)
                    setattr(owner, name + "_oracle", OracleW4A4Linear(ql, codes))
                    setattr(owner, name + "_kernel", ql)
            for attn in (blk.attn1, blk.attn2):
                attn.use_fused_qkv_kernel = True
                attn.qkv_kernel_backend = "vdm"
                # one copy of the fused projection's weights from the start (what enable_fused_qkv does
                # for a model loaded from a packed checkpoint)
                from dsaquant_b200.attention_qkv import prepare_fused_projections

                prepare_fused_projections(attn)
        self.set_backend(backend)

    def set_backend(self, backend: str):
        assert backend in ("kernel", "oracle")
        for blk in self.blocks:
            for owner, names in ((blk.attn1, self._QUANT_NAMES), (blk.attn2, self._QUANT_NAMES),
                                 (blk, ("ffn_up", "ffn_down"))):
                for name in names:
                    twin = getattr(owner, f"{name}_{backend}", None)
                    if twin is not None:
                        setattr(owner, name, twin)
            for attn in (blk.attn1, blk.attn2):
                attn.use_fused_qkv_kernel = backend == "kernel"
        self.backend = backend
        if backend != "kernel":
            self.set_fused(False)

    def set_fused(self, on: bool):
        """Fold norms / modulation / GELU / gated skips into the W4A4 calls (kernel back-end only)."""
        assert not on or self.backend == "kernel"
        for blk in self.blocks:
            blk.fused = bool(on)

    # ---- forward ------------------------------------------------------------------------
    def make_kv_exchange(self, group):
        """Exchange memory for row-sharded self-attention over `group` (one PeerKVExchange shared by
        all blocks): K and V travel by peer stores from the kernels that produce them instead of
        two all-gathers per block.  Collective: every rank of the group must call it."""
        from dsaquant_b200.peer_exchange import PeerKVExchange

        world, rank = dist.get_world_size(group), dist.get_rank(group)
        m_total = self.cfg.tokens
        parts = sharding.row_partition(m_total, world)
        cap = sharding.shard_capacity(m_total, world) * world
        ex = PeerKVExchange.from_symmetric_memory(group, cap, self.cfg.dim, parts[rank][0],
                                                  shard_rows=[e - s for s, e in parts])
        ex.senders = sum(1 for s, e in parts if e > s)
        return ex

    def set_kv_exchange(self, exchange, overlap: bool = False) -> None:
        """Route of the K/V exchange: a PeerKVExchange (fused kernel route only), or None for the
        NCCL all-gathers.  overlap=True places own rows first in the gather buffers and splits the
        attention into a local and a remote part so that the exchange hides behind the local part.
        Collective in effect: switch it on every rank of the group alike, between steps."""
        if exchange is not None:
            exchange.set_rotated(overlap)
        for blk in self.blocks:
            blk.attn1.kv_exchange = exchange
            blk.attn1.kv_senders = None if exchange is None else exchange.senders

    def enable_kv_push(self, group) -> None:
        self.set_kv_exchange(self.make_kv_exchange(group))

    def embed_time(self, timestep: torch.Tensor):
        half = self.cfg.freq_dim // 2
        freqs = torch.pow(10000, -torch.arange(half, dtype=torch.float64, device=timestep.device) / half)
        ang = torch.outer(timestep.double(), freqs)
        emb = torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(self.time_embedder[0].weight.dtype)
        temb = self.time_embedder(emb)
        return temb, self.time_proj(F.silu(temb)).unflatten(1, (6, -1))

    @torch.no_grad()
    def forward(self, latent: torch.Tensor, timestep: torch.Tensor, text: torch.Tensor,
                group=None) -> torch.Tensor:
        """latent [1,C,F,H,W], timestep [1], text [1,T,text_dim] -> noise prediction [1, L*4, out_ch]
        (the reference's packed output layout, model.py:346-352).  With `group` set the token
        rows are sharded over the ranks of that group and the result is gathered at the end."""
        cfg = self.cfg
        c1, c2, c3 = cfg.patch
        _, c, f, h, w = latent.shape
        fp, hp, wp = f // c1, h // c2, w // c3
        x = latent.reshape(1, c, fp, c1, hp, c2, wp, c3).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(1, fp * hp * wp, -1)
        m_total = x.shape[1]
        key = (fp, hp, wp, str(latent.device))
        if getattr(self, "_rope_key", None) != key:     # the table depends on the grid only: build it once
            self._rope_key, self._rope = key, rope_table(cfg.dim // cfg.heads, fp, hp, wp, latent.device)
        freqs = self._rope
        _mark("other")
        if group is not None:
            rank, world = dist.get_rank(group), dist.get_world_size(group)
            s, e = sharding.row_partition(m_total, world)[rank]
            x, freqs = x[:, s:e], freqs[s:e]
        x = self.patch_embedding_mlp(x.to(self.patch_embedding_mlp.weight.dtype))
        temb, temb6 = self.embed_time(timestep)
        ctx = self.text_embedder(text.to(x.dtype))
        for blk in self.blocks:
            x = blk(x, ctx, temb6, freqs, group, m_total)
        _mark("other")
        mod = self.scale_shift_table.float() + temb.float()[:, None]
        shift, scale = mod[:, 0][None], mod[:, 1][None]
        x = (fp32_layer_norm(x, cfg.eps) * (1 + scale) + shift).to(x.dtype)
        x = self.proj_out(x)
        if group is not None:
            x = sharding.all_gather_rows(x[0].contiguous(), m_total, group)[None]
        n = math.prod(cfg.patch)
        _mark("end")
        return x.reshape(1, m_total, n, -1).reshape(1, m_total * n, -1)


def build_model(cfg: WanConfig, device, seed: int = 0, backend: str = "kernel", keep_oracle: bool = False) -> WanDiT:
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device(device):
            model = WanDiT(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.init_weights(seed)
    model.quantize_blocks(backend, keep_oracle)
    for m in (model.time_embedder, model.time_proj):
        m.float()
    return model.eval()


def synth_inputs(cfg: WanConfig, device, seed: int = 0, negative: bool = False):
    g = torch.Generator(device=device).manual_seed(seed)
    latent = torch.randn((1,) + cfg.latent, generator=g, device=device).half()
    text = torch.randn((1, cfg.text_len, cfg.text_dim), generator=g, device=device).half()
    if negative:
        text = torch.randn((1, cfg.text_len, cfg.text_dim), generator=g, device=device).half()
    timestep = torch.rand(1, generator=g, device=device) * 1000.0
    return latent, timestep, text


@torch.no_grad()
def cfg_step(model: WanDiT, latent, timestep, text_cond, text_uncond, guidance: float = 5.0,
             branch_group=None, world_group=None, branch: Optional[int] = None) -> torch.Tensor:
    """One classifier-free-guidance denoising step: noise_uncond + s * (noise_cond - noise_uncond)
    (vdm_infer/models/wan_vdm/pipelines/text2video.py:576-609).  Single GPU: two sequential
    forwards.  Multi GPU: `branch` in {0,1} selects which forward this rank's group computes;
    the two predictions are exchanged with one all-gather over `world_group`."""
    if branch is None:
        cond = model(latent, timestep, text_cond)
        uncond = model(latent, timestep, text_uncond)
        return uncond + guidance * (cond - uncond)
    mine = model(latent, timestep, text_cond if branch == 0 else text_uncond, group=branch_group)
    world = dist.get_world_size(world_group)
    both = torch.empty((world,) + mine.shape, dtype=mine.dtype, device=mine.device)
    if mine.is_cuda:
        dist.all_gather_into_tensor(both, mine.contiguous(), group=world_group)
    else:  # CPU back-ends take the list form
        dist.all_gather(list(both.unbind(0)), mine.contiguous(), group=world_group)
    half = world // 2
    cond, uncond = both[0], both[half]
    return uncond + guidance * (cond - uncond)
