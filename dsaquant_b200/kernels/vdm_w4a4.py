"""B200 (sm_100a) implementation of the DSAQuant W4A4 kernel wrapper.

Drop-in for the reference module vdm_infer/kernels/vdm_w4a4.py: same public
names, argument order, defaults and error types
(build_config / is_available / load_error :115-179, pack_weight_with_scale
:209-214, quantize_weight_per_channel :217-219, linear_vdm_w4a4 :222-244,
quantize_activation_per_token :247-250, linear_prequantized :253-256,
linear_vdm_w4a4_qkv :259-298).  The work is done by libb200w4a4.so through its
C ABI; there is no Triton, no other backend and no CPU fallback: without the
library (or without a compute-capability-10.0 device) every op raises.

Behavioural notes for callers of the reference module:

* `qweight` / `wscales` are still the vdm_w4a4_packed_v1 buffers
  (`vdm_weight_packed` [N,K/2] u8, `vdm_weight_scale_packed` [N,K/64] f16).  On
  first use each pair is repacked once into the layout the tcgen05 GEMM stages
  with TMA, plus the plain per-channel scale [N]; the result is cached per
  tensor object and dropped when the tensor is garbage collected.
* `x` is read as it is (fp16, bf16 or fp32) instead of through an fp16 copy
  (vdm_w4a4.py:182-184); for fp16 callers the result is the same.
* Activation scales stay fp32 end to end, and codes use true IEEE division, so
  codes and accumulators are bit-identical to the reference's PyTorch W4A4 path.
* `quantize_activation_per_token` / `linear_prequantized` keep their signatures
  but exchange this library's activation container: int8 codes [M,K] (one code
  per byte, no padding of M to 256) and fp32 scales [M].
"""
from __future__ import annotations

import ctypes
import os
import weakref
from pathlib import Path
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib
from ..csrc import build as _build

BLOCK_M = 256
BLOCK_N = 128
WARP_K = 64

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
QACT_INT8 = 0
QACT_NIBBLE = 1

_SM100_ALIASES = {
    "b200": "10.0a", "blackwell": "10.0a", "sm100": "10.0a", "sm100a": "10.0a",
    "sm_100": "10.0a", "sm_100a": "10.0a", "10.0": "10.0a", "10.0a": "10.0a",
}


# --------------------------------------------------------------------------- build / arch selection
def _configure_cuda_home() -> None:
    if os.environ.get("CUDA_HOME"):
        return
    if Path("/usr/local/cuda").exists():
        os.environ["CUDA_HOME"] = "/usr/local/cuda"


def _detect_arch_list() -> str:
    """Same precedence as the reference (TORCH_CUDA_ARCH_LIST, then VDM_W4A4_TARGET_ARCH alias,
    then the visible device), with the sm_100a aliases added and 10.0a as the fallback."""
    explicit = os.environ.get("TORCH_CUDA_ARCH_LIST")
    if explicit:
        return explicit
    target = os.environ.get("VDM_W4A4_TARGET_ARCH", "auto").strip().lower()
    if target in _SM100_ALIASES:
        return _SM100_ALIASES[target]
    if torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability()
        return "10.0a" if (major, minor) == (10, 0) else f"{major}.{minor}"
    return "10.0a"


def _arch_tag(arch_list: str) -> str:
    tags = []
    for token in arch_list.replace(";", " ").replace(",", " ").split():
        ptx = "+ptx" in token.lower()
        token = token.lower().replace("+ptx", "")
        if token.startswith("sm_"):
            tag = "sm" + token[3:]
        elif "." in token:
            major, minor = token.split(".", 1)
            tag = f"sm{major}{minor}"
        else:
            tag = token.replace("-", "_")
        tags.append(tag + ("ptx" if ptx else ""))
    return "_".join(tags) if tags else "sm100a"


def build_config() -> dict:
    _configure_cuda_home()
    arch_list = _detect_arch_list()
    tag = _arch_tag(arch_list)
    return {
        "cuda_home": os.environ.get("CUDA_HOME"),
        "torch_cuda": torch.version.cuda,
        "arch_list": arch_list,
        "arch_tag": tag,
        "build_dir": str(_build.lib_path().parent),
        "extension_name": os.environ.get("VDM_W4A4_EXT_NAME", _build.LIB_NAME),
    }


_EXT = None


def _load_ext():
    """The loaded library.  Arch selection and loading run once; later calls are a global read (the
    reference keeps its extension in a module-level singleton the same way, vdm_w4a4.py:19,130-133)."""
    global _EXT
    if _EXT is not None:
        return _EXT
    _EXT = _load_ext_once()
    return _EXT


def _load_ext_once():
    tag = _arch_tag(_detect_arch_list())
    if "sm100a" not in tag.split("_") and "sm100" not in tag.split("_"):
        raise RuntimeError(f"b200 W4A4 kernels target sm_100a only, selected arch is {tag!r}")
    _configure_cuda_home()
    return _lib.load()


def is_available() -> bool:
    try:
        _load_ext()
        return True
    except BaseException:
        return False


def load_error() -> Optional[BaseException]:
    return _lib.load_error()


# --------------------------------------------------------------------------- helpers
def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (the W4A4 path has no CPU fallback)")


def _as_2d_contiguous(x: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, ...]]:
    orig_shape = tuple(x.shape[:-1])
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype not in _DTYPE_CODE:
        x2 = x2.float()
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if x2.data_ptr() % 16 != 0:
        x2 = x2.clone()
    return x2, orig_shape


def _bias_f16(b: Optional[torch.Tensor], n: int) -> Optional[torch.Tensor]:
    """Bias as a contiguous, 16-byte aligned fp16 [N] vector (or None)."""
    if b is None:
        return None
    b = b.detach().reshape(-1)
    if b.dtype != torch.float16 or not b.is_contiguous() or b.data_ptr() % 16 != 0:
        b = b.half().contiguous().clone()
    if b.numel() != n:
        raise ValueError("bias must have N elements")
    return b


def _check_linear_shapes(x_2d: torch.Tensor, qweight: torch.Tensor, wscales: torch.Tensor) -> None:
    if x_2d.shape[1] % WARP_K != 0:
        raise ValueError(f"K={x_2d.shape[1]} must be a multiple of {WARP_K}")
    if qweight.shape[0] % BLOCK_N != 0:
        raise ValueError(f"N={qweight.shape[0]} must be a multiple of {BLOCK_N}")
    if qweight.shape[1] != x_2d.shape[1] // 2:
        raise ValueError("qweight shape must be [N, K/2]")
    if wscales.shape != (qweight.shape[0], x_2d.shape[1] // WARP_K):
        raise ValueError("wscales shape must be [N, K/64]")


class _DeviceGuard:
    """Makes `device` current for the duration of a call when it is not already."""

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


# --------------------------------------------------------------------------- weight side
def pack_weight_with_scale(weight: torch.Tensor, channel_scale: torch.Tensor):
    """fp weight [N,K] + caller-provided per-channel scale -> the three vdm_w4a4_packed_v1
    buffers (qweight u8 [N,K/2], packed_scales f16 [N,K/64], channel_scales f16 [N])."""
    lib = _load_ext()
    _require_cuda(weight, "weight")
    weight_h = weight.detach().half().contiguous()
    scale_h = channel_scale.detach().reshape(-1).half().contiguous().to(weight_h.device)
    return _pack(lib, weight_h, scale_h)


def quantize_weight_per_channel(weight: torch.Tensor):
    lib = _load_ext()
    _require_cuda(weight, "weight")
    return _pack(lib, weight.detach().half().contiguous(), None)


def _pack(lib, weight_h: torch.Tensor, scale_h: Optional[torch.Tensor]):
    if weight_h.dim() != 2:
        raise RuntimeError("weight must be [N, K]")
    n, k = weight_h.shape
    if scale_h is not None and scale_h.numel() != n:
        raise RuntimeError("channel_scale must have N elements")
    dev = weight_h.device
    qweight = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
    packed_scales = torch.empty((n, max(k // 64, 1)), dtype=torch.float16, device=dev)
    channel_scales = torch.empty((n,), dtype=torch.float16, device=dev)
    with _DeviceGuard(dev):
        rc = lib.b200w4a4_pack_weight(
            weight_h.data_ptr(), scale_h.data_ptr() if scale_h is not None else None,
            qweight.data_ptr(), packed_scales.data_ptr(), channel_scales.data_ptr(), n, k,
            _stream_ptr(dev))
    _lib.check(rc, "pack_weight")
    return qweight, packed_scales, channel_scales


_PREPARED: dict = {}

# Optional profiling hook: when set, it is called with "quant" right before an activation
# quantiser is enqueued and with "gemm" right before a GEMM (a benchmark records CUDA events
# there).  None in normal use: the calls below then cost one comparison.
_PHASE_HOOK = None


def set_phase_hook(fn) -> None:
    global _PHASE_HOOK
    _PHASE_HOOK = fn


def _version_of(t: torch.Tensor) -> int:
    try:
        return t._version
    except RuntimeError:  # inference tensors carry no version counter
        return -1


def prepare_b200_weight(qweight: torch.Tensor, wscales: torch.Tensor):
    """Load-time repack of one layer: (vdm_weight_packed, vdm_weight_scale_packed) ->
    (w_b200 u8 [N,K/2] in the TMA/tcgen05 staging layout, plain scale f16 [N]).  Cached."""
    lib = _load_ext()
    staging = _weight_staging(lib)
    key = (qweight.data_ptr(), _version_of(qweight), tuple(qweight.shape), qweight.device.index,
           wscales.data_ptr(), _version_of(wscales), staging)
    hit = _PREPARED.get(key)
    if hit is not None:
        return hit
    _require_cuda(qweight, "qweight")
    n, k2 = qweight.shape
    k = 2 * k2
    if qweight.dtype != torch.uint8 or wscales.dtype != torch.float16:
        raise RuntimeError("qweight must be uint8 and wscales float16")
    qw = qweight if qweight.is_contiguous() else qweight.contiguous()
    ws = wscales if wscales.is_contiguous() else wscales.contiguous()
    dev = qweight.device
    w_b200 = torch.empty((n, lib.b200w4a4_repack_bytes(n, k) // n), dtype=torch.uint8, device=dev)
    w_scale = torch.empty((n,), dtype=torch.float16, device=dev)
    with _DeviceGuard(dev):
        rc = lib.b200w4a4_repack_weight(qw.data_ptr(), w_b200.data_ptr(), ws.data_ptr(),
                                        w_scale.data_ptr(), n, k, _stream_ptr(dev))
    _lib.check(rc, "repack_weight")
    _PREPARED[key] = (w_b200, w_scale)
    weakref.finalize(qweight, _PREPARED.pop, key, None)
    return w_b200, w_scale


_STAGING = None


def _weight_staging(lib) -> int:
    global _STAGING
    if _STAGING is None:
        _STAGING = lib.b200w4a4_set_weight_staging(0)   # 0: query only
    return _STAGING


def set_weight_staging(bits: int) -> int:
    """How the GEMM stages weights: 4 = packed int4 in HBM, widened to int8 in shared memory (default);
    8 = int8 in HBM (twice the weight bytes, no widening work in the GEMM).  Process-wide; weights
    repacked under the other setting are repacked again on their next use.  Returns the previous value."""
    global _STAGING
    rc = _load_ext().b200w4a4_set_weight_staging(int(bits))
    if rc < 0:
        _lib.check(rc, "set_weight_staging")
    _STAGING = int(bits)
    return rc


def release_b200_weight(qweight: torch.Tensor) -> int:
    """Drops the cached repack of `qweight` (e.g. a layer that from now on is only evaluated as
    part of a fused projection).  Returns the number of entries released; a later call with the
    same tensor simply repacks again."""
    ptr, dev = qweight.data_ptr(), qweight.device.index
    dead = [k for k in _PREPARED if k[0] == ptr and k[3] == dev]
    for k in dead:
        _PREPARED.pop(k, None)
    return len(dead)


# --------------------------------------------------------------------------- forward ops
def _workspace_bytes(m: int, k: int) -> int:
    """b200w4a4_linear_workspace_bytes(m, k) without the foreign call: codes and scales, each rounded
    up to 256 bytes (checked against the library in tests/test_host.py)."""
    return ((m * k + 255) & ~255) + ((m * 4 + 255) & ~255)


def _linear_prepared(x_2d: torch.Tensor, w_b200: torch.Tensor, w_scale: torch.Tensor,
                     bias_h: Optional[torch.Tensor], clip_ratio: float) -> torch.Tensor:
    lib = _load_ext()
    m, k = x_2d.shape
    n = w_b200.shape[0]
    dev = x_2d.device
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    if m == 0:
        return out
    ws_bytes = _workspace_bytes(m, k)
    workspace = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
    with _DeviceGuard(dev):
        rc = lib.b200w4a4_linear(
            x_2d.data_ptr(), _DTYPE_CODE[x_2d.dtype], w_b200.data_ptr(), w_scale.data_ptr(),
            bias_h.data_ptr() if bias_h is not None else None, out.data_ptr(),
            workspace.data_ptr(), ws_bytes, m, n, k, float(clip_ratio), _stream_ptr(dev))
    _lib.check(rc, "linear")
    return out


def linear_vdm_w4a4(
    x: torch.Tensor,
    qweight: torch.Tensor,
    wscales: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    clip_ratio: float = 1.0,
    bias_half: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    _load_ext()
    _require_cuda(x, "x")
    x_2d, orig_shape = _as_2d_contiguous(x)
    _check_linear_shapes(x_2d, qweight, wscales)
    w_b200, w_scale = prepare_b200_weight(qweight, wscales)
    b = _bias_f16(bias_half if bias_half is not None else bias, qweight.shape[0])
    out = _linear_prepared(x_2d, w_b200, w_scale, b, clip_ratio)
    return out.view(*orig_shape, -1)


def quantize_activation_per_token(x: torch.Tensor, clip_ratio: float = 1.0):
    """Returns (qact int8 [M,K], ascales fp32 [M], act_scales fp16 [M]).

    `ascales` are the exact scales the GEMM uses; `act_scales` is their fp16 rounding, kept
    for signature compatibility with the reference (which returns fp16 scales)."""
    lib = _load_ext()
    _require_cuda(x, "x")
    x_2d, _ = _as_2d_contiguous(x)
    m, k = x_2d.shape
    if k % WARP_K != 0:
        raise ValueError(f"K={k} must be a multiple of {WARP_K}")
    dev = x_2d.device
    qact = torch.empty((m, k), dtype=torch.int8, device=dev)
    ascales = torch.empty((m,), dtype=torch.float32, device=dev)
    if m > 0:
        with _DeviceGuard(dev):
            rc = lib.b200w4a4_quantize_act(x_2d.data_ptr(), _DTYPE_CODE[x_2d.dtype],
                                           qact.data_ptr(), QACT_INT8, ascales.data_ptr(), m, k,
                                           float(clip_ratio), _stream_ptr(dev))
        _lib.check(rc, "quantize_act")
    return qact, ascales, ascales.half()


def quantize_activation_nibbles(x: torch.Tensor, clip_ratio: float = 1.0):
    """Same quantiser, packed container: (u8 [M,K/2] with code 2b in the low and 2b+1 in the
    high nibble, fp32 scales [M])."""
    lib = _load_ext()
    _require_cuda(x, "x")
    x_2d, _ = _as_2d_contiguous(x)
    m, k = x_2d.shape
    if k % WARP_K != 0:
        raise ValueError(f"K={k} must be a multiple of {WARP_K}")
    dev = x_2d.device
    qact = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    ascales = torch.empty((m,), dtype=torch.float32, device=dev)
    if m > 0:
        with _DeviceGuard(dev):
            rc = lib.b200w4a4_quantize_act(x_2d.data_ptr(), _DTYPE_CODE[x_2d.dtype],
                                           qact.data_ptr(), QACT_NIBBLE, ascales.data_ptr(), m, k,
                                           float(clip_ratio), _stream_ptr(dev))
        _lib.check(rc, "quantize_act")
    return qact, ascales


def linear_prequantized(qact: torch.Tensor, ascales: torch.Tensor, qweight: torch.Tensor,
                        wscales: torch.Tensor, *, return_acc: bool = False):
    """GEMM only, no bias: qact int8 [M,K] and fp32 ascales [M] as returned by
    quantize_activation_per_token.  With return_acc=True also returns the int32 accumulators."""
    lib = _load_ext()
    _require_cuda(qact, "qact")
    if qact.dtype != torch.int8 or ascales.dtype != torch.float32:
        raise RuntimeError("qact must be int8 [M,K] and ascales float32 [M]")
    qact = qact.contiguous()
    ascales = ascales.contiguous()
    _check_linear_shapes(qact, qweight, wscales)
    w_b200, w_scale = prepare_b200_weight(qweight, wscales)
    m, k = qact.shape
    n = qweight.shape[0]
    dev = qact.device
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    acc = torch.empty((m, n), dtype=torch.int32, device=dev) if return_acc else None
    if m > 0:
        with _DeviceGuard(dev):
            rc = lib.b200w4a4_gemm(qact.data_ptr(), ascales.data_ptr(), w_b200.data_ptr(),
                                   w_scale.data_ptr(), None, out.data_ptr(),
                                   acc.data_ptr() if acc is not None else None, m, n, k,
                                   _stream_ptr(dev))
        _lib.check(rc, "gemm")
    return (out, acc) if return_acc else out


def linear_vdm_w4a4_qkv(
    x: torch.Tensor,
    q_weight_packed: torch.Tensor,
    q_weight_scale: torch.Tensor,
    k_weight_packed: torch.Tensor,
    k_weight_scale: torch.Tensor,
    v_weight_packed: torch.Tensor,
    v_weight_scale: torch.Tensor,
    q_bias: Optional[torch.Tensor] = None,
    k_bias: Optional[torch.Tensor] = None,
    v_bias: Optional[torch.Tensor] = None,
    clip_ratio: float = 1.0,
    w_qkv_packed: Optional[torch.Tensor] = None,
    w_qkv_scale: Optional[torch.Tensor] = None,
    qkv_bias_half: Optional[torch.Tensor] = None,
    contiguous_outputs: bool = False,
):
    """One activation quantisation and one GEMM with N = 3*D; returns three views split along
    the last dimension (contiguous_outputs=True: three contiguous tensors written by the GEMM
    itself, same values).  Concatenating v1 buffers along dim 0 is valid because one 128-channel
    block of the v1 layout is exactly 128 rows of the [N,K/2] view."""
    if w_qkv_packed is None or w_qkv_scale is None:
        w_qkv_packed = torch.cat([q_weight_packed, k_weight_packed, v_weight_packed], dim=0).contiguous()
        w_qkv_scale = torch.cat([q_weight_scale, k_weight_scale, v_weight_scale], dim=0).contiguous()
    n = q_weight_packed.shape[0]
    if qkv_bias_half is None and (q_bias is not None or k_bias is not None or v_bias is not None):
        device = w_qkv_packed.device

        def _b(b):
            return b.half().contiguous() if b is not None else torch.zeros(n, dtype=torch.float16, device=device)

        qkv_bias_half = torch.cat([_b(q_bias), _b(k_bias), _b(v_bias)], dim=0)
    if contiguous_outputs and n % 64 == 0:
        return linear_vdm_w4a4_split(x, w_qkv_packed, w_qkv_scale, 3, qkv_bias_half, clip_ratio)
    qkv = linear_vdm_w4a4(x, w_qkv_packed, w_qkv_scale, bias=None, clip_ratio=clip_ratio,
                          bias_half=qkv_bias_half)
    return qkv.split(n, dim=-1)


# --------------------------------------------------------------------------- test / debug helpers
def unpack_codes(packed: torch.Tensor, rows: int, k: int, which: int) -> torch.Tensor:
    """int8 codes [rows,k] of a packed buffer: which = 1 repacked weight, 2 v1 weight, 3 nibble rows."""
    lib = _load_ext()
    _require_cuda(packed, "packed")
    codes = torch.empty((rows, k), dtype=torch.int8, device=packed.device)
    with _DeviceGuard(packed.device):
        rc = lib.b200w4a4_unpack_codes(packed.contiguous().data_ptr(), codes.data_ptr(), rows, k,
                                       which, _stream_ptr(packed.device))
    _lib.check(rc, "unpack_codes")
    return codes


def set_cta_group(cta_group: int) -> int:
    """Selects the GEMM variant (1: one CTA per 128x256 tile, 2: CTA pair per 256x256 tile)."""
    rc = _load_ext().b200w4a4_set_cta_group(int(cta_group))
    if rc < 0:
        _lib.check(rc, "set_cta_group")
    return rc


def last_device_status(device: Optional[int] = None) -> int:
    """Synchronises the device and returns (and clears) the kernels' time-out status word."""
    idx = torch.cuda.current_device() if device is None else int(device)
    return _load_ext().b200w4a4_last_device_status(idx)


def check_device(device: Optional[int] = None) -> None:
    """Synchronises the device and raises B200W4A4Error (code B200W4A4_EDEVICE) if a kernel has
    recorded a time-out since the status word was last cleared; the word is left in place."""
    idx = torch.cuda.current_device() if device is None else int(device)
    _lib.check(_load_ext().b200w4a4_check_device(idx), "check_device")


def map_cache_stats() -> Tuple[int, int]:
    """(hits, misses) of the library's tensor-map table since it was loaded."""
    h, m = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
    _load_ext().b200w4a4_map_cache_stats(ctypes.byref(h), ctypes.byref(m))
    return int(h.value), int(m.value)


# --------------------------------------------------------------------------- fused variants
_PROLOGUES = {None: 0, "none": 0, "gelu_tanh": 1, "layernorm_mod": 2}
_EPILOGUES = {None: 0, "none": 0, "gelu_tanh": 1, "gate_residual": 2}


def _f32_vec(t: torch.Tensor, width: int, rows: int, name: str):
    """fp32 [width] (stride 0) or [rows, width] (stride = width), contiguous and 16-byte aligned."""
    t = t.detach()
    if t.dtype != torch.float32:
        t = t.float()
    t = t.reshape(-1, width) if t.numel() != width else t.reshape(1, width)
    if t.shape[0] not in (1, rows):
        raise ValueError(f"{name} must have {width} or {rows}x{width} elements")
    t = t.contiguous()
    if t.data_ptr() % 16 != 0:
        t = t.clone()
    return t, (0 if t.shape[0] == 1 else width)


def linear_vdm_w4a4_fused(
    x: torch.Tensor,
    qweight: torch.Tensor,
    wscales: torch.Tensor,
    bias_half: Optional[torch.Tensor] = None,
    clip_ratio: float = 1.0,
    *,
    prologue: Optional[str] = None,
    mod_scale: Optional[torch.Tensor] = None,
    mod_shift: Optional[torch.Tensor] = None,
    ln_eps: float = 1e-6,
    epilogue: Optional[str] = None,
    residual: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """linear_vdm_w4a4 with the surrounding elementwise work of a DiT block folded in.

    prologue  "layernorm_mod": x <- fp16(fp16(layer_norm(x)) * (1 + mod_scale) + mod_shift)
              "gelu_tanh":     x <- fp16(gelu_tanh(x))
    epilogue  "gelu_tanh":     y <- fp16(gelu_tanh(y))
              "gate_residual": y <- fp16(residual.float() + y.float() * gate)
    (the reference runs these as separate PyTorch ops around QuantLinear,
    vdm_infer/models/wan_vdm/modules/dit_block.py:103-115).  x must be fp16 when a prologue is
    used; without one it may also be bf16 or fp32 (quantised from its exact values)."""
    lib = _load_ext()
    _require_cuda(x, "x")
    if prologue not in _PROLOGUES or epilogue not in _EPILOGUES:
        raise ValueError("unknown prologue / epilogue")
    pre, epi = _PROLOGUES[prologue], _EPILOGUES[epilogue]
    if x.dtype != torch.float16 and pre != 0:
        raise RuntimeError("the fused prologues take fp16 activations")
    x_2d, orig_shape = _as_2d_contiguous(x)
    _check_linear_shapes(x_2d, qweight, wscales)
    w_b200, w_scale = prepare_b200_weight(qweight, wscales)
    m, k = x_2d.shape
    n = qweight.shape[0]
    dev = x_2d.device
    ms = mh = None
    m_stride = 0
    if pre == 2:
        if mod_scale is None or mod_shift is None:
            raise ValueError("layernorm_mod needs mod_scale and mod_shift")
        ms, m_stride = _f32_vec(mod_scale, k, m, "mod_scale")
        mh, h_stride = _f32_vec(mod_shift, k, m, "mod_shift")
        if h_stride != m_stride:
            raise ValueError("mod_scale and mod_shift must have the same shape")
    res = gt = None
    g_stride = 0
    if epi == 2:
        if residual is None or gate is None:
            raise ValueError("gate_residual needs residual and gate")
        res = residual.reshape(-1, n)
        if res.dtype != torch.float16 or res.shape[0] != m or not res.is_contiguous():
            raise ValueError("residual must be a contiguous fp16 [M, N] tensor")
        gt, g_stride = _f32_vec(gate, n, m, "gate")
    b = _bias_f16(bias_half, n)
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    if m == 0:
        return out.view(*orig_shape, n)
    hook = _PHASE_HOOK
    if x_2d.dtype != torch.float16 or hook is not None:
        # bf16 / fp32 activations (e.g. the attention output) are quantised from their exact
        # values, then the GEMM with the fused epilogue runs: two library calls.  A profiling
        # hook takes the same route so that it can put a mark between the two kernels.
        qact = torch.empty((m, k), dtype=torch.int8, device=dev)
        act_scale = torch.empty((m,), dtype=torch.float32, device=dev)
        with _DeviceGuard(dev):
            stream = _stream_ptr(dev)
            if hook is not None:
                hook("quant")
            if pre == 0:
                rc = lib.b200w4a4_quantize_act(x_2d.data_ptr(), _DTYPE_CODE[x_2d.dtype], qact.data_ptr(), 0,
                                               act_scale.data_ptr(), m, k, float(clip_ratio), stream)
            else:
                rc = lib.b200w4a4_quantize_act_fused(
                    x_2d.data_ptr(), pre, ms.data_ptr() if ms is not None else None,
                    mh.data_ptr() if mh is not None else None, m_stride, float(ln_eps), qact.data_ptr(),
                    act_scale.data_ptr(), m, k, float(clip_ratio), stream)
            _lib.check(rc, "quantize_act")
            if hook is not None:
                hook("gemm")
            rc = lib.b200w4a4_gemm_fused(
                qact.data_ptr(), act_scale.data_ptr(), w_b200.data_ptr(), w_scale.data_ptr(),
                b.data_ptr() if b is not None else None, out.data_ptr(), epi,
                res.data_ptr() if res is not None else None,
                gt.data_ptr() if gt is not None else None, g_stride, m, n, k, stream)
        _lib.check(rc, "gemm_fused")
        return out.view(*orig_shape, n)
    ws_bytes = _workspace_bytes(m, k)
    workspace = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
    with _DeviceGuard(dev):
        rc = lib.b200w4a4_linear_fused(
            x_2d.data_ptr(), pre, ms.data_ptr() if ms is not None else None,
            mh.data_ptr() if mh is not None else None, m_stride, float(ln_eps),
            w_b200.data_ptr(), w_scale.data_ptr(), b.data_ptr() if b is not None else None,
            out.data_ptr(), epi, res.data_ptr() if res is not None else None,
            gt.data_ptr() if gt is not None else None, g_stride, workspace.data_ptr(), ws_bytes,
            m, n, k, float(clip_ratio), _stream_ptr(dev))
    _lib.check(rc, "linear_fused")
    return out.view(*orig_shape, n)


def linear_vdm_w4a4_split(
    x: torch.Tensor,
    qweight: torch.Tensor,
    wscales: torch.Tensor,
    segments: int,
    bias_half: Optional[torch.Tensor] = None,
    clip_ratio: float = 1.0,
    *,
    prologue: Optional[str] = None,
    mod_scale: Optional[torch.Tensor] = None,
    mod_shift: Optional[torch.Tensor] = None,
    ln_eps: float = 1e-6,
    outs: Optional[Sequence[torch.Tensor]] = None,
):
    """Fused QKV / KV projection whose GEMM writes each of the `segments` equal column groups as
    its own [M, N/segments] fp16 matrix (the reference returns strided views of one [M,N] matrix,
    vdm_w4a4.py:297-298).  `outs`, when given, are the destinations: 2-D fp16 tensors of that shape
    whose rows may be strided (e.g. this rank's rows of an all-gather buffer); otherwise new
    contiguous tensors are returned.  Values are those of linear_vdm_w4a4(...).split(...).
    x must be fp16 when a prologue is used."""
    lib = _load_ext()
    _require_cuda(x, "x")
    if prologue not in _PROLOGUES:
        raise ValueError("unknown prologue")
    x_2d, orig_shape = _as_2d_contiguous(x)
    _check_linear_shapes(x_2d, qweight, wscales)
    w_b200, w_scale = prepare_b200_weight(qweight, wscales)
    m, k = x_2d.shape
    n = qweight.shape[0]
    if segments not in (1, 2, 3) or n % segments or (n // segments) % 64:
        raise ValueError("segments must be 1..3 and N / segments a multiple of 64")
    seg = n // segments
    dev = x_2d.device
    pre = _PROLOGUES[prologue]
    if pre != 0 and x_2d.dtype != torch.float16:
        raise RuntimeError("the fused prologues take fp16 activations")
    ms = mh = None
    m_stride = 0
    if pre == 2:
        if mod_scale is None or mod_shift is None:
            raise ValueError("layernorm_mod needs mod_scale and mod_shift")
        ms, m_stride = _f32_vec(mod_scale, k, m, "mod_scale")
        mh, h_stride = _f32_vec(mod_shift, k, m, "mod_shift")
        if h_stride != m_stride:
            raise ValueError("mod_scale and mod_shift must have the same shape")
    b = _bias_f16(bias_half, n)
    own = outs is None
    if own:
        outs = [torch.empty((m, seg), dtype=torch.float16, device=dev) for _ in range(segments)]
    else:
        if len(outs) != segments:
            raise ValueError("one destination per segment")
        for o in outs:
            if (o.dtype != torch.float16 or o.dim() != 2 or tuple(o.shape) != (m, seg) or o.device != dev
                    or (m > 0 and o.stride(1) != 1) or (m > 1 and o.stride(0) < seg)):
                raise ValueError("each destination must be a fp16 [M, N/segments] tensor with unit column stride")
    if m == 0:
        return tuple(o.view(*orig_shape, seg) for o in outs) if own else tuple(outs)
    qact = torch.empty((m, k), dtype=torch.int8, device=dev)
    act_scale = torch.empty((m,), dtype=torch.float32, device=dev)
    ptrs = (ctypes.c_void_p * segments)(*[o.data_ptr() for o in outs])
    lds = (ctypes.c_longlong * segments)(*[(o.stride(0) if m > 1 else seg) for o in outs])
    with _DeviceGuard(dev):
        stream = _stream_ptr(dev)
        hook = _PHASE_HOOK
        if hook is not None:
            hook("quant")
        if pre == 0:
            rc = lib.b200w4a4_quantize_act(x_2d.data_ptr(), _DTYPE_CODE[x_2d.dtype], qact.data_ptr(), 0,
                                           act_scale.data_ptr(), m, k, float(clip_ratio), stream)
        else:
            rc = lib.b200w4a4_quantize_act_fused(
                x_2d.data_ptr(), pre, ms.data_ptr() if ms is not None else None,
                mh.data_ptr() if mh is not None else None, m_stride, float(ln_eps), qact.data_ptr(),
                act_scale.data_ptr(), m, k, float(clip_ratio), stream)
        _lib.check(rc, "quantize_act")
        if hook is not None:
            hook("gemm")
        rc = lib.b200w4a4_gemm_split(qact.data_ptr(), act_scale.data_ptr(), w_b200.data_ptr(),
                                     w_scale.data_ptr(), b.data_ptr() if b is not None else None,
                                     ptrs, lds, segments, m, n, k, stream)
    _lib.check(rc, "gemm_split")
    return tuple(o.view(*orig_shape, seg) for o in outs) if own else tuple(outs)
