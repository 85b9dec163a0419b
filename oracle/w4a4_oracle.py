"""CPU oracle for the W4A4 linear-layer path (TEST INFRASTRUCTURE, not product code).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import
this module; the product path never does.  It restates, in numpy, the integer
semantics of the reference's own PyTorch W4A4 path:

  * activation quantiser: UniformQuantizer.init_qparams / quant, symmetric 4-bit
    (vdm_infer/quantization/quant_linear.py:43-48, :64-66), evaluated per token
    on a 2-D fp32 input, with the kernel path's clip ratio folded into the scale
    ((absmax/7)*clip, vdm_infer/kernels/csrc/vdm_w4a4_kernel.cu:478 and
    tests/test_vdm_w4a4_kernel_smoke.py:25);
  * weight codes: clamp(round(w / scale), -8, 7) (quant_linear.py:64-66;
    tests/test_vdm_w4a4_kernel_smoke.py:27);
  * exact integer accumulation and dequantisation
    (tests/test_vdm_w4a4_kernel_smoke.py:28; vdm_w4a4_kernel.cu:243-274);
  * the vdm_w4a4_packed_v1 byte layouts written by
    weight_quantize_per_channel_kernel / pack_wscales (vdm_w4a4_kernel.cu:518-551, :286-294).

Parity status: pinned.  tests/golden/make_golden.py runs the reference's own
QuantLinear / UniformQuantizer (imported from the reference tree) on seeded
inputs and stores its codes, scales, accumulators and outputs; tests/test_oracle.py
checks this module against those fixtures bit for bit.

All floating-point steps are IEEE fp32 with one rounding per operation.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
QMIN, QMAX = -8, 7


# --------------------------------------------------------------------------- quantisers
def act_scale(x: np.ndarray, clip: float = 1.0) -> np.ndarray:
    """Per-token scale s[m] = (max(absmax, 1e-5) / 7) * clip, fp32 [M]."""
    x = np.asarray(x, dtype=F32)
    amax = np.abs(x).max(axis=1) if x.shape[1] else np.zeros(x.shape[0], F32)
    s = np.maximum(amax.astype(F32), F32(1e-5)) / F32(7.0)
    return (s * F32(clip)).astype(F32)


def quantize_act(x: np.ndarray, clip: float = 1.0):
    """x [M,K] (values exactly representable in fp32) -> (codes int8 [M,K], scale fp32 [M])."""
    x = np.asarray(x, dtype=F32)
    s = act_scale(x, clip)
    q = np.rint(x / s[:, None])  # true division, ties to even
    return np.clip(q, QMIN, QMAX).astype(np.int8), s


def weight_scale_absmax(w: np.ndarray) -> np.ndarray:
    """Per-channel fp16 scale amax/7 (1 for an all-zero row), as quantize_weight_per_channel does
    (vdm_w4a4_kernel.cu:459-481 applied to weight rows with clip 1, :747)."""
    w = np.asarray(w, dtype=F32)
    amax = np.abs(w).max(axis=1).astype(F32)
    s = np.where(amax > 0, amax / F32(7.0), F32(1.0)).astype(F32)
    return s.astype(np.float16)


def quantize_weight(w: np.ndarray, ch_scale) -> np.ndarray:
    """w [N,K], per-channel scale [N] (stored as fp16 in the format) -> codes int8 [N,K]."""
    w = np.asarray(w, dtype=F32)
    s = np.asarray(ch_scale).reshape(-1).astype(np.float16).astype(F32)
    q = np.rint(w / s[:, None])
    return np.clip(q, QMIN, QMAX).astype(np.int8)


# --------------------------------------------------------------------------- GEMM + dequant
def int_gemm(qa: np.ndarray, qw: np.ndarray) -> np.ndarray:
    """acc[m,n] = sum_k qa[m,k]*qw[n,k], exact int32.

    Uses an fp32 BLAS matmul: every partial sum is an integer of magnitude
    <= 64*K < 2**24 for K < 262144, so fp32 arithmetic is exact."""
    K = qa.shape[1]
    assert qw.shape[1] == K and 64 * K < (1 << 24)
    acc = qa.astype(F32) @ qw.astype(F32).T
    return acc.astype(np.int32)


def dequant(acc: np.ndarray, a_scale: np.ndarray, w_scale, bias=None) -> np.ndarray:
    """fp16_rn( fl(fl(float(acc) * fl(sa*sw)) + bias) ): three fp32 roundings, then fp16."""
    sa = np.asarray(a_scale, dtype=F32).reshape(-1, 1)
    sw = np.asarray(w_scale).reshape(1, -1).astype(np.float16).astype(F32)
    prod = (sa * sw).astype(F32)
    v = (acc.astype(F32) * prod).astype(F32)
    if bias is not None:
        b = np.asarray(bias).reshape(1, -1).astype(np.float16).astype(F32)
        v = (v + b).astype(F32)
    return v.astype(np.float16)


def linear_w4a4(x, w_codes, w_scale, bias=None, clip: float = 1.0):
    """Full path. Returns dict(codes, a_scale, acc, out)."""
    qa, sa = quantize_act(x, clip)
    acc = int_gemm(qa, np.asarray(w_codes, dtype=np.int8))
    return {"codes": qa, "a_scale": sa, "acc": acc, "out": dequant(acc, sa, w_scale, bias)}


# --------------------------------------------------------------------------- nibble helpers
def _nib(codes: np.ndarray) -> np.ndarray:
    return (codes.astype(np.int16) & 0xF).astype(np.uint8)


def _sext(nib: np.ndarray) -> np.ndarray:
    return (((nib.astype(np.int16) ^ 8) - 8)).astype(np.int8)


def pack_nibble_rows(codes: np.ndarray) -> np.ndarray:
    """int8 [M,K] -> u8 [M,K/2]: element 2b low nibble, 2b+1 high nibble
    (the reference's nibble rule, vdm_w4a4_kernel.cu:95-102, :324-330)."""
    n = _nib(codes)
    return (n[:, 0::2] | (n[:, 1::2] << 4)).astype(np.uint8)


def unpack_nibble_rows(packed: np.ndarray) -> np.ndarray:
    M, K2 = packed.shape
    out = np.empty((M, 2 * K2), np.uint8)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = packed >> 4
    return _sext(out)


# --------------------------------------------------------------------------- vdm_w4a4_packed_v1
def _v1_word_index(n: np.ndarray, k8: np.ndarray, K: int) -> np.ndarray:
    """32-bit-word index, inside the flat v1 code tensor, of codes k8..k8+7 of row n."""
    bn, r = n >> 7, n & 127
    tile, rr = r >> 4, r & 15
    hi8, lrow = rr >> 3, rr & 7
    bk, kk = k8 >> 6, k8 & 63
    khalf, kq = kk >> 5, (kk & 31) >> 3
    lane = lrow * 4 + kq
    word = hi8 * 2 + khalf
    return ((((bn * (K >> 6) + bk) * 8 + tile) * 32 + lane) << 2) + word


def pack_weight_v1(codes: np.ndarray) -> np.ndarray:
    """int8 codes [N,K] -> vdm_weight_packed u8 [N,K/2] (flat 16-byte entries
    [n/128][k/64][tile][lane], words {row n0 k0.., row n0 k0+32.., row n0+8 k0.., row n0+8 k0+32..};
    vdm_w4a4_kernel.cu:518-551 with the y/z swap at :542-544)."""
    N, K = codes.shape
    assert N % 128 == 0 and K % 64 == 0
    nib = _nib(codes).astype(np.uint32).reshape(N, K // 8, 8)
    words = np.zeros((N, K // 8), np.uint32)
    for e in range(8):
        words |= nib[:, :, e] << np.uint32(4 * e)
    n_idx, k_idx = np.meshgrid(np.arange(N), np.arange(0, K, 8), indexing="ij")
    flat = np.empty(N * K // 8, np.uint32)
    flat[_v1_word_index(n_idx, k_idx, K).ravel()] = words.ravel()
    return flat.view(np.uint8).reshape(N, K // 2)


def unpack_weight_v1(packed: np.ndarray) -> np.ndarray:
    N, K2 = packed.shape
    K = 2 * K2
    flat = np.ascontiguousarray(packed).reshape(-1).view(np.uint32)
    n_idx, k_idx = np.meshgrid(np.arange(N), np.arange(0, K, 8), indexing="ij")
    words = flat[_v1_word_index(n_idx, k_idx, K)]
    out = np.empty((N, K // 8, 8), np.uint8)
    for e in range(8):
        out[:, :, e] = (words >> np.uint32(4 * e)) & 0xF
    return _sext(out.reshape(N, K))


def _v1_scale_index(n: np.ndarray, bk: np.ndarray, K: int) -> np.ndarray:
    bn, r = n >> 7, n & 127
    g, rr = r >> 4, r & 15
    hi, rrr = rr >> 3, rr & 7
    lane = g * 4 + (rrr >> 1)
    idx = hi * 2 + (rrr & 1)
    return (((bn * (K >> 6) + bk) * 32 + lane) << 2) + idx


def pack_wscale_v1(ch_scale, K: int) -> np.ndarray:
    """fp16 [N] -> vdm_weight_scale_packed fp16 [N,K/64]: flat [n/128][k/64][lane][4] where a
    lane's four halfs are channels (lane/4)*16 + (lane%4)*2 + {0,1,8,9}; every k-block repeats
    the channel scale (vdm_w4a4_kernel.cu:286-294, :548-550)."""
    s = np.asarray(ch_scale).reshape(-1).astype(np.float16)
    N = s.shape[0]
    n_idx, bk_idx = np.meshgrid(np.arange(N), np.arange(K // 64), indexing="ij")
    flat = np.empty(N * (K // 64), np.float16)
    flat[_v1_scale_index(n_idx, bk_idx, K).ravel()] = np.broadcast_to(s[:, None], n_idx.shape).ravel()
    return flat.reshape(N, K // 64)


def unpack_wscale_v1(scale_packed: np.ndarray) -> np.ndarray:
    N, KB = scale_packed.shape
    flat = np.ascontiguousarray(scale_packed).reshape(-1)
    return flat[_v1_scale_index(np.arange(N), np.zeros(N, np.int64), KB * 64)]


# --------------------------------------------------------------------------- B200 weight layout
def repack_b200(codes: np.ndarray) -> np.ndarray:
    """int8 codes [N,K] -> u8 [N,K/2] in the layout the tcgen05 GEMM stages: for every run of
    32 consecutive k (k32), output byte i (0..15) = code[k32+i] << 4 | code[k32+16+i] & 0xF."""
    N, K = codes.shape
    nib = _nib(codes).reshape(N, K // 32, 2, 16)
    return ((nib[:, :, 0, :] << 4) | nib[:, :, 1, :]).astype(np.uint8).reshape(N, K // 2)


def unpack_b200(wr: np.ndarray) -> np.ndarray:
    N, K2 = wr.shape
    b = wr.reshape(N, K2 // 16, 16)
    out = np.empty((N, K2 // 16, 2, 16), np.uint8)
    out[:, :, 0, :] = b >> 4
    out[:, :, 1, :] = b & 0xF
    return _sext(out.reshape(N, 2 * K2))
