"""GPU parity tests: the sm_100a kernels (through the C ABI / python wrappers) against the CPU
oracle and the reference-generated fixtures.  Integer results (codes, accumulators) and the fp16
outputs of the oracle's pinned rounding order must match bit for bit; against the reference's
fp32 fake-quant output the tolerance is 1e-2 relative / 5e-3 absolute per element."""
from pathlib import Path

import numpy as np
import pytest
import torch

from _cases import CASES, digest, make_case
from oracle import w4a4_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def vdm():
    from dsaquant_b200.kernels import vdm_w4a4 as v

    assert v.is_available(), f"libb200w4a4.so not loadable: {v.load_error()}"
    yield v
    assert v.last_device_status() == 0, "a kernel recorded a device-side time-out"


def _cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _v1_buffers(w16, ws16):
    qw = orc.quantize_weight(w16, ws16)
    return qw, _cuda(orc.pack_weight_v1(qw)), _cuda(orc.pack_wscale_v1(ws16, w16.shape[1]))


# ------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,K", [(1, 64), (15, 128), (257, 1536), (33, 3072), (40, 5120), (9, 8960),
                                 (5, 13824), (3, 16448)])
@pytest.mark.parametrize("clip", [1.0, 0.95, 0.5])   # 0.5: quotients beyond +-7.5, the clamping path
def test_quantize_act_codes_bit_exact(vdm, dtype, M, K, clip):
    x16, _, _ = make_case(100 + M + K, M, K, 128, bias=False)
    xt = _cuda(x16).to(dtype)                       # exact for fp32; bf16 rounds: oracle sees the same values
    x_ref = xt.float().cpu().numpy()
    q_ref, s_ref = orc.quantize_act(x_ref, clip)
    qact, ascales, act_h = vdm.quantize_activation_per_token(xt, clip)
    assert qact.shape == (M, K) and qact.dtype == torch.int8
    np.testing.assert_array_equal(ascales.cpu().numpy(), s_ref)
    np.testing.assert_array_equal(qact.cpu().numpy(), q_ref)
    np.testing.assert_array_equal(act_h.cpu().numpy(), s_ref.astype(np.float16))
    qn, s2 = vdm.quantize_activation_nibbles(xt, clip)
    np.testing.assert_array_equal(qn.cpu().numpy(), orc.pack_nibble_rows(q_ref))
    np.testing.assert_array_equal(vdm.unpack_codes(qn, M, K, 3).cpu().numpy(), q_ref)
    np.testing.assert_array_equal(s2.cpu().numpy(), s_ref)


def test_quantize_act_ties_zero_rows_and_saturation(vdm):
    K = 64
    x = np.zeros((4, K), np.float32)
    x[0, :12] = [7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 6.5, -5.5, -6.5, 3.49, -3.51]
    x[2, :3] = [-7.0, 7.0, 3.5]
    x[3, :] = 1e-7
    for clip in (1.0, 0.5):
        q, s, _ = vdm.quantize_activation_per_token(_cuda(x), clip)
        q_ref, s_ref = orc.quantize_act(x, clip)
        np.testing.assert_array_equal(q.cpu().numpy(), q_ref)
        np.testing.assert_array_equal(s.cpu().numpy(), s_ref)


# ------------------------------------------------------------------ weights
@pytest.mark.parametrize("N,K", [(128, 64), (256, 192), (384, 1536)])
def test_pack_weight_matches_v1_layout(vdm, N, K):
    _, w16, _ = make_case(3, 8, K, N, bias=False)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    packed, scale_packed, scale = vdm.pack_weight_with_scale(_cuda(w16), _cuda(ws))
    np.testing.assert_array_equal(packed.cpu().numpy(), orc.pack_weight_v1(qw))
    np.testing.assert_array_equal(scale_packed.cpu().numpy(), orc.pack_wscale_v1(ws, K))
    np.testing.assert_array_equal(scale.cpu().numpy(), ws)
    np.testing.assert_array_equal(vdm.unpack_codes(packed, N, K, 2).cpu().numpy(), qw)
    # absmax/7 scales computed on the device
    p2, sp2, s2 = vdm.quantize_weight_per_channel(_cuda(w16))
    np.testing.assert_array_equal(s2.cpu().numpy(), ws)
    np.testing.assert_array_equal(p2.cpu().numpy(), orc.pack_weight_v1(qw))
    # load-time repack
    w_b200, w_scale = vdm.prepare_b200_weight(packed, scale_packed)
    np.testing.assert_array_equal(w_b200.cpu().numpy(), orc.repack_b200(qw))
    np.testing.assert_array_equal(w_scale.cpu().numpy(), ws)
    np.testing.assert_array_equal(vdm.unpack_codes(w_b200, N, K, 1).cpu().numpy(), qw)


# ------------------------------------------------------------------ GEMM
def _gemm_case(vdm, M, K, N, seed, clip=1.0, bias=True):
    x16, w16, b16 = make_case(seed, M, K, N, bias=bias)
    ws = orc.weight_scale_absmax(w16)
    qw, packed, scale_packed = _v1_buffers(w16, ws)
    ref = orc.linear_w4a4(x16, qw, ws, b16, clip)
    xt = _cuda(x16)
    qact, ascales, _ = vdm.quantize_activation_per_token(xt, clip)
    out_nb, acc = vdm.linear_prequantized(qact, ascales, packed, scale_packed, return_acc=True)
    np.testing.assert_array_equal(acc.cpu().numpy(), ref["acc"])
    np.testing.assert_array_equal(out_nb.cpu().numpy().view(np.uint16),
                                  orc.dequant(ref["acc"], ref["a_scale"], ws, None).view(np.uint16))
    out = vdm.linear_vdm_w4a4(xt, packed, scale_packed, _cuda(b16) if bias else None, clip_ratio=clip)
    assert out.shape == (M, N) and out.dtype == torch.float16
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("M", [1, 15, 16, 127, 128, 129, 255, 256, 257, 700])
@pytest.mark.parametrize("K,N", [(64, 128), (128, 256), (192, 384), (1536, 128), (1536, 1536)])
def test_gemm_bit_exact_small_shapes(vdm, cta_group, M, K, N):
    prev = vdm.set_cta_group(cta_group)
    try:
        _gemm_case(vdm, M, K, N, seed=1000 + M + K + N, clip=0.95)
    finally:
        vdm.set_cta_group(prev)


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("name", list(CASES))
def test_linear_against_reference_fixtures(vdm, cta_group, name):
    seed, M, K, N, kw, clip = CASES[name]
    g = np.load(GOLD / f"{name}.npz")
    x16, w16, b16 = make_case(seed, M, K, N, **kw)
    assert str(g["input_digest"]) == digest(x16, w16, b16)
    ws = g["w_scale"]
    qw, packed, scale_packed = _v1_buffers(w16, ws)
    prev = vdm.set_cta_group(cta_group)
    try:
        xt = _cuda(x16)
        qact, ascales, _ = vdm.quantize_activation_per_token(xt, clip)
        _, acc = vdm.linear_prequantized(qact, ascales, packed, scale_packed, return_acc=True)
        out = vdm.linear_vdm_w4a4(xt, packed, scale_packed, _cuda(b16), clip_ratio=clip)
    finally:
        vdm.set_cta_group(prev)
    codes, acc, out = qact.cpu().numpy(), acc.cpu().numpy(), out.float().cpu().numpy()
    np.testing.assert_array_equal(ascales.cpu().numpy(), g["a_scale"])
    if "a_codes" in g.files:
        np.testing.assert_array_equal(codes, g["a_codes"])
        np.testing.assert_array_equal(acc, g["acc"])
        np.testing.assert_allclose(out, g["ref_out_f32"], rtol=1e-2, atol=5e-3)
    else:
        assert digest(codes) == str(g["a_codes_digest"])
        assert digest(acc) == str(g["acc_digest"])
        np.testing.assert_allclose(out[::61, ::53], g["ref_out_f32_sample"], rtol=1e-2, atol=5e-3)


def test_c_abi_rejects_bad_arguments_without_launching(vdm):
    """Error codes of the C ABI on a live device: nothing is launched, the status word stays clean."""
    from dsaquant_b200 import _lib

    lib = _lib.load()
    s = torch.cuda.current_stream().cuda_stream
    x = torch.zeros(64 * 128 + 8, dtype=torch.float16, device="cuda")
    q = torch.zeros(64 * 128 + 16, dtype=torch.int8, device="cuda")
    sc = torch.zeros(64, dtype=torch.float32, device="cuda")
    w = torch.zeros(128 * 64, dtype=torch.uint8, device="cuda")
    ws = torch.ones(128, dtype=torch.float16, device="cuda")
    out = torch.zeros(64 * 128, dtype=torch.float16, device="cuda")
    work = torch.zeros(lib.b200w4a4_linear_workspace_bytes(64, 128) + 256, dtype=torch.uint8, device="cuda")
    ok = lambda: lib.b200w4a4_quantize_act(x.data_ptr(), 0, q.data_ptr(), 0, sc.data_ptr(), 64, 128, 1.0, s)
    assert ok() == 0
    assert lib.b200w4a4_quantize_act(x.data_ptr(), 0, q.data_ptr(), 0, sc.data_ptr(), 64, 96, 1.0, s) == -2    # K % 64
    assert lib.b200w4a4_quantize_act(x.data_ptr(), 0, q.data_ptr(), 0, sc.data_ptr(), 0, 128, 1.0, s) == -2     # M < 1
    assert lib.b200w4a4_quantize_act(x.data_ptr(), 7, q.data_ptr(), 0, sc.data_ptr(), 64, 128, 1.0, s) == -1    # dtype enum
    assert lib.b200w4a4_quantize_act(x.data_ptr(), 0, q.data_ptr(), 5, sc.data_ptr(), 64, 128, 1.0, s) == -1    # container enum
    assert lib.b200w4a4_quantize_act(x.data_ptr(), 0, q.data_ptr(), 0, sc.data_ptr(), 64, 128, 0.0, s) == -1    # clip
    assert lib.b200w4a4_quantize_act(x.data_ptr() + 2, 0, q.data_ptr(), 0, sc.data_ptr(), 64, 128, 1.0, s) == -3  # alignment
    gemm = lambda n, k, o=out: lib.b200w4a4_gemm(q.data_ptr(), sc.data_ptr(), w.data_ptr(), ws.data_ptr(), None,
                                                 o.data_ptr(), None, 64, n, k, s)
    assert gemm(128, 128) == 0
    assert gemm(100, 128) == -2 and gemm(128, 100) == -2
    assert lib.b200w4a4_gemm(q.data_ptr() + 1, sc.data_ptr(), w.data_ptr(), ws.data_ptr(), None, out.data_ptr(),
                             None, 64, 128, 128, s) == -3
    lin = lambda wsp, nbytes: lib.b200w4a4_linear(x.data_ptr(), 0, w.data_ptr(), ws.data_ptr(), None, out.data_ptr(),
                                                  wsp, nbytes, 64, 128, 128, 1.0, s)
    assert lin(work.data_ptr(), work.numel()) == 0
    assert lin(work.data_ptr(), 16) == -6                       # workspace too small
    assert lin(work.data_ptr() + 16, work.numel() - 16) == -3   # workspace not 256-byte aligned
    assert lin(None, work.numel()) == -1
    assert lib.b200w4a4_gemm_fused(q.data_ptr(), sc.data_ptr(), w.data_ptr(), ws.data_ptr(), None, out.data_ptr(), 2,
                                   None, None, 0, 64, 128, 128, s) == -1   # gate_residual without operands
    assert lib.b200w4a4_gemm_fused(q.data_ptr(), sc.data_ptr(), w.data_ptr(), ws.data_ptr(), None, out.data_ptr(), 9,
                                   None, None, 0, 64, 128, 128, s) == -1
    assert lib.b200w4a4_quantize_act_fused(x.data_ptr(), 2, None, None, 0, 1e-6, q.data_ptr(), sc.data_ptr(), 64, 128,
                                           1.0, s) == -1
    assert lib.b200w4a4_unpack_codes(w.data_ptr(), q.data_ptr(), 100, 128, 2, s) == -2   # v1 needs rows % 128 == 0
    torch.cuda.synchronize()
    assert lib.b200w4a4_last_device_status(torch.cuda.current_device()) == 0


def test_random_shape_sweep_bit_exact(vdm):
    """Seeded sweep over ragged shapes: every M, K multiple of 64, N multiple of 128, clip, bias on/off,
    both GEMM variants; codes, accumulators and fp16 outputs must equal the oracle bit for bit."""
    rng = np.random.default_rng(2024)
    for i in range(36):
        M = int(rng.integers(1, 1500))
        K = 64 * int(rng.integers(1, 40))
        N = 128 * int(rng.integers(1, 9))
        clip = float(rng.choice([1.0, 0.95, 0.9, 0.5]))
        bias = bool(rng.integers(0, 2))
        prev = vdm.set_cta_group(1 + i % 2)
        try:
            _gemm_case(vdm, M, K, N, seed=3000 + i, clip=clip, bias=bias)
        finally:
            vdm.set_cta_group(prev)


def test_tensor_maps_are_reused_between_identical_launches(vdm):
    """Second launch with the same buffers finds all three TMA descriptors in the library's table."""
    x16, w16, _ = make_case(5, 300, 256, 256, bias=False)
    ws = orc.weight_scale_absmax(w16)
    qw, qweight, wscales = _v1_buffers(w16, ws)
    qact, ascales, _ = vdm.quantize_activation_per_token(_cuda(x16), 1.0)
    lib = __import__("dsaquant_b200")._lib.load()
    w_b200, w_scale = vdm.prepare_b200_weight(qweight, wscales)
    out = torch.empty(300, 256, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream

    def launch():
        rc = lib.b200w4a4_gemm(qact.data_ptr(), ascales.data_ptr(), w_b200.data_ptr(), w_scale.data_ptr(), None,
                               out.data_ptr(), None, 300, 256, 256, s)
        assert rc == 0

    launch()
    h0, m0 = vdm.map_cache_stats()
    first = out.clone()
    launch()
    h1, m1 = vdm.map_cache_stats()
    assert (h1 - h0, m1 - m0) == (3, 0)
    torch.cuda.synchronize()
    assert torch.equal(out, first)


def test_int8_staged_weights_give_identical_results(vdm):
    """B200W4A4_WEIGHT_STAGING=int8 / set_weight_staging(8): the load-time step writes int8 [N,K]
    (16 * code) and the GEMM stages it with TMA instead of widening packed tiles in shared memory.
    Codes, accumulators and outputs must be the ones of the default packed path, for both CTA groups,
    a ragged M and every epilogue input the plain call takes."""
    M, K, N = 777, 1536, 640
    x16, w16, b16 = make_case(31, M, K, N)
    ws = orc.weight_scale_absmax(w16)
    qw, qweight, wscales = _v1_buffers(w16, ws)
    ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)
    prev = vdm.set_weight_staging(8)
    try:
        w8, w_scale = vdm.prepare_b200_weight(qweight, wscales)
        assert tuple(w8.shape) == (N, K)
        np.testing.assert_array_equal(w8.view(torch.int8).cpu().numpy(), qw.astype(np.int16) * 16)
        np.testing.assert_array_equal(vdm.unpack_codes(w8, N, K, 1).cpu().numpy(), qw)
        for cg in (2, 1):
            old = vdm.set_cta_group(cg)
            try:
                out = vdm.linear_vdm_w4a4(_cuda(x16), qweight, wscales, _cuda(b16), 0.95)
                qact, ascales, _ = vdm.quantize_activation_per_token(_cuda(x16), 0.95)
                _, acc = vdm.linear_prequantized(qact, ascales, qweight, wscales, return_acc=True)
            finally:
                vdm.set_cta_group(old)
            np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))
            np.testing.assert_array_equal(acc.cpu().numpy(), ref["acc"])
    finally:
        vdm.set_weight_staging(prev)
    out4 = vdm.linear_vdm_w4a4(_cuda(x16), qweight, wscales, _cuda(b16), 0.95)   # back on the packed path
    np.testing.assert_array_equal(out4.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))
