"""Fused prologues / epilogues of the W4A4 linear against the same work done as separate PyTorch
ops around the plain kernel (what the reference's DiT block does, dit_block.py:103-115).
gate_residual is elementwise with a pinned rounding order: bit-exact.  layernorm_mod and gelu_tanh
contain reductions / transcendental calls whose last fp32 bit differs from PyTorch's kernels, so
their fp16 intermediates may differ by one ulp in rare elements: checked by tolerance."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from _cases import make_case
from oracle import w4a4_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vdm():
    from dsaquant_b200.kernels import vdm_w4a4 as v

    assert v.is_available(), v.load_error()
    yield v
    assert v.last_device_status() == 0


def _layer(vdm, K, N, seed):
    _, w16, b16 = make_case(seed, 8, K, N)
    packed, scale_packed, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w16).cuda())
    return packed, scale_packed, torch.from_numpy(b16).cuda()


@pytest.mark.parametrize("M,K,N", [(300, 1536, 1536), (1000, 5120, 384), (77, 256, 128)])
@pytest.mark.parametrize("per_token", [False, True])
def test_gate_residual_epilogue_bit_exact(vdm, M, K, N, per_token):
    packed, sp, bias = _layer(vdm, K, N, 50)
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, generator=g, device="cuda").half()
    res = torch.randn(M, N, generator=g, device="cuda").half()
    gate = torch.randn((M, N) if per_token else (N,), generator=g, device="cuda")
    y = vdm.linear_vdm_w4a4(x, packed, sp, None, 0.95, bias_half=bias)
    want = (res.float() + y.float() * gate).half()
    got = vdm.linear_vdm_w4a4_fused(x, packed, sp, bias, 0.95, epilogue="gate_residual", residual=res, gate=gate)
    assert torch.equal(got, want)


@pytest.mark.parametrize("M,K,N", [(300, 1536, 8960), (129, 256, 256)])
def test_gelu_epilogue_and_prologue(vdm, M, K, N):
    packed, sp, bias = _layer(vdm, K, N, 51)
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, generator=g, device="cuda").half()
    y = vdm.linear_vdm_w4a4(x, packed, sp, None, 0.95, bias_half=bias)
    want = F.gelu(y, approximate="tanh")
    got = vdm.linear_vdm_w4a4_fused(x, packed, sp, bias, 0.95, epilogue="gelu_tanh")
    diff = (got.float() - want.float()).abs()
    assert (got != want).float().mean().item() < 1e-3            # at most a stray 1-ulp difference
    assert diff.max().item() <= 2e-3 * max(1.0, want.abs().max().item())
    # prologue form: quantise gelu(h) without materialising it
    packed2, sp2, bias2 = _layer(vdm, N, 256, 52)
    h = y
    want2 = vdm.linear_vdm_w4a4(F.gelu(h, approximate="tanh"), packed2, sp2, None, 0.95, bias_half=bias2)
    got2 = vdm.linear_vdm_w4a4_fused(h, packed2, sp2, bias2, 0.95, prologue="gelu_tanh")
    rel = torch.linalg.vector_norm(got2.float() - want2.float()) / torch.linalg.vector_norm(want2.float())
    assert rel.item() < 5e-3


@pytest.mark.parametrize("M,K,N", [(300, 1536, 1536), (200, 5120, 256), (64, 13824, 128)])
@pytest.mark.parametrize("per_token", [False, True])
def test_layernorm_mod_prologue(vdm, M, K, N, per_token):
    packed, sp, bias = _layer(vdm, K, N, 53)
    g = torch.Generator(device="cuda").manual_seed(K)
    x = (torch.randn(M, K, generator=g, device="cuda") * 3 + 0.5).half()
    scale = torch.randn((M, K) if per_token else (K,), generator=g, device="cuda") * 0.1
    shift = torch.randn((M, K) if per_token else (K,), generator=g, device="cuda") * 0.1
    ln = F.layer_norm(x.float(), (K,), None, None, 1e-6).half()              # FP32LayerNorm, cast back
    h = (ln.float() * (1 + scale) + shift).half()
    want = vdm.linear_vdm_w4a4(h, packed, sp, None, 0.95, bias_half=bias)
    got = vdm.linear_vdm_w4a4_fused(x, packed, sp, bias, 0.95, prologue="layernorm_mod",
                                    mod_scale=scale, mod_shift=shift, ln_eps=1e-6)
    rel = torch.linalg.vector_norm(got.float() - want.float()) / torch.linalg.vector_norm(want.float())
    assert rel.item() < 5e-3
    # the quantiser's own view: codes of the fused prologue vs codes of the materialised tensor
    from dsaquant_b200 import _lib
    lib = _lib.load()
    q_f = torch.empty(M, K, dtype=torch.int8, device="cuda")
    s_f = torch.empty(M, dtype=torch.float32, device="cuda")
    sc, sh = scale.contiguous(), shift.contiguous()
    rc = lib.b200w4a4_quantize_act_fused(x.data_ptr(), 2, sc.data_ptr(), sh.data_ptr(), K if per_token else 0, 1e-6,
                                         q_f.data_ptr(), s_f.data_ptr(), M, K, 0.95,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    q_u, s_u, _ = vdm.quantize_activation_per_token(h, 0.95)
    assert (q_f != q_u).float().mean().item() < 2e-3
    assert (q_f.int() - q_u.int()).abs().max().item() <= 1
    assert torch.allclose(s_f, s_u, rtol=2e-3)


@pytest.mark.parametrize("M,K,D,segments", [(300, 1536, 1536, 3), (1000, 5120, 384, 3), (513, 3072, 3072, 2),
                                           (77, 256, 64, 2), (257, 1536, 128, 1), (32760, 1536, 1536, 3)])
@pytest.mark.parametrize("cta_group", [1, 2])
def test_split_outputs_bit_identical(vdm, M, K, D, segments, cta_group):
    """The split epilogue stores the same values as the one-matrix GEMM, as separate tensors."""
    if (segments * D) % 128:
        pytest.skip("N must be a multiple of 128")
    N = segments * D
    packed, sp, bias = _layer(vdm, K, N, 61)
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = torch.randn(M, K, generator=g, device="cuda").half()
    prev = vdm.set_cta_group(cta_group)
    try:
        want = vdm.linear_vdm_w4a4(x, packed, sp, None, 0.95, bias_half=bias).split(D, dim=-1)
        got = vdm.linear_vdm_w4a4_split(x, packed, sp, segments, bias, 0.95)
        assert len(got) == segments
        for a, b in zip(got, want):
            assert a.is_contiguous() and a.shape == (M, D)
            assert torch.equal(a, b)
        # destinations inside larger buffers: rows at an offset, wider row pitch; the rest untouched
        pad_rows, pitch = 40, D + 64
        bufs = [torch.full((M + 2 * pad_rows, pitch), 7.0, dtype=torch.float16, device="cuda") for _ in range(segments)]
        views = [bf[pad_rows:pad_rows + M, 8:8 + D] for bf in bufs]
        vdm.linear_vdm_w4a4_split(x, packed, sp, segments, bias, 0.95, outs=views)
        for bf, v, b in zip(bufs, views, want):
            assert torch.equal(v, b)
            assert (bf[:pad_rows] == 7).all() and (bf[pad_rows + M:] == 7).all()
            assert (bf[:, :8] == 7).all() and (bf[:, 8 + D:] == 7).all()
    finally:
        vdm.set_cta_group(prev)


def test_split_with_layernorm_prologue_matches_fused(vdm):
    M, K, D = 500, 1536, 1536
    packed, sp, bias = _layer(vdm, K, 3 * D, 67)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(M, K, generator=g, device="cuda") * 2).half()
    scale = torch.randn(K, generator=g, device="cuda") * 0.1
    shift = torch.randn(K, generator=g, device="cuda") * 0.1
    want = vdm.linear_vdm_w4a4_fused(x, packed, sp, bias, 0.95, prologue="layernorm_mod", mod_scale=scale,
                                     mod_shift=shift).split(D, dim=-1)
    got = vdm.linear_vdm_w4a4_split(x, packed, sp, 3, bias, 0.95, prologue="layernorm_mod", mod_scale=scale,
                                    mod_shift=shift)
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_split_rejects_bad_arguments(vdm):
    from dsaquant_b200 import _lib
    lib = _lib.load()
    import ctypes
    M, K, N = 64, 256, 384
    packed, sp, _ = _layer(vdm, K, N, 71)
    x = torch.randn(M, K, device="cuda").half()
    with pytest.raises(ValueError):
        vdm.linear_vdm_w4a4_split(x, packed, sp, 4)
    with pytest.raises(ValueError):
        vdm.linear_vdm_w4a4_split(x, packed, sp, 3, outs=[torch.empty(M, 128, device="cuda").half()] * 2)
    packed2, sp2, _ = _layer(vdm, K, 128, 73)
    with pytest.raises(ValueError):
        vdm.linear_vdm_w4a4_split(x, packed2, sp2, 3)        # 128 / 3
    # C ABI: a row pitch that is not a multiple of 8 elements, and one below the segment width
    w_b200, w_scale = vdm.prepare_b200_weight(packed, sp)
    qa = torch.zeros(M, K, dtype=torch.int8, device="cuda")
    sa = torch.ones(M, dtype=torch.float32, device="cuda")
    o = torch.empty(M, 200, dtype=torch.float16, device="cuda")
    ptrs = (ctypes.c_void_p * 3)(o.data_ptr(), o.data_ptr(), o.data_ptr())
    for ld, code in ((132, -3), (64, -2)):
        lds = (ctypes.c_longlong * 3)(ld, ld, ld)
        rc = lib.b200w4a4_gemm_split(qa.data_ptr(), sa.data_ptr(), w_b200.data_ptr(), w_scale.data_ptr(), None,
                                     ptrs, lds, 3, M, N, K, None)
        assert rc == code
