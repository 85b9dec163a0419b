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
