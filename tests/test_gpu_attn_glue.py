"""qk_norm_rope (RMSNorm across heads + rotary embedding + cast, one pass) against the same work
done with the PyTorch ops of the reference's attention processor
(vdm_infer/models/wan_vdm/modules/attention.py:131-135, :167-177, :208-216).  The roundings are
placed where the reference ops round, so almost every element is bit-identical; the row reduction
runs in a different order than torch's mean, which can move single values across an fp16 rounding
boundary: checked as a mismatch rate plus a bound of two output ulps."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def glue():
    from dsaquant_b200 import attention_qkv as a
    from dsaquant_b200.kernels import vdm_w4a4 as v

    assert v.is_available(), v.load_error()
    yield a
    assert v.last_device_status() == 0


def _torch_glue(x, w, freqs, eps, heads, out_dtype):
    """The reference's op sequence on [L, D] fp16 (RMSNorm.forward, apply_rotary_emb fp32 variant)."""
    y = x
    if w is not None:
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(x.dtype) * w
    if freqs is not None:
        y4 = y.view(1, y.shape[0], heads, -1)
        yc = torch.view_as_complex(y4.float().reshape(*y4.shape[:-1], -1, 2))
        y = torch.view_as_real(yc * freqs[None]).flatten(3).to(x.dtype).reshape(y.shape)
    return y.to(out_dtype)


def _freqs(L, hd, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ang = torch.rand(L, 1, hd // 2, generator=g, device="cuda") * 6.2831853
    return torch.polar(torch.ones_like(ang), ang).to(torch.complex64)


def _compare(got, want, out_dtype):
    assert got.dtype == out_dtype and got.shape == want.shape
    g, w = got.float(), want.float()
    ulp = 2.0 ** (-7 if out_dtype == torch.bfloat16 else -10)
    # A rotation can cancel (re = a*cos - b*sin near 0), so the error of an element scales with the
    # magnitude of its pair, which the rotation preserves.
    pair = w.reshape(*w.shape[:-1], -1, 2).norm(dim=-1, keepdim=True).expand(*w.shape[:-1], w.shape[-1] // 2, 2)
    assert ((g - w).abs() <= 2 * ulp * pair.reshape(w.shape) + 1e-6).all()
    assert (g != w).float().mean().item() < 5e-3


@pytest.mark.parametrize("L,D,heads", [(1000, 1536, 12), (517, 5120, 40), (300, 3072, 24), (77, 256, 2),
                                       (4096, 1024, 8), (33, 12288, 96)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_norm_rope_matches_reference_ops(glue, L, D, heads, out_dtype):
    g = torch.Generator(device="cuda").manual_seed(L + D)
    x = (torch.randn(L, D, generator=g, device="cuda") * 1.7).half()
    w = (1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")).half()
    fr = _freqs(L, D // heads, 3)
    want = _torch_glue(x, w, fr, 1e-6, heads, out_dtype)
    got = glue.qk_norm_rope(x, w, glue.rope_cos_sin(fr), 1e-6, D // heads, out_dtype)
    _compare(got, want, out_dtype)
    # norm only (cross-attention: no rotation)
    _compare(glue.qk_norm_rope(x, w, None, 1e-6, D // heads, out_dtype), _torch_glue(x, w, None, 1e-6, heads, out_dtype),
             out_dtype)


def test_cast_only_is_exact_and_strided_rows_are_read_in_place(glue):
    L, D = 999, 1536
    qkv = torch.randn(L, 3 * D, device="cuda").half()
    for i in range(3):
        part = qkv[:, i * D:(i + 1) * D]                       # row pitch 3*D, 16-byte aligned columns
        assert torch.equal(glue.qk_norm_rope(part, None, None, 1e-6, 128, torch.bfloat16), part.to(torch.bfloat16))
        assert torch.equal(glue.qk_norm_rope(part, None, None, 1e-6, 128, torch.float16), part)
    # rotation only: elementwise with pinned roundings -> bit-exact against the torch ops
    fr = _freqs(L, 128, 9)
    want = _torch_glue(qkv[:, :D].contiguous(), None, fr, 1e-6, D // 128, torch.float16)
    got = glue.qk_norm_rope(qkv[:, :D], None, glue.rope_cos_sin(fr), 1e-6, 128, torch.float16)
    assert (got != want).float().mean().item() < 1e-3          # fma contraction inside torch's complex multiply
    _compare(got, want, torch.float16)


def test_leading_dims_and_errors(glue):
    x = torch.randn(2, 50, 512, device="cuda").half()
    w = torch.ones(512, device="cuda").half()
    out = glue.qk_norm_rope(x, w, None, 1e-6, 128)
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    with pytest.raises(RuntimeError):
        glue.qk_norm_rope(x.float(), w, None, 1e-6, 128)
    with pytest.raises(ValueError):
        glue.qk_norm_rope(x, w[:100], None, 1e-6, 128)
    with pytest.raises(ValueError):
        glue.qk_norm_rope(x, w, torch.zeros(3, 64, 2, device="cuda"), 1e-6, 128)
    from dsaquant_b200 import _lib
    lib = _lib.load()
    o = torch.empty(10, 516, dtype=torch.float16, device="cuda")
    xs = torch.zeros(10, 516, dtype=torch.float16, device="cuda")
    assert lib.b200w4a4_qk_norm_rope(xs.data_ptr(), 516, None, None, 1e-6, 128, o.data_ptr(), 0, 516, 10, 516, None) == -2
    assert lib.b200w4a4_qk_norm_rope(xs.data_ptr(), 512, None, None, 1e-6, 128, o.data_ptr(), 7, 512, 10, 512, None) == -1


def test_bf16_activation_into_fused_linear(glue):
    """The attention output stays bf16: the output projection quantises it from its exact values."""
    from dsaquant_b200.kernels import vdm_w4a4 as vdm
    from _cases import make_case

    M, K, N = 300, 1536, 1536
    _, w16, b16 = make_case(91, 8, K, N)
    packed, sp, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w16).cuda())
    bias = torch.from_numpy(b16).cuda()
    xb = torch.randn(M, K, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").half()
    gate = torch.randn(N, device="cuda")
    want = vdm.linear_vdm_w4a4_fused(xb.half(), packed, sp, bias, 0.95, epilogue="gate_residual", residual=res, gate=gate)
    got = vdm.linear_vdm_w4a4_fused(xb, packed, sp, bias, 0.95, epilogue="gate_residual", residual=res, gate=gate)
    assert torch.equal(got, want)      # bf16 values in fp16 range convert exactly
