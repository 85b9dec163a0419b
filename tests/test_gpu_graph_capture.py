"""The library calls are stream-ordered and allocate nothing behind torch's back (tensor maps travel
as kernel parameters), so a caller can capture them in a CUDA graph and replay it on new data."""
import pytest
import torch

from _cases import make_case

pytestmark = pytest.mark.gpu


def test_linear_fused_split_and_glue_replay_from_a_cuda_graph():
    from dsaquant_b200 import attention_qkv as aq
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    assert vdm.is_available(), vdm.load_error()
    M, K, D = 700, 1536, 512
    _, w16, b16 = make_case(101, 8, K, 3 * D)
    packed, sp, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w16).cuda())
    bias = torch.from_numpy(b16).cuda()
    _, w2, b2 = make_case(103, 8, D, K)
    packed2, sp2, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w2).cuda())
    bias2 = torch.from_numpy(b2).cuda()
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(M, K, generator=g, device="cuda").half()
    scale = torch.randn(K, generator=g, device="cuda") * 0.1
    shift = torch.randn(K, generator=g, device="cuda") * 0.1
    gate = torch.randn(K, generator=g, device="cuda")
    nw = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).half()
    ang = torch.rand(M, 1, 32, generator=g, device="cuda") * 6.28
    cs = aq.rope_cos_sin(torch.polar(torch.ones_like(ang), ang))

    def chain(inp):
        y = vdm.linear_vdm_w4a4(inp, packed, sp, None, 0.95, bias_half=bias)
        q, k, v = vdm.linear_vdm_w4a4_split(inp, packed, sp, 3, bias, 0.95, prologue="layernorm_mod",
                                            mod_scale=scale, mod_shift=shift)
        qb = aq.qk_norm_rope(q, nw, cs, 1e-6, 64)
        out = vdm.linear_vdm_w4a4_fused(qb, packed2, sp2, bias2, 0.95, epilogue="gate_residual", residual=inp, gate=gate)
        return y, k, v, qb, out

    for _ in range(2):                       # one-time set-up (weight repack, per-device state) outside the capture
        chain(x)
    torch.cuda.synchronize()
    static_x = x.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(static_x)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        captured = chain(static_x)
    for seed in (11, 12):
        fresh = torch.randn(M, K, generator=torch.Generator(device="cuda").manual_seed(seed), device="cuda").half()
        static_x.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        want = chain(fresh)
        for a, b in zip(captured, want):
            assert torch.equal(a, b)
    assert vdm.last_device_status() == 0
