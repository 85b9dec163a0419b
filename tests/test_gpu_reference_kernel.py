"""Cross-checks against the REFERENCE's own CUDA extension (built for sm_100a by
oracle/build_ref_ext.py into oracle/_ref/; skipped when it is absent):
  * the vdm_w4a4_packed_v1 byte layout written by this library equals the reference packer's,
    byte for byte, on weights whose codes are unambiguous (exact multiples of a power-of-two scale);
  * on random weights the two packers agree except at rounding ties (the reference multiplies by an
    approximate reciprocal, vdm_w4a4_kernel.cu:319-328);
  * the reference kernel's output is statistically close to the oracle (its smoke tests print the
    same statistics, tests/test_vdm_w4a4_kernel_smoke.py:29-34) while this library's is bit-exact."""
import numpy as np
import pytest
import torch

from _cases import make_case
from oracle import _ref_loader
from oracle import w4a4_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mod = _ref_loader.load()
    if mod is None:
        pytest.skip("oracle/_ref/vdm_w4a4_ref_ext.so not built")
    return mod


@pytest.fixture(scope="module")
def vdm():
    from dsaquant_b200.kernels import vdm_w4a4 as v

    assert v.is_available(), v.load_error()
    return v


@pytest.mark.parametrize("N,K", [(128, 64), (256, 192), (384, 1536)])
def test_v1_layout_equals_reference_packer_bytes(ref, vdm, N, K):
    rng = np.random.default_rng(N + K)
    codes = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    scale = np.full(N, 2.0 ** -6, np.float16) * (1 + (np.arange(N) % 3)).astype(np.float16)  # 1,2,3 x 2^-6
    w = (codes.astype(np.float32) * scale.astype(np.float32)[:, None]).astype(np.float16)
    assert np.array_equal(orc.quantize_weight(w, scale), codes)          # unambiguous codes
    wt, st = torch.from_numpy(w).cuda(), torch.from_numpy(scale).cuda()
    r_q, r_sp, r_s = ref.pack_weight_with_scale(wt, st)
    m_q, m_sp, m_s = vdm.pack_weight_with_scale(wt, st)
    assert r_q.shape == (N, K // 2) and r_sp.shape == (N, K // 64) and r_s.shape == (N,)
    assert torch.equal(r_q, m_q), "vdm_weight_packed differs from the reference packer"
    assert torch.equal(r_sp, m_sp), "vdm_weight_scale_packed differs from the reference packer"
    assert torch.equal(r_s, m_s)
    np.testing.assert_array_equal(r_q.cpu().numpy(), orc.pack_weight_v1(codes))
    np.testing.assert_array_equal(r_sp.cpu().numpy(), orc.pack_wscale_v1(scale, K))


def test_random_weights_agree_except_at_ties(ref, vdm):
    _, w16, _ = make_case(9, 8, 1536, 1536, bias=False)
    ws = orc.weight_scale_absmax(w16)
    wt, st = torch.from_numpy(w16).cuda(), torch.from_numpy(ws).cuda()
    r_q = ref.pack_weight_with_scale(wt, st)[0]
    m_q = vdm.pack_weight_with_scale(wt, st)[0]
    r_codes = vdm.unpack_codes(r_q, 1536, 1536, 2)
    m_codes = vdm.unpack_codes(m_q, 1536, 1536, 2)
    np.testing.assert_array_equal(m_codes.cpu().numpy(), orc.quantize_weight(w16, ws))
    diff = (r_codes != m_codes)
    assert diff.float().mean().item() < 1e-3
    assert (r_codes.int() - m_codes.int()).abs().max().item() <= 1


def test_reference_kernel_statistics_and_this_kernel_exact(ref, vdm):
    """Seed / shape / clip of the reference's kernel smoke test."""
    torch.manual_seed(0)
    m, k, n, clip = 257, 1536, 1536, 0.95
    x = torch.randn(m, k, device="cuda", dtype=torch.float16)
    w = torch.randn(n, k, device="cuda", dtype=torch.float16)
    b = torch.randn(n, device="cuda", dtype=torch.float16)
    wscale = (w.abs().amax(dim=1).clamp_min(1e-6) / 7).half()
    qw, wps, _ = ref.pack_weight_with_scale(w, wscale)
    out_ref = ref.linear_dynamic_bias(x, qw, wps, b, clip)
    out_mine = vdm.linear_vdm_w4a4(x, qw, wps, b, clip_ratio=clip)         # same v1 buffers, drop-in
    codes = vdm.unpack_codes(qw, n, k, 2).cpu().numpy()
    oracle = orc.linear_w4a4(x.cpu().numpy(), codes, wscale.cpu().numpy(), b.cpu().numpy(), clip)["out"]
    np.testing.assert_array_equal(out_mine.cpu().numpy().view(np.uint16), oracle.view(np.uint16))
    o = torch.from_numpy(oracle.astype(np.float32)).cuda()
    rel_ref = (torch.linalg.vector_norm(out_ref.float() - o) / torch.linalg.vector_norm(o)).item()
    assert out_ref.shape == (m, n) and rel_ref < 0.05
    print(f"reference kernel vs oracle: rel_l2 {rel_ref:.3e}, max_abs {(out_ref.float() - o).abs().max().item():.3e}")


def test_exported_checkpoint_equals_reference_packer_layer_by_layer(ref, vdm, tmp_path):
    """Exporter (dsaquant_b200/checkpoints/export.py): a multi-layer model in its full quantised
    form (fp weights + wquantizer scales) -> vdm_w4a4_packed_v1 file.  Every layer's three buffers
    in the file equal what the reference's own packer writes for the same weight and scale, and
    the file loads back into a fresh model that evaluates like the exported one."""
    import torch.nn as nn

    from dsaquant_b200.checkpoints import export as ex
    from dsaquant_b200.checkpoints import packed_checkpoint as pc
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    qp = {"w": {"bit": 4, "sym": True, "granularity": "per_channel"}, "act": {"bit": 4, "sym": True}}
    shapes = [(256, 128), (128, 256), (384, 128), (128, 384)]            # (N, K)

    def build():
        torch.manual_seed(0)
        m = nn.Sequential(*[nn.Linear(k, n, bias=(i % 2 == 0)) for i, (n, k) in enumerate(shapes)])
        for i in range(len(shapes)):
            m[i] = QuantLinear(m[i], {"w": "lsq", "act": "dynamic"}, qp)
        return m

    # Full quantised state with unambiguous codes: weight = code * scale, scale = s * 2^-6.
    rng = np.random.default_rng(3)
    state, truth = {}, {}
    for i, (n, k) in enumerate(shapes):
        codes = rng.integers(-7, 8, size=(n, k), dtype=np.int8)
        scale = (np.full(n, 2.0 ** -6, np.float32) * (1 + (np.arange(n) % 3))).astype(np.float16)
        w = (codes.astype(np.float32) * scale.astype(np.float32)[:, None]).astype(np.float16)
        state[f"{i}.weight"] = torch.from_numpy(w)
        state[f"{i}.wquantizer.scale"] = torch.from_numpy(scale.astype(np.float32)).view(n, 1)
        if i % 2 == 0:
            state[f"{i}.bias"] = torch.from_numpy(rng.standard_normal(n).astype(np.float16))
        truth[i] = (w, scale)
    out = tmp_path / "packed.pt"
    stats = ex.export_packed_checkpoint(build(), {"model": state}, str(out), metadata={"model": "synthetic"})
    assert stats["layers"] == len(shapes)
    ckpt = torch.load(out, map_location="cpu", weights_only=True)
    assert pc.is_packed_checkpoint(ckpt) and ckpt["metadata"]["model"] == "synthetic"
    for i, (w, scale) in truth.items():
        r_q, r_sp, r_s = ref.pack_weight_with_scale(torch.from_numpy(w).cuda(), torch.from_numpy(scale).cuda())
        assert torch.equal(ckpt["model"][f"{i}.vdm_weight_packed"], r_q.cpu())
        assert torch.equal(ckpt["model"][f"{i}.vdm_weight_scale_packed"], r_sp.cpu())
        assert torch.equal(ckpt["model"][f"{i}.vdm_weight_scale"], r_s.half().cpu())
        assert f"{i}.weight" not in ckpt["model"]
    fresh = build()
    pc.load_packed_quantized_model(fresh, ckpt, quant_linear_cls=QuantLinear, dtype=torch.float16,
                                   device=torch.device("cuda"))
    x = torch.randn(70, 128, device="cuda", dtype=torch.float16)
    w0, s0 = truth[0]
    want = orc.linear_w4a4(x.cpu().numpy(), orc.quantize_weight(w0, s0), s0, state["0.bias"].numpy(), 0.95)["out"]
    np.testing.assert_array_equal(fresh[0](x).cpu().numpy().view(np.uint16), want.view(np.uint16))
