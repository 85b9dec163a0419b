"""CPU-only tests: the C-ABI library loads and exports what the header declares, the python
mirror keeps the reference's interface, the fake-quant branch reproduces the reference fixtures,
and the packed-checkpoint loader handles the vdm_w4a4_packed_v1 format."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

from _cases import CASES, make_case
from oracle import w4a4_oracle as orc

ROOT = Path(__file__).resolve().parent.parent
GOLD = Path(__file__).resolve().parent / "golden"
QPARAMS = {"w": {"bit": 4, "sym": True, "granularity": "per_channel", "group_size": -1,
                 "round_zero": True, "use_grad_scaling": True, "cali": "mse"},
           "act": {"bit": 4, "sym": True}}


def test_library_exports_every_declared_symbol():
    from dsaquant_b200 import _lib

    header = (ROOT / "include" / "b200w4a4.h").read_text()
    declared = set(re.findall(r"\b(b200w4a4_[a-z0-9_]+)\s*\(", header))
    assert len(declared) == 29
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == declared
    assert lib.b200w4a4_version() == 1 == int(re.search(r"B200W4A4_ABI_VERSION (\d+)", header).group(1))


def test_host_only_entry_points():
    from dsaquant_b200 import _lib

    lib = _lib.load()
    assert lib.b200w4a4_repack_bytes(1536, 1536) == 1536 * 768
    assert lib.b200w4a4_repack_bytes(100, 64) == 0 and lib.b200w4a4_repack_bytes(128, 96) == 0
    assert lib.b200w4a4_qact_bytes(257, 1536, 0) == 257 * 1536
    assert lib.b200w4a4_qact_bytes(257, 1536, 1) == 257 * 768
    assert lib.b200w4a4_qact_bytes(0, 1536, 0) == 0
    ws = lib.b200w4a4_linear_workspace_bytes(257, 1536)
    assert ws >= 257 * 1536 + 257 * 4 and ws % 256 == 0
    assert lib.b200w4a4_linear_noalloc_max_codes() == 8 << 20
    assert lib.b200w4a4_set_cta_group(3) == -1
    for code in range(0, -9, -1):
        text = lib.b200w4a4_strerror(code).decode()
        assert text and "unknown" not in text
    assert "unknown" in lib.b200w4a4_strerror(-99).decode()
    # argument checks come before any CUDA call
    assert lib.b200w4a4_gemm(None, None, None, None, None, None, None, 1, 128, 64, None) == -1
    assert lib.b200w4a4_linear_noalloc(None, 0, None, None, None, None, 9000, 128, 64, 1.0, None) == -8


def test_arch_selection_gains_sm100a(monkeypatch):
    from dsaquant_b200.kernels import vdm_w4a4 as v

    monkeypatch.delenv("TORCH_CUDA_ARCH_LIST", raising=False)
    for alias in ("b200", "blackwell", "sm100", "sm100a", "sm_100a", "10.0", "10.0a"):
        monkeypatch.setenv("VDM_W4A4_TARGET_ARCH", alias)
        assert v._detect_arch_list() == "10.0a"
    monkeypatch.setenv("TORCH_CUDA_ARCH_LIST", "10.0a")
    cfg = v.build_config()
    assert set(cfg) == {"cuda_home", "torch_cuda", "arch_list", "arch_tag", "build_dir", "extension_name"}
    assert cfg["arch_tag"] == "sm100a"
    assert v._arch_tag("8.6;10.0a+PTX") == "sm86_sm100aptx"
    monkeypatch.setenv("TORCH_CUDA_ARCH_LIST", "8.6")
    with pytest.raises(RuntimeError):
        v._load_ext()
    assert (v.BLOCK_M, v.BLOCK_N, v.WARP_K) == (256, 128, 64)


def test_wrapper_rejects_cpu_tensors_and_bad_shapes():
    from dsaquant_b200.kernels import vdm_w4a4 as v

    x = torch.zeros(4, 128)
    qw = torch.zeros(128, 64, dtype=torch.uint8)
    ws = torch.zeros(128, 2, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        v.linear_vdm_w4a4(x, qw, ws)
    with pytest.raises(RuntimeError):
        v.pack_weight_with_scale(torch.zeros(128, 64), torch.ones(128))
    # the fused / split entry points and the attention glue have no CPU route either
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        v.linear_vdm_w4a4_fused(x.half(), qw, ws, epilogue="gelu_tanh")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        v.linear_vdm_w4a4_split(x.half(), qw, ws, 2)
    from dsaquant_b200 import attention_qkv as aq
    with pytest.raises(RuntimeError, match="CUDA"):
        aq.qk_norm_rope(torch.zeros(4, 128, dtype=torch.float16), None, None, 1e-6, 64)
    cs = aq.rope_cos_sin(torch.polar(torch.ones(5, 1, 8), torch.arange(40.0).reshape(5, 1, 8)))
    assert cs.shape == (5, 8, 2) and cs.dtype == torch.float32
    assert torch.allclose(cs[..., 0], torch.cos(torch.arange(40.0).reshape(5, 8)), atol=1e-6)
    # C ABI argument checks of the new entries come before any CUDA call
    from dsaquant_b200 import _lib
    lib = _lib.load()
    assert lib.b200w4a4_gemm_split(None, None, None, None, None, None, None, 3, 1, 384, 64, None) == -1
    assert lib.b200w4a4_qk_norm_rope(None, 128, None, None, 1e-6, 64, None, 1, 128, 4, 128, None) == -1
    with pytest.raises(ValueError, match="multiple of 64"):
        v._check_linear_shapes(torch.zeros(4, 96), qw, ws)
    with pytest.raises(ValueError, match="multiple of 128"):
        v._check_linear_shapes(x, torch.zeros(100, 64, dtype=torch.uint8), ws)
    with pytest.raises(ValueError, match=r"\[N, K/2\]"):
        v._check_linear_shapes(x, torch.zeros(128, 32, dtype=torch.uint8), ws)
    with pytest.raises(ValueError, match=r"\[N, K/64\]"):
        v._check_linear_shapes(x, qw, torch.zeros(128, 3, dtype=torch.float16))


@pytest.mark.parametrize("name", ["tiny", "cfg0"])
def test_fake_quant_branch_reproduces_reference_fixture(name):
    """The mirror's PyTorch branch must equal the reference's own fake-quant forward."""
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    seed, M, K, N, kw, clip = CASES[name]
    g = np.load(GOLD / f"{name}.npz")
    x16, w16, b16 = make_case(seed, M, K, N, **kw)
    lin = nn.Linear(K, N)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(w16).float())
        lin.bias.copy_(torch.from_numpy(b16).float())
    ql = QuantLinear(lin, {"w": "lsq", "act": "dynamic"}, QPARAMS)
    with torch.no_grad():
        ql.wquantizer(ql.weight.detach())
        ql.wquantizer.scale.copy_(ql.wquantizer.scale.half().float())
        ql.set_quant_state(True, True)
        out = ql(torch.from_numpy(x16).float()).numpy()
    np.testing.assert_array_equal(ql.aquantizer.scale.reshape(-1).numpy(), g["a_scale"])
    if "ref_out_f32" in g.files:
        np.testing.assert_array_equal(out, g["ref_out_f32"])
    else:
        np.testing.assert_array_equal(out[::61, ::53], g["ref_out_f32_sample"])
    # second call keeps the first call's scale, like the reference (init stays True)
    assert ql.aquantizer.init
    with pytest.raises(NotImplementedError):
        ql.set_hadamard(True)
    assert "use_vdm_kernel=False" in ql.extra_repr()


def test_fakequant_cpu_port_matches_oracle():
    from oracle.fakequant_cpu import fakequant_linear

    x16, w16, b16 = make_case(3, 64, 256, 128)
    ws = orc.weight_scale_absmax(w16)
    ref = orc.linear_w4a4(x16, orc.quantize_weight(w16, ws), ws, b16, 1.0)
    got = fakequant_linear(torch.from_numpy(x16).float(), torch.from_numpy(w16).float(),
                           torch.from_numpy(ws).float(), torch.from_numpy(b16).float(), 1.0).numpy()
    np.testing.assert_allclose(got, ref["out"].astype(np.float32), rtol=1e-2, atol=5e-3)


class _TinyAttn(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
        self.cross_attention_dim_head = None


class _TinyModel(nn.Module):
    def __init__(self, dim=128):
        super().__init__()
        self.embed = nn.Linear(8, dim)            # stays fp
        self.blocks = nn.ModuleList([_TinyAttn(dim)])


def _quantize_blocks(model, cls):
    for blk in model.blocks:
        for name in ("to_q", "to_k", "to_v"):
            setattr(blk, name, cls(getattr(blk, name), {"w": "lsq", "act": "dynamic"}, QPARAMS))


def _packed_state(model, rng, legacy=False):
    state = {k: v.detach().clone() for k, v in model.state_dict().items()
             if ".wquantizer." not in k and ".aquantizer." not in k}
    for name, mod in model.named_modules():
        if type(mod).__name__ != "QuantLinear":
            continue
        n, k = mod.out_features, mod.in_features
        codes = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
        scale = (rng.random(n) * 0.01 + 0.001).astype(np.float16)
        prefix = "diy_" if legacy else "vdm_"
        state[f"{name}.{prefix}weight_packed"] = torch.from_numpy(orc.pack_weight_v1(codes))
        state[f"{name}.{prefix}weight_scale_packed"] = torch.from_numpy(orc.pack_wscale_v1(scale, k))
        state[f"{name}.{prefix}weight_scale"] = torch.from_numpy(scale)
        del state[f"{name}.weight"]
    return state


@pytest.mark.parametrize("legacy", [False, True])
def test_packed_checkpoint_round_trip_on_cpu(tmp_path, legacy):
    from dsaquant_b200.checkpoints import packed_checkpoint as pc
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    rng = np.random.default_rng(1)
    src = _TinyModel()
    _quantize_blocks(src, QuantLinear)
    fmt = pc._LEGACY_PACKED_CHECKPOINT_FORMAT if legacy else pc.PACKED_CHECKPOINT_FORMAT
    ckpt = {"format": fmt, "metadata": {"note": "synthetic"}, "model": _packed_state(src, rng, legacy)}
    path = tmp_path / "packed.pt"
    torch.save(ckpt, path)
    loaded = pc.load_quant_checkpoint(str(path), dcp_loader=None)
    assert pc.is_packed_checkpoint(loaded) and not pc.is_packed_checkpoint({"format": "other", "model": {}})

    model = _TinyModel()
    _quantize_blocks(model, QuantLinear)
    missing, unexpected = pc.load_packed_quantized_model(
        model, loaded, quant_linear_cls=QuantLinear, dtype=torch.float16, device=torch.device("cpu"),
        require_vdm_kernel=False, repack_for_b200=False)
    assert missing == [] and unexpected == []
    q = model.blocks[0].to_q
    assert q.use_vdm_kernel and q.weight is None and q.wquantizer is None and q.aquantizer is None
    assert q.vdm_weight_packed.dtype == torch.uint8 and q.vdm_weight_packed.shape == (128, 64)
    assert q.vdm_weight_scale_packed.shape == (128, 2) and q.vdm_weight_scale.shape == (128,)
    assert q._bias_half.dtype == torch.float16 and model.embed.weight.dtype == torch.float16
    key = "blocks.0.to_q." + ("diy_" if legacy else "vdm_") + "weight_packed"
    assert torch.equal(q.vdm_weight_packed, ckpt["model"][key])

    pc.enable_fused_qkv(model, quant_linear_cls=QuantLinear, attention_cls=_TinyAttn, use_fused_qkv=True)
    assert model.blocks[0].use_fused_qkv_kernel and model.blocks[0].qkv_kernel_backend == "vdm"

    # writer: the saved state has the three buffers + bias and no fp weight / quantizer state
    out_path = tmp_path / "resaved.pt"
    pc.save_packed_checkpoint(model, str(out_path), metadata={"a": 1})
    again = torch.load(out_path, weights_only=True)
    assert again["format"] == pc.PACKED_CHECKPOINT_FORMAT and again["metadata"] == {"a": 1}
    keys = set(again["model"])
    assert "blocks.0.to_q.vdm_weight_packed" in keys and "blocks.0.to_q.bias" in keys
    assert not any(k.endswith(".weight") and "blocks" in k for k in keys)
    assert not any("quantizer" in k or k.endswith("_bias_half") for k in keys)

    # a checkpoint that lacks a buffer is refused
    broken = dict(ckpt, model={k: v for k, v in ckpt["model"].items() if "to_v" not in k or "scale" not in k})
    fresh = _TinyModel()
    _quantize_blocks(fresh, QuantLinear)
    with pytest.raises(KeyError, match="missing"):
        pc.load_packed_quantized_model(fresh, broken, quant_linear_cls=QuantLinear, dtype=torch.float16,
                                       device=torch.device("cpu"), require_vdm_kernel=False)
    with pytest.raises(ValueError, match="Unsupported checkpoint format"):
        pc.load_packed_quantized_model(fresh, {"format": "x", "model": {}}, quant_linear_cls=QuantLinear,
                                       dtype=torch.float16, device=torch.device("cpu"))


def test_fused_qkv_cache_concatenates_v1_buffers():
    from dsaquant_b200 import attention_qkv as aq
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    rng = np.random.default_rng(2)
    attn = _TinyAttn(128)
    _quantize_blocks(type("M", (), {"blocks": [attn]})(), QuantLinear)
    codes = []
    for lin, has_bias in ((attn.to_q, True), (attn.to_k, False), (attn.to_v, True)):
        c = rng.integers(-8, 8, size=(128, 128), dtype=np.int8)
        codes.append(c)
        lin.register_buffer("vdm_weight_packed", torch.from_numpy(orc.pack_weight_v1(c)))
        lin.register_buffer("vdm_weight_scale_packed", torch.from_numpy(orc.pack_wscale_v1(np.ones(128, np.float16), 128)))
        lin._bias_half = torch.ones(128, dtype=torch.float16) if has_bias else None
    aq._cat_cached(attn, "_vdm_qkv", (attn.to_q, attn.to_k, attn.to_v))
    np.testing.assert_array_equal(attn._vdm_qkv_weight_packed.numpy(), orc.pack_weight_v1(np.concatenate(codes)))
    assert attn._vdm_qkv_weight_scale.shape == (384, 2)
    assert attn._vdm_qkv_bias_half.tolist() == [1.0] * 128 + [0.0] * 128 + [1.0] * 128


def test_install_as_vdm_infer_aliases_modules():
    import sys

    import dsaquant_b200

    saved = {k: v for k, v in sys.modules.items() if k == "vdm_infer" or k.startswith("vdm_infer.")}
    for k in saved:
        del sys.modules[k]
    try:
        dsaquant_b200.install_as_vdm_infer()
        from vdm_infer.kernels import vdm_w4a4
        from vdm_infer.quantization.quant_linear import QuantLinear

        assert vdm_w4a4.__name__ == "dsaquant_b200.kernels.vdm_w4a4"
        assert QuantLinear.__module__ == "dsaquant_b200.quantization.quant_linear"
    finally:
        for k in [k for k in sys.modules if k == "vdm_infer" or k.startswith("vdm_infer.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_missing_library_fails_loudly(tmp_path):
    """Without libb200w4a4.so (and with the JIT build disabled) nothing falls back to the CPU:
    is_available() is False, load_error() keeps the reason and every op raises."""
    import subprocess
    import sys

    code = r"""
import torch
from dsaquant_b200.kernels import vdm_w4a4 as v
assert v.is_available() is False
assert isinstance(v.load_error(), FileNotFoundError), repr(v.load_error())
x = torch.zeros(4, 128); qw = torch.zeros(128, 64, dtype=torch.uint8); ws = torch.zeros(128, 2, dtype=torch.float16)
for fn in (lambda: v.linear_vdm_w4a4(x, qw, ws), lambda: v.quantize_activation_per_token(x),
           lambda: v.pack_weight_with_scale(torch.zeros(128, 64), torch.ones(128))):
    try:
        fn()
    except FileNotFoundError:
        pass
    else:
        raise SystemExit("op did not raise")
from dsaquant_b200.quantization.quant_linear import QuantLinear
ql = QuantLinear(torch.nn.Linear(128, 128), {"w": "lsq", "act": "dynamic"}, {"w": {}, "act": {}})
ql.wquantizer(ql.weight.detach())
try:
    ql.enable_vdm_kernel_mode()
except AssertionError as e:
    assert "not compiled/available" in str(e)
else:
    raise SystemExit("enable_vdm_kernel_mode did not fail")
print("ok")
"""
    env = dict(__import__("os").environ, VDM_W4A4_EXTENSIONS_DIR=str(tmp_path), B200W4A4_NO_JIT="1",
               PYTHONPATH=str(ROOT))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=str(tmp_path))
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr


def test_peer_exchange_layout_is_disjoint_and_sized():
    """Host bookkeeping of the K/V exchange memory: regions are 256-byte aligned, do not overlap and
    fit exactly in exchange_bytes; every rank's map has the same shape at its own base."""
    from dsaquant_b200 import peer_exchange as px

    for cap, dim, group in ((512, 256, 2), (32768, 5120, 4), (1280, 1536, 8)):
        total = px.exchange_bytes(cap, dim, group)
        base = 0x7000_0000_0000
        m = px.layout(base, cap, dim, group)
        regions = []
        for p in range(2):
            for i in range(2):
                regions.append((m.kv[p][i], cap * dim * 2))
                regions.append((m.ready[p][i], 4 * group))
            regions.append((m.done[p], 4 * group))
        assert len(regions) == 10
        regions.sort()
        for (a, n), (b, _) in zip(regions, regions[1:]):
            assert a % 256 == 0 and a + n <= b
        last, n = regions[-1]
        assert base <= regions[0][0] and last + n <= base + total
        other = px.layout(base + (1 << 32), cap, dim, group)
        assert other.kv[1][1] - m.kv[1][1] == 1 << 32 and other.done[0] - m.done[0] == 1 << 32


def test_public_header_is_plain_c(tmp_path):
    """The drop-in boundary is a C ABI: the header must compile as C99 (and as C++) on its own,
    and a C program must link against the library through it."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    from dsaquant_b200.csrc import build as b

    src = tmp_path / "use_abi.c"
    src.write_text('#include "b200w4a4.h"\n#include <stdio.h>\n'
                   'int main(void) { printf("%d %s\\n", b200w4a4_version(), b200w4a4_strerror(-2));\n'
                   '  return b200w4a4_repack_bytes(1536, 1536) == 1536u * 768u ? 0 : 1; }\n')
    inc = str(ROOT / "include")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I", inc, str(src)],
                   check=True)
    gxx = shutil.which("g++")
    if gxx is not None:
        subprocess.run([gxx, "-std=c++11", "-fsyntax-only", "-x", "c++", "-I", inc, str(src)], check=True)
    lib = b.lib_path()
    exe = tmp_path / "use_abi"
    subprocess.run([gcc, "-std=c99", "-I", inc, str(src), "-o", str(exe), str(lib), f"-Wl,-rpath,{lib.parent}"],
                   check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.startswith("1 unsupported shape")


def test_quantiser_fast_path_bracket_is_exact():
    """CPU emulation of the quantiser's fast path (dsaquant_b200/csrc/quant_act.cuh, chunk_codes):
    two fused multiply-adds with the reciprocal nudged up / down by 2^-20 must agree whenever the
    pinned definition clamp(rint(x / s)) is not within reach of a rounding tie, and when they agree
    they must equal it.  fp64 holds the product of two fp32 numbers exactly, and adding the 1.5*2^23
    constant in one rounding is rint() of that exact product, so numpy reproduces the GPU bits."""
    import numpy as np

    rng = np.random.default_rng(5)
    one_up, one_dn = np.float32(1.0 + 2.0 ** -20), np.float32(1.0 - 2.0 ** -20)
    checked = 0
    for clip in (1.0, 0.95, 0.934, 0.5):
        amax = np.abs(rng.standard_normal(4000).astype(np.float16).astype(np.float32)) * np.float32(30.0) + np.float32(1e-3)
        s = ((np.maximum(amax, np.float32(1e-5)) / np.float32(7.0)) * np.float32(clip)).astype(np.float32)
        r = (np.float32(1.0) / s).astype(np.float32)
        r_up, r_dn = (r * one_up).astype(np.float32), (r * one_dn).astype(np.float32)
        # values spread over [-amax, amax] plus neighbours of every half-integer multiple of s
        u = (rng.uniform(-1, 1, (4000, 256)).astype(np.float32) * amax[:, None]).astype(np.float16).astype(np.float32)
        ties = (np.arange(-15, 16, 2, dtype=np.float32) * np.float32(0.5))[None, :] * s[:, None]
        near = np.concatenate([np.nextafter(ties, np.float32(np.inf)), ties, np.nextafter(ties, np.float32(-np.inf)),
                               ties.astype(np.float16).astype(np.float32)], axis=1)
        near = np.clip(near, -amax[:, None], amax[:, None]).astype(np.float32)
        x = np.concatenate([u, near], axis=1)
        want = np.clip(np.rint((x / s[:, None]).astype(np.float32)), -8, 7)
        ya = np.rint(x.astype(np.float64) * r_up[:, None].astype(np.float64))
        yb = np.rint(x.astype(np.float64) * r_dn[:, None].astype(np.float64))
        if not clip >= 0.934:
            ya, yb = np.clip(ya, -8, 7), np.clip(yb, -8, 7)
        agree = ya == yb
        assert np.array_equal(ya[agree], want[agree])
        assert agree[:, :256].mean() > 0.9999           # on ordinary values the division fallback stays rare
        assert not agree[:, 256:].all()                 # and the planted ties do reach it
        if clip >= 0.934:
            assert np.abs(ya).max() <= 7                # no clamp needed on this path
        checked += x.size
    assert checked > 4_000_000


def test_reference_fused_call_site_binds_against_this_package():
    """The reference's fused-QKV call site (modules/attention.py, `_get_qkv_projections`) imports
    names from vdm_infer.kernels.vdm_w4a4 and calls them with keyword arguments.  Read from a
    DSAQuant checkout when one is present (skipped otherwise): after install_as_vdm_infer() every
    imported name must resolve, and every call must bind against this package's signatures."""
    import ast
    import inspect
    import sys

    import dsaquant_b200
    from harness.bench_cpu import reference_checkout

    ref = reference_checkout()
    if ref is None:
        pytest.skip("no DSAQuant checkout (DSAQUANT_REFERENCE)")
    src = (Path(ref) / "vdm_infer" / "models" / "wan_vdm" / "modules" / "attention.py").read_text()
    fn = next(n for n in ast.walk(ast.parse(src)) if isinstance(n, ast.FunctionDef) and n.name == "_get_qkv_projections")
    imported = {}
    for node in ast.walk(fn):
        if isinstance(node, ast.ImportFrom) and node.module and node.module.startswith("vdm_infer."):
            for alias in node.names:
                imported[alias.asname or alias.name] = (node.module, alias.name)
    assert set(imported) >= {"linear_vdm_w4a4", "linear_vdm_w4a4_qkv"}

    saved = {k: v for k, v in sys.modules.items() if k == "vdm_infer" or k.startswith("vdm_infer.")}
    for k in saved:
        del sys.modules[k]
    try:
        dsaquant_b200.install_as_vdm_infer()
        resolved = {}
        for local, (module, name) in imported.items():
            mod = __import__(module, fromlist=[name])
            resolved[local] = getattr(mod, name)
        calls = 0
        for node in ast.walk(fn):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in resolved:
                sig = inspect.signature(resolved[node.func.id])
                sig.bind(*[object()] * len(node.args), **{kw.arg: object() for kw in node.keywords if kw.arg})
                calls += 1
        assert calls >= 2
        # the attributes the call site reads on the projection layers exist on this QuantLinear
        from vdm_infer.quantization.quant_linear import QuantLinear
        ql = QuantLinear(torch.nn.Linear(128, 128), {"w": "lsq", "act": "dynamic"}, {"w": {}, "act": {}})
        for attr in ("kernel_clip_ratio", "_bias_half"):
            assert hasattr(ql, attr)
    finally:
        for k in [k for k in sys.modules if k == "vdm_infer" or k.startswith("vdm_infer.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_cpu_arm_port_matches_the_reference_quantlinear(monkeypatch):
    """The benchmark's CPU arm: with a DSAQuant checkout it times the reference's own QuantLinear, without
    one the restatement under oracle/.  Where both exist they must compute the same thing (clip 1.0)."""
    from harness import bench_cpu
    from oracle.fakequant_cpu import fakequant_linear

    layers = [("a", 128, 256), ("b", 256, 128)]
    monkeypatch.setattr(bench_cpu, "reference_checkout", lambda: None)
    port = bench_cpu.CpuArm(layers, 32, 1.0, port_fn=fakequant_linear)
    assert port.kind == "port" and port.time(1, 0) > 0
    with pytest.raises(RuntimeError):
        bench_cpu.CpuArm(layers, 32, 1.0)              # neither a checkout nor a port: nothing to time
    monkeypatch.undo()
    if bench_cpu.reference_checkout() is None:
        pytest.skip("no DSAQuant checkout (DSAQUANT_REFERENCE)")
    ref = bench_cpu.CpuArm(layers, 32, 1.0, port_fn=fakequant_linear)
    assert ref.kind == "reference"
    with torch.no_grad():
        for (x, ql), (x2, (w, ws, b)) in zip(ref.items, port.items):
            assert torch.equal(x, x2)
            ql.aquantizer.init = False
            want = ql(x)
            # the port takes the fp16-rounded channel scale of the packed format; give it the reference's own
            got = fakequant_linear(x2, w, ql.wquantizer.scale.reshape(-1).float(), b, 1.0)
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    assert bench_cpu.sized_rows(layers, 2, 1, 1.0, port_fn=fakequant_linear, budget_s=1e-9, lo=64, hi=256) == 64


def test_reference_fused_call_site_runs_unchanged_against_these_modules(monkeypatch):
    """Executes the reference's own `_get_qkv_projections` (source text read from a DSAQuant checkout,
    compiled unchanged; skipped when there is none) on an attention object whose projections are
    this package's QuantLinear layers holding vdm_w4a4_packed_v1 buffers.  The two kernel entry
    points it imports are replaced by CPU stand-ins that decode the v1 buffers with the oracle, so the
    test covers what the call site relies on: attribute names, the concatenation of v1 buffers along
    dim 0, the cached `_vdm_qkv_*` / `_vdm_kv_*` attributes, bias handling and the split of the result."""
    import ast
    import sys

    import dsaquant_b200
    from dsaquant_b200.kernels import vdm_w4a4 as vdm
    from dsaquant_b200.quantization.quant_linear import QuantLinear
    from harness.bench_cpu import reference_checkout

    ref = reference_checkout()
    if ref is None:
        pytest.skip("no DSAQuant checkout (DSAQUANT_REFERENCE)")
    path = Path(ref) / "vdm_infer" / "models" / "wan_vdm" / "modules" / "attention.py"
    src = path.read_text()
    fn = next(n for n in ast.walk(ast.parse(src)) if isinstance(n, ast.FunctionDef) and n.name == "_get_qkv_projections")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), str(path), "exec"), ns)   # the reference's code, as it is
    ref_get_qkv = ns["_get_qkv_projections"]

    def cpu_linear(x, qweight, wscales, bias=None, clip_ratio=1.0, bias_half=None):
        codes = orc.unpack_weight_v1(qweight.numpy())
        ws = orc.unpack_wscale_v1(wscales.numpy())
        b = bias_half if bias_half is not None else bias
        shape = x.shape[:-1]
        out = orc.linear_w4a4(x.reshape(-1, x.shape[-1]).numpy(), codes, ws,
                              None if b is None else b.numpy(), clip_ratio)["out"]
        return torch.from_numpy(out).reshape(*shape, -1)

    def cpu_qkv(x, qp, qs, kp, ks, vp, vs, q_bias=None, k_bias=None, v_bias=None, clip_ratio=1.0,
                w_qkv_packed=None, w_qkv_scale=None, qkv_bias_half=None):
        assert w_qkv_packed is not None and w_qkv_scale is not None     # the call site passes its caches
        return cpu_linear(x, w_qkv_packed, w_qkv_scale, None, clip_ratio, qkv_bias_half).split(qp.shape[0], dim=-1)

    monkeypatch.setattr(vdm, "linear_vdm_w4a4", cpu_linear)
    monkeypatch.setattr(vdm, "linear_vdm_w4a4_qkv", cpu_qkv)
    saved = {k: v for k, v in sys.modules.items() if k == "vdm_infer" or k.startswith("vdm_infer.")}
    for k in saved:
        del sys.modules[k]
    try:
        dsaquant_b200.install_as_vdm_infer()
        rng = np.random.default_rng(11)
        D = 128
        for cross in (False, True):
            attn = _TinyAttn(D)
            attn.cross_attention_dim_head = 64 if cross else None
            separate = {}
            for i, name in enumerate(("to_q", "to_k", "to_v")):
                lin = getattr(attn, name)
                ql = QuantLinear(lin, {"w": "lsq", "act": "dynamic"}, {"w": {}, "act": {}})
                codes = rng.integers(-8, 8, size=(D, D), dtype=np.int8)
                ws = (np.full(D, 2.0 ** -6, np.float32) * (1 + (np.arange(D) % 3))).astype(np.float16)
                ql.register_buffer("vdm_weight_packed", torch.from_numpy(orc.pack_weight_v1(codes)))
                ql.register_buffer("vdm_weight_scale_packed", torch.from_numpy(orc.pack_wscale_v1(ws, D)))
                ql.register_buffer("vdm_weight_scale", torch.from_numpy(ws))
                ql._bias_half = torch.from_numpy(rng.standard_normal(D).astype(np.float16)) if i != 1 else None
                ql.use_vdm_kernel = True
                setattr(attn, name, ql)
                separate[name] = (codes, ws, ql._bias_half)
            attn.use_fused_qkv_kernel, attn.qkv_kernel_backend = True, "vdm"
            x = torch.from_numpy(rng.standard_normal((1, 37, D)).astype(np.float16))
            ctx = torch.from_numpy(rng.standard_normal((1, 21, D)).astype(np.float16)) if cross else None
            q, k, v = ref_get_qkv(attn, x, ctx)
            for name, got, inp in (("to_q", q, x), ("to_k", k, ctx if cross else x), ("to_v", v, ctx if cross else x)):
                codes, ws, b = separate[name]
                want = orc.linear_w4a4(inp.reshape(-1, D).numpy(), codes, ws, None if b is None else b.numpy(),
                                       attn.to_q.kernel_clip_ratio)["out"]
                np.testing.assert_array_equal(got.reshape(-1, D).numpy().view(np.uint16), want.view(np.uint16))
            cache = "_vdm_kv_weight_packed" if cross else "_vdm_qkv_weight_packed"
            assert getattr(attn, cache).shape == ((2 if cross else 3) * D, D // 2)
    finally:
        for k in [k for k in sys.modules if k == "vdm_infer" or k.startswith("vdm_infer.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_packed_checkpoint_files_interoperate_with_the_reference_modules(tmp_path):
    """vdm_w4a4_packed_v1 files cross between the two implementations (CPU; needs a DSAQuant checkout,
    skipped otherwise): a file written by this package's writer loads through the reference's
    load_packed_quantized_model into the reference's QuantLinear, a file written by the reference's
    writer loads through this package's loader, and both directions keep every buffer bit for bit."""
    import importlib
    import sys

    from dsaquant_b200.checkpoints import packed_checkpoint as mine
    from dsaquant_b200.quantization.quant_linear import QuantLinear as MyQL
    from harness.bench_cpu import reference_checkout

    ref = reference_checkout()
    if ref is None:
        pytest.skip("no DSAQuant checkout (DSAQUANT_REFERENCE)")
    saved = {k: v for k, v in sys.modules.items() if k == "vdm_infer" or k.startswith("vdm_infer.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, ref)
    try:
        theirs = importlib.import_module("vdm_infer.checkpoints.packed_checkpoint")
        RefQL = importlib.import_module("vdm_infer.quantization.quant_linear").QuantLinear
        assert theirs.PACKED_CHECKPOINT_FORMAT == mine.PACKED_CHECKPOINT_FORMAT
        assert tuple(theirs.VDM_BUFFER_SUFFIXES) == tuple(mine.VDM_BUFFER_SUFFIXES)
        rng = np.random.default_rng(21)

        def model_with(cls):
            m = _TinyModel()
            _quantize_blocks(m, cls)
            return m

        def load(module, cls, ckpt):
            m = model_with(cls)
            kw = dict(quant_linear_cls=cls, dtype=torch.float16, device=torch.device("cpu"), require_vdm_kernel=False)
            if module is mine:
                kw["repack_for_b200"] = False
            missing, unexpected = module.load_packed_quantized_model(m, ckpt, **kw)
            assert list(missing) == [] and list(unexpected) == []
            return m

        truth = {"format": mine.PACKED_CHECKPOINT_FORMAT, "metadata": {}, "model": _packed_state(model_with(MyQL), rng)}
        # this package's writer -> the reference's loader and layer class
        a = tmp_path / "mine.pt"
        mine.save_packed_checkpoint(load(mine, MyQL, truth), str(a), metadata={"by": "b200"})
        into_ref = load(theirs, RefQL, theirs.load_quant_checkpoint(str(a), None))
        # the reference's writer -> this package's loader and layer class
        b = tmp_path / "theirs.pt"
        theirs.save_packed_checkpoint(into_ref, str(b), metadata={"by": "reference"})
        into_mine = load(mine, MyQL, mine.load_quant_checkpoint(str(b), None))
        for name in ("to_q", "to_k", "to_v"):
            for suffix in mine.VDM_BUFFER_SUFFIXES:
                want = truth["model"][f"blocks.0.{name}.{suffix}"]
                assert torch.equal(getattr(getattr(into_ref.blocks[0], name), suffix), want)
                assert torch.equal(getattr(getattr(into_mine.blocks[0], name), suffix), want)
            assert getattr(into_ref.blocks[0], name).use_vdm_kernel and getattr(into_mine.blocks[0], name).use_vdm_kernel
        fa, fb = torch.load(a, weights_only=True), torch.load(b, weights_only=True)
        assert set(fa["model"]) == set(fb["model"])
        for key in fa["model"]:
            assert torch.equal(fa["model"][key], fb["model"][key]), key
    finally:
        sys.path.remove(ref)
        for k in [k for k in sys.modules if k == "vdm_infer" or k.startswith("vdm_infer.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_python_workspace_size_matches_the_library():
    from dsaquant_b200 import _lib
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    lib = _lib.load()
    for m, k in ((1, 64), (257, 1536), (300, 5120), (32760, 13824), (4095, 8960)):
        assert vdm._workspace_bytes(m, k) == lib.b200w4a4_linear_workspace_bytes(m, k)
