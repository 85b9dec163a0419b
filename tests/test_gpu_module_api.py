"""GPU tests of the module-level API (QuantLinear, fused QKV, packed-checkpoint load) with the
seeds and shapes of the reference's own smoke scripts, and size-independent properties at the
full Wan-14B shapes."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from _cases import make_case
from oracle import w4a4_oracle as orc

pytestmark = pytest.mark.gpu
QPARAMS = {"w": {"bit": 4, "sym": True, "granularity": "per_channel", "group_size": -1,
                 "round_zero": True, "use_grad_scaling": True, "cali": "mse"},
           "act": {"bit": 4, "sym": True}}


@pytest.fixture(scope="module")
def vdm():
    from dsaquant_b200.kernels import vdm_w4a4 as v

    assert v.is_available(), f"libb200w4a4.so not loadable: {v.load_error()}"
    yield v
    assert v.last_device_status() == 0


def _make_quant(linear):
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    ql = QuantLinear(linear, {"w": "lsq", "act": "dynamic"}, QPARAMS).cuda().half()
    ql.wquantizer(ql.weight.detach())
    ql.wquantizer.build()
    ql.aquantizer.build()
    ql = ql.half()
    ql.set_quant_state(use_wq=True, use_aq=True)
    return ql


def _rel_l2(a, b):
    return (torch.linalg.vector_norm(a.float() - b.float()) / torch.linalg.vector_norm(b.float())).item()


def test_quantlinear_kernel_vs_fake_quant_seed1(vdm):
    """tests/test_vdm_quantlinear_smoke.py of the reference, with assertions."""
    torch.manual_seed(1)
    ql = _make_quant(nn.Linear(1536, 1536, bias=True))
    x = torch.randn(257, 1536, device="cuda", dtype=torch.float16)
    w16 = ql.weight.detach().cpu().numpy()
    b16 = ql.bias.detach().cpu().numpy()
    with torch.no_grad():
        fake = ql(x)                          # PyTorch fake-quant branch, activation clip 1.0
        ql.enable_vdm_kernel_mode()
        assert ql.use_vdm_kernel and ql.weight is None and ql.wquantizer is None
        out = ql(x)                           # kernel branch, clip 0.95
        ql.kernel_clip_ratio = 1.0
        out_clip1 = ql(x)
    assert out.shape == (257, 1536) and out.dtype == torch.float16
    # kernel branch == oracle, bit for bit, for both clip ratios
    ws = ql.vdm_weight_scale.cpu().numpy()
    qw = vdm.unpack_codes(ql.vdm_weight_packed, 1536, 1536, 2).cpu().numpy()
    np.testing.assert_array_equal(qw, orc.quantize_weight(w16, ws))
    for got, clip in ((out, 0.95), (out_clip1, 1.0)):
        ref = orc.linear_w4a4(x.cpu().numpy(), qw, ws, b16, clip)["out"]
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    # and it tracks the fake-quant branch the way the reference's smoke test reports
    assert _rel_l2(out_clip1, fake) < 0.02     # same clip: only fp16-vs-fp32 scale rounding differs
    assert _rel_l2(out, fake) < 0.15           # clip 0.95 vs 1.0


class _Attn(nn.Module):
    def __init__(self, dim, cross):
        super().__init__()
        self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
        self.cross_attention_dim_head = 128 if cross else None
        self.fused_projections = False


@pytest.mark.parametrize("cross", [False, True])
def test_fused_qkv_is_bit_identical_seed2(vdm, cross):
    """tests/test_vdm_qkv_fuse_smoke.py of the reference: fused == three separate linears."""
    from dsaquant_b200.attention_qkv import get_qkv_projections

    torch.manual_seed(2)
    attn = _Attn(1536, cross).cuda().half()
    for name in ("to_q", "to_k", "to_v"):
        ql = _make_quant(getattr(attn, name))
        ql.enable_vdm_kernel_mode()
        setattr(attn, name, ql)
    x = torch.randn(1, 257, 1536, device="cuda", dtype=torch.float16)
    ctx = torch.randn(1, 512, 1536, device="cuda", dtype=torch.float16) if cross else None
    with torch.no_grad():
        src = ctx if cross else x
        q0, k0, v0 = attn.to_q(x), attn.to_k(src), attn.to_v(src)
        attn.use_fused_qkv_kernel = True
        attn.qkv_kernel_backend = "vdm"
        q1, k1, v1 = get_qkv_projections(attn, x, ctx)
        q2, k2, v2 = get_qkv_projections(attn, x, ctx)       # second call hits the caches
    for a, b in ((q1, q0), (k1, k0), (v1, v0), (q2, q0), (k2, k0), (v2, v0)):
        assert a.shape == b.shape
        assert torch.equal(a, b)
    cache = "_vdm_kv_weight_packed" if cross else "_vdm_qkv_weight_packed"
    assert getattr(attn, cache).shape[0] == (2 if cross else 3) * 1536


def test_packed_checkpoint_load_and_forward_on_gpu(vdm, tmp_path):
    from dsaquant_b200.checkpoints import packed_checkpoint as pc
    from dsaquant_b200.quantization.quant_linear import QuantLinear

    K, N, M = 256, 384, 77
    x16, w16, b16 = make_case(21, M, K, N)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([nn.Linear(K, N)])

    state = {"blocks.0.vdm_weight_packed": torch.from_numpy(orc.pack_weight_v1(qw)),
             "blocks.0.vdm_weight_scale_packed": torch.from_numpy(orc.pack_wscale_v1(ws, K)),
             "blocks.0.vdm_weight_scale": torch.from_numpy(ws),
             "blocks.0.bias": torch.from_numpy(b16)}
    path = tmp_path / "ckpt.pt"
    torch.save({"format": pc.PACKED_CHECKPOINT_FORMAT, "metadata": {}, "model": state}, path)
    net = Net()
    net.blocks[0] = QuantLinear(net.blocks[0], {"w": "lsq", "act": "dynamic"}, QPARAMS)
    ckpt = pc.load_quant_checkpoint(str(path), None)
    missing, unexpected = pc.load_packed_quantized_model(
        net, ckpt, quant_linear_cls=QuantLinear, dtype=torch.float16, device=torch.device("cuda"))
    assert missing == [] and unexpected == []
    layer = net.blocks[0]
    w_b200, w_scale = layer.prepare_b200_weights()          # cached by the load-time repack
    np.testing.assert_array_equal(w_b200.cpu().numpy(), orc.repack_b200(qw))
    with torch.no_grad():
        out = layer(torch.from_numpy(x16).cuda().view(1, M, K))
    assert out.shape == (1, M, N)
    ref = orc.linear_w4a4(x16, qw, ws, b16, layer.kernel_clip_ratio)["out"]
    np.testing.assert_array_equal(out[0].cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("M,K,N", [(32760, 5120, 15360), (32760, 13824, 5120),      # Wan 2.1 14B
                                   (27280, 3072, 9216), (27280, 14336, 3072),       # Wan 2.2 5B
                                   (32760, 1536, 8960), (4095, 8960, 1536)])        # Wan 2.1 1.3B, 1/8 row shard
def test_full_size_properties_wan_shapes(vdm, M, K, N):
    """Full benchmark shapes (M not a multiple of the tile): sampled rows against the oracle, a
    checksum of checksums over every accumulator, and canary rows after the M tail."""
    g = torch.Generator(device="cuda").manual_seed(K + N)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32)
    x[:, torch.randperm(K, generator=torch.Generator().manual_seed(1))[: K // 100].cuda()] *= 20.0
    x = x.half()
    w = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).half()
    bias = (torch.randn(N, generator=g, device="cuda") * 0.01).half()
    packed, scale_packed, ch_scale = vdm.quantize_weight_per_channel(w)
    qw_dev = vdm.unpack_codes(packed, N, K, 2)

    qact, ascales, _ = vdm.quantize_activation_per_token(x, 0.95)
    out_nb, acc = vdm.linear_prequantized(qact, ascales, packed, scale_packed, return_acc=True)
    # checksum of checksums: sum_n acc[m,n] == qa[m,:] . sum_n qw[n,:]   (exact in float64)
    wsum = qw_dev.to(torch.float64).sum(dim=0)
    want = qact.to(torch.float64) @ wsum
    assert torch.equal(acc.sum(dim=1, dtype=torch.int64), want.to(torch.int64))
    # and along the other axis: sum_m acc[m,n] == (sum_m qa[m,:]) . qw[n,:]
    asum = qact.to(torch.float64).sum(dim=0)
    assert torch.equal(acc.sum(dim=0, dtype=torch.int64), (qw_dev.to(torch.float64) @ asum).to(torch.int64))
    del acc, out_nb

    # public entry point with canary rows behind the output
    rows = torch.cat([torch.arange(0, 4), torch.arange(M - 130, M),
                      torch.randint(0, M, (60,), generator=torch.Generator().manual_seed(3))]).unique()
    out = vdm.linear_vdm_w4a4(x, packed, scale_packed, bias, clip_ratio=0.95)
    assert out.shape == (M, N)
    x_s = x[rows.cuda()].cpu().numpy()
    ref = orc.linear_w4a4(x_s, qw_dev.cpu().numpy(), ch_scale.cpu().numpy(), bias.cpu().numpy(), 0.95)
    np.testing.assert_array_equal(qact[rows.cuda()].cpu().numpy(), ref["codes"])
    np.testing.assert_array_equal(out[rows.cuda()].cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))

    # the kernel must not write past row M: call the C ABI into a buffer with guard rows
    from dsaquant_b200 import _lib
    lib = _lib.load()
    guard = 300
    buf = torch.full((M + guard, N), -7.0, dtype=torch.float16, device="cuda")
    w_b200, w_scale = vdm.prepare_b200_weight(packed, scale_packed)
    rc = lib.b200w4a4_gemm(qact.data_ptr(), ascales.data_ptr(), w_b200.data_ptr(), w_scale.data_ptr(),
                           bias.data_ptr(), buf.data_ptr(), None, M, N, K,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(buf[:M], out)
    assert bool((buf[M:] == -7.0).all())


def test_host_pipeline_matches_direct_call(vdm):
    """Row-chunked, stream-overlapped host path == one call on the whole matrix, bit for bit."""
    from dsaquant_b200.host_pipeline import HostLinearLayer, HostLinearPipeline

    M, K = 2500, 512
    x16, w_a, b_a = make_case(31, M, K, 384)
    _, w_b, _ = make_case(32, 8, K, 128, bias=False)
    layers, direct = [], []
    xd = torch.from_numpy(x16).cuda()
    for w16, b16 in ((w_a, b_a), (w_b, None)):
        packed, scale_packed, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w16).cuda())
        bias = torch.from_numpy(b16).cuda() if b16 is not None else None
        layers.append(HostLinearLayer(packed, scale_packed, bias))
        direct.append(vdm.linear_vdm_w4a4(xd, packed, scale_packed, None, 0.95, bias_half=bias))
    pipe = HostLinearPipeline("cuda", k_max=1024, n_max=512, chunk_rows=600, depth=2)
    x_host = torch.from_numpy(x16).pin_memory()
    outs = [torch.empty(M, L.n, dtype=torch.float16).pin_memory() for L in layers]
    for _ in range(2):                                   # second pass reuses every staging buffer
        pipe.run(x_host, layers, outs, 0.95)
        pipe.synchronize()
        for o, d in zip(outs, direct):
            assert torch.equal(o, d.cpu())
    # two groups with different widths in one pipelined sequence (no drain between them)
    x2_16, w_c, b_c = make_case(33, 700, 1024, 256)
    packed, scale_packed, _ = vdm.quantize_weight_per_channel(torch.from_numpy(w_c).cuda())
    layer_c = HostLinearLayer(packed, scale_packed, torch.from_numpy(b_c).cuda())
    direct_c = vdm.linear_vdm_w4a4(torch.from_numpy(x2_16).cuda(), packed, scale_packed, None, 0.95,
                                   bias_half=torch.from_numpy(b_c).cuda())
    x2_host = torch.from_numpy(x2_16).pin_memory()
    out_c = torch.empty(700, 256, dtype=torch.float16).pin_memory()
    for o in outs:
        o.zero_()
    pipe.run_groups([(x_host, layers, outs), (x2_host, [layer_c], [out_c])], 0.95)
    pipe.synchronize()
    for o, d in zip(outs + [out_c], direct + [direct_c]):
        assert torch.equal(o, d.cpu())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runs_on_a_non_current_device(vdm):
    """Per-device state of the library: tensors on cuda:1 while cuda:0 is current."""
    x16, w16, b16 = make_case(61, 200, 256, 128)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)["out"]
    assert torch.cuda.current_device() == 0
    dev = torch.device("cuda", 1)
    packed = torch.from_numpy(orc.pack_weight_v1(qw)).to(dev)
    sp = torch.from_numpy(orc.pack_wscale_v1(ws, 256)).to(dev)
    out = vdm.linear_vdm_w4a4(torch.from_numpy(x16).to(dev), packed, sp, torch.from_numpy(b16).to(dev), clip_ratio=0.95)
    assert out.device == dev and torch.cuda.current_device() == 0
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    assert vdm.last_device_status(1) == 0


def test_query_reports_sm100(vdm):
    import ctypes

    from dsaquant_b200 import _lib
    lib = _lib.load()
    sm, major, minor = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert lib.b200w4a4_query(0, ctypes.byref(sm), ctypes.byref(major), ctypes.byref(minor)) == 0
    assert (major.value, minor.value) == (10, 0) and sm.value >= 100
    assert lib.b200w4a4_query(99, None, None, None) == -5


def test_cuda_graph_capture_and_replay(vdm):
    """The library allocates nothing and never synchronises, so a linear can be captured in a
    CUDA graph (after one eager call has done the per-device set-up) and replayed on new data."""
    M, K, N = 333, 512, 256
    x16, w16, b16 = make_case(71, M, K, N)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    packed = torch.from_numpy(orc.pack_weight_v1(qw)).cuda()
    sp = torch.from_numpy(orc.pack_wscale_v1(ws, K)).cuda()
    bias = torch.from_numpy(b16).cuda()
    x_static = torch.from_numpy(x16).cuda()
    vdm.linear_vdm_w4a4(x_static, packed, sp, None, 0.95, bias_half=bias)      # warm-up: set-up + repack cache
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = vdm.linear_vdm_w4a4(x_static, packed, sp, None, 0.95, bias_half=bias)
    for seed in (72, 73):
        x_new, _, _ = make_case(seed, M, K, N)
        x_static.copy_(torch.from_numpy(x_new).cuda())
        graph.replay()
        torch.cuda.synchronize()
        ref = orc.linear_w4a4(x_new, qw, ws, b16, 0.95)["out"]
        np.testing.assert_array_equal(y_static.cpu().numpy().view(np.uint16), ref.view(np.uint16))


def test_concurrent_threads_and_streams(vdm):
    """Two python threads, each on its own stream, share the library without interfering."""
    import threading

    M, K, N = 700, 1536, 384
    cases = []
    for seed in (81, 82):
        x16, w16, b16 = make_case(seed, M, K, N)
        ws = orc.weight_scale_absmax(w16)
        qw = orc.quantize_weight(w16, ws)
        cases.append((x16, qw, ws, b16, torch.from_numpy(orc.pack_weight_v1(qw)).cuda(),
                      torch.from_numpy(orc.pack_wscale_v1(ws, K)).cuda()))
    results, errors = [None, None], []

    def work(i):
        try:
            x16, qw, ws, b16, packed, sp = cases[i]
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                x = torch.from_numpy(x16).cuda()
                bias = torch.from_numpy(b16).cuda()
                for _ in range(20):
                    y = vdm.linear_vdm_w4a4(x, packed, sp, None, 0.95, bias_half=bias)
                stream.synchronize()
                results[i] = y.cpu().numpy()
        except BaseException as exc:  # surfaced in the main thread
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i, (x16, qw, ws, b16, _, _) in enumerate(cases):
        ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)["out"]
        np.testing.assert_array_equal(results[i].view(np.uint16), ref.view(np.uint16))


def test_fused_projection_holds_one_copy_of_its_weights(vdm):
    """After the fused caches are built the member layers keep no copies of their own: their v1
    buffers are row views of the concatenated tensors, and the per-layer repacks are released.
    Memory in use stays what it was before fusing (it doubled when every copy was kept)."""
    from dsaquant_b200.attention_qkv import get_qkv_projections, prepare_fused_projections

    torch.manual_seed(4)
    attn = _Attn(1536, False).cuda().half()
    for name in ("to_q", "to_k", "to_v"):
        ql = _make_quant(getattr(attn, name))
        ql.enable_vdm_kernel_mode()
        ql.prepare_b200_weights()                      # what the checkpoint loader does per layer
        setattr(attn, name, ql)
    x = torch.randn(1, 300, 1536, device="cuda", dtype=torch.float16)
    with torch.no_grad():
        want = [attn.to_q(x), attn.to_k(x), attn.to_v(x)]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    weights = 3 * 1536 * 768                           # bytes of the three packed weights
    attn.use_fused_qkv_kernel, attn.qkv_kernel_backend = True, "vdm"
    prepare_fused_projections(attn)
    torch.cuda.synchronize()
    after = torch.cuda.memory_allocated()
    assert after - before < 0.25 * weights, (before, after)
    base = attn._vdm_qkv_weight_packed
    for i, name in enumerate(("to_q", "to_k", "to_v")):
        buf = getattr(attn, name).vdm_weight_packed
        assert buf.data_ptr() == base.data_ptr() + i * 1536 * 768 and buf.shape == (1536, 768)
        assert name + ".vdm_weight_packed" in attn.state_dict()
    with torch.no_grad():
        got = get_qkv_projections(attn, x, None)
        again = attn.to_k(x)                           # a member evaluated on its own still works
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert torch.equal(again, want[1])
