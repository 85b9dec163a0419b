"""qk_norm_rope_push + wait_flags: the K/V exchange of a row-sharded attention group done by the
producing kernel (stores to every rank's gather buffer, then a completion flag) instead of a
separate all-gather.  One GPU stands in for the whole group here: every "rank" owns a buffer, a
flag array and a ticket in the same device memory and the ranks' kernels run one after the other on
one stream, so no kernel ever waits for another one.  The time-out path is exercised with a flag
that nothing sets."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from dsaquant_b200 import attention_qkv as aq
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    assert vdm.is_available(), vdm.load_error()
    yield aq, vdm
    assert vdm.last_device_status() == 0


@pytest.mark.parametrize("ranks,D,heads", [(4, 1536, 12), (2, 5120, 40), (8, 256, 2)])
def test_group_exchange_emulated_on_one_gpu(mods, ranks, D, heads):
    aq, vdm = mods
    from dsaquant_b200.sharding import row_partition

    total = 2048 + 77
    parts = row_partition(total, ranks)
    hd = D // heads
    g = torch.Generator(device="cuda").manual_seed(ranks + D)
    x = torch.randn(total, D, generator=g, device="cuda").half()
    w = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).half()
    ang = torch.rand(total, 1, hd // 2, generator=g, device="cuda") * 6.28
    cs = aq.rope_cos_sin(torch.polar(torch.ones_like(ang), ang))
    bufs = [torch.full((total, D), -3.0, dtype=torch.bfloat16, device="cuda") for _ in range(ranks)]
    flags = [torch.zeros(ranks, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    tickets = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    for epoch in (1, 2):
        if epoch == 2:
            x = (x.float() * 0.5 + 0.25).half()
        want = aq.qk_norm_rope(x, w, cs, 1e-6, hd, torch.bfloat16)
        for r, (s, e) in enumerate(parts):
            if e == s:
                continue
            aq.qk_norm_rope_push(x[s:e], w, cs[s:e], 1e-6, hd, [b.data_ptr() for b in bufs], D, s, torch.bfloat16,
                                 flag_ptrs=[f.data_ptr() for f in flags], flag_index=r, epoch=epoch, ticket=tickets[r])
        live = [r for r, (s, e) in enumerate(parts) if e > s]
        for r in range(ranks):
            # every rank waits for the ranks that sent something (empty shards raise no flag)
            aq.wait_flags(flags[r][:len(live)] if live == list(range(len(live))) else flags[r], epoch, 200)
        torch.cuda.synchronize()
        assert vdm.last_device_status() == 0
        for r in range(ranks):
            assert torch.equal(bufs[r], want)
            assert (flags[r][live] == epoch).all()
            assert int(tickets[r].item()) == 0


def test_wait_that_runs_out_reports_a_status_and_leaves_the_context_usable(mods):
    aq, vdm = mods
    flags = torch.zeros(3, dtype=torch.int32, device="cuda")
    flags[0] = 7
    aq.wait_flags(flags, 7, timeout_ms=30)            # flags 1 and 2 never reach 7
    torch.cuda.synchronize()
    assert vdm.last_device_status() == 105
    assert vdm.last_device_status() == 0              # read-and-clear
    flags.fill_(9)                                    # later epochs pass (>= comparison)
    aq.wait_flags(flags, 8, timeout_ms=30)
    x = torch.randn(64, 256, device="cuda").half()
    assert torch.equal(aq.qk_norm_rope(x, None, None, 1e-6, 128, torch.float16), x)
    assert vdm.last_device_status() == 0


def test_push_argument_checks(mods):
    aq, _ = mods
    from dsaquant_b200 import _lib

    lib = _lib.load()
    x = torch.zeros(8, 256, dtype=torch.float16, device="cuda")
    o = torch.zeros(8, 256, dtype=torch.float16, device="cuda")
    t = torch.zeros(1, dtype=torch.int32, device="cuda")
    f = torch.zeros(4, dtype=torch.int32, device="cuda")
    outs9 = (ctypes.c_void_p * 9)(*[o.data_ptr()] * 9)
    flg = (ctypes.c_void_p * 9)(*[f.data_ptr()] * 9)
    call = lib.b200w4a4_qk_norm_rope_push
    assert call(x.data_ptr(), 256, None, None, 1e-6, 128, outs9, 9, 0, 256, 0, None, 0, 0, None, 8, 256, None) == -1
    assert call(x.data_ptr(), 256, None, None, 1e-6, 128, outs9, 0, 0, 256, 0, None, 0, 0, None, 8, 256, None) == -1
    assert call(x.data_ptr(), 256, None, None, 1e-6, 128, outs9, 2, 0, 256, 0, flg, 0, 1, None, 8, 256, None) == -1
    assert call(x.data_ptr(), 256, None, None, 1e-6, 128, outs9, 2, 0, 256, -1, None, 0, 0, None, 8, 256, None) == -1
    assert lib.b200w4a4_wait_flags(f.data_ptr(), 33, 1, 10, None) == -1
    assert lib.b200w4a4_wait_flags(f.data_ptr(), 4, 1, 0, None) == -1
    with pytest.raises(ValueError):
        aq.qk_norm_rope_push(x, None, None, 1e-6, 128, [o.data_ptr()], 256, 0, torch.float16, flag_ptrs=[f.data_ptr()])
    # plain two-destination push without flags
    o2 = torch.ones(8, 256, dtype=torch.float16, device="cuda")
    xr = torch.randn(8, 256, device="cuda").half()
    aq.qk_norm_rope_push(xr, None, None, 1e-6, 128, [o.data_ptr(), o2.data_ptr()], 256, 0, torch.float16)
    assert torch.equal(o, xr) and torch.equal(o2, xr)


@pytest.mark.parametrize("ranks", [2, 4])
def test_exchange_protocol_over_several_blocks_emulated(mods, ranks):
    """PeerKVExchange bookkeeping (epochs, the two buffer sets, ready / done flags) with every rank of
    the group living in this process: four consecutive attention blocks, results equal to the
    single-call kernel on the whole matrix, no wait runs out."""
    aq, vdm = mods
    from dsaquant_b200 import peer_exchange as px
    from dsaquant_b200.sharding import row_partition, shard_capacity

    D, heads, total = 512, 4, 1500
    hd = D // heads
    parts = row_partition(total, ranks)
    cap = shard_capacity(total, ranks) * ranks
    senders = sum(1 for s, e in parts if e > s)
    mem = [torch.zeros(px.exchange_bytes(cap, D, ranks), dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    members = [px.layout(m.data_ptr(), cap, D, ranks) for m in mem]
    group = [px.PeerKVExchange(r, members, mem[r], cap, D, parts[r][0], timeout_ms=200) for r in range(ranks)]
    g = torch.Generator(device="cuda").manual_seed(ranks)
    w = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).half()
    ang = torch.rand(total, 1, hd // 2, generator=g, device="cuda") * 6.28
    cs = aq.rope_cos_sin(torch.polar(torch.ones_like(ang), ang))
    for block in range(4):
        k = torch.randn(total, D, generator=g, device="cuda").half()
        v = torch.randn(total, D, generator=g, device="cuda").half()
        want_k = aq.qk_norm_rope(k, w, cs, 1e-6, hd)
        want_v = v.to(torch.bfloat16)
        for ex in group:
            assert ex.begin_block() == block + 1
        for r, ex in enumerate(group):
            s, e = parts[r]
            if e > s:
                ex.push("v", v[s:e], None, None, 1e-6, hd)
                ex.push("k", k[s:e], w, cs[s:e], 1e-6, hd)
        for ex in group:
            got_k, got_v = ex.gathered(total, senders)
            assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
        for ex in group:
            ex.end_block()
    torch.cuda.synchronize()
    assert vdm.last_device_status() == 0


def test_exchange_reports_a_missing_peer(mods):
    aq, vdm = mods
    from dsaquant_b200 import peer_exchange as px

    D, ranks, cap = 256, 2, 512
    mem = [torch.zeros(px.exchange_bytes(cap, D, ranks), dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    members = [px.layout(m.data_ptr(), cap, D, ranks) for m in mem]
    ex0 = px.PeerKVExchange(0, members, mem[0], cap, D, 0, timeout_ms=30)
    ex0.begin_block()
    x = torch.randn(256, D, device="cuda").half()
    ex0.push("v", x, None, None, 1e-6, 128)
    ex0.push("k", x, None, None, 1e-6, 128)
    ex0.gathered(512)                                  # rank 1 never pushes: both waits run out
    torch.cuda.synchronize()
    assert vdm.last_device_status() == 105
    with pytest.raises(ValueError):
        ex0.push("k", torch.zeros(600, D, device="cuda").half(), None, None, 1e-6, 128)


def test_unread_timeout_does_not_cancel_later_gemms(mods):
    """The status word is a report, not a kill switch: a wait_flags time-out that the host has not
    read yet must not make a later GEMM drain early.  The GEMM stays bit-exact, check_device
    answers EDEVICE, and the code is still there to be read (and cleared) afterwards."""
    import numpy as np

    from _cases import make_case
    from dsaquant_b200 import _lib
    from oracle import w4a4_oracle as orc

    aq, vdm = mods
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    aq.wait_flags(flags, 5, timeout_ms=30)            # nothing ever sets these flags
    torch.cuda.synchronize()                          # the time-out is recorded, and deliberately not read

    M, K, N = 3000, 1536, 1536                        # 72 tiles of 12 k-blocks: many barrier waits that spin
    x16, w16, b16 = make_case(77, M, K, N)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    qweight = torch.from_numpy(orc.pack_weight_v1(qw)).cuda()
    wscales = torch.from_numpy(orc.pack_wscale_v1(ws, K)).cuda()
    for cg in (2, 1):
        prev = vdm.set_cta_group(cg)
        try:
            out = vdm.linear_vdm_w4a4(torch.from_numpy(x16).cuda(), qweight, wscales, torch.from_numpy(b16).cuda(), 0.95)
        finally:
            vdm.set_cta_group(prev)
        ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)
        np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))
    with pytest.raises(_lib.B200W4A4Error) as err:
        vdm.check_device()
    assert err.value.code == -7
    assert vdm.last_device_status() == 105            # still readable, cleared by this read
    vdm.check_device()                                # clean again


@pytest.mark.parametrize("ranks", [2, 4])
def test_rotated_placement_puts_own_rows_first_emulated(mods, ranks):
    """Rotated placement of PeerKVExchange (own shard at row 0, peers after it in ascending rank order):
    on every emulated rank the local range is its own shard and the remote range is the other shards,
    in order, without holes (the last shard is shorter); and attention over local + remote keys merged
    by log-sum-exp equals attention over all keys in their natural order."""
    aq, vdm = mods
    from dsaquant_b200 import peer_exchange as px
    from dsaquant_b200.sharding import row_partition, shard_capacity
    from harness import wan_dit

    D, heads, total = 512, 4, 1900
    hd = D // heads
    parts = row_partition(total, ranks)
    rows = [e - s for s, e in parts]                  # 1024 + 876, or 512 x 3 + 364
    assert min(rows) > 0 and rows[-1] < rows[0]
    cap = shard_capacity(total, ranks) * ranks
    mem = [torch.zeros(px.exchange_bytes(cap, D, ranks), dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    members = [px.layout(m.data_ptr(), cap, D, ranks) for m in mem]
    group = [px.PeerKVExchange(r, members, mem[r], cap, D, parts[r][0], timeout_ms=200, shard_rows=rows) for r in range(ranks)]
    for ex in group:
        ex.set_rotated(True)
    g = torch.Generator(device="cuda").manual_seed(10 + ranks)
    for block in range(3):
        k = torch.randn(total, D, generator=g, device="cuda").half()
        v = torch.randn(total, D, generator=g, device="cuda").half()
        want_k, want_v = k.to(torch.bfloat16), v.to(torch.bfloat16)
        for ex in group:
            ex.begin_block()
        for r, ex in enumerate(group):
            s, e = parts[r]
            ex.push("v", v[s:e], None, None, 1e-6, hd)
            ex.push("k", k[s:e], None, None, 1e-6, hd)
        for r, ex in enumerate(group):
            s, e = parts[r]
            lk, lv = ex.local_rows()
            rk, rv = ex.remote_rows()
            others = torch.cat([want_k[a:b] for x, (a, b) in enumerate(parts) if x != r])
            assert torch.equal(lk, want_k[s:e]) and torch.equal(lv, want_v[s:e])
            assert torch.equal(rk, others) and rk.shape[0] == total - (e - s)
            assert torch.equal(rv, torch.cat([want_v[a:b] for x, (a, b) in enumerate(parts) if x != r]))
            if block == 0:
                q = torch.randn(1, heads, 200, hd, generator=g, device="cuda").to(torch.bfloat16)
                split = lambda t: t.view(1, -1, heads, hd).transpose(1, 2)
                o1, l1 = wan_dit.sdpa_with_lse(q, split(lk), split(lv))
                o2, l2 = wan_dit.sdpa_with_lse(q, split(rk), split(rv))
                merged = wan_dit.merge_attention(o1, l1, o2, l2)
                # the library's one-pass merge kernel against the PyTorch formula
                fused = aq.merge_attention(o1, l1, o2, l2)
                assert fused.shape == (200, D) and fused.dtype == torch.bfloat16
                want_m = merged.transpose(1, 2).reshape(200, D).float()
                assert (fused.float() - want_m).abs().max().item() <= 2 ** -7 * want_m.abs().max().item()
                full = torch.nn.functional.scaled_dot_product_attention(q, split(want_k), split(want_v))
                assert (merged.float() - full.float()).abs().max().item() < 2e-2
                cos = torch.nn.functional.cosine_similarity(merged.float().flatten(), full.float().flatten(), dim=0)
                assert cos.item() > 0.9999
        for ex in group:
            ex.end_block()
    torch.cuda.synchronize()
    assert vdm.last_device_status() == 0
