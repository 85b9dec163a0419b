"""The CPU oracle against fixtures produced by the reference's own PyTorch W4A4 path
(tests/golden/make_golden.py) and against its own layout round trips.  CPU only."""
from pathlib import Path

import numpy as np
import pytest

from _cases import CASES, digest, make_case
from oracle import w4a4_oracle as orc

GOLD = Path(__file__).resolve().parent / "golden"


def _load(name):
    return np.load(GOLD / f"{name}.npz")


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_fixture(name):
    seed, M, K, N, kw, clip = CASES[name]
    g = _load(name)
    x16, w16, b16 = make_case(seed, M, K, N, **kw)
    assert str(g["input_digest"]) == digest(x16, w16, b16), "seeded inputs drifted from the fixture"
    assert float(g["clip"]) == np.float32(clip)

    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    r = orc.linear_w4a4(x16, qw, ws, b16, clip)
    np.testing.assert_array_equal(ws, g["w_scale"])
    np.testing.assert_array_equal(r["a_scale"], g["a_scale"])          # bit-exact fp32 scales
    if "a_codes" in g.files:
        np.testing.assert_array_equal(r["codes"], g["a_codes"])
        np.testing.assert_array_equal(qw, g["w_codes"])
        np.testing.assert_array_equal(r["acc"], g["acc"])
        ref = g["ref_out_f32"]
        acc_s = r["acc"]
    else:
        assert digest(r["codes"]) == str(g["a_codes_digest"])
        assert digest(qw) == str(g["w_codes_digest"])
        assert digest(r["acc"]) == str(g["acc_digest"])
        np.testing.assert_array_equal(r["acc"][::61, ::53], g["acc_sample"])
        ref = g["ref_out_f32_sample"]
        acc_s = None
    out = r["out"].astype(np.float32)
    if acc_s is None:
        out = out[::61, ::53]
    # The reference fake-quant output is an fp32 GEMM of dequantised values; the oracle rounds
    # an exact integer result once to fp16: 1e-2 relative / 5e-3 absolute per element.
    np.testing.assert_allclose(out, ref, rtol=1e-2, atol=5e-3)


def test_ties_round_to_even_and_clamp():
    # scale = 7/7 = 1 -> x/scale = x; halves must round to even, range clamps at -8/7.
    x = np.array([[7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 6.5, -5.5, -6.5, 3.49, -3.51] + [0.0] * 52],
                 np.float32)
    q, s = orc.quantize_act(x, 1.0)
    assert s[0] == np.float32(1.0)
    assert q[0, :12].tolist() == [7, 0, 2, 2, 0, -2, -2, 6, -6, -6, 3, -4]
    q2, s2 = orc.quantize_act(-x, 0.5)      # clip 0.5 halves the scale: +-7 -> +-14 -> clamped
    assert s2[0] == np.float32(0.5) and q2[0, 0] == -8 and q2.max() == 7 and q2.min() == -8


def test_zero_row_uses_floor_scale():
    x = np.zeros((3, 64), np.float32)
    q, s = orc.quantize_act(x, 0.95)
    assert np.all(q == 0)
    np.testing.assert_array_equal(s, np.full(3, np.float32(np.float32(1e-5) / np.float32(7)) * np.float32(0.95)))


@pytest.mark.parametrize("N,K", [(128, 64), (256, 192), (384, 1536)])
def test_v1_layout_round_trip_and_closed_form(N, K):
    rng = np.random.default_rng(N * 7 + K)
    codes = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    packed = orc.pack_weight_v1(codes)
    assert packed.shape == (N, K // 2) and packed.dtype == np.uint8
    np.testing.assert_array_equal(orc.unpack_weight_v1(packed), codes)
    # Spot-check the closed form against an independent lane-level walk of one 16-byte entry.
    flat = packed.reshape(-1).view(np.uint32).reshape(-1, 4)
    bn, bk, tile, lane = (N // 128 - 1), (K // 64 - 1), 5, 22
    entry = flat[((bn * (K // 64) + bk) * 8 + tile) * 32 + lane]
    n0, k0 = bn * 128 + tile * 16 + lane // 4, bk * 64 + (lane % 4) * 8
    for word, (n, k) in enumerate([(n0, k0), (n0, k0 + 32), (n0 + 8, k0), (n0 + 8, k0 + 32)]):
        nibs = [(int(entry[word]) >> (4 * e)) & 0xF for e in range(8)]
        assert nibs == [int(c) & 0xF for c in codes[n, k:k + 8]]
    # Concatenating packed tensors along dim 0 equals packing the concatenated codes (fused QKV).
    other = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    cat = np.concatenate([packed, orc.pack_weight_v1(other)], axis=0)
    np.testing.assert_array_equal(cat, orc.pack_weight_v1(np.concatenate([codes, other], axis=0)))


def test_v1_scale_layout():
    N, K = 256, 192
    s = (np.arange(N) + 1).astype(np.float16)
    sp = orc.pack_wscale_v1(s, K)
    assert sp.shape == (N, K // 64)
    np.testing.assert_array_equal(orc.unpack_wscale_v1(sp), s)
    flat = sp.reshape(-1).reshape(N // 128, K // 64, 32, 4)
    for bn, bk, lane in [(0, 0, 0), (1, 2, 13), (1, 1, 31)]:
        base = bn * 128 + (lane // 4) * 16 + (lane % 4) * 2
        np.testing.assert_array_equal(flat[bn, bk, lane], s[[base, base + 1, base + 8, base + 9]])


def test_b200_weight_layout_round_trip():
    rng = np.random.default_rng(5)
    codes = rng.integers(-8, 8, size=(128, 256), dtype=np.int8)
    wr = orc.repack_b200(codes)
    np.testing.assert_array_equal(orc.unpack_b200(wr), codes)
    # byte i of a 16-byte run: high nibble k32+i, low nibble k32+16+i; x16 trick of the GEMM.
    b = int(wr[3, 16 + 5])
    assert (b >> 4) == (int(codes[3, 32 + 5]) & 0xF) and (b & 0xF) == (int(codes[3, 32 + 16 + 5]) & 0xF)
    assert np.int8(np.uint8(b & 0xF0)) == 16 * codes[3, 32 + 5]
    assert np.int8(np.uint8((b << 4) & 0xF0)) == 16 * codes[3, 32 + 16 + 5]


def test_nibble_rows_round_trip():
    rng = np.random.default_rng(6)
    codes = rng.integers(-8, 8, size=(5, 64), dtype=np.int8)
    np.testing.assert_array_equal(orc.unpack_nibble_rows(orc.pack_nibble_rows(codes)), codes)
