"""b200w4a4_linear_noalloc: the entry point for callers that cannot allocate device memory
(it keeps the quantised activations in a device array built into the library).  Called through
the C ABI, twice in a row, and compared bit for bit with b200w4a4_linear, which takes a
caller-allocated workspace.  Collected last on purpose: a failure here cannot hide another test."""
import ctypes

import numpy as np
import pytest
import torch

from _cases import make_case
from oracle import w4a4_oracle as orc

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_noalloc_entry_matches_workspace_entry_twice():
    from dsaquant_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    max_codes = lib.b200w4a4_linear_noalloc_max_codes()
    max_rows = lib.b200w4a4_linear_noalloc_max_rows()
    assert max_codes == 8 << 20 and max_rows == 8192

    # Two different shapes back to back: the second call finds the first call's data in the scratch.
    for seed, (M, K, N) in enumerate([(512, 5120, 1536), (300, 1536, 384)]):
        assert M <= max_rows and M * K <= max_codes
        x16, w16, b16 = make_case(40 + seed, M, K, N)
        ws = orc.weight_scale_absmax(w16)
        qw = orc.quantize_weight(w16, ws)
        x = torch.from_numpy(x16).to(dev)
        w_b200 = torch.from_numpy(orc.repack_b200(qw)).to(dev)
        w_scale = torch.from_numpy(ws).to(dev)
        bias = torch.from_numpy(b16).to(dev)

        ws_bytes = lib.b200w4a4_linear_workspace_bytes(M, K)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        want = torch.empty(M, N, dtype=torch.float16, device=dev)
        rc = lib.b200w4a4_linear(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), _ptr(bias), _ptr(want),
                                 _ptr(workspace), ws_bytes, M, N, K, 0.95, stream)
        assert rc == 0, _lib.strerror(rc)

        got = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
        rc = lib.b200w4a4_linear_noalloc(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), _ptr(bias), _ptr(got),
                                         M, N, K, 0.95, stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
        # and both equal the oracle
        ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))

    # Exactly at both limits (rows = max_rows, codes = max_codes): the last code byte sits next to
    # the first scale and the whole scale region is in use.  Issued on a second stream after a
    # device synchronisation, which is all the ordering the shared scratch asks for.
    M, K, N = max_rows, max_codes // max_rows, 128
    x16, w16, b16 = make_case(43, M, K, N)
    ws = orc.weight_scale_absmax(w16)
    qw = orc.quantize_weight(w16, ws)
    x = torch.from_numpy(x16).to(dev)
    w_b200 = torch.from_numpy(orc.repack_b200(qw)).to(dev)
    w_scale = torch.from_numpy(ws).to(dev)
    bias = torch.from_numpy(b16).to(dev)
    ws_bytes = lib.b200w4a4_linear_workspace_bytes(M, K)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    want = torch.empty(M, N, dtype=torch.float16, device=dev)
    got = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    side_ptr = ctypes.c_void_p(side.cuda_stream)
    rc = lib.b200w4a4_linear(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), _ptr(bias), _ptr(want),
                             _ptr(workspace), ws_bytes, M, N, K, 0.95, side_ptr)
    assert rc == 0, _lib.strerror(rc)
    rc = lib.b200w4a4_linear_noalloc(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), _ptr(bias), _ptr(got),
                                     M, N, K, 0.95, side_ptr)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
    ref = orc.linear_w4a4(x16, qw, ws, b16, 0.95)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref["out"].view(np.uint16))

    # Sizes beyond the built-in scratch are refused with a clear error and launch nothing.
    out = torch.empty(8, dtype=torch.float16, device=dev)
    rc = lib.b200w4a4_linear_noalloc(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), None, _ptr(out),
                                     max_rows + 1, 128, 64, 1.0, stream)
    assert rc == -8 and "scratch" in _lib.strerror(rc)
    rc = lib.b200w4a4_linear_noalloc(_ptr(x), 0, _ptr(w_b200), _ptr(w_scale), None, _ptr(out),
                                     4096, 128, 4096, 1.0, stream)
    assert rc == -8
    assert lib.b200w4a4_last_device_status(dev.index) == 0
