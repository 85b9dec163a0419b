#!/usr/bin/env python
"""Runs one library kernel a few times on a small case, through the C ABI, and exits.

Meant for profiler captures (a few hundred MB on the device, a handful of launches) and for quick
timing of a single shape:

    python harness/kernel_case.py gemm  --m 8192 --k 5120 --n 15360 [--cta-group 2] [--iters 2]
    python harness/kernel_case.py quant --m 8192 --k 5120 [--prologue layernorm_mod|gelu_tanh]
    python harness/kernel_case.py gemm  --m 8192 --k 5120 --n 15360 --weight-staging int8
    python harness/kernel_case.py glue  --m 16384 --k 5120 --heads 40      # qk_norm_rope, k = model width

`gemm` launches the quantiser and the GEMM `--iters` times each (the quantiser fills the codes the
GEMM reads); `--time` adds CUDA-event timing of the last kernel of each iteration and prints it.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "quant", "glue"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--n", type=int, default=15360)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--weight-staging", default="int4", choices=["int4", "int8"])
    ap.add_argument("--prologue", default="none", choices=["none", "layernorm_mod", "gelu_tanh"])
    args = ap.parse_args()

    import torch

    from dsaquant_b200 import _lib
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    lib = _lib.load()
    vdm.set_cta_group(args.cta_group)
    if args.weight_staging == "int8":
        vdm.set_weight_staging(8)
    M, K, N = args.m, args.k, args.n
    torch.manual_seed(0)
    s = torch.cuda.current_stream().cuda_stream
    x = torch.randn(M, K, device="cuda", dtype=torch.float16)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.iters)]

    if args.kernel in ("gemm", "quant"):
        qact = torch.empty(M, K, device="cuda", dtype=torch.int8)
        asc = torch.empty(M, device="cuda", dtype=torch.float32)
        mod = torch.randn(K, device="cuda", dtype=torch.float32) * 0.02
        if args.kernel == "gemm":
            if args.weight_staging == "int8":
                wq = (torch.randint(-8, 8, (N, K), device="cuda", dtype=torch.int16) * 16).to(torch.int8)
            else:
                wq = torch.randint(0, 256, (N, K // 2), device="cuda", dtype=torch.uint8)   # repacked-layout bytes
            ws = (torch.rand(N, device="cuda") * 0.01 + 0.001).half()
            bias = torch.randn(N, device="cuda").half()
            out = torch.empty(M, N, device="cuda", dtype=torch.float16)
        for a, b in ev:
            if args.kernel == "quant":
                a.record()
            if args.prologue == "none":
                _lib.check(lib.b200w4a4_quantize_act(x.data_ptr(), 0, qact.data_ptr(), 0, asc.data_ptr(), M, K, 0.95, s),
                           "quantize_act")
            else:
                pre = {"gelu_tanh": 1, "layernorm_mod": 2}[args.prologue]
                _lib.check(lib.b200w4a4_quantize_act_fused(x.data_ptr(), pre, mod.data_ptr(), mod.data_ptr(), 0, 1e-6,
                                                           qact.data_ptr(), asc.data_ptr(), M, K, 0.95, s),
                           "quantize_act_fused")
            if args.kernel == "gemm":
                a.record()
                _lib.check(lib.b200w4a4_gemm(qact.data_ptr(), asc.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                             bias.data_ptr(), out.data_ptr(), None, M, N, K, s), "gemm")
            b.record()
        work = 2.0 * M * N * K if args.kernel == "gemm" else M * (3.0 * K + 4)
        unit = "TOP/s" if args.kernel == "gemm" else "GB/s"
        scale = 1e9 if args.kernel == "gemm" else 1e6
    else:
        hd = K // args.heads
        w = (1.0 + 0.1 * torch.randn(K, device="cuda")).half()
        cs = torch.randn(M, hd // 2, 2, device="cuda", dtype=torch.float32)
        out = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        for a, b in ev:
            a.record()
            _lib.check(lib.b200w4a4_qk_norm_rope(x.data_ptr(), K, w.data_ptr(), cs.data_ptr(), 1e-6, hd, out.data_ptr(),
                                                 1, K, M, K, s), "qk_norm_rope")
            b.record()
        work, unit, scale = M * K * 4.0, "GB/s", 1e6

    torch.cuda.synchronize()
    assert vdm.last_device_status() == 0
    if args.time:
        ms = min(a.elapsed_time(b) for a, b in ev)
        print(f"{args.kernel} M={M} K={K} N={N}: {ms * 1e3:.1f} us = {work / ms / scale:.0f} {unit}")
    print("ok")


if __name__ == "__main__":
    main()
