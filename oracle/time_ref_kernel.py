"""Times the REFERENCE's own CUDA kernel (oracle/_ref, built by oracle/build_ref_ext.py) on the
benchmark's GEMM shapes on the current GPU: the same-box "kernel to beat".  BASELINE
INFRASTRUCTURE, not product code.  Prints one JSON line per shape."""
from __future__ import annotations

import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from oracle import _ref_loader

SHAPES = [(32760, 5120, 15360), (32760, 5120, 5120), (32760, 5120, 13824), (32760, 13824, 5120),
          (32760, 1536, 4608), (32760, 1536, 8960), (32760, 8960, 1536)]


def main():
    ref = _ref_loader.load()
    if ref is None:
        print(json.dumps({"unavailable": "oracle/_ref/vdm_w4a4_ref_ext.so not built"}))
        return
    for m, k, n in SHAPES:
        x = torch.randn(m, k, device="cuda", dtype=torch.float16)
        w = (torch.randn(n, k, device="cuda") * 0.02).half()
        b = (torch.randn(n, device="cuda") * 0.01).half()
        qw, wps, _ = ref.quantize_weight_per_channel(w)
        for _ in range(2):
            ref.linear_dynamic_bias(x, qw, wps, b, 0.95)
        torch.cuda.synchronize()
        it = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(it):
            ref.linear_dynamic_bias(x, qw, wps, b, 0.95)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / it
        print(json.dumps({"kernel": "reference vdm_w4a4 linear_dynamic_bias (mma.sync s4, sm_100a build)",
                          "M": m, "K": k, "N": n, "ms": round(ms, 3), "tops": round(2.0 * m * n * k / ms / 1e9, 1)}),
              flush=True)


if __name__ == "__main__":
    main()
