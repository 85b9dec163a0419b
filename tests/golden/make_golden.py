"""Regenerates tests/golden/*.npz by running the REFERENCE's own PyTorch W4A4 path.

Run where a DSAQuant checkout exists (DSAQUANT_REFERENCE, or a directory called
`reference` next to this repository):

    python tests/golden/make_golden.py

For every case of tests/_cases.CASES it imports the reference's QuantLinear /
UniformQuantizer (vdm_infer/quantization/quant_linear.py), runs the fake-quant
forward in fp32 on CPU on a 2-D [M,K] input (per-token dynamic activation
scales: aquantizer.init is reset before the call), and records the reference's
activation codes and scales, weight codes, the exact integer accumulators of
those codes and the reference's fp32 output.  Cases with clip != 1 take the
scale from the formula of the reference's kernel smoke test,
(absmax.clamp_min(.)/7*clip) evaluated in fp32
(tests/test_vdm_w4a4_kernel_smoke.py:25), and quantise with the reference's
UniformQuantizer.quant.  Small cases store every array; large ones store
SHA-256 digests plus a strided sample.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
_REF = os.environ.get("DSAQUANT_REFERENCE") or str(HERE.parent.parent.parent / "reference")
if not (Path(_REF) / "vdm_infer").is_dir():
    raise SystemExit("set DSAQUANT_REFERENCE to a DSAQuant checkout (or place one next to this repository)")
sys.path.insert(0, _REF)

from _cases import CASES, digest, make_case  # noqa: E402
from vdm_infer.quantization.quant_linear import QuantLinear  # noqa: E402  (reference code)

QPARAMS = {
    "w": {"bit": 4, "sym": True, "granularity": "per_channel", "group_size": -1, "round_zero": True,
          "cali": "mse"},
    "act": {"bit": 4, "sym": True},
}


def run_reference(x16, w16, b16, clip):
    x = torch.from_numpy(x16).float()
    w = torch.from_numpy(w16).float()
    lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=b16 is not None)
    with torch.no_grad():
        lin.weight.copy_(w)
        if b16 is not None:
            lin.bias.copy_(torch.from_numpy(b16).float())
    ql = QuantLinear(lin, {"w": "lsq", "act": "dynamic"}, QPARAMS)
    with torch.no_grad():
        ql.wquantizer(ql.weight.detach())          # absmax/7 per output channel, fp32
        # The packed format stores the channel scale as fp16 (quant_linear.py:144): use that value.
        ws16 = ql.wquantizer.scale.detach().half()
        ql.wquantizer.scale.copy_(ws16.float())
        ql.set_quant_state(use_wq=True, use_aq=True)
        if clip == 1.0:
            ql.aquantizer.init = False
            out = ql(x)
            a_scale = ql.aquantizer.scale.detach().clone()
        else:
            a_scale = (x.abs().amax(dim=1, keepdim=True).clamp_min(1e-5) / 7 * clip).float()
            del ql.aquantizer.scale                      # same replacement init_qparams does (:51-53)
            ql.aquantizer.register_buffer("scale", a_scale)
            ql.aquantizer.init = True
            out = ql(x)
        a_codes = ql.aquantizer.quant(x, a_scale, None)
        w_codes = ql.wquantizer.quant(ql.weight.detach(), ql.wquantizer.scale, None)
        acc = (a_codes.double() @ w_codes.double().t()).round().to(torch.int32)
    return {
        "a_codes": a_codes.to(torch.int8).numpy(),
        "a_scale": a_scale.reshape(-1).float().numpy(),
        "w_codes": w_codes.to(torch.int8).numpy(),
        "w_scale": ws16.reshape(-1).numpy(),
        "acc": acc.numpy(),
        "ref_out_f32": out.float().numpy(),
    }


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    for name, (seed, M, K, N, kw, clip) in CASES.items():
        x16, w16, b16 = make_case(seed, M, K, N, **kw)
        r = run_reference(x16, w16, b16, clip)
        rec = {"clip": np.float32(clip), "input_digest": np.array(digest(x16, w16, b16))}
        if M * N <= 64 * 1024:
            rec.update(r)
        else:
            for k in ("a_codes", "a_scale", "w_codes", "w_scale", "acc"):
                rec[k + "_digest"] = np.array(digest(r[k]))
            rec["acc_sample"] = r["acc"][::61, ::53].copy()
            rec["ref_out_f32_sample"] = r["ref_out_f32"][::61, ::53].copy()
            rec["a_scale"] = r["a_scale"]
            rec["w_scale"] = r["w_scale"]
        path = HERE / f"{name}.npz"
        np.savez_compressed(path, **rec)
        print(f"{name}: M={M} K={K} N={N} clip={clip} -> {path.name} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
