"""CPU arm of the benchmark: the reference's PyTorch W4A4 (fake-quant) forward timed on the host
cores.  BASELINE INFRASTRUCTURE -- bench.py calls this for `cpu_baseline` and `--impl reference`;
nothing in the product path imports it.

Two back-ends:
  "reference"  the reference's own QuantLinear (vdm_infer/quantization/quant_linear.py:162-178),
               imported from the checkout (DSAQUANT_REFERENCE, or `reference` beside this repository), with
               aquantizer.init reset before every call so the activation scale is per call
               (per-token dynamic), as BASELINE config 0 describes;
  "port"       a restatement of that forward handed in by the caller (bench.py passes the one
               under oracle/), used where no checkout is present (a checkout cannot travel
               with this repository).
Both quantise-dequantise the weights on every call, as the reference's forward does.
"""
from __future__ import annotations

import os
import sys
import time
from pathlib import Path
from typing import List, Tuple

QPARAMS = {
    "w": {"bit": 4, "sym": True, "granularity": "per_channel", "group_size": -1, "round_zero": True,
          "cali": "mse"},
    "act": {"bit": 4, "sym": True},
}


def reference_checkout() -> str | None:
    """DSAQUANT_REFERENCE, else a directory called `reference` next to this repository."""
    for ref in (os.environ.get("DSAQUANT_REFERENCE"), str(Path(__file__).resolve().parent.parent.parent / "reference")):
        if ref and (Path(ref) / "vdm_infer" / "quantization" / "quant_linear.py").exists():
            return ref
    return None


class CpuArm:
    """Holds the four layers of a workload on the CPU and times one pass over `rows` tokens."""

    def __init__(self, layers: List[Tuple[str, int, int]], rows: int, clip: float, port_fn=None):
        import torch

        self.torch = torch
        self.layers_def = layers
        self.rows = rows
        self.clip = clip
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        ref = reference_checkout()
        self.kind = "reference" if ref else "port"
        self.port_fn = port_fn
        if not ref and port_fn is None:
            raise RuntimeError("no reference checkout (DSAQUANT_REFERENCE) and no port function given")
        g = torch.Generator().manual_seed(0)
        self.items = []
        for _, k, n in layers:
            x = torch.randn(rows, k, generator=g)
            x[:, torch.randperm(k, generator=g)[: max(1, k // 100)]] *= 20.0
            w = torch.randn(n, k, generator=g) * 0.02
            b = torch.randn(n, generator=g) * 0.01
            x, w = x.half().float(), w.half().float()
            if ref:
                self.items.append((x, self._reference_layer(ref, w, b)))
            else:
                ws = (w.abs().amax(dim=1) / 7).half().float()
                self.items.append((x, (w, ws, b)))

    def _reference_layer(self, ref: str, w, b):
        torch = self.torch
        if ref not in sys.path:
            sys.path.insert(0, ref)
        from vdm_infer.quantization.quant_linear import QuantLinear  # reference code, unmodified

        lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=True)
        with torch.no_grad():
            lin.weight.copy_(w)
            lin.bias.copy_(b)
        ql = QuantLinear(lin, {"w": "lsq", "act": "dynamic"}, QPARAMS)
        with torch.no_grad():
            ql.wquantizer(ql.weight.detach())
            ql.set_quant_state(use_wq=True, use_aq=True)
        return ql

    def step(self) -> None:
        torch = self.torch
        with torch.no_grad():
            if self.kind == "reference":
                for x, ql in self.items:
                    ql.aquantizer.init = False
                    ql(x)
            else:
                for x, (w, ws, b) in self.items:
                    self.port_fn(x, w, ws, b, self.clip)

    def time(self, steps: int, warmup: int) -> float:
        """Mean seconds per step over `steps` timed steps after `warmup` untimed ones."""
        for _ in range(warmup):
            self.step()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step()
        return (time.perf_counter() - t0) / max(1, steps)

    def describe(self, m_total: int) -> str:
        note = "" if self.kind == "port" else " (activation clip 1.0: the reference's fake-quant path has no clip)"
        return (f"{self.rows} of {m_total} token rows of each of the {len(self.layers_def)} layers per step, "
                f"fp32, {self.cores} threads{note}")


def sized_rows(layers, steps: int, warmup: int, clip: float, port_fn=None, budget_s: float = 60.0,
               lo: int = 256, hi: int = 4096) -> int:
    """Rows per step such that warmup + steps passes take about budget_s on this host."""
    probe = CpuArm(layers, lo, clip, port_fn)
    probe.step()
    per_row = probe.time(1, 0) / lo
    rows = int(budget_s / max(per_row * (steps + warmup), 1e-9))
    return max(lo, min(hi, rows // 64 * 64))
