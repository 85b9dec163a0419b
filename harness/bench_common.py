"""Pieces shared by bench.py and harness/dit_step.py: workloads, synthetic inputs, clock sampling,
measured peaks.  Benchmark infrastructure, not product code."""
from __future__ import annotations

import json
import statistics
import subprocess
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

M_TOKENS = 32760
CLIP = 0.95
INT8_NOMINAL_TOPS = 4500.0

# name -> [(layer, K, N)]: the four W4A4 GEMM shapes of one DiT block at 32760 tokens.
WORKLOADS = {
    # Wan 2.1 T2V 14B (the configuration the metric is quoted on)
    "wan14b_linear_set_M32760": [("qkv", 5120, 15360), ("attn_out", 5120, 5120),
                                 ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120)],
    # Wan 2.1 T2V 1.3B: short reductions, narrow outputs
    "wan13b_linear_set_M32760": [("qkv", 1536, 4608), ("attn_out", 1536, 1536),
                                 ("ffn_up", 1536, 8960), ("ffn_down", 8960, 1536)],
}
DEFAULT_WORKLOAD = "wan14b_linear_set_M32760"


def total_ops(layers, m: int) -> float:
    return float(sum(2.0 * m * k * n for _, k, n in layers))


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {}


class ClockSampler:
    """Samples SM clock, power and throttle reasons while a timed region runs (NVML, ~20 ms
    period; falls back to one nvidia-smi query per 200 ms).  Read-only: changes no GPU setting."""

    _BITS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
             "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80}

    def __init__(self, index: int):
        self.index = index
        self.samples, self.power = [], []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    n = self._nvml
                    self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                    try:
                        self.power.append(n.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                    except Exception:
                        pass
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) \
                        if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
                        else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                    for k, bit in self._BITS.items():
                        if mask & bit:
                            self.reasons.add(k)
                    time.sleep(0.02)
                else:
                    out = subprocess.run(
                        ["nvidia-smi", f"--id={self.index}",
                         "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                         "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits"],
                        capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                    self.samples.append(int(out[0]))
                    self.max_mhz = int(out[1])
                    for k, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                     "sw_power_cap"), out[2:]):
                        if v.strip().lower().startswith("active"):
                            self.reasons.add(k)
                    time.sleep(0.2)
            except Exception:
                time.sleep(0.05)

    def stop(self, settle_fraction: float = 0.0) -> dict:
        """settle_fraction: ignore that leading share of the samples when taking the median (a
        long loop is judged on the clocks it settles at, not on its first burst)."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        tail = self.samples[int(len(self.samples) * settle_fraction):]
        return {
            "sm_mhz": int(statistics.median(tail)) if tail else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "power_w_max": round(max(self.power), 1) if self.power else None,
        }


# --------------------------------------------------------------------------- inputs
def make_activations(torch, m: int, k: int, seed: int, device):
    """fp16 [m,k]: N(0,1) with 1 % of the input channels scaled x20 (the benchmark's outliers)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.randperm(k, generator=g)[: max(1, k // 100)]
    gd = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(m, k, generator=gd, device=device, dtype=torch.float32)
    x[:, idx.to(device)] *= 20.0
    return x.half()


def make_layer(torch, vdm, k: int, n: int, seed: int, device):
    """Weights N(0,0.02) quantised per output channel (absmax/7), packed to vdm_w4a4_packed_v1 and
    repacked for the GEMM; bias N(0,0.01)."""
    gd = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn(n, k, generator=gd, device=device, dtype=torch.float32) * 0.02).half()
    b = (torch.randn(n, generator=gd, device=device, dtype=torch.float32) * 0.01).half()
    qweight, wscales, _ = vdm.quantize_weight_per_channel(w)
    w_b200, w_scale = vdm.prepare_b200_weight(qweight, wscales)
    return {"qweight": qweight, "wscales": wscales, "w_b200": w_b200, "w_scale": w_scale, "bias": b,
            "w_fp16": w, "k": k, "n": n}
