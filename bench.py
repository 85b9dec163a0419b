#!/usr/bin/env python
"""Benchmark of the W4A4 linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload = "wan14b_linear_set_M32760"): the four W4A4 GEMM shapes of one
Wan-2.1-14B DiT block at 32760 tokens -- fused QKV 5120->15360, attention out 5120->5120,
FFN up 5120->13824, FFN down 13824->5120 -- with synthetic inputs of the benchmark's
distributions (activations N(0,1) with 1 % of channels x20, weights N(0,0.02), bias N(0,0.01),
fp16).  One step = dynamic per-token A4 quantise + W4A4 GEMM (+ dequant, bias) for each of
the four layers.  The metric is tera-operations per second, ops = 2*M*N*K with the unpadded M.

`value`     device-resident inputs, C-ABI calls (b200w4a4_quantize_act + b200w4a4_gemm), CUDA
            events on the launching stream, max over ranks.
`e2e`       the public python API for host-resident activations (HostLinearPipeline): every step
            copies the two fp16 activation matrices from pinned host memory and reads all four
            fp16 outputs back into pinned host memory, copies and compute overlapped per row chunk.
`roofline`  the GEMM kernel: algorithmic ops per launch / its mean launch time (events around
            each GEMM launch inside the timed region), against 2 x the measured bf16 matmul
            peak (the int8 tensor pipe runs at twice the bf16 rate).
`cpu_baseline` / `--impl reference`: the reference's PyTorch fake-quant W4A4 forward restated
            for CPU (oracle/fakequant_cpu.py), all host threads, on a bounded row sample.

With N > 1 every rank runs the same set on its own tokens (independent prompts / CFG branches,
weights replicated, no collective on the data path): weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_TOKENS = 32760
LAYERS = [  # name, K, N
    ("qkv", 5120, 15360),
    ("attn_out", 5120, 5120),
    ("ffn_up", 5120, 13824),
    ("ffn_down", 13824, 5120),
]
CLIP = 0.95
WORKLOAD = "wan14b_linear_set_M32760"
INT8_NOMINAL_TOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum of one QKV-shaped GEMM launch, scaled from the
# ncu capture summarised in profiles/ (M=8192 case, traffic proportional to M); None if unknown.
GEMM_DRAM_TRAFFIC_BYTES = int(409.7e6 * 32760 / 8192)  # 197.7 MB read + 212.0 MB written at M=8192


def total_ops(m: int) -> float:
    return float(sum(2.0 * m * k * n for _, k, n in LAYERS))


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs (NVML, ~20 ms period;
    falls back to one nvidia-smi query per 200 ms)."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
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

    def _run(self):
        names = {
            "hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
            "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80,
        }
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    n = self._nvml
                    self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) \
                        if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
                        else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                    for k, bit in names.items():
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

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------- inputs
def make_activations(torch, m: int, k: int, seed: int, device):
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.randperm(k, generator=g)[: max(1, k // 100)]
    gd = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(m, k, generator=gd, device=device, dtype=torch.float32)
    x[:, idx.to(device)] *= 20.0
    return x.half()


def make_layer(torch, vdm, k: int, n: int, seed: int, device):
    gd = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn(n, k, generator=gd, device=device, dtype=torch.float32) * 0.02).half()
    b = (torch.randn(n, generator=gd, device=device, dtype=torch.float32) * 0.01).half()
    qweight, wscales, ch_scale = vdm.quantize_weight_per_channel(w)
    w_b200, w_scale = vdm.prepare_b200_weight(qweight, wscales)
    return {"qweight": qweight, "wscales": wscales, "w_b200": w_b200, "w_scale": w_scale, "bias": b,
            "w_fp16": w, "k": k, "n": n}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_sample(rows: int, steps: int = 1, warmup: int = 0) -> dict:
    """Times the CPU restatement of the reference's fake-quant forward on `rows` tokens of
    every layer of the set; returns TOPS-equivalent (2*rows*N*K summed / time)."""
    import torch

    from oracle.fakequant_cpu import fakequant_linear

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layers = []
    g = torch.Generator().manual_seed(0)
    for _, k, n in LAYERS:
        x = torch.randn(rows, k, generator=g)
        x[:, torch.randperm(k, generator=g)[: k // 100]] *= 20.0
        w = torch.randn(n, k, generator=g) * 0.02
        b = torch.randn(n, generator=g) * 0.01
        ws = (w.abs().amax(dim=1) / 7).half().float()
        layers.append((x.half().float(), w.half().float(), ws, b))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for x, w, ws, b in layers:
            fakequant_linear(x, w, ws, b, 1.0)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    return {"value": total_ops(rows) / t / 1e12, "seconds_per_step": t, "cores": cores}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    # Bound the run: one probing pass, then as many of the requested steps as fit in ~90 s.
    probe = cpu_reference_sample(rows, steps=1, warmup=0)
    fit = max(1, int(90.0 / max(probe["seconds_per_step"], 1e-3)))
    args.steps = max(1, min(args.steps, fit))
    args.warmup = max(0, min(args.warmup, 1))
    r = cpu_reference_sample(rows, steps=args.steps, warmup=args.warmup)
    sample = f"{rows} of {M_TOKENS} token rows of each of the 4 layers per step"
    line = {
        "impl": "reference", "metric": "w4a4_linear_tops", "value": r["value"], "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": max(1, args.steps), "warmup": max(0, args.warmup),
        "ms_per_step": r["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M_TOKENS, "layers": [[k, n] for _, k, n in LAYERS],
                   "sample": sample},
        "cpu_baseline": {"value": r["value"], "unit": "TOP/s", "cores": r["cores"], "kind": "port",
                         "sample": sample},
        "e2e": {"value": r["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-rows", type=int, default=4096)
    ap.add_argument("--e2e-chunk-rows", type=int, default=2048)
    ap.add_argument("--e2e-depth", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=M_TOKENS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="linear_set",
                    choices=["linear_set", "dit_wan21_1.3b", "dit_wan22_5b", "dit_wan21_14b"],
                    help="linear_set (default, the headline GEMM set) or one CFG step of a harness DiT")
    args, extra = ap.parse_known_args()
    if args.workload.startswith("dit_"):
        # Full-step configurations live in the harness; same launch contract, one JSON line.
        from harness import dit_step

        sys.argv = [sys.argv[0], "--model", args.workload[4:], "--steps", str(args.steps),
                    "--warmup", str(args.warmup)] + extra
        dit_step.main()
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(3, args.warmup)

    import ctypes

    import torch
    import torch.distributed as dist

    from dsaquant_b200 import _lib
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the W4A4 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if not vdm.is_available():
        raise SystemExit(f"libb200w4a4.so not available: {vdm.load_error()}")
    lib = _lib.load()
    cta_group = int(os.environ.get("B200W4A4_CTA_GROUP", "2"))
    vdm.set_cta_group(cta_group)

    m = args.tokens
    layers = [make_layer(torch, vdm, k, n, 100 + i, device) for i, (_, k, n) in enumerate(LAYERS)]
    xs = {k: make_activations(torch, m, k, 7 + rank, device) for k in sorted({k for _, k, _ in LAYERS})}
    outs = [torch.empty(m, L["n"], dtype=torch.float16, device=device) for L in layers]
    kmax = max(k for _, k, _ in LAYERS)
    qact = torch.empty(m * kmax, dtype=torch.int8, device=device)
    ascale = torch.empty(m, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)

    def step_device(gemm_events=None):
        for i, L in enumerate(layers):
            x = xs[L["k"]]
            if gemm_events is not None:
                gemm_events[i][2].record(stream)
            rc = lib.b200w4a4_quantize_act(x.data_ptr(), 0, qact.data_ptr(), 0, ascale.data_ptr(), m,
                                           L["k"], CLIP, sp)
            if gemm_events is not None:
                gemm_events[i][0].record(stream)
            rc |= lib.b200w4a4_gemm(qact.data_ptr(), ascale.data_ptr(), L["w_b200"].data_ptr(),
                                    L["w_scale"].data_ptr(), L["bias"].data_ptr(), outs[i].data_ptr(),
                                    None, m, L["n"], L["k"], sp)
            if gemm_events is not None:
                gemm_events[i][1].record(stream)
            if rc != 0:
                raise RuntimeError(f"b200w4a4 call failed: {rc}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------
    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
            torch.cuda.Event(enable_timing=True)) for _ in layers] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record(stream)
    for s in range(args.steps):
        step_device(ev[s])
    t_end.record(stream)
    barrier()
    clocks = sampler.stop()
    total_ms = t_start.elapsed_time(t_end)
    status = vdm.last_device_status(local_rank)
    if status != 0:
        raise RuntimeError(f"device-side time-out recorded by a kernel (role code {status})")
    gemm_ms = [[a.elapsed_time(b) for a, b, _ in step] for step in ev]
    gemm_mean_ms = [sum(step[i] for step in gemm_ms) / args.steps for i in range(len(layers))]
    quant_ms = [[q.elapsed_time(a) for a, _, q in step] for step in ev]
    quant_mean_ms = [sum(step[i] for step in quant_ms) / args.steps for i in range(len(layers))]

    # Library int8 x int8 GEMM (cuBLASLt through torch._int_mm) on the QKV shape: context for
    # the roofline, measured in a short burst after the timed region.
    lib_int8_tops = None
    if rank == 0 and m % 8 == 0:
        try:
            k0, n0 = LAYERS[0][1], LAYERS[0][2]
            a8 = torch.randint(-8, 8, (m, k0), device=device, dtype=torch.int8)
            b8 = torch.randint(-8, 8, (n0, k0), device=device, dtype=torch.int8).t()
            for _ in range(3):
                torch._int_mm(a8, b8)
            l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0.record(stream)
            for _ in range(10):
                torch._int_mm(a8, b8)
            l1.record(stream)
            torch.cuda.synchronize()
            lib_int8_tops = 2.0 * m * k0 * n0 / (l0.elapsed_time(l1) / 10 * 1e-3) / 1e12
            del a8, b8
        except Exception:
            lib_int8_tops = None

    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = world * total_ops(m) / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the python API, host buffers -------------------------
    # Inputs and outputs are pinned host tensors; the public helper HostLinearPipeline chunks
    # rows and overlaps H2D, quantise + GEMM and D2H.  Layers that read the same activation
    # are evaluated per chunk, so each activation matrix crosses the link once per step.
    from dsaquant_b200.host_pipeline import HostLinearLayer, HostLinearPipeline

    hx = {k: v.cpu().pin_memory() for k, v in xs.items()}
    hout = [torch.empty(m, L["n"], dtype=torch.float16).pin_memory() for L in layers]
    host_layers = [HostLinearLayer(L["qweight"], L["wscales"], L["bias"]) for L in layers]
    pipe = HostLinearPipeline(device, k_max=kmax, n_max=max(L["n"] for L in layers), chunk_rows=args.e2e_chunk_rows, depth=args.e2e_depth)
    groups = {}
    for i, L in enumerate(layers):
        groups.setdefault(L["k"], []).append(i)

    def step_e2e():
        for k, idx in groups.items():
            pipe.run(hx[k], [host_layers[i] for i in idx], [hout[i] for i in idx], CLIP)

    e2e_steps = max(1, args.e2e_steps)
    for _ in range(2):
        step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        step_e2e()
    e1.record(stream)
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / e2e_steps
    e2e_value = world * total_ops(m) / (e2e_ms * 1e-3) / 1e12
    h2d = sum(v.numel() * 2 for v in hx.values())
    d2h = sum(v.numel() * 2 for v in hout)

    if rank == 0:
        peaks = measured_peaks()
        if "bf16_tflops_sustained" in peaks:
            peak, peak_src = 2.0 * float(peaks["bf16_tflops_sustained"]), \
                "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (of measured)"
        else:
            peak, peak_src = 2.0 * 1400.0, "2 x 1.4 PFLOP/s sustained bf16 (of fallback)"
        # dominant kernel = the QKV-shaped GEMM (largest share of the step)
        k0, n0 = LAYERS[0][1], LAYERS[0][2]
        achieved = 2.0 * m * k0 * n0 / (gemm_mean_ms[0] * 1e-3) / 1e12
        gemm_all = sum(2.0 * m * k * n for _, k, n in LAYERS) / (sum(gemm_mean_ms) * 1e-3) / 1e12
        line = {
            "metric": "w4a4_linear_tops", "value": value, "unit": "TOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": m, "layers": [[k, n] for _, k, n in LAYERS],
                       "clip": CLIP, "act_dtype": "f16", "parallelism": f"dp{world}",
                       "l2": "inputs_exceed_l2 (activations 335-906 MB per layer vs 126 MB L2)",
                       "gemm_variant": f"cta_group::{cta_group}"},
            "e2e": {"value": e2e_value, "unit": "TOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": 2 * len(LAYERS) * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm_w4a4_kernel (QKV 5120->15360)",
                         "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak,
                         "peak_source": peak_src, "frac_of_nominal_int8_4500": achieved / INT8_NOMINAL_TOPS,
                         "all_gemms_achieved": gemm_all,
                         "gemm_ms": {LAYERS[i][0]: gemm_mean_ms[i] for i in range(len(LAYERS))},
                         "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                         "library_int8_mm_tops_same_shape": lib_int8_tops},
            "quantizer": {"bound": "hbm", "kernel": "quant_act_rows_kernel",
                          "gb_per_s": {LAYERS[i][0]: m * (3.0 * LAYERS[i][1] + 4) / (quant_mean_ms[i] * 1e-3) / 1e9
                                       for i in range(len(LAYERS))},
                          "peak_gb_per_s": peaks.get("hbm_gbs"),
                          "bytes_per_row": "2K (fp16 read) + K (int8 codes) + 4 (fp32 scale)"},
        }
        if not args.no_cpu_baseline and world == 1:
            r = cpu_reference_sample(args.cpu_rows)
            line["cpu_baseline"] = {
                "value": r["value"], "unit": "TOP/s", "cores": r["cores"], "kind": "port",
                "sample": f"{args.cpu_rows} of {m} token rows of each of the 4 layers, one pass "
                          f"({r['seconds_per_step']:.1f} s)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
