#!/usr/bin/env python
"""Benchmark of the W4A4 linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload, default "wan14b_linear_set_M32760"): the four W4A4 GEMM shapes of one
Wan-2.1-14B DiT block at 32760 tokens -- fused QKV 5120->15360, attention out 5120->5120, FFN up
5120->13824, FFN down 13824->5120 -- with synthetic inputs of the benchmark's distributions
(activations N(0,1) with 1 % of channels x20, weights N(0,0.02), bias N(0,0.01), fp16).
"wan13b_linear_set_M32760" is the Wan-2.1-1.3B set (K = 1536 / 8960).  One step = dynamic
per-token A4 quantise + W4A4 GEMM (+ dequant, bias) for each of the four layers.  The metric is
tera-operations per second, ops = 2*M*N*K with the unpadded M.

`value`      device-resident inputs, C-ABI calls (b200w4a4_quantize_act + b200w4a4_gemm), CUDA
             events on the launching stream, max over ranks.
`e2e`        the public python API for host-resident activations (HostLinearPipeline): every
             step copies this rank's activation rows from pinned host memory and reads all four
             fp16 outputs back into pinned host memory, copies and compute overlapped per chunk.
`roofline`   the QKV GEMM kernel: algorithmic ops per launch / its mean launch time (events
             around each GEMM launch inside the timed region), burst against 2 x the measured
             burst bf16 matmul rate; `sustained` repeats the step for >= 2 s and pairs it with
             2 x the measured sustained bf16 rate (the int8 tensor pipe runs at twice the bf16
             rate; MEASURED_PEAKS.json has no int8 entry), with the library int8 GEMM on the
             same codes in the same regime beside it.
`cpu_baseline` / `--impl reference`: the reference's PyTorch fake-quant W4A4 forward on the host
             cores (its own QuantLinear when DSAQUANT_REFERENCE names a checkout, else the
             restatement under oracle/), all host threads, on a bounded row sample.
`gpu_baseline` the reference's own CUDA kernel (oracle/_ref, built unmodified for sm_100a) on the
             QKV shape in the same run: the kernel this library replaces.
`dit_step`   N = 1 default run and every N > 1 run: one Wan-2.1-14B CFG denoising step of the
             harness model at this N (harness/dit_step.py), with its own clocks, per-phase split
             and sharded-vs-unsharded check.

With N > 1 the 32760 token rows of every layer are split over the ranks (weights replicated,
dsaquant_b200.sharding.row_partition): strong scaling, no collective on the data path; the run
proves in place that the sharded outputs equal the unsharded ones bit for bit.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from harness.bench_common import (CLIP, DEFAULT_WORKLOAD, INT8_NOMINAL_TOPS, M_TOKENS, WORKLOADS,  # noqa: E402
                                  ClockSampler, make_activations, make_layer, measured_peaks, total_ops)

# dram__bytes_read.sum + dram__bytes_write.sum of one QKV-shaped GEMM launch at M = 32760, scaled
# from the ncu capture summarised in profiles/ (M = 8192 case; traffic grows in proportion to M).
GEMM_DRAM_TRAFFIC_BYTES = {"wan14b_linear_set_M32760": int((193.1e6 + 208.1e6) * 32760 / 8192),   # QKV 5120->15360
                           "wan13b_linear_set_M32760": int((16.2e6 + 75.5e6) * 32760 / 8192)}     # QKV 1536->4608: reads + the full output
# (at K = 1536 the 75.5 MB output was still in L2 when the captured launch ended: ncu saw 17.7 MB written)


def base_config(workload: str, m: int, world: int, cta_group: int) -> dict:
    layers = WORKLOADS[workload]
    return {"workload": workload, "M": m, "layers": [[k, n] for _, k, n in layers], "clip": CLIP,
            "act_dtype": "f16",
            "parallelism": "single GPU" if world == 1 else f"token rows split over {world} GPUs, weights replicated",
            "l2": "inputs_exceed_l2 (activation matrices of 100-906 MB rotate through the step vs 126 MB L2)",
            "gemm_variant": f"cta_group::{cta_group}"}


# --------------------------------------------------------------------------- CPU arm
def cpu_arm(layers, rows: int, clip: float):
    from harness.bench_cpu import CpuArm
    from oracle.fakequant_cpu import fakequant_linear   # the checker's restatement, timed as a baseline only

    return CpuArm(layers, rows, clip, port_fn=fakequant_linear)


def run_reference_arm(args) -> None:
    """`--impl reference`: the reference's CPU implementation of the path on the host cores, same
    config / metric / unit as the GPU arm, each step a bounded row sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from harness.bench_cpu import sized_rows
    from oracle.fakequant_cpu import fakequant_linear

    layers = WORKLOADS[args.workload]
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    rows = sized_rows(layers, steps, warmup, CLIP, port_fn=fakequant_linear, budget_s=75.0)
    arm = cpu_arm(layers, rows, CLIP)
    sec = arm.time(steps, warmup)
    value = total_ops(layers, rows) / sec / 1e12
    sample = arm.describe(args.tokens)
    line = {
        "impl": "reference", "metric": "w4a4_linear_tops", "value": value, "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": base_config(args.workload, args.tokens, args.gpus, int(os.environ.get("B200W4A4_CTA_GROUP", "2"))),
        "cpu_baseline": {"value": value, "unit": "TOP/s", "cores": arm.cores, "kind": arm.kind, "sample": sample},
        "e2e": {"value": value, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm helpers
def timed_loop(torch, stream, fn, seconds: float, est_ms: float, device_index: int):
    """Runs fn back to back for about `seconds`; returns (mean ms over the second half, clocks with
    the median SM clock of that half).  The first half lets power and clocks settle."""
    n = max(20, int(seconds * 1e3 / max(est_ms, 1e-3)))
    a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    sampler = ClockSampler(device_index).start()
    a.record(stream)
    for i in range(n):
        if i == n // 2:
            b.record(stream)
        fn()
    c.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop(settle_fraction=0.5)
    return b.elapsed_time(c) / (n - n // 2), a.elapsed_time(c) * 1e-3, clocks


def library_int8(torch, vdm, stream, qact, layer, m, seconds, device_index):
    """cuBLASLt int8 x int8 -> int32 (torch._int_mm) on the SAME activation and weight codes the
    W4A4 GEMM consumes (data decides how much power a tensor-core GEMM draws), burst and sustained.
    No dequantisation or bias: a lower bound on the library's time for the layer."""
    k, n = layer["k"], layer["n"]
    m8 = m - m % 8
    if m8 < 32:
        return None
    try:
        a8 = qact[: m8 * k].view(m8, k)
        b8 = vdm.unpack_codes(layer["qweight"], n, k, 2).t()
        for _ in range(3):
            torch._int_mm(a8, b8)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(10):
            torch._int_mm(a8, b8)
        e1.record(stream)
        torch.cuda.synchronize()
        burst_ms = e0.elapsed_time(e1) / 10
        ops = 2.0 * m8 * k * n
        rec = {"burst_tops": ops / (burst_ms * 1e-3) / 1e12}
        if seconds > 0:
            time.sleep(0.5)
            ms, _, clocks = timed_loop(torch, stream, lambda: torch._int_mm(a8, b8), seconds, burst_ms, device_index)
            rec.update({"sustained_tops": ops / (ms * 1e-3) / 1e12, "sustained_sm_mhz": clocks["sm_mhz"]})
        return rec
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:160]}


def reference_gpu_kernel(torch, m: int, k: int, n: int, device) -> dict:
    """The reference's own CUDA kernel (vdm_w4a4_kernel.cu built unmodified for sm_100a into
    oracle/_ref by oracle/build_ref_ext.py) on one layer shape: the same-box kernel to beat."""
    try:
        from oracle import _ref_loader

        ref = _ref_loader.load()
        if ref is None:
            return {"unavailable": "oracle/_ref/vdm_w4a4_ref_ext.so is not built on this machine"}
        x = make_activations(torch, m, k, 7, device)
        gd = torch.Generator(device=device).manual_seed(100)
        w = (torch.randn(n, k, generator=gd, device=device) * 0.02).half()
        b = (torch.randn(n, generator=gd, device=device) * 0.01).half()
        qw, wps, _ = ref.quantize_weight_per_channel(w)
        for _ in range(2):
            ref.linear_dynamic_bias(x, qw, wps, b, CLIP)
        torch.cuda.synchronize()
        it = 3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(it):
            ref.linear_dynamic_bias(x, qw, wps, b, CLIP)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / it
        return {"kernel": "reference linear_dynamic_bias (3 launches: abs-max, quantise, mma.sync s4 GEMM), sm_100a build",
                "shape": [m, k, n], "ms": ms, "value": 2.0 * m * n * k / (ms * 1e-3) / 1e12, "unit": "TOP/s"}
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


# --------------------------------------------------------------------------- GPU arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=M_TOKENS)
    ap.add_argument("--sustain-seconds", type=float, default=2.5, help="length of the sustained leg (0: skip)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunk-rows", type=int, default=4096)
    ap.add_argument("--e2e-depth", type=int, default=3)
    ap.add_argument("--cpu-rows", type=int, default=4096)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true")
    ap.add_argument("--no-dit", action="store_true", help="skip the Wan-14B DiT-step key")
    ap.add_argument("--dit-model", default="wan21_14b", choices=["wan21_1.3b", "wan22_5b", "wan21_14b"])
    ap.add_argument("--dit-steps", type=int, default=5)
    ap.add_argument("--dit-warmup", type=int, default=2)
    ap.add_argument("--dit-layers", type=int, default=0, help="override the DiT's block count (0: the model's own)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(3, args.warmup)

    import torch
    import torch.distributed as dist

    from dsaquant_b200 import _lib, sharding
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

    LAYERS = WORKLOADS[args.workload]
    m_total = args.tokens
    row0, row1 = sharding.row_partition(m_total, world)[rank]
    m = row1 - row0                                     # this rank's token rows (all of them at N = 1)
    layers = [make_layer(torch, vdm, k, n, 100 + i, device) for i, (_, k, n) in enumerate(LAYERS)]
    # Every rank draws the same full activation matrices (same seed) and keeps its own rows.
    x_full = {k: make_activations(torch, m_total, k, 7, device) for k in sorted({k for _, k, _ in LAYERS})}
    xs = {k: (v if world == 1 else v[row0:row1].contiguous()) for k, v in x_full.items()}
    outs = [torch.empty(max(m, 1), L["n"], dtype=torch.float16, device=device) for L in layers]
    kmax = max(k for _, k, _ in LAYERS)
    qact = torch.empty(max(m, 1) * kmax, dtype=torch.int8, device=device)
    ascale = torch.empty(max(m, 1), dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)

    def step_device(gemm_events=None):
        if m == 0:
            return
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

    def new_events(n_steps):
        return [[tuple(torch.cuda.Event(enable_timing=True) for _ in range(3)) for _ in layers]
                for _ in range(n_steps)]

    def per_layer_ms(ev):
        n = len(ev)
        g = [sum(s[i][0].elapsed_time(s[i][1]) for s in ev) / n for i in range(len(layers))]
        q = [sum(s[i][2].elapsed_time(s[i][0]) for s in ev) / n for i in range(len(layers))]
        return g, q

    # ---- device-resident timing (the headline `value`) ---------------------------------
    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank).start()
    ev = new_events(args.steps)
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
    gemm_mean_ms, quant_mean_ms = per_layer_ms(ev) if m > 0 else ([0.0] * len(layers), [0.0] * len(layers))
    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = total_ops(LAYERS, m_total) / (ms_per_step * 1e-3) / 1e12

    # ---- sharded == unsharded, proven inside the multi-GPU run ----------------------------
    # Every rank has the full activations: it runs each layer unsharded on all rows, gathers the
    # ranks' sharded outputs (an all-gather outside every timed region) and compares bit for bit.
    shard_check = None
    if world > 1:
        equal = []
        for i, L in enumerate(layers):
            xf = x_full[L["k"]]
            full = vdm.linear_vdm_w4a4(xf, L["qweight"], L["wscales"], L["bias"], CLIP)
            gathered = sharding.all_gather_rows(outs[i][:m], m_total)
            equal.append(bool(torch.equal(full, gathered)))
            del full, gathered
        ok = torch.tensor([1 if all(equal) else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        shard_check = {"layers_bit_equal_to_unsharded": equal, "all_ranks_ok": bool(ok.item()),
                       "rows_per_rank": [e - s for s, e in sharding.row_partition(m_total, world)]}
    del x_full
    torch.cuda.empty_cache()

    # ---- sustained regime: the same step repeated for >= sustain-seconds ---------------------
    sustained = None
    if args.sustain_seconds > 0 and m > 0:
        n_rep = max(20, int(args.sustain_seconds * 1e3 / max(total_ms / args.steps, 1e-3)))
        ev2 = new_events(n_rep - n_rep // 2)
        time.sleep(0.5)
        barrier()
        samp2 = ClockSampler(local_rank).start()
        s0, s1, s2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        s0.record(stream)
        for i in range(n_rep):
            if i == n_rep // 2:
                s1.record(stream)
            step_device(ev2[i - n_rep // 2] if i >= n_rep // 2 else None)
        s2.record(stream)
        torch.cuda.synchronize()
        clocks2 = samp2.stop(settle_fraction=0.5)
        sus_ms = s1.elapsed_time(s2) / (n_rep - n_rep // 2)
        sus_gemm_ms, sus_quant_ms = per_layer_ms(ev2)
        sustained = {"seconds": s0.elapsed_time(s2) * 1e-3, "steps": n_rep, "ms_per_step": sus_ms,
                     "value": total_ops(LAYERS, m) / (sus_ms * 1e-3) / 1e12, "unit": "TOP/s (this rank's rows)",
                     "gemm_ms": {LAYERS[i][0]: sus_gemm_ms[i] for i in range(len(LAYERS))},
                     "quant_ms": {LAYERS[i][0]: sus_quant_ms[i] for i in range(len(LAYERS))},
                     "clocks": clocks2, "measured_over": "second half of the loop (clocks settled)"}

    # ---- library int8 GEMM on the same codes (rank 0) ---------------------------------------
    lib_int8 = None
    if rank == 0 and m > 0:
        L0 = layers[0]
        lib.b200w4a4_quantize_act(xs[L0["k"]].data_ptr(), 0, qact.data_ptr(), 0, ascale.data_ptr(), m, L0["k"], CLIP, sp)
        lib_int8 = library_int8(torch, vdm, stream, qact, L0, m, args.sustain_seconds if world == 1 else 0.0, local_rank)

    # ---- end to end through the python API, host buffers ---------------------------------------
    # Inputs and outputs are pinned host tensors; HostLinearPipeline chunks rows and overlaps H2D,
    # quantise + GEMM and D2H.  Layers that read the same activation are evaluated per chunk, so
    # each activation matrix crosses the link once per step.
    from dsaquant_b200.host_pipeline import HostLinearLayer, HostLinearPipeline

    e2e = None
    if m > 0:
        hx = {k: v.cpu().pin_memory() for k, v in xs.items()}
        hout = [torch.empty(m, L["n"], dtype=torch.float16).pin_memory() for L in layers]
        host_layers = [HostLinearLayer(L["qweight"], L["wscales"], L["bias"]) for L in layers]
        pipe = HostLinearPipeline(device, k_max=kmax, n_max=max(L["n"] for L in layers),
                                  chunk_rows=args.e2e_chunk_rows, depth=args.e2e_depth)
        groups = {}
        for i, L in enumerate(layers):
            groups.setdefault(L["k"], []).append(i)

        plan = [(hx[k], [host_layers[i] for i in idx], [hout[i] for i in idx]) for k, idx in groups.items()]

        def step_e2e():
            pipe.run_groups(plan, CLIP)
    else:
        hx, hout = {}, []

        def step_e2e():
            return None

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
    hb = torch.tensor([sum(v.numel() * 2 for v in hx.values()), sum(v.numel() * 2 for v in hout)],
                      dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        dist.all_reduce(hb, op=dist.ReduceOp.SUM)
    e2e_ms = float(te.item()) / e2e_steps
    e2e = {"value": total_ops(LAYERS, m_total) / (e2e_ms * 1e-3) / 1e12, "unit": "TOP/s",
           "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item()),
           "ms_per_step": e2e_ms, "steps": e2e_steps,
           "note": "bytes are the sum over ranks; every rank copies its own rows through pinned host memory"}
    # Same-run check of the host pipeline against the device-resident path (same rows, same bits).
    if m > 0:
        torch.cuda.synchronize()
        e2e["matches_device_path"] = bool(torch.equal(hout[1], outs[1][:m].cpu()))
    del hx, hout

    # ---- baselines on rank 0 of a single-GPU run ----------------------------------------------------
    gpu_baseline = cpu_baseline = None
    if rank == 0 and world == 1:
        if not args.no_gpu_baseline:
            del outs, qact
            torch.cuda.empty_cache()
            gpu_baseline = reference_gpu_kernel(torch, m_total, LAYERS[0][1], LAYERS[0][2], device)
        if not args.no_cpu_baseline:
            arm = cpu_arm(LAYERS, args.cpu_rows, CLIP)
            arm.step()
            sec = arm.time(3, 0)
            cpu_baseline = {"value": total_ops(LAYERS, args.cpu_rows) / sec / 1e12, "unit": "TOP/s",
                            "cores": arm.cores, "kind": arm.kind,
                            "sample": arm.describe(m_total) + f"; 3 timed passes after 1 warm-up ({sec:.2f} s each)"}
    outs = qact = None
    layers_meta = [(L["k"], L["n"]) for L in layers]
    del layers, xs
    torch.cuda.empty_cache()

    # ---- the full DiT step at this N -----------------------------------------------------------------
    dit = None
    if not args.no_dit:
        from harness import dit_step

        try:
            dit = dit_step.measure(args.dit_model, args.dit_steps, args.dit_warmup, layers=args.dit_layers)
        except Exception as exc:  # keep the linear-set line even if the harness model cannot run here
            dit = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        peaks = measured_peaks()
        if "bf16_tflops" in peaks:
            burst_peak = 2.0 * float(peaks["bf16_tflops"])
            sus_peak = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
            src = "of measured"
        else:
            burst_peak, sus_peak, src = 2.0 * 1590.0, 2.0 * 1400.0, "of fallback"
        k0, n0 = layers_meta[0]
        qkv_ops = 2.0 * m * k0 * n0
        achieved = qkv_ops / (gemm_mean_ms[0] * 1e-3) / 1e12 if m > 0 else 0.0
        gemm_all = sum(2.0 * m * k * n for k, n in layers_meta) / (sum(gemm_mean_ms) * 1e-3) / 1e12 if m > 0 else 0.0
        sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        # Issue bound of the tensor pipe itself: 8192 int8 MAC per clock per SM at the sampled clock.
        clock_peak = 2.0 * 8192 * sm_count * (clocks["sm_mhz"] or 0) * 1e6 / 1e12
        traffic = GEMM_DRAM_TRAFFIC_BYTES.get(args.workload)
        roofline = {
            "bound": "tensor", "kernel": f"gemm_w4a4_kernel ({LAYERS[0][0]} {k0}->{n0}, {m} rows)",
            "regime": "burst (the timed region is shorter than the power controller's reaction)",
            "achieved": achieved, "peak": burst_peak, "unit": "TOP/s", "frac": achieved / burst_peak,
            "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({src}); no int8 entry there",
            "frac_of_nominal_int8_4500": achieved / INT8_NOMINAL_TOPS,
            "frac_of_tensor_pipe_at_sampled_clock": achieved / clock_peak if clock_peak else None,
            "tensor_pipe_peak_at_sampled_clock": clock_peak,
            "all_gemms_achieved": gemm_all,
            "gemm_ms": {LAYERS[i][0]: gemm_mean_ms[i] for i in range(len(LAYERS))},
            "traffic": int(traffic * m / m_total) if traffic else None,
        }
        if lib_int8 and "burst_tops" in lib_int8:
            roofline["library_int8_mm_burst_tops_same_codes"] = lib_int8["burst_tops"]
            roofline["frac_of_library_int8_burst"] = achieved / lib_int8["burst_tops"]
        elif lib_int8:
            roofline["library_int8_mm"] = lib_int8
        if sustained is not None:
            sus_qkv = qkv_ops / (sustained["gemm_ms"][LAYERS[0][0]] * 1e-3) / 1e12
            mhz = sustained["clocks"]["sm_mhz"] or 0
            sustained.update({
                "qkv_gemm_tops": sus_qkv, "peak": sus_peak,
                "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({src})",
                "frac": sus_qkv / sus_peak, "frac_of_nominal_int8_4500": sus_qkv / INT8_NOMINAL_TOPS,
                "all_gemms_tops": sum(2.0 * m * k * n for k, n in layers_meta) /
                                  (sum(sustained["gemm_ms"].values()) * 1e-3) / 1e12,
                "qkv_gemm_ms_x_sm_mhz": sustained["gemm_ms"][LAYERS[0][0]] * mhz,
                "frac_of_tensor_pipe_at_sampled_clock":
                    sus_qkv / (2.0 * 8192 * sm_count * mhz * 1e6 / 1e12) if mhz else None})
            if lib_int8 and "sustained_tops" in lib_int8:
                sustained["library_int8_mm_sustained_tops_same_codes"] = lib_int8["sustained_tops"]
                sustained["library_int8_mm_sustained_sm_mhz"] = lib_int8["sustained_sm_mhz"]
                sustained["frac_of_library_int8_sustained"] = sus_qkv / lib_int8["sustained_tops"]
        hbm = peaks.get("hbm_gbs")
        quantizer = {"bound": "hbm", "kernel": "quant_act_rows_kernel", "peak_gb_per_s": hbm,
                     "bytes_per_row": {"container": "2K (fp16 read) + K (int8 codes) + 4 (fp32 scale)",
                                       "algorithmic_int4": "2K (fp16 read) + K/2 (int4 codes) + 2 (fp16 scale)"},
                     "gb_per_s": {}, "frac_of_measured_copy": {}, "gb_per_s_algorithmic_int4": {},
                     "frac_algorithmic_int4": {}}
        for i, (name, k, _) in enumerate(LAYERS):
            if m == 0 or quant_mean_ms[i] <= 0:
                continue
            sec = quant_mean_ms[i] * 1e-3
            a, b = m * (3.0 * k + 4) / sec / 1e9, m * (2.5 * k + 2) / sec / 1e9
            quantizer["gb_per_s"][name], quantizer["gb_per_s_algorithmic_int4"][name] = a, b
            if hbm:
                quantizer["frac_of_measured_copy"][name], quantizer["frac_algorithmic_int4"][name] = a / hbm, b / hbm
        line = {
            "metric": "w4a4_linear_tops", "value": value, "unit": "TOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic", "config": base_config(args.workload, m_total, world, cta_group),
            "e2e": e2e, "gpu_launches": 2 * len(LAYERS) * args.steps, "clocks": clocks,
            "roofline": roofline, "sustained": sustained, "quantizer": quantizer,
        }
        if shard_check is not None:
            line["sharded_vs_unsharded"] = shard_check
        if gpu_baseline is not None:
            line["gpu_baseline"] = gpu_baseline
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        if dit is not None:
            line["dit_step"] = dit
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
