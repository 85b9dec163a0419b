#!/usr/bin/env python
"""Times one classifier-free-guidance DiT denoising step of the harness model (harness/wan_dit.py)
with every block linear running through the W4A4 library.

    python harness/dit_step.py --model wan21_14b --steps 5 --warmup 2
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P harness/dit_step.py --model wan21_14b

Parallel layout (one process per GPU, weights replicated; the work of a step is fixed, so
scaling is strong):
  N = 1   cond and uncond forwards run back to back on the one GPU
  N = 2   one CFG branch per GPU, one all-gather of the two noise predictions
  N = 4/8 N/2 GPUs per branch: token rows sharded inside the branch, K and V of every
          self-attention exchanged inside the branch, then the same exchange of predictions
The cond-only step (after the guidance boundary) row-shards the single forward over all N GPUs.
The K/V exchange has three routes: "nccl" (two asynchronous all-gathers per block, overlapped with
the q/k glue kernels), "peer_stores" (the kernels that produce K and V store their rows into every
rank's gather buffer, dsaquant_b200/peer_exchange.py; the default, bit-identical to "nccl") and,
reported beside them, "peer_stores_overlap" (the same stores, with attention split into a local and
a remote part merged by log-sum-exp so that the exchange hides behind the local part; not
bit-identical: the merge rounds twice).

`measure()` is what bench.py calls for its `dit_step` key; `main()` prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

DEFAULT_ROUTE = "peer_stores"


class Layout:
    """Process groups of the two layouts.  Collective constructor: every rank builds it once."""

    def __init__(self, dist, world: int, rank: int):
        self.world, self.rank = world, rank
        self.world_group = dist.group.WORLD if world > 1 else None
        self.branch = None            # CFG layout: which forward this rank computes
        self.branch_group = None      # CFG layout: row-sharding group inside the branch (None: unsharded)
        if world > 1:
            half = world // 2
            groups = [dist.new_group(list(range(0, half))), dist.new_group(list(range(half, world)))]
            self.branch = 0 if rank < half else 1
            self.branch_group = groups[self.branch] if half > 1 else None

    def cfg_name(self) -> str:
        if self.world == 1:
            return "sequential cond+uncond"
        return "cfg2" if self.world == 2 else f"cfg2 x rows{self.world // 2}"

    def cond_name(self) -> str:
        return f"rows{self.world}" if self.world > 1 else "single"


def _barrier(torch, dist, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def time_steps(torch, dist, world, device, step_fn, steps: int, warmup: int):
    """(ms per step as the max over ranks, last output).  CUDA events on the current stream,
    barrier + synchronize on both sides."""
    out = None
    for _ in range(warmup):
        out = step_fn()
    _barrier(torch, dist, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step_fn()
    e1.record()
    _barrier(torch, dist, world)
    ms = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()), out


def _cosine(torch, a, b) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b / (a.norm() * b.norm()).clamp_min(1e-300)).item())


def sharded_vs_unsharded(torch, dist, wan_dit, cfg, device, world_group, exchange, inputs, overlap_ok=False) -> dict:
    """Correctness record carried by the multi-GPU run itself: a 2-block model of the same width,
    the same weights on every rank; one forward unsharded on this GPU, one row-sharded over all
    ranks with the NCCL route, one with the peer-store route and one with the peer-store route
    hidden behind local attention.  The first two must agree bit for bit (the third merges two
    partial attention results, so it is held to the cosine bound); against the unsharded forward only the attention kernel's tiling of the query
    rows differs, so cosine similarity (>= 0.999) and the largest difference are reported."""
    small = wan_dit.WanConfig(cfg.name + "_2blk", cfg.dim, cfg.heads, cfg.ffn, 2, cfg.in_ch, cfg.out_ch, cfg.latent)
    model = wan_dit.build_model(small, device, seed=3, backend="kernel")
    model.set_fused(True)
    latent, timestep, text = inputs
    ref = model(latent, timestep, text)
    model.set_kv_exchange(None)
    a = model(latent, timestep, text, group=world_group)
    rec = {"model": f"{small.dim}-wide, 2 blocks, {small.tokens} tokens, rows{dist.get_world_size(world_group)}",
           "cosine_nccl_vs_unsharded": _cosine(torch, a, ref),
           "max_abs_diff_nccl_vs_unsharded": float((a.float() - ref.float()).abs().max().item()),
           "output_abs_max": float(ref.float().abs().max().item())}
    if exchange is not None:
        model.set_kv_exchange(exchange)
        b = model(latent, timestep, text, group=world_group)
        model.set_kv_exchange(None)
        rec["peer_stores_equals_nccl"] = bool(torch.equal(a, b))
        if overlap_ok:
            model.set_kv_exchange(exchange, overlap=True)
            c = model(latent, timestep, text, group=world_group)
            model.set_kv_exchange(None)
            rec["cosine_overlap_vs_unsharded"] = _cosine(torch, c, ref)
            rec["max_abs_diff_overlap_vs_unsharded"] = float((c.float() - ref.float()).abs().max().item())
    # every rank must have seen the same thing
    # The overlap route is reported, not required: merging two bf16 partial attention results moves the
    # attention output by about one bf16 ulp, which a random-weight 4-bit model amplifies (see the
    # fused-vs-op-by-op note in tests/test_dit_harness.py); it is opt-in for that reason.
    ok = torch.tensor([1 if (rec["cosine_nccl_vs_unsharded"] >= 0.999 and rec.get("peer_stores_equals_nccl", True)) else 0],
                      device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=world_group)
    rec["all_ranks_ok"] = bool(ok.item())
    del model
    torch.cuda.empty_cache()
    return rec


def measure(model_name: str, steps: int, warmup: int, *, layers: int = 0, fused: bool = True,
            with_routes: bool = True, with_phases: bool = True, with_check: bool = True,
            cond_only: bool = True, default_route: str = DEFAULT_ROUTE) -> dict:
    """Times the CFG step (and the cond-only step) of `model_name` at the current world size.
    Expects torch.distributed to be initialised when WORLD_SIZE > 1.  Returns a dict (same on
    every rank except the per-phase split, which is this rank's own)."""
    import torch
    import torch.distributed as dist

    from dsaquant_b200.kernels import vdm_w4a4 as vdm
    from harness import wan_dit
    from harness.bench_common import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    device = torch.device("cuda", torch.cuda.current_device())
    steps, warmup = max(1, steps), max(1, warmup)

    cfg = wan_dit.CONFIGS[model_name]
    if layers:
        cfg = wan_dit.WanConfig(cfg.name + f"_{layers}blk", cfg.dim, cfg.heads, cfg.ffn, layers,
                                cfg.in_ch, cfg.out_ch, cfg.latent)
    layout = Layout(dist, world, rank)
    t0 = time.time()
    model = wan_dit.build_model(cfg, device, seed=0, backend="kernel")
    torch.cuda.synchronize()
    build_s = time.time() - t0
    model_gb = torch.cuda.memory_allocated(device) / 1e9
    model.set_fused(fused)
    latent, timestep, text = wan_dit.synth_inputs(cfg, device, seed=1)
    _, _, text_neg = wan_dit.synth_inputs(cfg, device, seed=2, negative=True)

    # Exchange memory for the peer-store route, one per sharding group.
    ex_world = ex_branch = None
    ex_error = None
    if with_routes and fused and world > 1:
        try:
            ex_world = model.make_kv_exchange(layout.world_group)
            if layout.branch_group is not None:
                ex_branch = model.make_kv_exchange(layout.branch_group)
        except Exception as exc:  # symmetric memory not available on this box
            ex_world = ex_branch = None
            ex_error = f"{type(exc).__name__}: {exc}"[:200]

    # The overlap route needs a library attention call that returns the log-sum-exp: probe it once,
    # outside any exchange, so that a missing kernel never interrupts a block half way.
    lse_ok = False
    if ex_world is not None:
        try:
            hd = cfg.dim // cfg.heads
            probe = torch.randn(1, cfg.heads, 128, hd, device=device, dtype=torch.bfloat16)
            wan_dit.sdpa_with_lse(probe, probe, probe)
            lse_ok = True
        except RuntimeError as exc:
            result_note = str(exc)[:200]
        ok = torch.tensor([1 if lse_ok else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        lse_ok = bool(ok.item())

    def run_cfg():
        return wan_dit.cfg_step(model, latent, timestep, text, text_neg, 5.0, branch_group=layout.branch_group,
                                world_group=layout.world_group, branch=layout.branch)

    def run_cond():
        return model(latent, timestep, text, group=layout.world_group)

    plans = [("cfg_step", run_cfg, layout.cfg_name(), layout.branch_group is not None, ex_branch)]
    if cond_only:
        plans.append(("cond_only_step", run_cond, layout.cond_name(), world > 1, ex_world))

    d, f, L, m = cfg.dim, cfg.ffn, cfg.layers, cfg.tokens
    per_fwd = L * (2.0 * m * d * (3 * d + d + d + d) + 2.0 * cfg.text_len * d * 2 * d + 2.0 * m * d * f * 2)
    result = {"model": cfg.name, "tokens": m, "layers": L, "dim": d, "ffn": f, "heads": cfg.heads,
              "n_gpus": world, "steps": steps, "warmup": warmup, "guidance": 5.0, "fused_elementwise": bool(fused),
              "attention": "bf16 SDPA (library)", "model_build_s": round(build_s, 1),
              "model_memory_gb": round(model_gb, 2),
              "w4a4_linear_tera_ops_per_forward": per_fwd / 1e12}
    if ex_error:
        result["peer_stores_unavailable"] = ex_error
    if ex_world is not None and not lse_ok:
        result["overlap_unavailable"] = "no library attention kernel returned a log-sum-exp on this box"
    elif lse_ok:
        result["attention_with_lse"] = wan_dit._LSE_BACKEND

    for key, fn, name, has_exchange, exchange in plans:
        routes = ["none"]
        if has_exchange:
            routes = ["nccl"] + (["peer_stores"] if exchange is not None else []) + \
                     (["peer_stores_overlap"] if exchange is not None and lse_ok else [])
        rec = {"parallelism": name, "routes_ms": {}}
        for route in routes:
            model.set_kv_exchange(exchange if route != "nccl" else None, overlap=route.endswith("overlap"))
            sampler = ClockSampler(device.index).start()
            ms, out = time_steps(torch, dist, world, device, fn, steps, warmup)
            rec["routes_ms"][route] = ms
            rec.setdefault("clocks", {})[route] = sampler.stop()
            rec.setdefault("output_abs_sum", {})[route] = float(out.double().abs().sum().item())
            rec["output_finite"] = bool(torch.isfinite(out).all())
        chosen = next(r for r in (default_route, "peer_stores", "nccl", "none") if r in rec["routes_ms"])
        rec["kv_exchange"] = {"none": "none (no row sharding inside a forward)", "nccl": "nccl all-gather (async, overlapped)",
                              "peer_stores": "peer stores from the producing kernels",
                              "peer_stores_overlap": "peer stores from the producing kernels, hidden behind attention over "
                                                     "the local keys (two attention calls merged by log-sum-exp)"}[chosen]
        rec["ms"] = rec["routes_ms"][chosen]
        if "peer_stores" in rec["routes_ms"]:
            rec["routes_agree"] = rec["output_abs_sum"]["nccl"] == rec["output_abs_sum"]["peer_stores"]
        result[key] = rec
        model.set_kv_exchange(None)
    status = vdm.last_device_status(device.index)
    result["device_status"] = status

    if with_phases:
        # One extra, untimed CFG step with event marks between phases (this rank's own stream).
        chosen_ex = ex_branch if (default_route.startswith("peer_stores") and ex_branch is not None) else None
        phase_route = "none"
        if layout.branch_group is not None:
            phase_route = result["cfg_step"]["kv_exchange"]
        model.set_kv_exchange(chosen_ex, overlap=(chosen_ex is not None and default_route.endswith("overlap")
                                                  and "peer_stores_overlap" in result["cfg_step"]["routes_ms"]))
        timer = wan_dit.PhaseTimer()
        wan_dit.set_phase_timer(timer)
        try:
            run_cfg()
            torch.cuda.synchronize()
        finally:
            wan_dit.set_phase_timer(None)
            model.set_kv_exchange(None)
        tot = timer.totals_ms()
        names = {"gemm": "gemm_ms", "quant": "quantiser_ms", "glue": "glue_ms", "sdpa": "sdpa_ms",
                 "exchange_wait": "exchange_wait_ms", "other": "other_ms"}
        phases = {v: round(tot.get(k, 0.0), 3) for k, v in names.items()}
        phases["sum_ms"] = round(sum(tot.values()), 3)
        phases["limiting_phase"] = max(names, key=lambda k: tot.get(k, 0.0))
        phases["route"] = phase_route
        phases["note"] = ("CUDA events on rank 0's stream during one extra CFG step; 'glue' = qk_norm_rope passes, "
                          "'exchange_wait' = stream time blocked on K/V of peers, 'other' = embeddings, "
                          "modulation vectors, output projection, prediction gather")
        result["cfg_step"]["phases"] = phases

    if with_check and world > 1 and fused:
        result["sharded_vs_unsharded"] = sharded_vs_unsharded(
            torch, dist, wan_dit, cfg, device, layout.world_group, ex_world, (latent, timestep, text), overlap_ok=lse_ok)
    del model
    torch.cuda.empty_cache()
    return result


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="wan21_1.3b", choices=["wan21_1.3b", "wan22_5b", "wan21_14b"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0, help="override the number of blocks (0 = model's own)")
    ap.add_argument("--no-fused", action="store_true",
                    help="run norms / modulation / GELU / gated skips as separate PyTorch ops")
    ap.add_argument("--route", default=DEFAULT_ROUTE, choices=["nccl", "peer_stores", "peer_stores_overlap"],
                    help="K/V exchange whose time is reported as the headline (both are timed)")
    ap.add_argument("--no-check", action="store_true")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    assert vdm.is_available(), vdm.load_error()
    r = measure(args.model, args.steps, args.warmup, layers=args.layers, fused=not args.no_fused,
                with_check=not args.no_check, default_route=args.route)
    if rank == 0:
        line = {"metric": "dit_step_ms", "value": r["cfg_step"]["ms"], "unit": "ms", "n_gpus": world,
                "steps": r["steps"], "warmup": r["warmup"], "higher_is_better": False, "scaling": "strong",
                "dtype": "int8 linears / bf16 attention", "data": "synthetic",
                "config": {"workload": f"{r['model']} CFG step", "tokens": r["tokens"], "layers": r["layers"],
                           "parallelism": r["cfg_step"]["parallelism"], "kv_exchange": r["cfg_step"]["kv_exchange"]},
                "dit_step": r}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
