#!/usr/bin/env python
"""Times one classifier-free-guidance DiT denoising step of the harness model (harness/wan_dit.py)
with every block linear running through the W4A4 library.

    python harness/dit_step.py --model wan21_14b --steps 3 --warmup 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P harness/dit_step.py --model wan21_14b

Parallel layout (one process per GPU, weights replicated):
  N = 1   cond and uncond forwards run back to back on the one GPU
  N = 2   one CFG branch per GPU, one all-gather of the two noise predictions
  N = 4/8 N/2 GPUs per branch: token rows sharded inside the branch (all-gather of K and V per
          self-attention), then the same exchange of predictions
`--cond-only` times the single-branch step used after the guidance boundary (all N GPUs row-shard
the one forward).  The total work of a step is fixed, so scaling is strong.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="wan21_1.3b", choices=["wan21_1.3b", "wan22_5b", "wan21_14b"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="override the number of blocks (0 = model's own)")
    ap.add_argument("--cond-only", action="store_true")
    ap.add_argument("--fused", action="store_true",
                    help="fold layer norm + modulation, GELU and gated skips into the W4A4 library calls")
    ap.add_argument("--kv-push", action="store_true",
                    help="with --fused and row sharding: K/V exchange by peer stores from the producing kernels "
                         "(dsaquant_b200/peer_exchange.py) instead of NCCL all-gathers")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from harness import wan_dit
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    assert vdm.is_available(), vdm.load_error()

    cfg = wan_dit.CONFIGS[args.model]
    if args.layers:
        cfg = wan_dit.WanConfig(cfg.name + f"_{args.layers}blk", cfg.dim, cfg.heads, cfg.ffn, args.layers,
                                cfg.in_ch, cfg.out_ch, cfg.latent)
    t0 = time.time()
    model = wan_dit.build_model(cfg, device, seed=0, backend="kernel")
    build_s = time.time() - t0
    model.set_fused(args.fused)
    latent, timestep, text = wan_dit.synth_inputs(cfg, device, seed=1)
    _, _, text_neg = wan_dit.synth_inputs(cfg, device, seed=2, negative=True)

    branch, branch_group, world_group = None, None, None
    if world > 1:
        world_group = dist.group.WORLD
        if args.cond_only:
            branch_group = world_group
        else:
            half = world // 2
            groups = [dist.new_group(list(range(0, half))), dist.new_group(list(range(half, world)))]
            branch = 0 if rank < half else 1
            branch_group = groups[branch] if half > 1 else None

    if args.kv_push and args.fused and branch_group is not None:
        model.enable_kv_push(branch_group)

    def step():
        if args.cond_only:
            return model(latent, timestep, text, group=branch_group)
        return wan_dit.cfg_step(model, latent, timestep, text, text_neg, 5.0,
                                branch_group=branch_group, world_group=world_group, branch=branch)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup)):
        out = step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert vdm.last_device_status(local_rank) == 0
    finite = bool(torch.isfinite(out).all())
    checksum = float(out.double().abs().sum().item())

    if rank == 0:
        d, f, L, m = cfg.dim, cfg.ffn, cfg.layers, cfg.tokens
        per_fwd = L * (2.0 * m * d * (3 * d + d + d + d) + 2.0 * cfg.text_len * d * 2 * d + 2.0 * m * d * f * 2)
        forwards = 1 if args.cond_only else 2
        if args.cond_only:
            layout = f"rows{world}" if world > 1 else "single"
        else:
            layout = "sequential cond+uncond" if world == 1 else (
                "cfg2" if world == 2 else f"cfg2 x rows{world // 2}")
        print(json.dumps({
            "metric": "dit_step_ms", "value": float(ms.item()), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(1, args.warmup), "higher_is_better": False,
            "scaling": "strong", "dtype": "int8 linears / bf16 attention", "data": "synthetic",
            "config": {"workload": f"{cfg.name} CFG step" + (" (cond only)" if args.cond_only else ""),
                       "tokens": m, "layers": L, "dim": d, "ffn": f, "heads": cfg.heads,
                       "parallelism": layout, "guidance": 5.0,
                       "fused_elementwise": bool(args.fused),
                       "kv_exchange": "peer stores" if (args.kv_push and args.fused and branch_group is not None)
                       else ("nccl all-gather" if branch_group is not None else "none")},
            "w4a4_linear_tera_ops_per_step": forwards * per_fwd / 1e12,
            "output_finite": finite, "output_abs_sum": checksum, "model_build_s": round(build_s, 1),
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
