#!/usr/bin/env python
"""Strong-scaling M-split sweep of a Wan GEMM set: the 32760 token rows of every layer are
sharded over the ranks (dsaquant_b200.sharding.row_partition, weights replicated), each rank
runs quantise + W4A4 GEMM on its rows, and the step is timed without and with the all-gather
of the fp16 outputs (needed only by callers that want the full matrix on every rank).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P harness/msplit_bench.py --set wan1.3b

Prints one JSON line (rank 0): TOP/s = 2*M*sum(N*K) / max-over-ranks step time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

SETS = {
    "wan1.3b": [(1536, 4608), (1536, 1536), (1536, 8960), (8960, 1536)],
    "wan14b": [(5120, 15360), (5120, 5120), (5120, 13824), (13824, 5120)],
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--set", default="wan1.3b", choices=sorted(SETS))
    ap.add_argument("--tokens", type=int, default=32760)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import bench
    from dsaquant_b200 import sharding
    from dsaquant_b200.kernels import vdm_w4a4 as vdm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    assert vdm.is_available(), vdm.load_error()

    m_total = args.tokens
    start, end = sharding.row_partition(m_total, world)[rank]
    m = end - start
    shapes = SETS[args.set]
    layers = [bench.make_layer(torch, vdm, k, n, 100 + i, device) for i, (k, n) in enumerate(shapes)]
    xs = {k: bench.make_activations(torch, m_total, k, 7, device)[start:end].contiguous()
          for k in sorted({k for k, _ in shapes})}

    def step(gather: bool):
        outs = []
        for L in layers:
            y = vdm.linear_vdm_w4a4(xs[L["k"]], L["qweight"], L["wscales"], None, 0.95, bias_half=L["bias"])
            if gather and world > 1:
                y = sharding.all_gather_rows(y, m_total)
            outs.append(y)
        return outs

    def timed(gather: bool) -> float:
        for _ in range(max(3, args.warmup)):
            step(gather)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step(gather)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_local = timed(False)
    ms_gather = timed(True)
    assert vdm.last_device_status(local_rank) == 0
    if rank == 0:
        ops = sum(2.0 * m_total * k * n for k, n in shapes)
        print(json.dumps({
            "metric": "w4a4_linear_tops", "unit": "TOP/s", "n_gpus": world, "scaling": "strong",
            "value": ops / (ms_local * 1e-3) / 1e12, "ms_per_step": ms_local,
            "value_with_output_allgather": ops / (ms_gather * 1e-3) / 1e12, "ms_per_step_with_allgather": ms_gather,
            "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": f"{args.set}_linear_set_M{m_total}_msplit", "rows_per_rank": m,
                       "layers": [list(s) for s in shapes], "parallelism": f"rows{world}"},
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
