"""Natural sharding of the W4A4 linear layer across GPUs of one node.

Every output row depends on one input row only (per-token activation scale, replicated
weights), so the token dimension M splits across ranks with no communication inside the layer.
An all-gather of the fp16 outputs is needed only by callers that want the full [M,N] matrix on
every rank (self-attention keys/values under row sharding).  The reference is single-GPU
(its sequence-parallel hooks are identity stubs, vdm_infer/models/wan_vdm/modules/attention.py:20-32),
so this module has no counterpart there; it defines the partition the multi-GPU benchmarks use.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

ROW_ALIGN = 256  # one CTA-pair tile of the GEMM: keeps every shard but the last free of tail tiles


def row_partition(m: int, world: int, align: int = ROW_ALIGN) -> List[Tuple[int, int]]:
    """Contiguous [start, end) row ranges, one per rank; every boundary except the end of the
    matrix is a multiple of `align`; sizes differ by less than two aligned blocks; empty shards only
    when there are fewer blocks than ranks."""
    if m < 0 or world < 1 or align < 1:
        raise ValueError("row_partition needs m >= 0, world >= 1, align >= 1")
    blocks = (m + align - 1) // align
    base, extra = divmod(blocks, world)
    bounds, start = [], 0
    for r in range(world):
        nblk = base + (1 if r < extra else 0)
        end = min(m, start + nblk * align)
        bounds.append((start, end))
        start = end
    return bounds


def shard_rows(x: torch.Tensor, rank: int, world: int, align: int = ROW_ALIGN) -> torch.Tensor:
    """This rank's rows of a [M, ...] tensor (a view)."""
    start, end = row_partition(x.shape[0], world, align)[rank]
    return x[start:end]


def all_gather_rows(y_local: torch.Tensor, m_total: int, group=None, align: int = ROW_ALIGN) -> torch.Tensor:
    """All-gather row shards produced under row_partition into the full [m_total, N] tensor.
    Shards are padded to the largest shard for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    bounds = row_partition(m_total, world, align)
    max_rows = max(e - s for s, e in bounds)
    n = y_local.shape[1]
    padded = y_local.new_zeros((max_rows, n))
    padded[: y_local.shape[0]].copy_(y_local)
    gathered = y_local.new_empty((world * max_rows, n))
    dist.all_gather_into_tensor(gathered, padded, group=group)
    out = y_local.new_empty((m_total, n))
    for r, (s, e) in enumerate(bounds):
        out[s:e].copy_(gathered[r * max_rows: r * max_rows + (e - s)])
    return out


def linear_rows_sharded(x_local: torch.Tensor, qweight: torch.Tensor, wscales: torch.Tensor,
                        bias: Optional[torch.Tensor] = None, clip_ratio: float = 1.0, *,
                        m_total: Optional[int] = None, gather: bool = False, group=None,
                        linear_fn: Optional[Callable] = None) -> torch.Tensor:
    """W4A4 linear on this rank's token rows; with gather=True returns the full output."""
    if linear_fn is None:
        from .kernels.vdm_w4a4 import linear_vdm_w4a4 as linear_fn
    y = linear_fn(x_local, qweight, wscales, bias, clip_ratio)
    if not gather:
        return y
    if m_total is None:
        raise ValueError("gather=True needs m_total")
    return all_gather_rows(y, m_total, group)
