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
    """Contiguous [start, end) row ranges, one per rank.  Every rank gets the same number of
    aligned blocks, ceil(blocks / world), until the rows run out: all shards but the last
    non-empty one have equal size, so an all-gather of equally padded shards leaves its padding
    at the very end of the gathered buffer and the result is a plain prefix view.  The largest
    shard is as small as any aligned split allows; trailing ranks are empty only when there are
    fewer blocks than ranks."""
    if m < 0 or world < 1 or align < 1:
        raise ValueError("row_partition needs m >= 0, world >= 1, align >= 1")
    blocks = (m + align - 1) // align
    per = (blocks + world - 1) // world * align
    return [(min(m, r * per), min(m, (r + 1) * per)) for r in range(world)]


def shard_capacity(m: int, world: int, align: int = ROW_ALIGN) -> int:
    """Rows of the (equal) padded shard every rank contributes to an all-gather."""
    blocks = (m + align - 1) // align
    return (blocks + world - 1) // world * align


def shard_rows(x: torch.Tensor, rank: int, world: int, align: int = ROW_ALIGN) -> torch.Tensor:
    """This rank's rows of a [M, ...] tensor (a view)."""
    start, end = row_partition(x.shape[0], world, align)[rank]
    return x[start:end]


def all_gather_rows(y_local: torch.Tensor, m_total: int, group=None, align: int = ROW_ALIGN,
                    async_op: bool = False):
    """All-gather row shards produced under row_partition into the full [m_total, N] tensor.
    Full shards go into the collective as they are; only a short (last) shard is padded.  The
    result is a prefix view of the gathered buffer: no copy on the receiving side.
    With async_op=True returns (work, result_view); wait on `work` before reading the view."""
    world = dist.get_world_size(group)
    cap = shard_capacity(m_total, world, align)
    n = y_local.shape[1]
    if y_local.shape[0] != cap:
        padded = y_local.new_zeros((cap, n))
        padded[: y_local.shape[0]].copy_(y_local)
        y_local = padded
    elif not y_local.is_contiguous():
        y_local = y_local.contiguous()
    gathered = y_local.new_empty((world * cap, n))
    work = dist.all_gather_into_tensor(gathered, y_local, group=group, async_op=async_op)
    out = gathered[:m_total]
    return (work, out) if async_op else out


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
