"""K/V exchange of a row-sharded attention group through peer memory instead of an all-gather.

Row sharding (sharding.py) leaves every rank with its own rows of K and V, while each rank's
attention needs all rows of its group.  The reference planned a sequence-parallel exchange for
this (the Ulysses stubs in vdm_infer/models/wan_vdm/modules/attention.py:20-32, :173-174); the
harness first used an NCCL all-gather per tensor.  Here the kernel that produces K / V
(b200w4a4_qk_norm_rope_push) stores its rows straight into every rank's gather buffer, so the
exchange costs no extra pass and no extra launch on the producer side:

  per self-attention block with epoch e (parity p = e & 1 selects one of two buffer sets)
    1. wait  done[p][*]  >= e - 2      every rank has finished reading the set used two blocks ago
    2. push V, push K into set p of every rank; each push raises ready_v / ready_k[p][me] = e there
    3. wait  ready_k[p][*], ready_v[p][*] >= e      (bounded, on this rank's own flag arrays)
    4. attention reads set p of this rank
    5. signal done[p][me] = e on every rank           (ordered after the attention kernel)

`rotated=True` changes where rows land: every rank's own shard sits at rows [0, capacity) of its own
buffers and the peers' shards follow in ascending rank order from row `capacity` on (a softmax over
keys does not care about their order).  Local and remote keys are then two contiguous ranges, so
attention over the local range can run while the remote range is still arriving (`local_rows`
needs no wait at all, `remote_rows` enqueues the waits).  Requires every rank to own rows.

Every wait is bounded (b200w4a4_wait_flags): a peer that never arrives shows up as device status
105, not as a hang.  Only plain loads and stores touch peer memory; no multicast loads.

The class below is the bookkeeping.  It works on device addresses, so the same code serves real
peers (addresses from symmetric memory, `from_symmetric_memory`) and an emulated group inside one
process and one GPU (addresses of ordinary tensors), which is how it is tested where fewer GPUs
than ranks are available.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import _lib
from . import attention_qkv as aq

_KINDS = ("k", "v")


@dataclass
class RankMemory:
    """Device addresses of one rank's exchange memory as seen from the calling rank."""
    kv: List[List[int]]      # [parity][kind] -> base of a [capacity, D] matrix
    ready: List[List[int]]   # [parity][kind] -> base of an int32 [group] array
    done: List[int]          # [parity] -> base of an int32 [group] array


def exchange_bytes(capacity_rows: int, dim: int, group: int) -> int:
    """Bytes of exchange memory one rank needs (two buffer sets of K and V, plus flags)."""
    flags = 2 * (2 + 1) * _round_up(4 * group, 256)
    return 2 * 2 * _round_up(capacity_rows * dim * 2, 256) + flags


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def layout(base: int, capacity_rows: int, dim: int, group: int) -> RankMemory:
    """Carves one rank's exchange memory (exchange_bytes long, zero-initialised) starting at `base`."""
    mat = _round_up(capacity_rows * dim * 2, 256)
    fl = _round_up(4 * group, 256)
    kv, ready, done = [], [], []
    off = base
    for _ in range(2):
        row = []
        for _ in _KINDS:
            row.append(off)
            off += mat
        kv.append(row)
    for _ in range(2):
        row = []
        for _ in _KINDS:
            row.append(off)
            off += fl
        ready.append(row)
    for _ in range(2):
        done.append(off)
        off += fl
    return RankMemory(kv, ready, done)


class PeerKVExchange:
    def __init__(self, rank: int, members: Sequence[RankMemory], local: torch.Tensor, capacity_rows: int,
                 dim: int, row0: int, dtype: torch.dtype = torch.bfloat16, timeout_ms: int = 1000,
                 shard_rows: Optional[Sequence[int]] = None):
        """rank: index of this rank inside the group; members[r]: rank r's memory as mapped here
        (members[rank] must describe `local`, this rank's own zero-initialised exchange memory, a
        uint8 tensor of exchange_bytes); row0: first row of this rank's shard."""
        self.rank, self.members, self.local = rank, list(members), local
        self.group = len(self.members)
        if self.group > 8:
            raise ValueError("at most 8 ranks per attention group")
        self.capacity, self.dim, self.row0, self.dtype = capacity_rows, dim, row0, dtype
        self.timeout_ms = timeout_ms
        self.device = local.device
        self.rotated = False
        self.shard_rows = list(shard_rows) if shard_rows is not None else None
        self.epoch = 0                      # blocks use epochs 1, 2, ...: the first two wait for -1 and 0, both met by the zero-initialised flags
        self.ticket = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._lib = _lib.load()
        mine = self.members[rank]
        base = local.data_ptr()
        size = local.numel()

        def view(addr: int, nbytes: int, dt: torch.dtype, shape):
            o = addr - base
            if o < 0 or o + nbytes > size:
                raise ValueError("members[rank] does not describe the local exchange memory")
            return local[o:o + nbytes].view(dt).view(*shape)

        self._kv = [[view(mine.kv[p][i], capacity_rows * dim * 2, dtype, (capacity_rows, dim)) for i in range(2)]
                    for p in range(2)]
        self._ready = [[view(mine.ready[p][i], 4 * self.group, torch.int32, (self.group,)) for i in range(2)]
                       for p in range(2)]
        self._done = [view(mine.done[p], 4 * self.group, torch.int32, (self.group,)) for p in range(2)]

    # ---- rotated placement -----------------------------------------------------------------------
    def set_rotated(self, on: bool) -> None:
        """Own shard first, peers after it (see the module text).  Switch only between blocks, on
        every rank of the group alike."""
        if on:
            if self.shard_rows is None or len(self.shard_rows) != self.group or min(self.shard_rows) < 1:
                raise ValueError("rotated placement needs the row count of every rank's shard, all non-empty")
            per = self.capacity // self.group
            if any(r > per for r in self.shard_rows) or any(r != per for r in self.shard_rows[:-1]):
                raise ValueError("rotated placement expects equal shards except a shorter last one")
        self.rotated = bool(on)

    def _slot_row(self, sender: int, receiver: int) -> int:
        """First row of `sender`'s shard inside `receiver`'s buffers."""
        if not self.rotated:
            return self.row0 if sender == self.rank else -1     # plain layout: the global row offset
        per = self.capacity // self.group
        if sender == receiver:
            return 0
        others = [x for x in range(self.group) if x != receiver]
        return per * (1 + others.index(sender))

    # ---- one self-attention block ------------------------------------------------------------
    def begin_block(self) -> int:
        """Step 1: new epoch; waits until every rank has released the buffer set it will overwrite."""
        self.epoch += 1
        p = self.epoch & 1
        aq.wait_flags(self._done[p], self.epoch - 2, self.timeout_ms)
        return self.epoch

    def push(self, kind: str, x: torch.Tensor, norm_weight: Optional[torch.Tensor],
             cos_sin: Optional[torch.Tensor], eps: float, head_dim: int) -> None:
        """Step 2 for K (`kind="k"`: RMSNorm + rotary + cast) or V (`kind="v"`: cast only)."""
        i = _KINDS.index(kind)
        p = self.epoch & 1
        if x.reshape(-1, x.shape[-1]).shape[0] + self.row0 > self.capacity:
            raise ValueError("shard does not fit the gather buffer")
        if self.rotated:
            # per-destination row offsets are folded into the destination addresses
            pitch = self.dim * 2
            dests = [m.kv[p][i] + self._slot_row(self.rank, r) * pitch for r, m in enumerate(self.members)]
            row0 = 0
        else:
            dests, row0 = [m.kv[p][i] for m in self.members], self.row0
        aq.qk_norm_rope_push(
            x, norm_weight, cos_sin, eps, head_dim, dests, self.dim, row0,
            self.dtype, flag_ptrs=[m.ready[p][i] for m in self.members], flag_index=self.rank, epoch=self.epoch,
            ticket=self.ticket)

    def gathered(self, rows: int, senders: Optional[int] = None):
        """Steps 3-4: waits for the first `senders` ranks (default: all; ranks behind them own no rows
        under the equal-capacity partition and send nothing) and returns this rank's (K, V) [rows, D]."""
        p = self.epoch & 1
        n = self.group if senders is None else senders
        for i in range(2):
            aq.wait_flags(self._ready[p][i][:n], self.epoch, self.timeout_ms)
        return self._kv[p][0][:rows], self._kv[p][1][:rows]

    def local_rows(self):
        """Rotated placement: this rank's own (K, V) rows of the current block.  They were written by
        this rank's own push kernels, so stream order is all the synchronisation they need."""
        p = self.epoch & 1
        n = self.shard_rows[self.rank]
        return self._kv[p][0][:n], self._kv[p][1][:n]

    def remote_rows(self):
        """Rotated placement: enqueues the bounded waits for every peer's K and V and returns the
        peers' (K, V) rows as one contiguous range."""
        p = self.epoch & 1
        for i in range(2):
            aq.wait_flags(self._ready[p][i], self.epoch, self.timeout_ms)
        per = self.capacity // self.group
        n = sum(r for x, r in enumerate(self.shard_rows) if x != self.rank)
        return self._kv[p][0][per:per + n], self._kv[p][1][per:per + n]

    def end_block(self) -> None:
        """Step 5: after the attention kernel (stream order), release the buffer set on every rank."""
        p = self.epoch & 1
        ptrs = (ctypes.c_void_p * self.group)(*[m.done[p] for m in self.members])
        with torch.cuda.device(self.device):
            rc = self._lib.b200w4a4_signal_flags(ptrs, self.group, self.rank, self.epoch & 0xFFFFFFFF,
                                                 torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "signal_flags")

    # ---- real peers ---------------------------------------------------------------------------
    @classmethod
    def from_symmetric_memory(cls, group, capacity_rows: int, dim: int, row0: int,
                              dtype: torch.dtype = torch.bfloat16, timeout_ms: int = 1000,
                              shard_rows: Optional[Sequence[int]] = None) -> "PeerKVExchange":
        """Allocates the exchange memory with torch's symmetric memory on every rank of `group`
        (a torch.distributed process group on one NVLink domain) and maps the peers' copies."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        nbytes = exchange_bytes(capacity_rows, dim, world)
        local = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        local.zero_()
        handle = symm_mem.rendezvous(local, group=group)
        torch.cuda.synchronize()
        dist.barrier(group)                                # every rank's flags are zero before anyone pushes
        members = [layout(int(handle.buffer_ptrs[r]), capacity_rows, dim, world) for r in range(world)]
        if int(handle.buffer_ptrs[rank]) != local.data_ptr():
            members[rank] = layout(local.data_ptr(), capacity_rows, dim, world)
        ex = cls(rank, members, local, capacity_rows, dim, row0, dtype, timeout_ms, shard_rows)
        ex._handle = handle                                # keeps the mappings alive
        return ex
