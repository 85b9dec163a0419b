"""Row sharding of the linear layer: partition arithmetic, and a world-size-2 gloo run on CPU
in which every rank computes its own token rows (the oracle stands in for the GPU kernel) and
the gathered result equals the unsharded one."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from _cases import make_case
from dsaquant_b200 import sharding
from oracle import w4a4_oracle as orc


@pytest.mark.parametrize("m,world", [(32760, 1), (32760, 2), (32760, 4), (32760, 8), (27280, 8), (512, 8), (1, 2), (0, 3)])
def test_row_partition_properties(m, world):
    b = sharding.row_partition(m, world)
    assert len(b) == world and b[0][0] == 0 and b[-1][1] == m
    for (s0, e0), (s1, e1) in zip(b, b[1:]):
        assert e0 == s1 and s0 <= e0
    cap = sharding.shard_capacity(m, world)
    sizes = [e - s for s, e in b]
    assert cap % sharding.ROW_ALIGN == 0 and max(sizes, default=0) <= cap
    nonempty = [z for z in sizes if z]
    assert all(z == cap for z in nonempty[:-1])            # only the last non-empty shard may be short
    assert all(s == min(m, r * cap) for r, (s, _) in enumerate(b))
    # no aligned split has a smaller largest shard
    blocks = -(-m // sharding.ROW_ALIGN)
    assert cap == -(-blocks // world) * sharding.ROW_ALIGN
    if m == 32760 and world == 8:
        assert sizes[0] == 4096 and sizes[-1] == 32760 - 7 * 4096
    if m == 27280 and world == 8:
        assert sizes == [3584] * 7 + [27280 - 7 * 3584]


def _oracle_linear(codes, ws, bias):
    def fn(x, qweight, wscales, b, clip):
        r = orc.linear_w4a4(x.numpy(), codes, ws, bias, clip)
        return torch.from_numpy(r["out"])
    return fn


def _worker(rank, world, port, m, k, n, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x16, w16, b16 = make_case(5, m, k, n)
        ws = orc.weight_scale_absmax(w16)
        codes = orc.quantize_weight(w16, ws)
        x = torch.from_numpy(x16)
        x_local = sharding.shard_rows(x, rank, world, align=64)
        y = sharding.all_gather_rows(
            sharding.linear_rows_sharded(x_local, None, None, None, 0.95, linear_fn=_oracle_linear(codes, ws, b16)),
            m, align=64)
        full = orc.linear_w4a4(x16, codes, ws, b16, 0.95)["out"]
        ok = np.array_equal(y.numpy().view(np.uint16), full.view(np.uint16))
        local_only = sharding.linear_rows_sharded(x_local, None, None, None, 0.95,
                                                  linear_fn=_oracle_linear(codes, ws, b16))
        s, e = sharding.row_partition(m, world, 64)[rank]
        ok = ok and np.array_equal(local_only.numpy().view(np.uint16), full[s:e].view(np.uint16))
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_sharded_linear_matches_unsharded_gloo(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    mp.spawn(_worker, args=(world, port, 200, 128, 128, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
