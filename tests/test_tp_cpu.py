"""Host-side logic of the tensor-parallel path on CPU: head sharding arithmetic, and the gather
layout checked across two `gloo` ranks against the oracle's `gather_dim_last`."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def load_tp():
    # tp.py has no native dependency; import it without the package's library loading
    import importlib.util
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("_tp", os.path.join(here, "gaudirt_b200", "tp.py"))
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["_tp"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_head_shard_partitions_heads_and_columns():
    tp = load_tp()
    for world in (1, 2, 4, 8):
        seen_kv, seen_q = [], []
        for r in range(world):
            s = tp.HeadShard(r, world, 64, 8)
            assert s.local_kv_heads == 8 // world and s.local_q_heads == 64 // world
            seen_kv.extend(s.kv_head_range())
            cols = s.q_columns(128)
            seen_q.extend(range(cols.start, cols.stop))
            # the query heads of a rank are exactly the groups of its KV heads
            assert {h // 8 for h in range(cols.start // 128, cols.stop // 128)} == set(s.kv_head_range())
        assert seen_kv == list(range(8)) and seen_q == list(range(64 * 128))
    with pytest.raises(ValueError):
        tp.HeadShard(0, 3, 64, 8)
    with pytest.raises(ValueError):
        tp.HeadShard(2, 2, 64, 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, rows, cols, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = load_tp()
    gen = torch.Generator().manual_seed(1234)
    full = torch.randn(rows, world * cols, generator=gen).to(torch.bfloat16)     # what every rank must end with
    mine = full[:, rank * cols:(rank + 1) * cols].contiguous()
    gather = tp.OutputGather(rows, cols, "cpu", mode="nccl")
    got = gather.gather(mine)
    ok = torch.equal(got, full) and torch.equal(got, oracle.gather_dim_last(
        [full[:, r * cols:(r + 1) * cols] for r in range(world)]))
    again = gather.gather(mine)
    result[rank] = bool(ok and torch.equal(again, full))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_gather_dim_last_over_gloo(world):
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, 5, 24, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(result) == {r: True for r in range(world)}
