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


def _row_parallel_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = load_tp()
    rows, heads, d, hidden = 6, 4, 16, 48
    gen = torch.Generator().manual_seed(99)
    attn = torch.randn(rows, heads * d, generator=gen).to(torch.bfloat16)          # gathered attention output
    weight = (torch.randn(hidden, heads * d, generator=gen) / 8).to(torch.bfloat16)
    cols = tp.HeadShard(rank, world, heads, heads).q_columns(d)
    mine = oracle.linear_bf16(attn[:, cols], weight[:, cols])                      # this rank's o_proj partial
    row_parallel = tp.RowParallelOutput(rows, hidden, "cpu", mode="nccl")
    parts = row_parallel.exchange(mine)
    want = [oracle.linear_bf16(attn[:, tp.HeadShard(r, world, heads, heads).q_columns(d)],
                               weight[:, tp.HeadShard(r, world, heads, heads).q_columns(d)]) for r in range(world)]
    ok = len(parts) == world and all(torch.equal(a, b) for a, b in zip(parts, want))
    total = oracle.canonical_rank_sum(parts)
    # every rank holds the same bits, and the sharded sum is the unsharded product up to the partials' roundings
    everyone = [torch.empty_like(total) for _ in range(world)]
    dist.all_gather(everyone, total)
    ok = ok and all(torch.equal(t, total) for t in everyone)
    full = oracle.linear_bf16(attn, weight)
    ok = ok and float((total.double() - full.double()).abs().max()) <= 2 ** -6 * float(full.abs().max())
    result[rank] = bool(ok)
    dist.destroy_process_group()


def test_row_parallel_partials_and_rank_ordered_sum_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_row_parallel_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(result) == {r: True for r in range(world)}


def test_rank_ordered_sum_known_answers():
    """Order matters in fp32 and the reference fixes it (tests/tp4_gather_reduce_smoke.py:16-20)."""
    parts = [torch.full((4,), v).to(torch.bfloat16) for v in (2.0 ** 24, 1.0, 1.0, -(2.0 ** 24))]
    assert oracle.canonical_rank_sum(parts).tolist() == [0.0] * 4              # each +1 is absorbed by 2^24
    small_first = [parts[1], parts[2], parts[0], parts[3]]
    assert oracle.canonical_rank_sum(small_first).tolist() == [2.0] * 4          # (1 + 1 + 2^24) - 2^24
    one = [torch.tensor([1.0, -3.5]).to(torch.bfloat16)]
    assert torch.equal(oracle.canonical_rank_sum(one), one[0])
