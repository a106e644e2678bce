"""Tensor-parallel decode on 2 GPUs: KV heads sharded, attention output gathered along the last
dimension -- the fused push epilogue and the NCCL baseline against the full-head CPU oracle.
One process per GPU (spawned), rendezvous on 127.0.0.1."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    try:
        import torch.distributed as dist
        import oracle
        import gaudirt_b200 as rt
        from gaudirt_b200 import tp
        from tests import cases

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        q_heads, kv_heads, d, layers = 16, 4, 128, 3
        ctx = cases.lognormal_contexts(10, 20261103, median=300, sigma=1.0, lo=16, hi=3000)
        blocks = int(((ctx + 127) // 128).sum()) + 2
        shard = tp.HeadShard(rank, world, q_heads, kv_heads)
        hq, hkv = shard.local_q_heads, shard.local_kv_heads
        import dataclasses
        base = cases.decode_case(len(ctx), q_heads, kv_heads, d, 128, blocks, ctx, seed=500)
        layer_cases = [base]
        for l in range(1, layers):           # same block tables for every layer, fresh activations and pools
            other = cases.decode_case(len(ctx), q_heads, kv_heads, d, 128, blocks, ctx, seed=500 + l)
            layer_cases.append(dataclasses.replace(base, q=other.q, k=other.k, v=other.v, pool=other.pool))
        md = rt.PagedMetadata(base.locations, base.requests, base.positions, base.mapping, base.slots)
        md._set_split_tokens(256)                                  # exercise the split-KV combine as well
        outs = {}
        for mode in ("nccl", "push"):
            gather = tp.OutputGather(len(ctx), hq * d, dev, mode=mode)
            got = []
            for c in layer_cases:
                pool = c.pool[:, shard.kv_head_range().start:shard.kv_head_range().stop].contiguous().to(dev)
                kp, vp = pool[0].transpose(0, 1), pool[1].transpose(0, 1)
                full = gather.attention(c.q[:, shard.q_columns(d)].to(dev), c.k[:, shard.kv_columns(d)].to(dev),
                                        c.v[:, shard.kv_columns(d)].to(dev), kp, vp, md, d, c.scale)
                got.append(full.clone())
            torch.cuda.synchronize()
            outs[mode] = got
        ok = rt._C._take_device_status() == 0
        for c, a, b in zip(layer_cases, outs["nccl"], outs["push"]):
            assert a.shape == (len(ctx), q_heads * d) and torch.equal(a.view(torch.int16), b.view(torch.int16)), 'push != nccl'
            ref_pool = c.pool.clone()
            oracle.kv_store_head_major(ref_pool, c.k, c.v, c.locations)
            kp, vp = oracle.pool_views(ref_pool)
            ref = oracle.attend_fp32_softmax(c.q, kp, vp, c.requests, c.positions, c.mapping, q_heads, kv_heads, d, c.scale)
            oracle.fp32_softmax_gate(b.cpu().double(), ref)
        # o_proj on the un-gathered heads -> rank-ordered sum -> residual-add RMS norm: the partials
        # exchanged by the GEMM epilogue's peer stores against the NCCL all-gather of the same partials
        hidden, rows = 512, len(ctx)
        gen = torch.Generator().manual_seed(77)
        w_full = (torch.randn(hidden, q_heads * d, generator=gen) / (q_heads * d) ** 0.5).bfloat16()
        gamma = (1 + 0.02 * torch.randn(hidden, generator=gen)).bfloat16()
        residuals = [torch.randn(rows, hidden, generator=gen).bfloat16() for _ in layer_cases]
        w_mine = w_full[:, shard.q_columns(d)].contiguous().to(dev)
        chain = {}
        for mode in ("nccl", "push"):
            row_parallel = tp.RowParallelOutput(rows, hidden, dev, mode=mode)
            got = []
            for full, res in zip(outs["push"], residuals):
                mine = full[:, shard.q_columns(d)]                       # this rank's heads, a strided view
                y, u = row_parallel.forward(mine, w_mine, res.to(dev), gamma.to(dev), 1e-5, 0.0)
                got.append((y.clone(), u.clone(), row_parallel.all_reduce(mine, w_mine).clone()))
            torch.cuda.synchronize()
            chain[mode] = got
        ok = ok and rt._C._take_device_status() == 0
        for full, res, a, b in zip(outs["push"], residuals, chain["nccl"], chain["push"]):
            for x, y in zip(a, b):
                assert torch.equal(x.view(torch.int16), y.view(torch.int16)), "o_proj push != nccl"
            parts = [oracle.linear_bf16(full.cpu()[:, tp.HeadShard(r, world, q_heads, kv_heads).q_columns(d)],
                                        w_full[:, tp.HeadShard(r, world, q_heads, kv_heads).q_columns(d)])
                     for r in range(world)]
            reduced = oracle.canonical_rank_sum(parts)
            assert float((b[2].cpu() != reduced).double().mean()) < 0.03   # fp32 tensor-core sums vs binary64, last bit
            assert float((b[2].cpu().double() - reduced.double()).abs().max()) <= 2 ** -6 * float(reduced.abs().max())
            _, want_u = oracle.fused_add_rms_norm(b[2].cpu(), res, gamma, 1e-5, 0.0, dtype=torch.float64)
            assert torch.equal(b[1].cpu().double(), want_u)               # given the summed activation, bit-exact
        result[rank] = bool(ok)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # surfaced by the parent
        import traceback
        result[rank] = "".join(traceback.format_exception(exc))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_decode_push_and_nccl_gather():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert dict(result) == {r: True for r in range(world)}, dict(result)
