"""The tensor-parallel exchanges, checked on ONE GPU: every rank's shard is run in turn and stores its
block into W gathered buffers that all live on this device, exactly as it would into its peers'.

What is exchanged and how it must come out is the reference's: `AllGatherDimLast`
(src/bridge/segmented_runner.cpp:170-191: `[B, cols]` per rank -> `[B, W*cols]`, rank-major along the
last dimension) for the attention output, and the rank-ordered sum of the o_proj partials
(tests/tp4_gather_reduce_smoke.py:16-41, src/bridge/communicator.cpp:373-417).  The multi-process
forms of the same checks need two GPUs (tests/test_gpu_tp.py)."""
import pytest
import torch

import oracle
from gaudirt_b200 import tp
from tests import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def bits(t):
    return t.contiguous().view(torch.int16)


def shard_pool(pool, shard):
    heads = shard.kv_head_range()
    part = pool[:, heads.start:heads.stop].contiguous().to(DEV)
    return part, part[0].transpose(0, 1), part[1].transpose(0, 1)


def run_sharded_step(rt, case, md, world, q_heads, kv_heads, d, fill=float("nan")):
    """Every rank in turn: its heads' attention stored into column block `rank` of W gathered buffers, and the
    same rank's plain single-output call on a fresh copy of its pool.  Returns (buffers, per-rank outputs, pools)."""
    rows = case.q.size(0)
    buffers = [torch.full((rows, q_heads * d), fill, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    singles, pools = [], []
    for r in range(world):
        shard = tp.HeadShard(r, world, q_heads, kv_heads)
        q = case.q[:, shard.q_columns(d)].to(DEV)               # a column block of the full activation: row-strided
        k, v = case.k[:, shard.kv_columns(d)].to(DEV), case.v[:, shard.kv_columns(d)].to(DEV)
        plan = md.attention_plan(shard.local_q_heads, shard.local_kv_heads, d)
        pool, kp, vp = shard_pool(case.pool, shard)
        torch.ops.gaudirt._paged_attn_push(q, k, v, kp, vp, md.row_locations(), plan,
                                           [b[:, shard.q_columns(d)] for b in buffers], d, case.scale)
        pool2, kp2, vp2 = shard_pool(case.pool, shard)
        singles.append(torch.ops.gaudirt.paged_attn(q, k, v, kp2, vp2, md, d, case.scale))
        assert torch.equal(bits(pool), bits(pool2)), "the pushed form stores the same pool"
        pools.append(pool)
    torch.cuda.synchronize()
    return buffers, singles, pools


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("combine", ["separate", "fused", "unsplit"])
def test_sharded_decode_lands_in_every_ranks_gathered_buffer(rt, world, combine):
    q_heads, kv_heads, d = 32, 8, 128
    ctx = cases.lognormal_contexts(12, 20261103 + world, median=300, sigma=1.0, lo=16, hi=3000)
    blocks = int(((ctx + 127) // 128).sum()) + 2
    case = cases.decode_case(len(ctx), q_heads, kv_heads, d, 128, blocks, ctx, seed=900 + world)
    md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
    if combine != "unsplit":
        md._set_split_tokens(256)
        md._set_fused_combine(1 if combine == "fused" else 0)
    else:
        md._set_split_tokens(1 << 20)
    buffers, singles, pools = run_sharded_step(rt, case, md, world, q_heads, kv_heads, d)
    want = oracle.gather_dim_last([s.cpu() for s in singles])
    for b in buffers:
        assert torch.equal(bits(b.cpu()), bits(want)), "every rank holds the rank-major gather of the shards"
    ref_pool = case.pool.clone()
    oracle.kv_store_head_major(ref_pool, case.k, case.v, case.locations)
    full_pool = torch.cat([p.cpu() for p in pools], dim=1)
    assert torch.equal(bits(full_pool), bits(ref_pool)), "the shards' pools are the head slices of the full pool"
    kp, vp = oracle.pool_views(ref_pool)
    ref = oracle.attend_fp32_softmax(case.q, kp, vp, case.requests, case.positions, case.mapping, q_heads, kv_heads, d,
                                     case.scale)
    oracle.fp32_softmax_gate(buffers[0].cpu().double(), ref)
    assert rt._C._take_device_status() == 0


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("q_heads,kv_heads,d", [(32, 8, 128), (16, 8, 256), (16, 8, 64)])
def test_sharded_mixed_prefill_and_decode_step_is_gathered_by_the_kernels(rt, world, q_heads, kv_heads, d):
    """A step with extend chunks (tensor-core kernel), short chunks and decode rows (decode kernel) in one call."""
    prefixes, lengths = [0, 700, 130, 2000, 64, 5, 300], [200, 1, 70, 1, 3, 140, 1]
    case = cases.ragged_case(prefixes, lengths, q_heads, kv_heads, d, 128, seed=77 + world, std=0.5)
    md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
    md._set_split_tokens(256)
    buffers, singles, pools = run_sharded_step(rt, case, md, world, q_heads, kv_heads, d)
    want = oracle.gather_dim_last([s.cpu() for s in singles])
    for b in buffers:
        assert torch.equal(bits(b.cpu()), bits(want))
    ref_pool = case.pool.clone()
    oracle.kv_store_head_major(ref_pool, case.k, case.v, case.locations)
    assert torch.equal(bits(torch.cat([p.cpu() for p in pools], dim=1)), bits(ref_pool))
    kp, vp = oracle.pool_views(ref_pool)
    args = (case.q, kp, vp, case.requests, case.positions, case.mapping, q_heads, kv_heads, d, case.scale)
    got = buffers[-1].cpu().double()
    oracle.fp32_softmax_gate(got, oracle.attend_fp32_softmax(*args))
    oracle.isolated_errors(got, oracle.attend_fp64_rounded(*args),
                           oracle.tiled_bf16_pv(*args, kv_tile=64 if d == 256 else oracle.KV_TILE))
    assert rt._C._take_device_status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_row_parallel_oproj_partials_and_rank_ordered_sum(rt, world):
    """o_proj on each rank's heads with the partial stored into slot `rank` of every rank's receive buffer, then
    the rank-ordered sum fused into the residual-add RMS norm: all ranks end with the same bits, the sum is the
    reference's canonical one, and the updated residual is bit-exact given the summed activation."""
    rows, q_heads, kv_heads, d, hidden = 48, 32, 8, 128, 1024
    gen = torch.Generator().manual_seed(4100 + world)
    attn = torch.randn(rows, q_heads * d, generator=gen).bfloat16()
    w_full = (torch.randn(hidden, q_heads * d, generator=gen) / (q_heads * d) ** 0.5).bfloat16()
    gamma = (0.02 * torch.randn(hidden, generator=gen)).bfloat16()
    residual = torch.randn(rows, hidden, generator=gen).bfloat16()
    receive = torch.full((world, world, rows, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)   # [rank][slot]
    attn_d = attn.to(DEV)
    for r in range(world):
        cols = tp.HeadShard(r, world, q_heads, kv_heads).q_columns(d)
        torch.ops.gaudirt._oproj_push(attn_d[:, cols], w_full[:, cols].contiguous().to(DEV),
                                      [receive[p][r] for p in range(world)])
    results = []
    for p in range(world):
        y, u = torch.ops.gaudirt._rank_sum_add_rms_norm(list(receive[p].unbind(0)), residual.to(DEV), gamma.to(DEV),
                                                        1e-5, 1.0)
        results.append((y, u, torch.ops.gaudirt._rank_sum(list(receive[p].unbind(0)))))
    for y, u, x in results[1:]:
        assert torch.equal(bits(y), bits(results[0][0])) and torch.equal(bits(u), bits(results[0][1]))
        assert torch.equal(bits(x), bits(results[0][2]))
    parts_gpu = [receive[0][r].cpu() for r in range(world)]
    assert torch.equal(bits(results[0][2].cpu()), bits(oracle.canonical_rank_sum(parts_gpu))), "sum of what arrived"
    parts = [oracle.linear_bf16(attn[:, tp.HeadShard(r, world, q_heads, kv_heads).q_columns(d)],
                                w_full[:, tp.HeadShard(r, world, q_heads, kv_heads).q_columns(d)]) for r in range(world)]
    reduced = oracle.canonical_rank_sum(parts)
    got = results[0][2].cpu()
    assert float((got != reduced).double().mean()) < 0.03          # fp32 tensor-core sums vs binary64: last bit only
    assert float((got.double() - reduced.double()).abs().max()) <= 2 ** -6 * float(reduced.abs().max())
    _, want_u = oracle.fused_add_rms_norm(got, residual, gamma, 1e-5, 1.0, dtype=torch.float64)
    assert torch.equal(results[0][1].cpu().double(), want_u)
    assert rt._C._take_device_status() == 0
