"""The benchmark configurations at their full sizes, checked through properties that do not need
the CPU oracle to walk every row: a whole-pool audit of the store against an independent scatter,
run-to-run bit identity, invariance under a physical re-placement of the blocks, the softmax
normalisation on a constant-V pool for every row, causality inside a chunk, and the oracle itself on
a sample of rows (shortest, longest and tile-boundary ones)."""
import math

import pytest
import torch

import oracle
from tests import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def bits(t):
    return t.contiguous().view(torch.int16)


def tabulate(tables, block, context):
    pos = torch.arange(context)
    return (tables.long()[:, pos // block] * block + pos % block).to(torch.int32).contiguous()


def place_blocks(need, num_blocks, gen):
    perm = torch.randperm(num_blocks, generator=gen).to(torch.int32)
    tables = torch.zeros(len(need), int(need.max()), dtype=torch.int32)
    cursor = 0
    for b, n in enumerate(need.tolist()):
        tables[b, :n] = perm[cursor:cursor + n]
        cursor += n
    return tables


def device_pool(rt, slots, kv_heads, d, seed, std=1.0):
    pool = rt._C._allocate_paged_kv(1, slots, kv_heads, d)
    gen = torch.Generator(device=DEV).manual_seed(seed)
    pool.normal_(0.0, std, generator=gen)
    return pool, pool[0, 0].transpose(0, 1), pool[0, 1].transpose(0, 1)       # views [slots, kv_heads, d]


def sampled_oracle_gate(out, rows, q, key_pool, value_pool, mapping, requests, positions, heads, kv_heads, d, scale):
    """Oracle on a few rows: each row's visible keys are gathered into a compact CPU pool."""
    keys, values, tables, cursor = [], [], [], 1
    longest = max(int(positions[r]) + 1 for r in rows)
    for r in rows:
        n = int(positions[r]) + 1
        slots = mapping[int(requests[r]), :n].long().to(DEV)
        keys.append(key_pool[slots].cpu())
        values.append(value_pool[slots].cpu())
        table = torch.zeros(longest, dtype=torch.int32)
        table[:n] = torch.arange(cursor, cursor + n, dtype=torch.int32)
        tables.append(table)
        cursor += n
    pad = torch.zeros(1, kv_heads, d, dtype=torch.bfloat16)
    args = (q[rows].cpu(), torch.cat([pad] + keys), torch.cat([pad] + values), torch.arange(len(rows)),
            torch.tensor([int(positions[r]) for r in rows]), torch.stack(tables), heads, kv_heads, d, scale)
    got = out[rows].cpu().double()
    oracle.fp32_softmax_gate(got, oracle.attend_fp32_softmax(*args))
    return oracle.isolated_errors(got, oracle.attend_fp64_rounded(*args), oracle.tiled_bf16_pv(*args, kv_tile=oracle.KV_TILE))


def decode_step(rt, q, k, v, key_pool, value_pool, locations, requests, positions, mapping, slots, d, scale):
    md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
    return torch.ops.gaudirt.paged_attn(q, k, v, key_pool, value_pool, md, d, scale)


def full_size_decode(rt, batch, heads, kv_heads, d, block, ctx, num_blocks, seed, sample):
    gen = torch.Generator().manual_seed(seed)
    need = (ctx + block - 1) // block
    assert int(need.sum()) <= num_blocks
    tables = place_blocks(need, num_blocks, gen)
    context = int(need.max()) * block
    mapping = tabulate(tables, block, context)
    slots = num_blocks * block
    requests, positions = torch.arange(batch), ctx - 1
    locations = mapping[requests, positions].contiguous()
    dgen = torch.Generator(device=DEV).manual_seed(seed + 1)
    mk = lambda width: torch.randn(batch, width, generator=dgen, device=DEV).bfloat16()
    q, k, v = mk(heads * d), mk(kv_heads * d), mk(kv_heads * d)
    scale = torch.tensor(1.0 / math.sqrt(d), dtype=torch.float32).item()
    pool, key_pool, value_pool = device_pool(rt, slots, kv_heads, d, seed + 2)
    before = pool.clone()
    step = lambda kp, vp, loc, table: decode_step(rt, q, k, v, kp, vp, loc, requests, positions, table, slots, d, scale)
    step_v = lambda new_v: decode_step(rt, q, k, new_v, key_pool, value_pool, locations, requests, positions, mapping,
                                       slots, d, scale)
    out = step(key_pool, value_pool, locations, mapping)
    assert out.shape == (batch, heads * d) and bool(torch.isfinite(out.float()).all())

    # 1. the store is an exact scatter: every other byte of the pool is as it was
    want = before.clone()
    where = locations.long().to(DEV)
    want[0, 0].transpose(0, 1)[where] = k.view(batch, kv_heads, d)
    want[0, 1].transpose(0, 1)[where] = v.view(batch, kv_heads, d)
    assert torch.equal(bits(pool), bits(want)), "whole-pool audit after the store"
    del want

    # 2. same inputs, same bits
    assert torch.equal(bits(out), bits(step(key_pool, value_pool, locations, mapping)))

    # 3. the oracle on a sample of rows
    e64, et = sampled_oracle_gate(out, sample, q, key_pool, value_pool, mapping, requests, positions, heads, kv_heads,
                                  d, scale)
    print("sampled rel-l2 vs fp64", e64, "vs tiled", et)

    # 4. physical placement does not matter: move every block, rewrite the tables, same bits
    move = torch.randperm(num_blocks, generator=gen)
    pool2 = torch.empty_like(before)
    pool2.view(2, kv_heads, num_blocks, block, d)[:, :, move.to(DEV)] = before.view(2, kv_heads, num_blocks, block, d)
    del before
    tables2 = move.to(torch.int32)[tables.long()]
    mapping2 = tabulate(tables2, block, context)
    out2 = step(pool2[0, 0].transpose(0, 1), pool2[0, 1].transpose(0, 1), mapping2[requests, positions].contiguous(),
                mapping2)
    assert torch.equal(bits(out), bits(out2)), "block-table indirection changed the result"
    del pool2

    # 5. softmax weights sum to one on every row, split or not: constant V per channel comes back
    channel = ((torch.arange(d) % 17) - 8).to(torch.bfloat16) / 8                # exact in bf16
    value_pool.copy_(channel.to(DEV).expand(slots, kv_heads, d))
    flat = step_v(channel.to(DEV).repeat(batch, kv_heads))
    error = (flat.float().view(batch, heads, d) - channel.float().to(DEV)).abs()
    assert float(error.max()) <= 2e-2 and float(error.mean()) <= 2e-3, (float(error.max()), float(error.mean()))
    assert rt._C._take_device_status() == 0
    return out


def test_config2_batch256_ctx4096(rt):
    batch, block = 256, 128
    ctx = torch.full((batch,), 4096)
    full_size_decode(rt, batch, 32, 8, 128, block, ctx, int(batch * 32 * 1.1), 20261102, sample=[0, 101, 255])


def test_config3_skewed_lengths_split_kv(rt):
    batch, block = 128, 128
    ctx = cases.lognormal_contexts(batch, 20261103)
    blocks = int(int(((ctx + block - 1) // block).sum()) * 1.1)
    order = torch.argsort(ctx)
    sample = [int(order[0]), int(order[1]), int(order[batch // 2]), int(order[-2]), int(order[-1])]
    full_size_decode(rt, batch, 64, 8, 128, block, ctx, blocks, 20261103, sample=sample)


def test_config4_chunked_prefill_on_paged_prefixes(rt):
    seqs, chunk, heads, kv_heads, d, block = 16, 512, 32, 8, 128, 128
    gen = torch.Generator().manual_seed(20261104)
    prefixes = torch.randint(0, 8193, (seqs,), generator=gen)
    prefixes[0], prefixes[1] = 0, 8192                                          # both ends of the range
    need = (prefixes + chunk + block - 1) // block
    num_blocks = int(int(need.sum()) * 1.1)
    tables = place_blocks(need, num_blocks, gen)
    mapping = tabulate(tables, block, int(need.max()) * block)
    slots = num_blocks * block
    requests = torch.arange(seqs).repeat_interleave(chunk)
    positions = (prefixes[:, None] + torch.arange(chunk)[None, :]).reshape(-1)
    locations = mapping[requests, positions].contiguous()
    rows = seqs * chunk
    dgen = torch.Generator(device=DEV).manual_seed(7)
    mk = lambda width: (torch.randn(rows, width, generator=dgen, device=DEV) * 0.5).bfloat16()
    q, k, v = mk(heads * d), mk(kv_heads * d), mk(kv_heads * d)
    scale = torch.tensor(1.0 / math.sqrt(d), dtype=torch.float32).item()
    pool, key_pool, value_pool = device_pool(rt, slots, kv_heads, d, 8, std=0.5)
    before = pool.clone()
    out = decode_step(rt, q, k, v, key_pool, value_pool, locations, requests, positions, mapping, slots, d, scale)
    want = before.clone()
    where = locations.long().to(DEV)
    want[0, 0].transpose(0, 1)[where] = k.view(rows, kv_heads, d)
    want[0, 1].transpose(0, 1)[where] = v.view(rows, kv_heads, d)
    assert torch.equal(bits(pool), bits(want)), "whole-pool audit after the store"
    sample = [0, 127, 128, 511, 512, 512 + 300, 5 * 512 + 129, rows - 1]      # tile edges, no prefix, longest prefix
    e64, et = sampled_oracle_gate(out, sample, q, key_pool, value_pool, mapping, requests, positions, heads, kv_heads,
                                  d, scale)
    print("sampled rel-l2 vs fp64", e64, "vs tiled", et)
    # causal inside the chunk: new tokens at offsets >= 300 cannot change rows before them
    k2, v2 = k.clone(), v.clone()
    late = (torch.arange(rows) % chunk >= 300).to(DEV)
    k2[late] = -k2[late]
    v2[late] = v2[late] * 2
    pool.copy_(before)
    out2 = decode_step(rt, q, k2, v2, key_pool, value_pool, locations, requests, positions, mapping, slots, d, scale)
    assert torch.equal(bits(out[~late]), bits(out2[~late])) and not torch.equal(bits(out[late]), bits(out2[late]))
    assert rt._C._take_device_status() == 0
