"""Chunked prefill on the tensor-core kernel (tcgen05/TMEM) against the CPU oracle: causal mask
inside the chunk, paged prefix, GQA packing, ragged tiles, softcap and sliding window."""
import math

import numpy as np
import pytest
import torch

import oracle
from gaudirt_b200 import raw as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build(seqs, q_heads, kv_heads, d, page, seed, std=1.0):
    """seqs: [(prefix, length)].  Pages of `page` contiguous slots, shuffled over the pool."""
    gen = torch.Generator().manual_seed(seed)
    context = max(p + l for p, l in seqs)
    context = (context + page - 1) // page * page
    pages_per = context // page
    n_pages = len(seqs) * pages_per + 3
    slots = n_pages * page
    perm = torch.randperm(n_pages, generator=gen)[: len(seqs) * pages_per].reshape(len(seqs), pages_per)
    pos = torch.arange(context)
    mapping = (perm[:, pos // page] * page + pos % page).to(torch.int32)
    requests = torch.cat([torch.full((l,), i) for i, (_, l) in enumerate(seqs)])
    positions = torch.cat([torch.arange(p, p + l) for p, l in seqs])
    locations = mapping[requests, positions].contiguous()
    rows = len(requests)
    mk = lambda *s: (torch.randn(*s, generator=gen) * std).to(torch.bfloat16)
    q, k, v = mk(rows, q_heads * d), mk(rows, kv_heads * d), mk(rows, kv_heads * d)
    pool = mk(2, kv_heads, slots, d)
    return dict(mapping=mapping, requests=requests, positions=positions, locations=locations, q=q, k=k, v=v, pool=pool,
                slots=slots, rows=rows)


def run_case(seqs, q_heads, kv_heads, page, seed, softcap=0.0, window=-1, min_rows=0, std=1.0, d=128):
    c = build(seqs, q_heads, kv_heads, d, page, seed, std)
    pool = c["pool"].to(DEV)
    H.kv_store(pool, c["k"].to(DEV), c["v"].to(DEV), c["locations"].to(DEV))
    seq, detected = H.validate(c["locations"], c["requests"], c["positions"], c["mapping"], c["slots"])
    assert detected >= page
    work, rest = H.prefill_plan(seq, q_heads, kv_heads, window=window, min_rows=min_rows)
    scale = 1.0 / math.sqrt(d)
    out = torch.full((c["rows"], q_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = c["mapping"].to(DEV)
    if len(work):
        H.paged_prefill_tc(c["q"].to(DEV), pool, table, detected, work, out, q_heads, scale, softcap, window, status,
                           entry_stride=detected)
    if len(rest):
        dwork, dcomb, entries = H.plan(rest, q_heads, kv_heads, d, window=window)
        part = H.paged_attn(c["q"].to(DEV), pool, table, detected, dwork, dcomb, entries, q_heads, scale, softcap, window,
                            status, entry_stride=detected)
        rows = torch.cat([torch.arange(r[0], r[0] + r[1]) for r in rest]).to(DEV)
        out[rows] = part[rows]
    assert int(status.item()) == 0, "device status (4 = a bounded wait expired)"
    ref_pool = c["pool"].clone()
    oracle.kv_store_head_major(ref_pool, c["k"], c["v"], c["locations"])
    kp, vp = oracle.pool_views(ref_pool)
    args = (c["q"], kp, vp, c["requests"], c["positions"], c["mapping"], q_heads, kv_heads, d, scale)
    got = out.cpu().double()
    assert bool(torch.isfinite(got).all())
    ref32 = oracle.attend_fp32_softmax(*args, softcap=softcap, window=window)
    oracle.fp32_softmax_gate(got, ref32)
    oracle.isolated_errors(got, oracle.attend_fp64_rounded(*args, softcap=softcap, window=window),
                           oracle.tiled_bf16_pv(*args, kv_tile=64 if d == 256 else oracle.KV_TILE, softcap=softcap,
                                                window=window))
    return len(work), len(rest)


def test_single_short_chunk_without_prefix():
    n_tc, n_rest = run_case([(0, 40)], 8, 2, 128, seed=1)
    assert n_tc == 1 and n_rest == 0            # one record: a full tile of 32 rows x 4 heads and a tile of 8 rows


def test_records_of_one_and_two_query_tiles():
    """One record feeds two query tiles of 128 packed rows: exactly two full tiles, one tile only, a second
    tile of a single row, and a chunk whose tiles need different numbers of KV tiles (the causal limit of the
    first tile ends one KV tile earlier)."""
    for seqs, records in (([(300, 64)], 1), ([(5, 32)], 1), ([(0, 33)], 1), ([(96, 64)], 1), ([(1000, 65), (0, 129)], 5)):
        n_tc, n_rest = run_case(seqs, 8, 2, 128, seed=sum(p + l for p, l in seqs))
        assert n_tc == records and n_rest == 0


@pytest.mark.parametrize("q_heads,kv_heads", [(8, 2), (4, 4), (16, 2), (9, 3)])
@pytest.mark.parametrize("page", [128, 1])
def test_chunks_on_paged_prefixes(q_heads, kv_heads, page):
    seqs = [(0, 70), (300, 129), (1000, 33), (127, 1), (640, 2)]
    n_tc, n_rest = run_case(seqs, q_heads, kv_heads, page, seed=q_heads * 10 + page)
    assert n_tc > 0 and n_rest >= 1              # the single decode row stays on the decode kernel


def test_ragged_tile_boundaries():
    for prefix, length in ((1, 127), (128, 128), (129, 130), (255, 3), (0, 257)):
        run_case([(prefix, length)], 8, 2, 16, seed=prefix + length, min_rows=1)


def test_softcap_and_sliding_window():
    run_case([(0, 200), (500, 64)], 8, 2, 128, seed=5, softcap=30.0, window=96)
    run_case([(37, 150)], 4, 1, 8, seed=6, window=64)


@pytest.mark.parametrize("d", [64, 256])
def test_other_head_dims(d):
    """head_dim 64 (two query tiles per CTA, 64-column accumulators) and 256 (one query tile per CTA, KV tiles
    of 64 tokens): whole pages by TMA and token-granular tables, grouped heads, records of one and two query
    tiles, ragged ends, softcap and window."""
    seqs = [(0, 70), (300, 129), (1000, 33), (127, 1), (640, 2), (64, 64)]
    for page in (128, 16, 1):
        n_tc, n_rest = run_case(seqs, 8, 2, page, seed=d + page, d=d)
        assert n_tc > 0 and n_rest >= 1
    run_case([(0, 257), (129, 130)], 4, 4, 32, seed=d + 7, min_rows=1, d=d)
    run_case([(0, 200), (500, 64)], 16, 2, 128, seed=d + 9, softcap=30.0, window=96, d=d)
    run_case([(37, 150)], 4, 1, 8, seed=d + 11, window=64, d=d)


def test_config4_shape_scaled_down():
    """The chunked-prefill configuration with fewer sequences and a shorter chunk: N(0, 0.5) data,
    32 query / 8 KV heads, prefixes drawn from [0, 8192)."""
    gen = torch.Generator().manual_seed(20261104)
    prefixes = torch.randint(0, 8193, (3,), generator=gen).tolist()
    run_case([(p, 96) for p in prefixes], 32, 8, 128, seed=4, std=0.5)
