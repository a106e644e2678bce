"""Seeded synthetic inputs with the shapes of the benchmark configurations (CPU tensors, so the
oracle and the device see identical bits).  Seeds: configuration k uses 20261100 + k."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class DecodeCase:
    q_heads: int
    kv_heads: int
    head_dim: int
    block: int
    slots: int
    ctx: torch.Tensor            # [B] context length after the store
    block_tables: torch.Tensor   # [B, max_blocks] int32 (block ids)
    mapping: torch.Tensor        # [B, context] int32 token slots (tabulated block tables)
    locations: torch.Tensor      # [B] int32 slot of the new token
    requests: torch.Tensor       # [B] int64
    positions: torch.Tensor      # [B] int64 (= ctx - 1)
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    pool: torch.Tensor           # [2, kv_heads, slots, d] bf16 before the store
    scale: float


def decode_case(batch, q_heads, kv_heads, head_dim, block, num_blocks, ctx, seed, std=1.0) -> DecodeCase:
    gen = torch.Generator().manual_seed(seed)
    ctx = torch.as_tensor(ctx, dtype=torch.int64)
    need = (ctx + block - 1) // block
    max_blocks = int(need.max())
    assert int(need.sum()) <= num_blocks
    perm = torch.randperm(num_blocks, generator=gen)
    tables = torch.zeros(batch, max_blocks, dtype=torch.int32)
    cursor = 0
    for b in range(batch):
        n = int(need[b])
        tables[b, :n] = perm[cursor:cursor + n].to(torch.int32)
        cursor += n
    context = max_blocks * block
    pos = torch.arange(context)
    mapping = (tables.long()[:, pos // block] * block + pos % block).to(torch.int32)
    slots = num_blocks * block
    positions = ctx - 1
    requests = torch.arange(batch, dtype=torch.int64)
    locations = mapping[requests, positions].contiguous()
    mk = lambda *shape: (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)
    q, k, v = mk(batch, q_heads * head_dim), mk(batch, kv_heads * head_dim), mk(batch, kv_heads * head_dim)
    pool = mk(2, kv_heads, slots, head_dim)
    scale = torch.tensor(1.0 / math.sqrt(head_dim), dtype=torch.float32).item()
    return DecodeCase(q_heads, kv_heads, head_dim, block, slots, ctx, tables, mapping, locations, requests,
                      positions, q, k, v, pool, scale)


def config1(seed=20261101) -> DecodeCase:
    """CPU-runnable single-layer paged decode: batch 4, 32/8 heads, d 128, block 128, 256 blocks,
    context lengths uniform in [1, 2048]."""
    gen = torch.Generator().manual_seed(seed)
    ctx = torch.randint(1, 2049, (4,), generator=gen)
    return decode_case(4, 32, 8, 128, 128, 256, ctx, seed + 1000)


def lognormal_contexts(batch, seed, median=2048, sigma=1.0, lo=16, hi=32768):
    gen = torch.Generator().manual_seed(seed)
    z = torch.randn(batch, generator=gen, dtype=torch.float64)
    return torch.clamp(torch.round(torch.exp(math.log(median) + sigma * z)), lo, hi).to(torch.int64)


@dataclass
class ChunkCase:
    q_heads: int
    kv_heads: int
    head_dim: int
    slots: int
    mapping: torch.Tensor        # [seqs, context] int32
    requests: torch.Tensor       # [rows] int64
    positions: torch.Tensor      # [rows] int64
    locations: torch.Tensor      # [rows] int32
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    pool: torch.Tensor
    scale: float


def chunk_case(prefixes, chunk, q_heads, kv_heads, head_dim, block, seed, std=1.0) -> ChunkCase:
    """Chunked prefill: every sequence appends `chunk` new rows to a prefix already in the pool."""
    gen = torch.Generator().manual_seed(seed)
    prefixes = torch.as_tensor(prefixes, dtype=torch.int64)
    n = len(prefixes)
    need = (prefixes + chunk + block - 1) // block
    n_blocks = int(int(need.sum()) * 1.1) + 1
    perm = torch.randperm(n_blocks, generator=gen).to(torch.int32)
    tables = torch.zeros(n, int(need.max()), dtype=torch.int32)
    cursor = 0
    for b in range(n):
        tables[b, : int(need[b])] = perm[cursor:cursor + int(need[b])]
        cursor += int(need[b])
    pos = torch.arange(int(need.max()) * block)
    mapping = (tables.long()[:, pos // block] * block + pos % block).to(torch.int32).contiguous()
    requests = torch.arange(n).repeat_interleave(chunk)
    positions = (prefixes[:, None] + torch.arange(chunk)[None, :]).reshape(-1)
    locations = mapping[requests, positions].contiguous()
    rows = n * chunk
    mk = lambda *shape: (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)
    q, k, v = mk(rows, q_heads * head_dim), mk(rows, kv_heads * head_dim), mk(rows, kv_heads * head_dim)
    pool = mk(2, kv_heads, n_blocks * block, head_dim)
    scale = torch.tensor(1.0 / math.sqrt(head_dim), dtype=torch.float32).item()
    return ChunkCase(q_heads, kv_heads, head_dim, n_blocks * block, mapping, requests, positions, locations, q, k, v,
                     pool, scale)


def ragged_case(prefixes, lengths, q_heads, kv_heads, head_dim, block, seed, std=1.0) -> ChunkCase:
    """A mixed step: sequence i appends `lengths[i]` new rows to a prefix of `prefixes[i]` tokens
    already in the pool (length 1 = a decode row, more = a prefill / extend chunk)."""
    gen = torch.Generator().manual_seed(seed)
    prefixes = torch.as_tensor(prefixes, dtype=torch.int64)
    lengths = torch.as_tensor(lengths, dtype=torch.int64)
    n = len(prefixes)
    need = (prefixes + lengths + block - 1) // block
    n_blocks = int(int(need.sum()) * 1.1) + 1
    perm = torch.randperm(n_blocks, generator=gen).to(torch.int32)
    tables = torch.zeros(n, int(need.max()), dtype=torch.int32)
    cursor = 0
    for b in range(n):
        tables[b, : int(need[b])] = perm[cursor:cursor + int(need[b])]
        cursor += int(need[b])
    pos = torch.arange(int(need.max()) * block)
    mapping = (tables.long()[:, pos // block] * block + pos % block).to(torch.int32).contiguous()
    requests = torch.repeat_interleave(torch.arange(n), lengths)
    positions = torch.cat([torch.arange(int(p), int(p + l)) for p, l in zip(prefixes, lengths)])
    locations = mapping[requests, positions].contiguous()
    rows = int(lengths.sum())
    mk = lambda *shape: (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)
    q, k, v = mk(rows, q_heads * head_dim), mk(rows, kv_heads * head_dim), mk(rows, kv_heads * head_dim)
    pool = mk(2, kv_heads, n_blocks * block, head_dim)
    scale = torch.tensor(1.0 / math.sqrt(head_dim), dtype=torch.float32).item()
    return ChunkCase(q_heads, kv_heads, head_dim, n_blocks * block, mapping, requests, positions, locations, q, k, v,
                     pool, scale)
