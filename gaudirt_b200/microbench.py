"""Kernel-level timings of the small kernels of the path against the HBM roofline.

    python -m gaudirt_b200.microbench [rows|oproj|prefill|steps|vocab ...]      (no argument: all sections)

Times `kv_store`, `fused_add_rms_norm`, `rotary_embedding` and the split-KV combine alone with CUDA
events (inputs larger than L2 are cycled so no launch re-reads cached data) and prints algorithmic
bytes / time next to the measured copy bandwidth from MEASURED_PEAKS.json when that file exists."""
from __future__ import annotations

import json
import os

import torch


def _time(fn, sets, iters=20):
    for i in range(3):
        fn(*sets[i % len(sets)])
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(*sets[i % len(sets)])
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main(sections=()):
    import gaudirt_b200 as rt
    from gaudirt_b200 import raw as H
    dev = "cuda:0"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak = 6650.0
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peak = float(json.load(open(path))["hbm_gbs"])
    rows = []
    want = lambda name: not sections or name in sections
    if want("rows"):
        _row_kernels(rows, H, dev, peak)
    if want("oproj"):
        _oproj(dev, peak, path)
    if want("prefill"):
        _prefill(H, dev, path)
    if want("steps"):
        _steps(rt, dev)
    if want("vocab"):
        _vocab(dev, peak)


def _row_kernels(rows, H, dev, peak):
    # KV store, chunked-prefill size: 8192 rows x 8 KV heads x 128
    kv_heads, d, slots, n = 8, 128, 1 << 20, 8192
    sets = []
    for i in range(6):
        pool = torch.zeros(2, kv_heads, slots, d, dtype=torch.bfloat16, device=dev)
        k = torch.randn(n, kv_heads * d, device=dev).to(torch.bfloat16)
        loc = torch.randperm(slots, device=dev)[:n].to(torch.int32)
        sets.append((pool, k, k.clone(), loc))
    ms = _time(lambda pool, k, v, loc: H.kv_store(pool, k, v, loc), sets)
    rows.append(("kv_store_kernel<8>  8192 rows x 8 heads x 128", 2 * 2 * n * kv_heads * d * 2, ms))
    del sets

    # fused_add_rms_norm, 8192 rows x hidden 8192
    sets = []
    for i in range(4):
        x = torch.randn(8192, 8192, device=dev).to(torch.bfloat16)
        sets.append((x, x.clone(), torch.ones(8192, dtype=torch.bfloat16, device=dev)))
    ms = _time(lambda x, r, w: torch.ops.gaudirt.fused_add_rms_norm(x, r, w, 1e-5, 1.0), sets)
    rows.append(("rms_norm_kernel<8,fused>  8192 x 8192", 4 * 8192 * 8192 * 2, ms))
    ms = _time(lambda x, r, w: torch.ops.gaudirt.fused_add_rms_norm(x[:64], r[:64], w, 1e-5, 1.0), sets)
    rows.append(("rms_norm_kernel<8,fused>  64 x 8192 (decode step)", 4 * 64 * 8192 * 2, ms))
    del sets

    # rotary, 8192 rows, 32 q heads + 8 k heads x 128
    sets = []
    cache = torch.randn(16384, 128, device=dev).to(torch.bfloat16)
    for i in range(4):
        q = torch.randn(8192, 32 * 128, device=dev).to(torch.bfloat16)
        k = torch.randn(8192, 8 * 128, device=dev).to(torch.bfloat16)
        pos = torch.randint(0, 16384, (8192,), device=dev, dtype=torch.int32)
        sets.append((q, k, pos))
    ms = _time(lambda q, k, pos: torch.ops.gaudirt.rotary_embedding_positions(q, k, cache, pos, 128, 128, True), sets)
    rows.append(("rotary_kernel  8192 rows x (32+8) heads x 128", 2 * 8192 * 40 * 128 * 2, ms))

    print(f"{'kernel / case':58s} {'ms':>8s} {'GB/s':>9s} {'of measured copy peak':>22s}")
    for name, nbytes, ms in rows:
        gbs = nbytes / ms / 1e6
        print(f"{name:58s} {ms:8.4f} {gbs:9.1f} {gbs / peak:22.3f}")



def _prefill(H, dev, path):
    """The tensor-core prefill kernel at head_dim 64, 128 and 256 on the chunked-prefill shape (16 sequences x
    512 new rows on paged prefixes of up to 8192 tokens, 32 query / 8 KV heads, pages of 128): CUDA events around
    each launch, four pools cycled, against the measured bf16 tensor throughput."""
    import math
    import numpy as np
    from gaudirt_b200 import abi
    tpeak = 1590.0
    if os.path.exists(path):
        tpeak = float(json.load(open(path)).get("bf16_tflops", tpeak))
    batch, chunk, hq, hkv, page, pools_n = 16, 512, 32, 8, 128, 4
    gen = torch.Generator().manual_seed(20261104)
    prefix = torch.randint(0, 8193, (batch,), generator=gen)
    need = (prefix + chunk + page - 1) // page
    n_pages = int(int(need.sum()) * 1.1) + 1
    slots = n_pages * page
    perm = torch.randperm(n_pages, generator=gen).to(torch.int32)
    tables = torch.zeros(batch, int(need.max()), dtype=torch.int32)
    cursor = 0
    for b in range(batch):
        tables[b, :int(need[b])] = perm[cursor:cursor + int(need[b])]
        cursor += int(need[b])
    table = (tables * page).to(dev)                         # first slot of every page of 128 slot-contiguous tokens
    seq = np.array([[b * chunk, chunk, int(prefix[b]), b] for b in range(batch)], dtype=np.int32)
    work, _ = H.prefill_plan(seq, hq, hkv)
    work_d = torch.from_numpy(work).to(dev)
    visible = int((prefix * chunk).sum()) + batch * chunk * (chunk + 1) // 2
    lib, stream = abi.lib(), H.stream_ptr()
    print()
    print(f"{'paged_prefill_tc_kernel  16 x 512 rows, 32q/8kv':52s} {'ms':>8s} {'TFLOP/s':>9s} {'of measured bf16 peak':>22s}")
    for d in (64, 128, 256):
        pools = [(torch.randn(2, hkv, slots, d, device=dev) * 0.5).bfloat16() for _ in range(pools_n)]
        q = (torch.randn(batch * chunk, hq * d, device=dev) * 0.5).bfloat16()
        out = torch.empty_like(q)
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(pools_n)]
        for _ in range(3):
            for pool, (a, b) in zip(pools, events):
                a.record()
                abi.check(lib.gk_paged_prefill_tc_bf16(q.data_ptr(), q.stride(0), pool[0].data_ptr(), pool[1].data_ptr(), slots,
                                                       table.data_ptr(), table.stride(0), 1, page, None, work_d.data_ptr(),
                                                       len(work), out.data_ptr(), out.stride(0), 1 / math.sqrt(d), 0.0, -1, hq,
                                                       hkv, d, None, stream), "gk_paged_prefill_tc_bf16")
                b.record()
            torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in events) / pools_n
        tflops = 4.0 * d * hq * visible / ms / 1e9
        print(f"{f'head_dim {d}':52s} {ms:8.4f} {tflops:9.0f} {tflops / tpeak:22.3f}")
        del pools, q, out


def _oproj(dev, peak, path):
    # o_proj (tcgen05): time against max(weight + activation bytes / copy peak, flops / cuBLAS bf16 peak);
    # weights are cycled through more copies than L2 holds.  torch's library GEMM is timed beside it.
    tpeak = 1590.0
    if os.path.exists(path):
        tpeak = float(json.load(open(path)).get("bf16_tflops", tpeak))
    print()
    print(f"{'gk_oproj_bf16  m x n x k':44s} {'us':>8s} {'TFLOP/s':>9s} {'GB/s':>8s} {'of roofline':>12s} {'library us':>11s}")
    for label, m, n, k in (("TP8 shard, 70B geometry, batch 64", 64, 8192, 1024),
                           ("TP8 shard, 70B geometry, batch 256", 256, 8192, 1024),
                           ("1 GPU, 8B geometry, batch 256", 256, 4096, 4096),
                           ("1 GPU, 70B geometry, batch 256", 256, 8192, 8192),
                           ("chunked prefill, 8192 rows, 8B geometry", 8192, 4096, 4096)):
        copies = max(2, min(12, (160 << 20) // (n * k * 2) + 1))
        sets = [(torch.randn(m, k, device=dev).to(torch.bfloat16), (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16))
                for _ in range(copies)]
        ms = _time(lambda x, w: torch.ops.gaudirt._oproj(x, w), sets, iters=3 * copies)
        lib = _time(lambda x, w: torch.nn.functional.linear(x, w), sets, iters=3 * copies)
        flops, nbytes = 2.0 * m * n * k, 2.0 * (n * k + m * k + m * n)
        bound_ms = max(flops / tpeak / 1e9, nbytes / peak / 1e6)
        print(f"{label + f'  {m}x{n}x{k}':44s} {ms * 1e3:8.1f} {flops / ms / 1e9:9.1f} {nbytes / ms / 1e6:8.0f} "
              f"{bound_ms / ms:12.3f} {lib * 1e3:11.1f}")
        del sets

    # the sum of 8 ranks' partials fused into the residual-add norm (the partials live on this GPU here)
    sets = []
    for i in range(6):
        parts = torch.randn(8, 64, 8192, device=dev).to(torch.bfloat16)
        sets.append((list(parts.unbind(0)), torch.randn(64, 8192, device=dev).to(torch.bfloat16),
                     torch.ones(8192, dtype=torch.bfloat16, device=dev)))
    ms = _time(lambda parts, res, w: torch.ops.gaudirt._rank_sum_add_rms_norm(parts, res, w, 1e-5, 1.0), sets, iters=30)
    print(f"{'_rank_sum_add_rms_norm  8 ranks x 64 x 8192':44s} {ms * 1e3:8.1f} us  "
          f"({(8 + 3) * 64 * 8192 * 2 / ms / 1e6:.0f} GB/s)")


def _steps(rt, dev):
    # The steps either side of the path, timed through their operators (launch-bound: microseconds
    # per call, host time included).
    steps = []
    i64 = lambda values: torch.tensor(values, dtype=torch.int64, device=dev)
    free = torch.randperm(1 << 20, device=dev)
    for label, batch, prefix, length in (("decode step, 256 requests x 1 token", 256, 4095, 1),
                                         ("chunked prefill, 16 requests x 512 tokens", 16, 4096, 512)):
        last = i64([7 * 128 + 126] * batch)
        args = (last, free, [prefix] * batch, [length] * batch, 128)
        steps.append((f"_allocate_paged_slots  {label}", _time(lambda: torch.ops.gaudirt._allocate_paged_slots(*args), [()])))
    table = torch.arange(1, 1 + 256 * 4096, dtype=torch.int32, device=dev).view(256, 4096)
    steps.append(("_release_paged_slots  256 x 4096 slots -> 8192 pages",
                  _time(lambda: torch.ops.gaudirt._release_paged_slots(table.view(-1).long(), 128, 1 << 14), [()])))
    steps.append(("_release_paged_slots  one request, 4096 slots -> 32 pages",
                  _time(lambda: torch.ops.gaudirt._release_paged_slots(table[3].long(), 128, 1 << 14), [()])))
    seq, orig = i64([4096] * 256), torch.full((256,), 4096, dtype=torch.int32, device=dev)
    steps.append(("_advance_decode_lengths  256 requests",
                  _time(lambda: torch.ops.gaudirt._advance_decode_lengths(seq, orig), [()])))
    requests = torch.arange(256, dtype=torch.int32, device=dev)
    positions = torch.full((256,), 4095, dtype=torch.int32, device=dev)
    locations = table[:, 4095].contiguous()
    slots = 256 * 4096 + 1
    steps.append(("PagedMetadata.from_device  256 x ctx 4096 (checks 1M table entries)",
                  _time(lambda: rt.PagedMetadata.from_device(locations, requests, positions, table, [4095] * 256,
                                                             [1] * 256, slots), [()])))
    steps.append(("PagedMetadata._from_scheduler  same, no read-back",
                  _time(lambda: rt.PagedMetadata._from_scheduler(locations, requests, positions, table, [4095] * 256,
                                                                 [1] * 256, slots, None, 0), [()])))
    host = [t.cpu() for t in (locations, requests, positions, table)]
    steps.append(("PagedMetadata(host lists)  same step validated on the host",
                  _time(lambda: rt.PagedMetadata(host[0], host[1], host[2], host[3], slots), [()], iters=5)))
    print()
    for name, ms in steps:
        print(f"{name:72s} {ms * 1e3:9.1f} us per call")
    assert rt._C._take_device_status() == 0


def _vocab(dev, peak):
    # After the LM head: 256 rows x 131072 bf16 logits (67 MB per pass; more sets than L2 holds).
    rows, vocab = 256, 131072
    sets = [(torch.randn(rows, vocab, device=dev).mul_(3).to(torch.bfloat16),) for _ in range(4)]
    nbytes = rows * vocab * 2
    out = []
    ms = _time(lambda x: torch.ops.gaudirt._vocabulary_argmax(x), sets)
    out.append(("_vocabulary_argmax", ms, nbytes))
    ms = _time(lambda x: torch.argmax(x, dim=-1), sets)
    out.append(("torch.argmax (library)", ms, nbytes))
    mask = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, vocab // 32), device=dev, dtype=torch.int64).to(torch.int32)
    few = torch.zeros_like(mask)
    few[:, 7] = 5                                                      # two allowed tokens per row: nearly all is written
    ms = _time(lambda x: torch.ops.gaudirt.apply_token_bitmask_inplace_(x, mask), sets)
    out.append(("apply_token_bitmask_inplace_  random mask (half banned)", ms, nbytes // 2))
    ms = _time(lambda x: torch.ops.gaudirt.apply_token_bitmask_inplace_(x, few), sets)
    out.append(("apply_token_bitmask_inplace_  2 tokens allowed", ms, nbytes))
    sets = [(torch.randn(rows, vocab, device=dev).mul_(3).to(torch.bfloat16),) for _ in range(4)]
    f32 = lambda v: torch.full((rows,), v, device=dev)
    seeds, positions = torch.arange(rows, device=dev), torch.arange(rows, device=dev)
    k_all, k_50 = torch.full((rows,), vocab, dtype=torch.int32, device=dev), torch.full((rows,), 50, dtype=torch.int32, device=dev)
    for label, temp, top_p, top_k, min_p, passes in (("greedy (temperature 0)", 0.0, 1.0, k_all, 0.0, 1),
                                                     ("temperature only", 0.8, 1.0, k_all, 0.0, 2),
                                                     ("top_k 50 + top_p 0.9 + min_p 0.02", 0.8, 0.9, k_50, 0.02, 9)):
        ms = _time(lambda x: torch.ops.gaudirt.sample_from_logits(x, f32(temp), f32(top_p), top_k, f32(min_p), seeds, positions, True),
                   sets)
        out.append((f"sample_from_logits  {label}", ms, nbytes * passes))
    print()
    print(f"{'256 x 131072 bf16 logits':66s} {'us':>8s} {'GB/s moved (all passes)':>24s} {'of copy peak':>13s}")
    for name, ms, moved in out:
        print(f"{name:66s} {ms * 1e3:8.1f} {moved / ms / 1e6:24.0f} {moved / ms / 1e6 / peak:13.3f}")


if __name__ == "__main__":
    import sys
    main(tuple(sys.argv[1:]))
