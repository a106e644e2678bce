"""Parity of the CUDA kernels, called through the C ABI, against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
from gaudirt_b200 import raw as H
from tests import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def bits(t):
    return t.contiguous().view(torch.int16)


def oracle_gates(actual, args, tile=oracle.KV_TILE, **kw):
    ref32 = oracle.attend_fp32_softmax(*args, **kw)
    ref64 = oracle.attend_fp64_rounded(*args, **kw)
    tiled = oracle.tiled_bf16_pv(*args, kv_tile=tile, **kw)
    got = actual.cpu().double()
    oracle.fp32_softmax_gate(got, ref32)
    return oracle.isolated_errors(got, ref64, tiled)


# ------------------------------------------------------------------------------------------
# KV store
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kv_heads,d,rows,slots", [(8, 128, 4, 32768), (2, 64, 137, 8193), (3, 64, 1, 70), (1, 256, 33, 500)])
@pytest.mark.parametrize("layout", ["dense", "packed_qkv", "odd_offset"])
def test_kv_store_is_a_bit_exact_scatter(kv_heads, d, rows, slots, layout):
    gen = torch.Generator().manual_seed(rows * 7 + d)
    width = kv_heads * d
    guard = 64
    raw = torch.randn(2 * kv_heads * slots * d + 2 * guard, generator=gen).to(torch.bfloat16)
    raw_dev = raw.to(DEV)
    pool_dev = raw_dev[guard:-guard].view(2, kv_heads, slots, d)
    k = torch.randn(rows, width, generator=gen).to(torch.bfloat16)
    v = torch.randn(rows, width, generator=gen).to(torch.bfloat16)
    loc = torch.randperm(slots, generator=gen)[:rows].to(torch.int32)
    if layout == "dense":
        kd, vd = k.to(DEV), v.to(DEV)
    elif layout == "packed_qkv":            # column slices of one [rows, q|k|v] projection output
        packed = torch.zeros(rows, 3 * width + 64, dtype=torch.bfloat16, device=DEV)
        packed[:, width:2 * width] = k.to(DEV)
        packed[:, 2 * width:3 * width] = v.to(DEV)
        kd, vd = packed[:, width:2 * width], packed[:, 2 * width:3 * width]
    else:                                   # one-element offset: rows are only 2-byte aligned
        ks = torch.zeros(rows, width + 1, dtype=torch.bfloat16, device=DEV)
        vs = torch.zeros(rows, width + 1, dtype=torch.bfloat16, device=DEV)
        ks[:, 1:] = k.to(DEV)
        vs[:, 1:] = v.to(DEV)
        kd, vd = ks[:, 1:], vs[:, 1:]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    H.kv_store(pool_dev, kd, vd, loc.to(DEV), status)
    torch.cuda.synchronize()
    expect = raw.clone()
    oracle.kv_store_head_major(expect[guard:-guard].view(2, kv_heads, slots, d), k, v, loc)
    assert torch.equal(bits(raw_dev.cpu()), bits(expect)), "pool (guards included) differs"
    assert int(status.item()) == 0


def test_kv_store_skips_out_of_range_slots_and_reports():
    pool = torch.zeros(2, 2, 16, 64, dtype=torch.bfloat16, device=DEV)
    k = torch.ones(3, 128, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    H.kv_store(pool, k, k, torch.tensor([3, 16, -1], dtype=torch.int32, device=DEV), status)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert float(pool.float().sum()) == 2 * 2 * 64          # only slot 3 was written


# ------------------------------------------------------------------------------------------
# decode
# ------------------------------------------------------------------------------------------
def run_decode(case, page_tokens, split_tokens=0, softcap=0.0, window=-1, fused_combine=False):
    pool = case.pool.to(DEV)
    H.kv_store(pool, case.k.to(DEV), case.v.to(DEV), case.locations.to(DEV))
    seq, detected = H.validate(case.locations, case.requests, case.positions, case.mapping, case.slots)
    assert detected >= min(case.block, 128)
    work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, window=window,
                                    split_tokens=split_tokens)
    if page_tokens == 1:
        table = case.mapping.to(DEV)
    else:
        table = (case.mapping[:, ::page_tokens]).contiguous().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = H.paged_attn(case.q.to(DEV), pool, table, page_tokens, work, combine, entries, case.q_heads,
                       case.scale, softcap, window, status, fused_combine=fused_combine)
    assert int(status.item()) == 0
    return out, pool, len(combine)


def oracle_args(case):
    pool = case.pool.clone()
    oracle.kv_store_head_major(pool, case.k, case.v, case.locations)
    kp, vp = oracle.pool_views(pool)
    return pool, (case.q, kp, vp, case.requests, case.positions, case.mapping, case.q_heads, case.kv_heads,
                  case.head_dim, case.scale)


def test_config1_store_then_attend():
    case = cases.config1()
    pool_ref, args = oracle_args(case)
    out, pool, _ = run_decode(case, page_tokens=128)
    assert torch.equal(bits(pool.cpu()), bits(pool_ref)), "whole-pool audit after the store"
    e64, et = oracle_gates(out, args)
    print("config1 rel-l2 vs fp64", e64, "vs tiled", et)
    # the token-granular table (the reference's mapping) and the block table give the same bits
    out1, _, _ = run_decode(case, page_tokens=1)
    assert torch.equal(bits(out.cpu()), bits(out1.cpu()))
    # same inputs, same schedule -> same bits
    again, _, _ = run_decode(case, page_tokens=128)
    assert torch.equal(bits(out.cpu()), bits(again.cpu()))


@pytest.mark.parametrize("split", [64, 256, 1024])
def test_config1_split_kv_combine(split):
    case = cases.config1()
    _, args = oracle_args(case)
    out, _, n_combine = run_decode(case, page_tokens=128, split_tokens=split)
    assert n_combine == int((case.ctx > split + split // 4).sum()) and (split > 256 or n_combine > 0)
    oracle_gates(out, args)
    again, _, _ = run_decode(case, page_tokens=128, split_tokens=split)
    assert torch.equal(bits(out.cpu()), bits(again.cpu())), "split-KV combine must be deterministic"
    # the combine fused into the attention kernel (last split to finish merges) gives the same bits
    # as the separate combine kernel, run after run
    for _ in range(3):
        fused, _, _ = run_decode(case, page_tokens=128, split_tokens=split, fused_combine=True)
        assert torch.equal(bits(out.cpu()), bits(fused.cpu()))


@pytest.mark.parametrize("q_heads,kv_heads,d", [(8, 8, 64), (4, 2, 64), (9, 3, 64), (16, 8, 128), (56, 8, 128),
                                                (8, 1, 128), (16, 1, 128), (8, 4, 256), (8, 1, 256)])
def test_decode_edge_lengths(q_heads, kv_heads, d):
    ctx = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 257, 300]
    case = cases.decode_case(len(ctx), q_heads, kv_heads, d, 16, 128, ctx, seed=q_heads * 131 + d)
    _, args = oracle_args(case)
    for page, split in ((16, 0), (1, 0), (8, 48)):
        out, _, _ = run_decode(case, page_tokens=page, split_tokens=split)
        oracle_gates(out, args, tile=64)


@pytest.fixture
def attention_form():
    from gaudirt_b200 import abi
    lib = abi.lib()
    yield lambda form: abi.check(lib.gk_set_attention_form(form), "gk_set_attention_form")
    lib.gk_set_attention_form(0)


@pytest.mark.parametrize("q_heads,kv_heads,d", [(8, 2, 64), (32, 8, 128), (8, 1, 256)])
def test_box_and_row_forms_give_the_same_bits(attention_form, q_heads, kv_heads, d):
    """The two ways of staging a 16-token group (one TMA box / 16-byte row copies) feed the same arithmetic:
    same bits, whatever the launch size.  Covers whole groups, ragged ends, ranges of fewer groups than
    warps, split ranges that leave warps without a group, a window that starts ranges off a 16-token
    boundary (row copies inside the box form) and pages of exactly one group."""
    ctx = [1, 7, 16, 17, 49, 64, 113, 287, 519, 1167, 2048]
    case = cases.decode_case(len(ctx), q_heads, kv_heads, d, 128, 64, ctx, seed=d + q_heads)
    _, args = oracle_args(case)
    for page, split, window in ((128, 0, -1), (128, 64, -1), (16, 256, -1), (128, 0, 100), (16, 64, 333)):
        outs = []
        for form in (1, 2):            # GK_ATTENTION_FORM_ROWS, GK_ATTENTION_FORM_BOXES
            attention_form(form)
            out, _, _ = run_decode(case, page_tokens=page, split_tokens=split, window=window)
            outs.append(out.cpu())
        assert torch.equal(bits(outs[0]), bits(outs[1])), (page, split, window)
        if window < 0:
            oracle_gates(outs[1], args)
    with pytest.raises(Exception):
        attention_form(7)


def test_programmatic_launch_changes_no_bits():
    """With programmatic dependent launch every kernel still waits for its predecessor before its first
    access: a store -> attention -> combine chain gives the same bits with the switch on and off."""
    from gaudirt_b200 import abi
    lib = abi.lib()
    case = cases.config1()
    outs = []
    try:
        for on in (0, 1, 1):
            abi.check(lib.gk_set_programmatic_launch(on), "gk_set_programmatic_launch")
            out, pool, n_combine = run_decode(case, page_tokens=128, split_tokens=256)
            assert n_combine > 0
            outs.append((out.cpu(), pool.cpu()))
    finally:
        lib.gk_set_programmatic_launch(0)
    for out, pool in outs[1:]:
        assert torch.equal(bits(out), bits(outs[0][0])) and torch.equal(bits(pool), bits(outs[0][1]))


def test_skewed_lengths_with_automatic_split():
    ctx = cases.lognormal_contexts(24, 20261103, median=512, sigma=1.0, lo=16, hi=6000)
    blocks = int(((ctx + 127) // 128).sum()) + 3
    case = cases.decode_case(24, 16, 2, 128, 128, blocks, ctx, seed=99)
    _, args = oracle_args(case)
    out, _, n_combine = run_decode(case, page_tokens=128)
    assert n_combine > 0, "the automatic schedule should cut the long sequences"
    oracle_gates(out, args)


# ------------------------------------------------------------------------------------------
# fixtures computed by the reference's own CPU code
# ------------------------------------------------------------------------------------------
def _fixture_case(z, name):
    g = lambda k: z[f"{name}/{k}"]
    b16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    return g, b16


@pytest.mark.parametrize("name", ["gqa4_d64", "gqa8_d128", "mha_d64"])
def test_reference_fixture_attention(name):
    z = np.load(os.path.join(GOLDEN, "attention.npz"))
    g, b16 = _fixture_case(z, name)
    heads, kv_heads, d = int(g("heads")), int(g("kv_heads")), int(g("head_dim"))
    kp, vp = b16(g("key_pool")), b16(g("value_pool"))                  # [slots, kv_heads, d]
    pool = torch.stack((kp.transpose(0, 1), vp.transpose(0, 1))).contiguous().to(DEV)
    mapping = torch.from_numpy(g("mapping"))
    requests, positions = g("requests"), g("positions")
    seq = np.array([[i, 1, positions[i], requests[i]] for i in range(len(requests))], dtype=np.int32)
    work, combine, entries = H.plan(seq, heads, kv_heads, d)
    out = H.paged_attn(b16(g("q")).to(DEV), pool, mapping.to(DEV), 1, work, combine, entries, heads, float(g("scale")))
    got = out.cpu().double()
    oracle.fp32_softmax_gate(got, torch.from_numpy(g("unrounded32")).to(torch.bfloat16).double())
    oracle.isolated_errors(got, torch.from_numpy(g("fp64_bf16")), torch.from_numpy(g("tiled_512")))
    oracle.isolated_errors(got, torch.from_numpy(g("fp64_bf16")), torch.from_numpy(g("direct_bf16_pv")))


@pytest.mark.parametrize("name", ["softcap_swa", "swa_only", "softcap_only"])
def test_reference_fixture_softcap_and_window(name):
    z = np.load(os.path.join(GOLDEN, "softcap_window.npz"))
    g, b16 = _fixture_case(z, name)
    heads, kv_heads, d = int(g("heads")), int(g("kv_heads")), int(g("head_dim"))
    kp, vp = b16(g("key_pool")), b16(g("value_pool"))
    pool = torch.stack((kp.transpose(0, 1), vp.transpose(0, 1))).contiguous().to(DEV)
    mapping = torch.from_numpy(g("mapping"))
    requests, positions = g("requests"), g("positions")
    slots = kp.size(0)
    locations = mapping[torch.from_numpy(requests), torch.from_numpy(positions)]
    seq, _ = H.validate(locations, requests, positions, mapping, slots)
    assert len(seq) < len(requests), "these fixtures hold multi-row (prefill) sequences"
    work, combine, entries = H.plan(seq, heads, kv_heads, d, window=int(g("window")))
    out = H.paged_attn(b16(g("q")).to(DEV), pool, mapping.to(DEV), 1, work, combine, entries, heads,
                       float(g("scale")), float(g("softcap")), int(g("window")))
    ref = b16(g("out_bf16")).double()
    got = out.cpu().double()
    rel = (torch.linalg.vector_norm(got - ref, dim=-1) / torch.linalg.vector_norm(ref, dim=-1).clamp_min(1e-6)).max()
    assert float(rel) < 1.5e-2          # gate of the reference's tests/paged_attention_generalized_smoke.py:110-113
    oracle.fp32_softmax_gate(got, ref)


def test_multi_row_sequences_are_causal():
    """Prefill-style rows (several consecutive positions of one request) through the same kernel."""
    gen = torch.Generator().manual_seed(77)
    heads, kv_heads, d, slots = 8, 2, 128, 4200
    lens, prefixes = (19, 137, 1, 40), (0, 512, 800, 3)
    context = 1024
    mapping = (torch.randperm(slots - 1, generator=gen)[: 4 * context] .reshape(4, context) + 1).to(torch.int32)
    requests = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(prefixes, lens)])
    locations = mapping[requests, positions].contiguous()
    rows = len(requests)
    q, k, v = (torch.randn(rows, w, generator=gen).to(torch.bfloat16) for w in (heads * d, kv_heads * d, kv_heads * d))
    pool = torch.randn(2, kv_heads, slots, d, generator=gen).to(torch.bfloat16)
    pool_dev = pool.to(DEV)
    H.kv_store(pool_dev, k.to(DEV), v.to(DEV), locations.to(DEV))
    oracle.kv_store_head_major(pool, k, v, locations)
    assert torch.equal(bits(pool_dev.cpu()), bits(pool))
    seq, page = H.validate(locations, requests, positions, mapping, slots)
    assert [tuple(s) for s in seq] == [(0, 19, 0, 0), (19, 137, 512, 1), (156, 1, 800, 2), (157, 40, 3, 3)] and page == 1
    scale = 1.0 / d ** 0.5
    for split in (0, 96):
        work, combine, entries = H.plan(seq, heads, kv_heads, d, split_tokens=split)
        out = H.paged_attn(q.to(DEV), pool_dev, mapping.to(DEV), 1, work, combine, entries, heads, scale)
        kp, vp = oracle.pool_views(pool)
        oracle_gates(out, (q, kp, vp, requests, positions, mapping, heads, kv_heads, d, scale))


def test_bad_table_entry_is_reported_not_followed():
    case = cases.decode_case(2, 4, 2, 64, 16, 8, [20, 33], seed=3)
    table = case.mapping.clone()
    table[1, 5] = case.slots + 7
    seq = np.array([[0, 1, 19, 0], [1, 1, 32, 1]], dtype=np.int32)
    work, combine, entries = H.plan(seq, 4, 2, 64)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = H.paged_attn(case.q.to(DEV), case.pool.to(DEV), table.to(DEV), 1, work, combine, entries, 4, case.scale,
                       status=status)
    assert int(status.item()) == 2 and bool(torch.isfinite(out.float()).all())
