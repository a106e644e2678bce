"""Operator-level parity: torch.ops.gaudirt.* and PagedMetadata against the CPU oracle.

The scenarios follow the reference's own operator tests (two-layer audit of
tests/paged_attention_smoke.py, mixed prefill/decode of tests/paged_layer_store_smoke.py,
generalised geometries of tests/paged_attention_generalized_smoke.py, plan binding of
tests/attention_plan_smoke.py)."""
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


def make_pools(rt, slots, kv_heads, d, key_base=None, value_base=None):
    combined = rt._C._allocate_paged_kv(1, slots, kv_heads, d)
    assert combined.shape == (1, 2, kv_heads, slots, d) and float(combined.float().abs().sum()) == 0
    key_pool, value_pool = combined[0, 0].transpose(0, 1), combined[0, 1].transpose(0, 1)
    if key_base is not None:
        key_pool.copy_(key_base)
        value_pool.copy_(value_base)
    return combined, key_pool, value_pool


def gates(actual, args, **kw):
    got = actual.cpu().double()
    oracle.fp32_softmax_gate(got, oracle.attend_fp32_softmax(*args, **kw))
    return oracle.isolated_errors(got, oracle.attend_fp64_rounded(*args, **kw),
                                  oracle.tiled_bf16_pv(*args, kv_tile=oracle.KV_TILE, **kw))


@pytest.mark.parametrize("rows", [1, 3, 17, 137, 513, 1025])
def test_two_layer_attention_and_pool_audit(rt, rows):
    heads, kv_heads, d = 4, 2, 64
    n_req, context = 64, 128
    slots = n_req * context + 1
    scale = 1.0 / math.sqrt(d)
    scale32 = torch.tensor(scale, dtype=torch.float32).item()
    gen = torch.Generator().manual_seed(3127 + rows)
    mapping = torch.arange(1, slots, dtype=torch.int32).reshape(n_req, context)
    requests = torch.arange(rows, dtype=torch.int64) % n_req
    positions = torch.arange(rows, dtype=torch.int64) // n_req + 3
    locations = mapping[requests, positions].to(torch.int64)
    md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
    assert md.rows() == rows and md.slots() == slots and md.context() == context
    q, k, v = (torch.randn(rows, w, generator=gen).to(torch.bfloat16) for w in (heads * d, kv_heads * d, kv_heads * d))
    sliced = rows in (17, 137)
    outputs = []
    for layer in range(2):
        kb = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        vb = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        _, key_pool, value_pool = make_pools(rt, slots, kv_heads, d, kb, vb)
        if sliced:                                   # one-element offset views, rows only 2-byte aligned
            ks = torch.empty(rows, kv_heads * d + 1, dtype=torch.bfloat16, device=DEV)
            vs = torch.empty(rows, kv_heads * d + 1, dtype=torch.bfloat16, device=DEV)
            kd, vd = ks[:, 1:], vs[:, 1:]
            kd.copy_(k); vd.copy_(v)
        else:
            kd, vd = k.to(DEV), v.to(DEV)
        out = torch.ops.gaudirt.paged_attn(q.to(DEV), kd, vd, key_pool, value_pool, md, d, scale)
        assert out.shape == q.shape and out.is_contiguous() and out.dtype == torch.bfloat16
        ek, ev = kb.clone(), vb.clone()
        ek[locations] = k.reshape(-1, kv_heads, d)
        ev[locations] = v.reshape(-1, kv_heads, d)
        assert torch.equal(bits(key_pool.cpu()), bits(ek)) and torch.equal(bits(value_pool.cpu()), bits(ev))
        gates(out, (q, ek, ev, requests, positions, mapping, heads, kv_heads, d, scale32))
        outputs.append((out, key_pool, value_pool))
    if rows == 3:
        out, key_pool, value_pool = outputs[0]
        before = key_pool.cpu()
        with pytest.raises(RuntimeError, match="disjoint|combined storage"):
            torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, key_pool, md, d, scale)
        assert torch.equal(bits(key_pool.cpu()), bits(before)), "a rejected call must not touch the pool"
        with pytest.raises(RuntimeError, match="head dimension"):
            torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, 96, scale)
    if rows == 137:
        out, key_pool, value_pool = outputs[1]
        one = rt.PagedMetadata(locations[-1:].contiguous(), requests[-1:].contiguous(), positions[-1:].contiguous(),
                               mapping, slots)
        replay = torch.ops.gaudirt.paged_attn(q[-1:].to(DEV), k[-1:].to(DEV), v[-1:].to(DEV), key_pool, value_pool,
                                              one, d, scale)
        assert torch.equal(bits(replay.cpu()), bits(out.cpu()[-1:]))
    assert rt._C._take_device_status() == 0


def test_mixed_prefill_and_decode_rows_share_one_store(rt):
    gen = torch.Generator().manual_seed(41753)
    heads, kv_heads, d = 4, 2, 64
    context, n_req = 1024, 3
    slots = context * n_req + 1
    prefixes, lengths = (0, 512, 800), (19, 137, 1)
    mapping = torch.arange(1, slots, dtype=torch.int32).reshape(n_req, context)
    requests = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lengths)])
    positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in zip(prefixes, lengths)])
    locations = mapping[requests.long(), positions.long()].contiguous()
    rows = len(locations)
    md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
    assert md.sequences() == [0, 19, 0, 0, 19, 137, 512, 1, 156, 1, 800, 2] and md.page_tokens() == 128
    q, k, v = (torch.randn(rows, w, generator=gen).to(torch.bfloat16) for w in (heads * d, kv_heads * d, kv_heads * d))
    ok, ov = (torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16) for _ in range(2))
    _, key_pool, value_pool = make_pools(rt, slots, kv_heads, d, ok, ov)
    out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, d, 1 / math.sqrt(d))
    ek, ev = ok.clone(), ov.clone()
    ek[locations.long()] = k.reshape(rows, kv_heads, d)
    ev[locations.long()] = v.reshape(rows, kv_heads, d)
    assert torch.equal(bits(key_pool.cpu()), bits(ek)) and torch.equal(bits(value_pool.cpu()), bits(ev))
    gates(out, (q, ek, ev, requests.long(), positions.long(), mapping, heads, kv_heads, d, 1 / math.sqrt(d)))


def test_plan_is_cached_and_bound_to_its_geometry(rt):
    positions = torch.tensor([3, 4, 5, *range(7, 17)], dtype=torch.int32)
    row_requests = torch.tensor([0] * 3 + [1] * 10, dtype=torch.int32)
    n_req, context, slots = 2, 32, 4096
    mapping = ((torch.arange(n_req)[:, None] * 256 + torch.arange(context)[None, :]) % slots).to(torch.int32)
    locations = mapping[row_requests.long(), positions.long()].contiguous()
    md = rt.PagedMetadata(locations, row_requests, positions, mapping, slots)
    plan = md.attention_plan(4, 2, 64)
    assert md.attention_plan(4, 2, 64).data_ptr() == plan.data_ptr()
    with pytest.raises(RuntimeError, match="different head geometry"):
        md.attention_plan(8, 2, 64)
    assert torch.equal(md.row_locations().cpu(), locations) and torch.equal(md.request_mapping().cpu(), mapping)
    assert md.rotary_header().cpu().tolist() == [13] and torch.equal(md.rotary_positions().cpu(), positions)
    # a tensor that is not a plan is rejected
    q = torch.zeros(13, 4 * 64, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(13, 2 * 64, dtype=torch.bfloat16, device=DEV)
    _, kp, vp = make_pools(rt, slots, 2, 64)
    with pytest.raises(RuntimeError, match="invalid or expired metadata plan"):
        torch.ops.gaudirt._paged_attn_validated(q, kv, kv, kp, vp, md.row_locations(), md.row_requests(),
                                                md.rotary_positions(), md.request_mapping(), md.rotary_header(), 64, 0.125)
    out = torch.ops.gaudirt._paged_attn_validated(q, kv, kv, kp, vp, md.row_locations(), md.row_requests(),
                                                  md.rotary_positions(), plan, md.rotary_header(), 64, 0.125)
    assert float(out.float().abs().sum()) == 0
    other = torch.cuda.Stream()
    with torch.cuda.stream(other), pytest.raises(RuntimeError, match="stream"):
        torch.ops.gaudirt._paged_attn_validated(q, kv, kv, kp, vp, md.row_locations(), md.row_requests(),
                                                md.rotary_positions(), plan, md.rotary_header(), 64, 0.125)


@pytest.mark.parametrize("q_heads,kv_heads,d,seqs,softcap,window", [
    (9, 3, 64, [(0, 48), (19, 1)], 0.0, -1),
    (16, 8, 128, [(0, 96), (32, 1), (45, 1)], 0.0, -1),
    (8, 4, 256, [(0, 140), (70, 1)], 50.0, 64),
    (8, 1, 256, [(0, 300), (150, 1)], 30.0, 96),
])
def test_generalised_geometry_softcap_window_from_scheduler(rt, q_heads, kv_heads, d, seqs, softcap, window):
    gen = torch.Generator().manual_seed(7721 + q_heads)
    scale, slots = 1.0 / math.sqrt(d), 4096
    kp_cpu, vp_cpu = (torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16) for _ in range(2))
    _, key_pool, value_pool = make_pools(rt, slots, kv_heads, d, kp_cpu, vp_cpu)
    max_ctx = max(p + l for p, l in seqs)
    mapping = torch.zeros(len(seqs), max_ctx + 16, dtype=torch.int32)
    loc, cursor = [], 1
    for i, (prefix, length) in enumerate(seqs):
        ids = list(range(cursor, cursor + prefix + length))
        cursor += prefix + length + 3
        mapping[i, : prefix + length] = torch.tensor(ids, dtype=torch.int32)
        loc.extend(ids[prefix:])
    rows = len(loc)
    q, k, v = (torch.randn(rows, w, generator=gen).to(torch.bfloat16) for w in (q_heads * d, kv_heads * d, kv_heads * d))
    locations = torch.tensor(loc, dtype=torch.int64, device=DEV)
    positions = torch.tensor([p + i for p, l in seqs for i in range(l)], dtype=torch.int64, device=DEV)
    md = rt.PagedMetadata._from_scheduler(locations, torch.arange(len(seqs), dtype=torch.int64, device=DEV), positions,
                                          mapping.to(DEV), [p for p, _ in seqs], [l for _, l in seqs], slots, None, 0)
    out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, d, scale, softcap, window)
    kp_cpu[loc] = k.reshape(rows, kv_heads, d)
    vp_cpu[loc] = v.reshape(rows, kv_heads, d)
    requests = torch.tensor([i for i, (_, l) in enumerate(seqs) for _ in range(l)])
    ref = oracle.attend_fp32_softmax(q, kp_cpu, vp_cpu, requests, positions.cpu(), mapping, q_heads, kv_heads, d, scale,
                                     softcap=softcap, window=window)
    got = out.cpu().double()
    rel = (torch.linalg.vector_norm(got - ref, dim=-1) / torch.linalg.vector_norm(ref, dim=-1).clamp_min(1e-6)).max()
    assert bool(torch.isfinite(got).all()) and float(rel) < 1.5e-2
    oracle.fp32_softmax_gate(got, ref)
    assert torch.equal(md.row_requests().cpu(), requests.to(torch.int32))


def test_many_requests_fused_scheduler_metadata(rt):
    n = 300
    mapping = torch.arange(1, 1 + n * 8, dtype=torch.int32).reshape(n, 8)
    slots = n * 8 + 16
    _, kp, vp = make_pools(rt, slots, 2, 64)
    md = rt.PagedMetadata._from_scheduler_fused(mapping[:, 4].to(torch.int64).to(DEV), torch.arange(n, device=DEV),
                                                torch.full((n,), 4, dtype=torch.int64, device=DEV), mapping.to(DEV),
                                                [4] * n, [1] * n, slots, None, 0, 4, 2, 64)
    gen = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(n, w, generator=gen).to(torch.bfloat16) for w in (256, 128, 128))
    out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), kp, vp, md, 64, 0.125)
    # four zero keys/values and the new token: the softmax mixes v with zeros
    kcpu, vcpu = torch.zeros(slots, 2, 64, dtype=torch.bfloat16), torch.zeros(slots, 2, 64, dtype=torch.bfloat16)
    kcpu[mapping[:, 4].long()] = k.reshape(n, 2, 64)
    vcpu[mapping[:, 4].long()] = v.reshape(n, 2, 64)
    ref = oracle.attend_fp32_softmax(q, kcpu, vcpu, torch.arange(n), torch.full((n,), 4), mapping, 4, 2, 64, 0.125)
    oracle.fp32_softmax_gate(out.cpu().double(), ref)


def test_config1_through_the_operator(rt):
    case = cases.config1()
    md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
    assert md.page_tokens() == 128
    combined = rt._C._allocate_paged_kv(1, case.slots, case.kv_heads, case.head_dim)
    combined[0].copy_(case.pool)
    key_pool, value_pool = combined[0, 0].transpose(0, 1), combined[0, 1].transpose(0, 1)
    out = torch.ops.gaudirt.paged_attn(case.q.to(DEV), case.k.to(DEV), case.v.to(DEV), key_pool, value_pool, md,
                                       case.head_dim, case.scale)
    ref_pool = case.pool.clone()
    oracle.kv_store_head_major(ref_pool, case.k, case.v, case.locations)
    assert torch.equal(bits(combined[0].cpu()), bits(ref_pool))
    kp, vp = oracle.pool_views(ref_pool)
    gates(out, (case.q, kp, vp, case.requests, case.positions, case.mapping, case.q_heads, case.kv_heads,
                case.head_dim, case.scale))
    # forced split-KV schedule on fresh metadata: same result within the gates, bit-stable across runs
    md2 = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
    md2._set_split_tokens(128)
    a = torch.ops.gaudirt.paged_attn(case.q.to(DEV), case.k.to(DEV), case.v.to(DEV), key_pool, value_pool, md2,
                                     case.head_dim, case.scale)
    b = torch.ops.gaudirt.paged_attn(case.q.to(DEV), case.k.to(DEV), case.v.to(DEV), key_pool, value_pool, md2,
                                     case.head_dim, case.scale)
    assert torch.equal(bits(a.cpu()), bits(b.cpu()))
    gates(a, (case.q, kp, vp, case.requests, case.positions, case.mapping, case.q_heads, case.kv_heads,
              case.head_dim, case.scale))


def test_sequential_decode_steps_keep_state(rt):
    """A short version of the reference's 128-step decode (tests/paged_attention_128_state_smoke.py):
    every step stores one token and attends to everything stored so far."""
    heads, kv_heads, d, steps = 8, 2, 128, 40
    slots = 256
    gen = torch.Generator().manual_seed(128)
    mapping = (torch.randperm(slots - 1, generator=gen)[:steps] + 1).reshape(1, steps).to(torch.int32)
    combined, key_pool, value_pool = make_pools(rt, slots, kv_heads, d)
    kc, vc = torch.zeros(slots, kv_heads, d, dtype=torch.bfloat16), torch.zeros(slots, kv_heads, d, dtype=torch.bfloat16)
    for step in range(steps):
        q, k, v = (torch.randn(1, w, generator=gen).to(torch.bfloat16) for w in (heads * d, kv_heads * d, kv_heads * d))
        loc = mapping[0, step:step + 1].long()
        md = rt.PagedMetadata(loc, torch.zeros(1, dtype=torch.int64), torch.tensor([step]), mapping, slots)
        out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, d, d ** -0.5)
        kc[loc] = k.reshape(1, kv_heads, d)
        vc[loc] = v.reshape(1, kv_heads, d)
        ref = oracle.attend_fp32_softmax(q, kc, vc, torch.zeros(1, dtype=torch.int64), torch.tensor([step]), mapping,
                                         heads, kv_heads, d, d ** -0.5)
        oracle.fp32_softmax_gate(out.cpu().double(), ref)
    assert torch.equal(bits(key_pool.cpu()), bits(kc)) and torch.equal(bits(value_pool.cpu()), bits(vc))


def test_chunked_prefill_goes_to_the_tensor_core_kernel_and_matches_the_generic_path(rt):
    """Mixed step: two prefill chunks on paged prefixes plus decode rows, head_dim 128.  The default
    plan sends the chunks to the tcgen05 kernel; with the threshold disabled the same rows run on
    the generic kernel.  Both satisfy the oracle gates."""
    from tests import cases
    c = cases.chunk_case([300, 0, 1500], 96, 16, 4, 128, 128, seed=31, std=0.5)
    # turn the last sequence into a single decode row
    keep = torch.cat([torch.arange(0, 192), torch.arange(192 + 95, 192 + 96)])
    requests, positions, locations = c.requests[keep], c.positions[keep], c.locations[keep].contiguous()
    q, k, v = c.q[keep], c.k[keep], c.v[keep]
    # the dropped rows' positions must already be in the pool for the decode row: store them first
    pool_ref = c.pool.clone()
    oracle.kv_store_head_major(pool_ref, c.k, c.v, c.locations)
    outs = []
    for min_rows in (0, -1):
        combined = rt._C._allocate_paged_kv(1, c.slots, 4, 128)
        combined[0].copy_(pool_ref)
        kp, vp = combined[0, 0].transpose(0, 1), combined[0, 1].transpose(0, 1)
        md = rt.PagedMetadata(locations, requests, positions, c.mapping, c.slots)
        assert md.sequences() == [0, 96, 300, 0, 96, 96, 0, 1, 192, 1, 1595, 2]
        md._set_prefill_min_rows(min_rows)
        out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), kp, vp, md, 128, c.scale)
        assert torch.equal(bits(combined[0].cpu()), bits(pool_ref))
        kpc, vpc = oracle.pool_views(pool_ref)
        gates(out, (q, kpc, vpc, requests, positions, c.mapping, 16, 4, 128, c.scale))
        outs.append(out.cpu().double())
    assert rt._C._take_device_status() == 0
    assert float((outs[0] - outs[1]).abs().max()) <= 2e-2


def test_kv_store_inside_the_attention_launch_equals_the_separate_store(rt):
    """Decode steps carry the store in the attention launch (single-block recipe of the reference,
    src/bridge/paged_attention.cpp:74); pool and output must be the separate store's, bit for bit, with and
    without split KV ranges; a batch in which one request appears twice falls back to the separate launch."""
    ctx = [700, 33, 1500, 257, 64, 1023, 1, 16]
    case = cases.decode_case(len(ctx), 32, 8, 128, 128, 48, ctx, seed=606)
    ref_pool = case.pool.clone()
    oracle.kv_store_head_major(ref_pool, case.k, case.v, case.locations)
    try:
        for split in (0, 128):
            got = {}
            for fused in (True, False):
                torch.ops.gaudirt._set_fused_kv_store(fused)
                md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
                if split:
                    md._set_split_tokens(split)
                pool = case.pool.to(DEV)
                out = torch.ops.gaudirt.paged_attn(case.q.to(DEV), case.k.to(DEV), case.v.to(DEV), pool[0].transpose(0, 1),
                                                   pool[1].transpose(0, 1), md, 128, case.scale)
                assert torch.equal(bits(pool.cpu()), bits(ref_pool)), (split, fused)
                got[fused] = out
            assert torch.equal(bits(got[True]), bits(got[False])), split
    finally:
        torch.ops.gaudirt._set_fused_kv_store(True)
    # two decode rows of ONE request (positions p, p + 1 as separate sequences cannot exist; a chunk of 2 rows
    # followed by its continuation can): the later rows read the earlier rows' slots
    n_req, context, slots = 2, 256, 2 * 256 + 1
    mapping = torch.arange(1, slots, dtype=torch.int32).reshape(n_req, context)
    requests = torch.tensor([0, 0, 1, 0, 0], dtype=torch.int64)
    positions = torch.tensor([40, 41, 7, 42, 43], dtype=torch.int64)          # request 0: rows 0-1, then rows 3-4
    locations = mapping[requests, positions].to(torch.int64)
    md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
    assert md.sequences() == [0, 2, 40, 0, 2, 1, 7, 1, 3, 2, 42, 0]
    gen = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(5, w, generator=gen).bfloat16() for w in (8 * 64, 2 * 64, 2 * 64))
    kb, vb = (torch.randn(slots, 2, 64, generator=gen).bfloat16() for _ in range(2))
    _, key_pool, value_pool = make_pools(rt, slots, 2, 64, kb, vb)
    out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, 64, 0.125)
    ek, ev = kb.clone(), vb.clone()
    ek[locations] = k.reshape(-1, 2, 64)
    ev[locations] = v.reshape(-1, 2, 64)
    assert torch.equal(bits(key_pool.cpu()), bits(ek)) and torch.equal(bits(value_pool.cpu()), bits(ev))
    gates(out, (q, ek, ev, requests, positions, mapping, 8, 2, 64, 0.125))
    assert rt._C._take_device_status() == 0


def test_two_host_threads_call_the_operators_concurrently(rt):
    """The boundary promises calls from several host threads (the reference keeps thread-local recipe caches for
    that, src/bridge/paged_attention.cpp:139-151): two threads, each with its own stream, metadata, pool and head
    geometry -- so both take the first-use set-up paths of different kernels at the same time -- must each get
    the result a single-threaded call gives."""
    import threading
    specs = [(32, 8, 128, [300, 1500, 64, 900]), (8, 2, 64, [17, 700, 2000]), (4, 4, 256, [100, 130])]
    built = []
    for i, (hq, hkv, d, ctx) in enumerate(specs):
        blocks = sum((c + 127) // 128 for c in ctx) + 2
        built.append(cases.decode_case(len(ctx), hq, hkv, d, 128, blocks, ctx, seed=1200 + i))

    def run(case, results, key, repeats):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                outs = []
                for _ in range(repeats):
                    md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
                    md._set_split_tokens(256)
                    pool = case.pool.to(DEV)
                    outs.append(torch.ops.gaudirt.paged_attn(case.q.to(DEV), case.k.to(DEV), case.v.to(DEV),
                                                             pool[0].transpose(0, 1), pool[1].transpose(0, 1), md,
                                                             case.head_dim, case.scale))
                stream.synchronize()
            results[key] = outs
        except Exception as exc:          # surfaced by the parent
            results[key] = exc

    results = {}
    threads = [threading.Thread(target=run, args=(c, results, i, 6)) for i, c in enumerate(built)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    for i, case in enumerate(built):
        assert isinstance(results.get(i), list), results.get(i)
        alone = {}
        run(case, alone, 0, 1)
        for out in results[i]:
            assert torch.equal(bits(out), bits(alone[0][0]))
        ref_pool = case.pool.clone()
        oracle.kv_store_head_major(ref_pool, case.k, case.v, case.locations)
        kp, vp = oracle.pool_views(ref_pool)
        oracle.fp32_softmax_gate(results[i][0].cpu().double(),
                                 oracle.attend_fp32_softmax(case.q, kp, vp, case.requests, case.positions, case.mapping,
                                                            case.q_heads, case.kv_heads, case.head_dim, case.scale))
    assert rt._C._take_device_status() == 0
