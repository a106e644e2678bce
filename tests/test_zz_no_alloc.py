"""The allocation-free attention entry point against the regular one.

Some callers cannot allocate device memory when they launch attention (all HBM already belongs to
their KV pool, or they run where entering an allocator is not allowed), so
gk_paged_attn_static_scratch_bf16 keeps its split-KV state in an array inside the library.  The
results must be the regular entry point's, also on a second call that finds the first call's
leftovers in that array.  Collected last on purpose: it is an addition, every other test runs first.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gaudirt_b200 import abi
from gaudirt_b200 import raw as H
from tests import cases

DEV = "cuda:0"


def _call_static(case, pool, table, page, work, combine, entries, q_dev):
    out = torch.full((case.q.size(0), case.q_heads * case.head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    work_d = torch.from_numpy(work).to(DEV)
    comb_d = torch.from_numpy(np.ascontiguousarray(combine)).to(DEV) if len(combine) else None
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    st = abi.lib().gk_paged_attn_static_scratch_bf16(
        q_dev.data_ptr(), q_dev.stride(0), pool[0].data_ptr(), pool[1].data_ptr(), case.slots, table.data_ptr(),
        table.stride(0), page, page, None, work_d.data_ptr(), len(work),
        comb_d.data_ptr() if comb_d is not None else None, len(combine), entries, out.data_ptr(), out.stride(0),
        case.scale, 0.0, -1, case.q_heads, case.kv_heads, case.head_dim, None, H.stream_ptr())
    abi.check(st, "gk_paged_attn_static_scratch_bf16")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return out


@pytest.mark.gpu
def test_static_scratch_entry_point_matches_regular_entry_point_twice():
    ctx = [700, 33, 1500, 257, 64, 1023]
    case = cases.decode_case(len(ctx), 32, 8, 128, 128, 40, ctx, seed=4242)
    pool = case.pool.to(DEV)
    H.kv_store(pool, case.k.to(DEV), case.v.to(DEV), case.locations.to(DEV))
    seq, page = H.validate(case.locations, case.requests, case.positions, case.mapping, case.slots)
    table = case.mapping.to(DEV)
    q_dev = case.q.to(DEV)
    for split in (128, 320):                       # two calls in a row, different schedules
        work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, split_tokens=split)
        assert len(combine) > 0 and 0 < entries <= 8192
        want = H.paged_attn(q_dev, pool, table, page, work, combine, entries, case.q_heads, case.scale,
                            entry_stride=page)
        got = _call_static(case, pool, table, page, work, combine, entries, q_dev)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), split
    # an unsplit schedule needs no scratch at all and still goes through
    work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, split_tokens=1 << 20)
    assert entries == 0 and len(combine) == 0
    want = H.paged_attn(q_dev, pool, table, page, work, combine, entries, case.q_heads, case.scale, entry_stride=page)
    got = _call_static(case, pool, table, page, work, combine, entries, q_dev)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_static_scratch_entry_point_refuses_oversized_schedules():
    lib = abi.lib()
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    args = lambda entries, d: (dummy.data_ptr(), 128, dummy.data_ptr(), dummy.data_ptr(), 16, dummy.data_ptr(), 1, 1, 1,
                               None, dummy.data_ptr(), 1, dummy.data_ptr(), 1, entries, dummy.data_ptr(), 128, 0.1, 0.0,
                               -1, 1, 1, d, None, None)
    assert lib.gk_paged_attn_static_scratch_bf16(*args(8193, 128)) == 4
    assert b"too small" in lib.gk_status_string(4)
    assert lib.gk_paged_attn_static_scratch_bf16(*args(-1, 128)) == 1
