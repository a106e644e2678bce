"""The allocation-free attention entry point against the regular one.

Some callers cannot allocate device memory when they launch attention (all HBM already belongs to
their KV pool, or they run where entering an allocator is not allowed), so
gk_paged_attn_static_scratch_bf16 keeps its split-KV state in an array inside the library.  The
results must be the regular entry point's, also on a second call that finds the first call's
leftovers in that array.  Collected last on purpose: it is an addition, every other test runs first.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from gaudirt_b200 import abi
from gaudirt_b200 import raw as H
from tests import cases

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _call_static(case, pool, table, page, work, combine, entries, q_dev, status=None, measure=True):
    out = torch.full((case.q.size(0), case.q_heads * case.head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    work_d = torch.from_numpy(work).to(DEV)
    comb_d = torch.from_numpy(np.ascontiguousarray(combine)).to(DEV) if len(combine) else None
    torch.cuda.synchronize()
    # what the DRIVER has handed out on this device, which also sees a cudaMalloc made behind torch's back
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    st = abi.lib().gk_paged_attn_static_scratch_bf16(
        q_dev.data_ptr(), q_dev.stride(0), pool[0].data_ptr(), pool[1].data_ptr(), case.slots, table.data_ptr(),
        table.stride(0), page, page, None, work_d.data_ptr(), len(work),
        comb_d.data_ptr() if comb_d is not None else None, len(combine), entries, out.data_ptr(), out.stride(0),
        case.scale, 0.0, -1, case.q_heads, case.kv_heads, case.head_dim,
        status.data_ptr() if status is not None else None, H.stream_ptr())
    abi.check(st, "gk_paged_attn_static_scratch_bf16")
    torch.cuda.synchronize()
    if measure:
        assert torch.cuda.mem_get_info()[0] == free_before, "the call took device memory from the driver"
        assert torch.cuda.memory_allocated() == torch_before
    return out


def _prepared(ctx, q_heads, kv_heads, d, seed):
    blocks = sum((c + 127) // 128 for c in ctx) + 2
    case = cases.decode_case(len(ctx), q_heads, kv_heads, d, 128, blocks, ctx, seed=seed)
    pool = case.pool.to(DEV)
    H.kv_store(pool, case.k.to(DEV), case.v.to(DEV), case.locations.to(DEV))
    seq, page = H.validate(case.locations, case.requests, case.positions, case.mapping, case.slots)
    return case, pool, seq, page, case.mapping.to(DEV), case.q.to(DEV)


@pytest.mark.gpu
def test_static_scratch_entry_point_matches_regular_entry_point_twice():
    case, pool, seq, page, table, q_dev = _prepared([700, 33, 1500, 257, 64, 1023], 32, 8, 128, 4242)
    # the module (and with it the array) is loaded by the first use of the library on this device: that one
    # call is not measured, every later one is
    work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, split_tokens=1 << 20)
    _call_static(case, pool, table, page, work, combine, entries, q_dev, measure=False)
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
def test_static_scratch_at_the_capacity_boundary_and_at_head_dim_256():
    """Exactly GK_STATIC_SCRATCH_MAX_ENTRIES entries at the widest head: the array is used to its last float."""
    # 8 sequences x 16 splits x 64 query heads = 8192 entries; head_dim 256 fills every entry's O row
    case, pool, seq, page, table, q_dev = _prepared([2048] * 8, 64, 8, 256, 515)
    work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, split_tokens=128)
    assert entries == 8192 and len(combine) == 8
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for _ in range(2):
        want = H.paged_attn(q_dev, pool, table, page, work, combine, entries, case.q_heads, case.scale, entry_stride=page)
        got = _call_static(case, pool, table, page, work, combine, entries, q_dev, status=status)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert int(status.item()) == 0
    # one more sequence: 9216 entries, refused before anything is launched
    case2, pool2, seq2, page2, table2, q2 = _prepared([2048] * 9, 64, 8, 256, 516)
    work2, combine2, entries2 = H.plan(seq2, 64, 8, 256, split_tokens=128)
    assert entries2 == 9216
    out = torch.zeros(9, 64 * 256, dtype=torch.bfloat16, device=DEV)
    wd, cd = torch.from_numpy(work2).to(DEV), torch.from_numpy(np.ascontiguousarray(combine2)).to(DEV)
    st = abi.lib().gk_paged_attn_static_scratch_bf16(
        q2.data_ptr(), q2.stride(0), pool2[0].data_ptr(), pool2[1].data_ptr(), case2.slots, table2.data_ptr(),
        table2.stride(0), page2, page2, None, wd.data_ptr(), len(work2), cd.data_ptr(), len(combine2), entries2,
        out.data_ptr(), out.stride(0), case2.scale, 0.0, -1, 64, 8, 256, None, H.stream_ptr())
    torch.cuda.synchronize()
    assert st == 4 and float(out.float().abs().sum()) == 0.0


@pytest.mark.gpu
def test_static_scratch_records_beyond_the_declared_count_are_skipped_and_flagged():
    """A schedule that needs more split state than the caller declared must not write past the declared part of
    the array: the device skips those records and raises GK_DEV_BAD_SLOT, and the next, honest call is right."""
    case, pool, seq, page, table, q_dev = _prepared([700, 33, 1500, 257, 64, 1023], 32, 8, 128, 4243)
    work, combine, entries = H.plan(seq, case.q_heads, case.kv_heads, case.head_dim, split_tokens=128)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = H.paged_attn(q_dev, pool, table, page, work, combine, entries, case.q_heads, case.scale, entry_stride=page)
    lied = _call_static(case, pool, table, page, work, combine, entries // 2, q_dev, status=status)
    assert int(status.item()) & 1, "GK_DEV_BAD_SLOT"
    # rows whose records fit the declared half are still right; the skipped blocks' rows were never written (NaN fill)
    ok_rows = [int(c[0]) for c in combine if int(c[2]) + int(c[3]) * int(c[1]) * case.q_heads <= entries // 2]
    assert ok_rows, "the case is built so that some blocks fit"
    for r in ok_rows:
        assert torch.equal(lied[r].view(torch.int16), want[r].view(torch.int16))
    status.zero_()
    got = _call_static(case, pool, table, page, work, combine, entries, q_dev, status=status)
    assert int(status.item()) == 0 and torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_static_scratch_entry_point_refuses_inconsistent_or_oversized_schedules():
    lib = abi.lib()
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    args = lambda entries, d, n_work=1, n_combine=1, combine=dummy.data_ptr(): (
        dummy.data_ptr(), 128, dummy.data_ptr(), dummy.data_ptr(), 16, dummy.data_ptr(), 1, 1, 1, None, dummy.data_ptr(),
        n_work, combine, n_combine, entries, dummy.data_ptr(), 128, 0.1, 0.0, -1, 1, 1, d, None, None)
    assert lib.gk_paged_attn_static_scratch_bf16(*args(8193, 128)) == 4
    assert b"too small" in lib.gk_status_string(4)
    assert lib.gk_paged_attn_static_scratch_bf16(*args(-1, 128)) == 1
    # every argument is judged before anything is launched: nothing below may touch `dummy`
    assert lib.gk_paged_attn_static_scratch_bf16(*args(16, 128, combine=None)) == 1          # records missing
    assert lib.gk_paged_attn_static_scratch_bf16(*args(16, 128, n_combine=0)) == 1           # state without records
    assert lib.gk_paged_attn_static_scratch_bf16(*args(0, 128, n_combine=1)) == 1            # records without state
    assert lib.gk_paged_attn_static_scratch_bf16(*args(16, 128, n_work=0)) == 1              # would merge leftovers
    torch.cuda.synchronize()
    assert int(dummy.abs().sum()) == 0


@pytest.mark.gpu
def test_static_scratch_first_library_call_in_a_fresh_process():
    """The set-up (address lookup, module load) happens on the first call: here that call is the very first use
    of the library in a new process, and it must already give the regular entry point's result."""
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch\n"
        "from tests import test_zz_no_alloc as t\n"
        "from gaudirt_b200 import raw as H\n"
        "from tests import cases\n"
        "ctx = [900, 40, 300]\n"
        "case = cases.decode_case(3, 16, 4, 128, 128, 16, ctx, seed=99)\n"
        "pool = case.pool.to(t.DEV); q = case.q.to(t.DEV); table = case.mapping.to(t.DEV)\n"
        "seq, page = H.validate(case.locations, case.requests, case.positions, case.mapping, case.slots)\n"
        "work, combine, entries = H.plan(seq, 16, 4, 128, split_tokens=128)\n"
        "got = t._call_static(case, pool, table, page, work, combine, entries, q, measure=False)\n"
        "want = H.paged_attn(q, pool, table, page, work, combine, entries, 16, case.scale, entry_stride=page)\n"
        "assert torch.equal(got.view(torch.int16), want.view(torch.int16))\n"
        "print('fresh-process ok')\n") % ROOT
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and "fresh-process ok" in done.stdout, done.stdout + done.stderr
