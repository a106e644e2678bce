"""CPU-only checks of the C ABI: the library loads, exports every declared symbol, and its
host-side entry points (metadata validation, schedule) agree with the oracle's rules."""
import os
import re

import numpy as np
import pytest

import oracle
from gaudirt_b200 import abi
from gaudirt_b200 import raw as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported_and_bound():
    header = open(os.path.join(ROOT, "include", "gaudirt_b200.h")).read()
    declared = set(re.findall(r"GK_API\s+[\w\s\*]+?\b(gk_\w+)\s*\(", header))
    assert declared, "no declarations found"
    lib = abi.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(abi.PROTOTYPES), declared ^ set(abi.PROTOTYPES)
    assert lib.gk_abi_version() == 1
    assert lib.gk_status_string(0) == b"ok"


def test_pool_bytes_and_geometry_limits():
    import ctypes as C
    out = C.c_uint64(0)
    assert abi.lib().gk_paged_kv_pool_bytes(32, 1153408, 8, 128, C.byref(out)) == 0
    assert out.value == 32 * 2 * 8 * 1153408 * 128 * 2
    for bad in ((1, 16, 8, 96), (0, 16, 8, 128), (1, 0, 8, 128), (1, 16, 257, 128)):
        assert abi.lib().gk_paged_kv_pool_bytes(*bad, C.byref(out)) == 2


def test_metadata_validation_matches_oracle_rules():
    mapping = np.arange(1, 1 + 3 * 8).reshape(3, 8).astype(np.int32)
    good = ([3, 4, 5, 12], [0, 0, 0, 1], [2, 3, 4, 3])
    seq, page = H.validate(*good, mapping, 64)
    assert [tuple(s[:3]) for s in seq] == oracle.validate_paged_metadata(*good, mapping, 64)
    assert list(seq[:, 3]) == [0, 1] and page == 128   # every visible prefix is one contiguous run
    holes = mapping.copy(); holes[0, 1] = -1
    alias = mapping.copy(); alias[1, 0] = 3
    for args, table, text in (
            (([9], [0], [2]), mapping, "does not match"),
            (([3, 3], [0, 0], [2, 2]), mapping, "duplicate output KV slot"),
            (([3], [0], [9]), mapping, "out of range"),
            (([3], [0], [2]), holes, "missing KV slot"),
            (([3, 12], [0, 1], [2, 3]), alias, "aliases another visible prefix")):
        with pytest.raises(abi.GkError, match=text):
            H.validate(*args, table, 64)
        with pytest.raises(ValueError, match=text):
            oracle.validate_paged_metadata(*args, table, 64)


def test_page_detection():
    # pages of 16 contiguous slots, placed at arbitrary (unaligned) bases
    bases = np.array([[70, 5, 300], [200, 40, 130]])
    mapping = (bases[:, :, None] + np.arange(16)[None, None, :]).reshape(2, 48).astype(np.int32)
    seq, page = H.validate([mapping[0, 47], mapping[1, 20]], [0, 1], [47, 20], mapping, 400)
    assert page == 16
    mapping[1, 18] = 399                                    # break inside a visible page
    _, page = H.validate([mapping[0, 47], mapping[1, 20]], [0, 1], [47, 20], mapping, 400)
    assert page == 1
    full = np.arange(512, dtype=np.int32).reshape(1, 512)
    assert H.validate([300], [0], [300], full, 512)[1] == 128


def _coverage(work, combine, seq, q_heads, window):
    """Every (row, key) pair that must be attended is covered exactly once."""
    spans = {}
    for first_row, n_rows, first_pos, table_row, lo, hi, base, word in work:
        assert 0 < n_rows and lo < hi <= first_pos + n_rows
        spans.setdefault((first_row, n_rows, first_pos, table_row), []).append((lo, hi, base, word & 0xffff, word >> 16))
    merged = {(r, n): (b, s) for r, n, b, s in combine}
    rows_seen = set()
    for (first_row, n_rows, first_pos, _), parts in spans.items():
        parts.sort()
        lo0 = max(0, first_pos - window + 1) if window > 0 else 0
        assert parts[0][0] == lo0 and parts[-1][1] == first_pos + n_rows
        for a, b in zip(parts[:-1], parts[1:]):
            assert a[1] == b[0]
        if len(parts) == 1:
            assert parts[0][2] == -1 and (first_row, n_rows) not in merged
        else:
            base, splits = merged[(first_row, n_rows)]
            assert splits == len(parts)
            assert [p[2] for p in parts] == [base + i * n_rows * q_heads for i in range(splits)]
            assert [p[4] for p in parts] == list(range(splits)) and all(p[3] == splits for p in parts)
        for r in range(first_row, first_row + n_rows):
            assert r not in rows_seen
            rows_seen.add(r)
    return rows_seen


@pytest.mark.parametrize("split", [0, 64, 200, 4096])
@pytest.mark.parametrize("window", [-1, 100])
def test_schedule_covers_every_row_and_key_once(split, window):
    seq = np.array([[0, 1, 4095, 0], [1, 37, 100, 1], [38, 1, 0, 2], [39, 1, 20000, 3], [40, 3, 0, 4]], np.int32)
    for q_heads, kv_heads in ((32, 8), (8, 8), (64, 8), (7, 1)):
        work, combine, entries = H.plan(seq, q_heads, kv_heads, 128, window=window, split_tokens=split)
        rows = _coverage(work, combine, seq, q_heads, window)
        assert rows == set(range(43))
        spans = work[:, 5] - work[:, 4]
        assert (np.diff(spans) <= 0).all(), "longest first"
        assert entries == sum(n * q_heads * s for _, n, _, s in combine)
        if split:
            assert spans.max() <= max(split, 16) * 1.25 + 64


def test_schedule_rejects_unsupported_geometry():
    seq = np.array([[0, 1, 5, 0]], np.int32)
    for q_heads, kv_heads, d in ((32, 8, 96), (34, 1, 128), (9, 2, 128)):
        with pytest.raises(abi.GkError, match="unsupported"):
            H.plan(seq, q_heads, kv_heads, d)


def test_slot_layout_records_and_errors():
    """Host half of slot allocation: per-request records, totals and the reference's argument
    errors (src/bridge/paged_slot_allocator.cpp:95-112)."""
    import ctypes as C
    lib = abi.lib()

    def layout(prefixes, lengths, page, free):
        n = len(prefixes)
        p = (C.c_int64 * n)(*prefixes)
        l = (C.c_int64 * n)(*lengths)
        records = (C.c_int32 * (4 * n))()
        total, pages = C.c_int64(-1), C.c_int64(-1)
        status = lib.gk_paged_slots_layout(p, l, n, page, free, records, C.byref(total), C.byref(pages))
        return status, list(records), total.value, pages.value

    for page in (1, 16, 64):
        prefixes, lengths = [0, 7, page, 2 * page - 1], [19, 14, 20, 66]
        status, records, total, pages = layout(prefixes, lengths, page, 1 << 20)
        _, used = oracle.allocate_paged_slots([0] * 4, list(range(1 << 12)), prefixes, lengths, page)
        assert status == 0 and total == sum(lengths) and pages == used
        assert records[0::4] == prefixes and records[1::4] == lengths
        assert records[2::4] == list(np.cumsum([0] + lengths[:-1]))
        fresh = [(p + n + page - 1) // page - (p + page - 1) // page for p, n in zip(prefixes, lengths)]
        assert records[3::4] == list(np.cumsum([0] + fresh[:-1]))
    for args, text in ((([0], [40], 16, 2), b"insufficient free pages"), (([0], [0], 16, 2), b"invalid token count"),
                       (([-1], [4], 16, 2), b"invalid request lengths"), (([0], [4], 0, 2), b"unsupported page size"),
                       (([1 << 31], [4], 16, 2), b"invalid request lengths")):
        assert layout(*args)[0] == 5 and text in lib.gk_metadata_error()


def test_entry_points_reject_bad_arguments_before_touching_the_device():
    """Every check below fails in the host-side argument validation, so it runs without a GPU."""
    import ctypes as C
    lib = abi.lib()
    INVALID, UNSUPPORTED = 1, 2
    buf = (C.c_char * 4096)()
    a16 = (C.addressof(buf) + 255) & ~255                                  # a 256-byte aligned host address stands in
    ptr = C.c_void_p(a16)
    odd = C.c_void_p(a16 + 2)
    outs = (C.c_void_p * 1)(a16)
    # o_proj: null pointers, misaligned operands, shapes the tiling does not cover
    assert lib.gk_oproj_bf16(None, 64, ptr, 64, 8, 64, 64, outs, 1, 64, None, None) == INVALID
    assert lib.gk_oproj_bf16(odd, 64, ptr, 64, 8, 64, 64, outs, 1, 64, None, None) == INVALID
    assert lib.gk_oproj_bf16(ptr, 60, ptr, 64, 8, 64, 64, outs, 1, 64, None, None) == INVALID      # stride not 16-byte
    assert lib.gk_oproj_bf16(ptr, 64, ptr, 64, 8, 96, 64, outs, 1, 96, None, None) == UNSUPPORTED  # n % 64
    assert lib.gk_oproj_bf16(ptr, 100, ptr, 100, 8, 64, 100, outs, 1, 64, None, None) == UNSUPPORTED  # k % 64
    assert lib.gk_oproj_bf16(ptr, 64, ptr, 64, 8, 64, 64, outs, 9, 64, None, None) == INVALID      # too many destinations
    assert lib.gk_oproj_bf16(ptr, 64, ptr, 64, 0, 64, 64, outs, 1, 64, None, None) == 0            # nothing to do
    # rank-ordered sum
    parts = (C.c_void_p * 2)(a16, a16)
    assert lib.gk_rank_sum_bf16(parts, 0, 64, ptr, None) == INVALID
    assert lib.gk_rank_sum_bf16(parts, 2, 12, ptr, None) == UNSUPPORTED                             # count % 8
    assert lib.gk_rank_sum_add_rms_norm_bf16(parts, 2, 64, ptr, ptr, 0.0, 0.0, 4, 64, 64, ptr, ptr, None) == INVALID  # eps
    assert lib.gk_rank_sum_add_rms_norm_bf16(parts, 2, 16384, ptr, ptr, 1e-5, 0.0, 4, 16384, 16384, ptr, ptr, None) == UNSUPPORTED
    # slot allocator
    size = C.c_uint64(0)
    assert lib.gk_paged_slots_release_workspace_bytes(5000, 512, C.byref(size)) == 0 and size.value == 2048 + 256
    assert lib.gk_paged_slots_release_workspace_bytes(0, 512, C.byref(size)) == INVALID
    assert lib.gk_paged_slots_release(ptr, 8, 16, 512, odd, ptr, ptr, None) == INVALID            # workspace alignment
    assert lib.gk_paged_slots_allocate(ptr, ptr, odd, 1, 8, 16, ptr, None, 0, 0, 0, None, None, None, None) == INVALID
    assert lib.gk_paged_slots_allocate(ptr, ptr, ptr, 1, 8, 0, ptr, None, 0, 0, 0, None, None, None, None) == INVALID
    assert lib.gk_advance_decode_lengths(ptr, ptr, 0, ptr, ptr, None) == INVALID
    # device metadata validation
    assert lib.gk_paged_metadata_device_workspace_bytes(1 << 20, C.byref(size)) == 0 and size.value == (1 << 20) // 8
    assert lib.gk_paged_metadata_device_workspace_bytes(0, C.byref(size)) == INVALID
    assert lib.gk_paged_metadata_device_validate(ptr, ptr, ptr, None, 16, 0, ptr, 4, 64, 64, 100, ptr, 1, 1, ptr, ptr, ptr, ptr,
                                                 None, None, ptr, None, ptr, None, None) == INVALID   # unknown width bit
    assert lib.gk_paged_metadata_device_validate(ptr, ptr, ptr, None, 0, 0, ptr, 4, 64, 32, 100, ptr, 1, 1, ptr, ptr, ptr, ptr,
                                                 None, None, ptr, None, ptr, None, None) == INVALID   # table stride < context
    # after the LM head
    assert lib.gk_vocab_argmax(ptr, 0, 4, 0, 0, ptr, None) == INVALID
    assert lib.gk_apply_vocab_bitmask(ptr, 0, 4, 64, 64, ptr, 4, 1, None, 0, 64, 0, None, None) == INVALID   # 64 active > 32 mask bits
    assert lib.gk_sample_vocab(ptr, 0, 4, 64, 64, ptr, ptr, ptr, ptr, None, ptr, 0, 0, 1, ptr, None) == INVALID  # positions without seeds
    # peer barrier
    flags = (C.c_void_p * 2)(a16, a16)
    assert lib.gk_peer_barrier_counted(flags, 0, 2, None, 1000, None, None) == INVALID
    assert lib.gk_peer_barrier(flags, 2, 2, 1, 1000, None, None) == INVALID


def test_slot_layout_random_batches_agree_with_the_oracle():
    """Property check over random request mixes: totals, page counts and per-request offsets of the host
    layout equal what the oracle's allocation rule implies."""
    import ctypes as C
    from hypothesis import given, settings, strategies as st
    lib = abi.lib()

    @settings(max_examples=200, deadline=None)
    @given(st.integers(1, 200), st.lists(st.tuples(st.integers(0, 3000), st.integers(0, 700)), min_size=1, max_size=40))
    def check(page, requests):
        prefixes, lengths = [p for p, _ in requests], [n for _, n in requests]
        n = len(requests)
        records = (C.c_int32 * (4 * n))()
        total, pages = C.c_int64(-1), C.c_int64(-1)
        status = lib.gk_paged_slots_layout((C.c_int64 * n)(*prefixes), (C.c_int64 * n)(*lengths), n, page, 1 << 30, records,
                                           C.byref(total), C.byref(pages))
        if sum(lengths) == 0:
            assert status == 5
            return
        assert status == 0 and total.value == sum(lengths)
        free = list(range(10 ** 6, 10 ** 6 + sum(lengths) + n + 1))  # page = 1 needs one page per token
        slots, used = oracle.allocate_paged_slots([7] * n, free, prefixes, lengths, page)
        assert pages.value == used and len(slots) == total.value
        # the first fresh page of request r, as the oracle consumed them, is where the record points
        at = 0
        for r in range(n):
            open_tail = min(lengths[r], (-prefixes[r]) % page)
            assert records[4 * r + 2] == at
            if lengths[r] > open_tail:
                assert slots[at + open_tail] == free[records[4 * r + 3]] * page
            at += lengths[r]

    check()


def test_plan_cuts_partition_every_range_including_uneven_cuts():
    """Whatever cut the schedule search picks (none, even pieces, or pieces of the limit with the remainder last,
    which it may pick when the grid is a few waves), the pieces of a block tile its KV range exactly, in split
    order, and the split state is sized for them."""
    shapes = [
        (np.array([[i, 1, 4095, i] for i in range(256)], dtype=np.int32), 4, 1),      # one KV head of config 2: one wave
        (np.array([[i, 1, 4095, i] for i in range(256)], dtype=np.int32), 8, 2),
        (np.array([[i, 1, 4095, i] for i in range(256)], dtype=np.int32), 32, 8),     # the whole GPU: no cut
        (np.array([[i, 1, 300 + 97 * i, i] for i in range(40)], dtype=np.int32), 8, 1),
    ]
    saw_uneven = False
    for seq, hq, hkv in shapes:
        work, combine, entries = H.plan(seq, hq, hkv, 128, sm_count=148)
        by_row = {}
        for w in work:
            by_row.setdefault(int(w[0]), []).append(w)
        total = 0
        for first_row, n_rows, first_pos, table_row in seq:
            pieces = sorted(by_row[int(first_row)], key=lambda w: int(w[7]) >> 16)
            n_splits = int(pieces[0][7]) & 0xffff
            assert len(pieces) == n_splits and [int(p[7]) >> 16 for p in pieces] == list(range(n_splits))
            assert int(pieces[0][4]) == 0 and int(pieces[-1][5]) == first_pos + n_rows
            for a, b in zip(pieces, pieces[1:]):
                assert int(a[5]) == int(b[4]) and int(a[5]) > int(a[4])
            lengths = [int(p[5]) - int(p[4]) for p in pieces]
            saw_uneven |= n_splits > 1 and len(set(lengths[:-1] + [lengths[-1]])) > 1 and lengths[-1] < lengths[0] // 2
            if n_splits > 1:
                bases = [int(p[6]) for p in pieces]
                assert bases == [bases[0] + s * n_rows * hq for s in range(n_splits)]
                total += n_splits * n_rows * hq
            else:
                assert int(pieces[0][6]) == -1
        assert total == entries and len(combine) == sum(1 for r in by_row.values() if len(r) > 1)
    assert saw_uneven, "the skewed single-head batch is where the uneven cut is chosen"
    # equal ranges that fit the resident CTA slots in one wave are left whole: the launch is HBM-bound either
    # way, and a CTA next to an idle slot streams faster, so a cut would only add prologues and merges
    work, combine, _ = H.plan(shapes[0][0], 4, 1, 128, sm_count=148)
    assert len(work) == 256 and len(combine) == 0


def test_process_wide_switches_take_only_their_values():
    """The two host-side switches (how the decode kernel stages a group, programmatic dependent launch) need no
    GPU: valid values are accepted, anything else is GK_ERR_INVALID_ARGUMENT and changes nothing."""
    lib = abi.lib()
    try:
        for form in (0, 1, 2):
            assert lib.gk_set_attention_form(form) == 0
        for bad in (-1, 3, 99):
            assert lib.gk_set_attention_form(bad) != 0
        assert lib.gk_set_programmatic_launch(1) == 0 and lib.gk_set_programmatic_launch(0) == 0
    finally:
        lib.gk_set_attention_form(0)
        lib.gk_set_programmatic_launch(0)
