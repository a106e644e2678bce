"""Device slot allocation / release and the decode-length update against the oracle and the
reference's known-answer vectors (tests/paged_slots_device_smoke.py:16-45,
tests/paged_attention_generalized_smoke.py:137-158, tests/dynamic_eager_ops_smoke.py:383-412,
tests/decode_lengths_smoke.py:20-33)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def dev(values, dtype=torch.int64):
    return torch.tensor(values, dtype=dtype, device=DEV)


@pytest.mark.parametrize("page_size", [16, 64])
def test_allocate_and_release_known_answers(rt, page_size):
    prefixes, lengths = [0, 7, page_size, 2 * page_size - 1], [19, 14, 20, 66]
    previous = [-1, 81 * page_size + 6, 82 * page_size + page_size - 1, 83 * page_size + page_size - 2]
    pages = [13, 7, 23, 41, 12, 33, 55, 61, 15, 18, 19, 20, 21, 22, 24, 25]
    expected, used_expected = oracle.allocate_paged_slots(previous, pages, prefixes, lengths, page_size)
    slots, used = rt._C._allocate_paged_slots(dev(previous), dev(pages), prefixes, lengths, page_size)
    assert used == used_expected and slots.dtype == torch.int64 and slots.cpu().tolist() == expected
    # spot values a reader can check by hand: request 0 starts page 13, request 1 continues after slot 81p+6
    assert expected[0] == 13 * page_size and expected[19] == 81 * page_size + 7
    released = [13 * page_size + 7, 7 * page_size, 13 * page_size, 23 * page_size + page_size - 1, 7 * page_size + 3]
    unique = rt._C._release_paged_slots(dev(released), page_size, 512)
    assert unique.cpu().tolist() == [13, 7, 23] == oracle.release_paged_slots(released, page_size, 512)
    for invalid in (0, 513 * page_size, 1 << 40):
        with pytest.raises(RuntimeError, match="outside the KV pool"):
            rt._C._release_paged_slots(dev([invalid]), page_size, 512)


@pytest.mark.parametrize("page_size", [1, 8, 16, 32, 64, 128])
def test_allocator_page_sizes_and_many_pages(rt, page_size):
    prefixes, lengths = [0, 3, page_size], [5, 7, page_size + 2]
    prev = [-1, 100 * page_size + (2 % page_size), 200 * page_size + (page_size - 1)]
    pages = list(range(10, 80))
    expected, used_expected = oracle.allocate_paged_slots(prev, pages, prefixes, lengths, page_size)
    slots, used = rt._C._allocate_paged_slots(dev(prev), dev(pages), prefixes, lengths, page_size)
    assert used == used_expected and slots.cpu().tolist() == expected
    rel_in = [9000 * page_size, 9000 * page_size + (page_size - 1), 12000 * page_size]
    unique = rt._C._release_paged_slots(dev(rel_in), page_size, 16384)
    assert unique.cpu().tolist() == [9000, 12000]


def test_allocator_shapes_that_share_a_bucket_in_the_reference(rt):
    for prefixes, lengths, n_pages in (([0, 3], [5, 7], 12), ([0, 16, 4], [4, 5, 5], 18),
                                       ([1, 2, 3, 4, 5], [2, 3, 2, 2, 2], 30)):
        prev = [-1] * len(prefixes)
        pages = list(range(100, 100 + n_pages))
        expected, used_expected = oracle.allocate_paged_slots(prev, pages, prefixes, lengths, 16)
        slots, used = rt._C._allocate_paged_slots(dev(prev), dev(pages), prefixes, lengths, 16)
        assert used == used_expected and slots.cpu().tolist() == expected


def test_allocator_argument_errors(rt):
    ok = (dev([-1]), dev([3, 4]), [0], [5], 16)
    rt._C._allocate_paged_slots(*ok)
    for args, text in (
            ((dev([-1]), dev([3]), [0], [40], 16), "insufficient free pages"),
            ((dev([-1]), dev([3]), [0], [0], 16), "invalid token count"),
            ((dev([-1]), dev([3]), [-1], [4], 16), "invalid request lengths"),
            ((dev([-1]), dev([3]), [0], [4], 0), "unsupported page size"),
            ((dev([-1, -1]), dev([3]), [0], [4], 16), "request count"),
            ((dev([-1], torch.int32), dev([3]), [0], [4], 16), "int64 indices")):
        with pytest.raises(RuntimeError, match=text):
            rt._C._allocate_paged_slots(*args)
    with pytest.raises(RuntimeError, match="invalid release geometry"):
        rt._C._release_paged_slots(dev([5]), 16, 0)


def test_empty_requests_and_random_batches_match_the_oracle(rt):
    rng = np.random.default_rng(11)
    for page_size in (1, 4, 16, 48, 128):
        n = 97
        prefixes = rng.integers(0, 5 * page_size + 3, n).tolist()
        lengths = rng.integers(0, 3 * page_size + 2, n).tolist()
        lengths[0] = lengths[5] = lengths[-1] = 0
        lengths[1] = 2000                                              # one long prefill among decodes
        pages = rng.permutation(8192)[:4096].tolist()
        # a request with an open page continues right behind its last slot
        prev = [int(rng.integers(1, 5000)) * page_size + (p - 1) % page_size if p % page_size else -1
                for p in prefixes]
        expected, used_expected = oracle.allocate_paged_slots(prev, pages, prefixes, lengths, page_size)
        slots, used = rt._C._allocate_paged_slots(dev(prev), dev(pages), prefixes, lengths, page_size)
        assert used == used_expected and slots.cpu().tolist() == expected


def test_allocation_fused_with_table_and_location_scatter(rt):
    page_size, context, n_req = 16, 96, 12
    prefixes, lengths = [0, 5, 32, 47], [33, 1, 1, 20]
    batch = [7, 2, 9, 4]
    rng = np.random.default_rng(3)
    pages = (rng.permutation(200)[:32] + 1).tolist()
    table = torch.full((n_req, context), -1, dtype=torch.int32, device=DEV)
    prev = []
    for r, p in zip(batch, prefixes):                                   # cached prefixes live on their own pages
        own = [(300 + 10 * r + i // page_size) * page_size + i % page_size for i in range(p)]
        table[r, :p] = torch.tensor(own, dtype=torch.int32)
        prev.append(own[-1] if own else -1)
    before = table.clone()
    expected, used_expected = oracle.allocate_paged_slots(prev, pages, prefixes, lengths, page_size)
    slots, locations, used = rt._C._allocate_paged_slots_into(dev(prev), dev(pages), prefixes, lengths, page_size,
                                                              table, dev(batch, torch.int32))
    assert used == used_expected and slots.cpu().tolist() == expected
    assert locations.dtype == torch.int32 and locations.cpu().tolist() == expected
    want = before.cpu()
    at = 0
    for r, p, n in zip(batch, prefixes, lengths):
        want[r, p:p + n] = torch.tensor(expected[at:at + n], dtype=torch.int32)
        at += n
    assert torch.equal(table.cpu(), want)                               # every other cell untouched
    assert rt._C._take_device_status() == 0
    # the produced table and slot list are accepted by the device-side validator as they are
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(prefixes, lengths)]).to(DEV)
    md = rt.PagedMetadata.from_device(locations, dev(batch, torch.int32), positions, table, prefixes, lengths, 8192)
    assert md.rows() == sum(lengths) and md.row_locations().cpu().tolist() == expected
    with pytest.raises(RuntimeError, match="invalid request lengths"):
        rt._C._allocate_paged_slots_into(dev(prev), dev(pages), [0, 5, 32, 90], lengths, page_size, table,
                                         dev(batch, torch.int32))


@pytest.mark.parametrize("n_slots", [1, 8192, 8193, 50001])
def test_release_order_and_dedup_at_scale(rt, n_slots):
    rng = np.random.default_rng(n_slots)
    page_size, max_pages = 16, 4096
    slots = rng.integers(1, max_pages * page_size, n_slots).tolist()
    want = oracle.release_paged_slots(slots, page_size, max_pages)
    for _ in range(2):                                                  # workspace is rebuilt on every call
        got = rt._C._release_paged_slots(dev(slots), page_size, max_pages)
        assert got.cpu().tolist() == want
    if n_slots > 8192:
        bad = list(slots)
        bad[n_slots // 2] = max_pages * page_size
        with pytest.raises(RuntimeError, match="outside the KV pool"):
            rt._C._release_paged_slots(dev(bad), page_size, max_pages)


@pytest.mark.parametrize("count", [1, 3, 16, 4097])
def test_advance_decode_lengths_keeps_the_old_batch(rt, count):
    seq = torch.arange(count, dtype=torch.int64) * (2 ** 33) + 17
    orig = torch.arange(count, dtype=torch.int32) + 31
    device_seq, device_orig = seq.to(DEV), orig.to(DEV)
    next_seq, next_orig = torch.ops.gaudirt._advance_decode_lengths(device_seq, device_orig)
    assert next_seq.dtype == torch.int64 and next_orig.dtype == torch.int32
    assert torch.equal(next_seq.cpu(), seq + 1) and torch.equal(next_orig.cpu(), orig + 1)
    assert torch.equal(device_seq.cpu(), seq) and torch.equal(device_orig.cpu(), orig)
    with pytest.raises(RuntimeError, match="matching contiguous int64 and int32"):
        torch.ops.gaudirt._advance_decode_lengths(device_orig, device_orig)


def test_advance_decode_lengths_in_a_cuda_graph(rt):
    seq = torch.tensor([5, 1 << 40], dtype=torch.int64, device=DEV)
    orig = torch.tensor([5, 9], dtype=torch.int32, device=DEV)
    torch.ops.gaudirt._advance_decode_lengths(seq, orig)                # warm up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        a, b = torch.ops.gaudirt._advance_decode_lengths(seq, orig)
        seq.copy_(a)
        orig.copy_(b)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert seq.cpu().tolist() == [8, (1 << 40) + 3] and orig.cpu().tolist() == [8, 12]
