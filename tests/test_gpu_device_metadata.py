"""Device-resident metadata: validation on the GPU, row expansion and the error codes of the
reference's device-input constructor (tests/paged_device_metadata_smoke.py:31-56, 80-150)."""
import re

import numpy as np
import pytest
import torch

import oracle
from tests import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REQUESTS, CONTEXT = 8, 1024
SLOTS = REQUESTS * CONTEXT + 1
ORDER = [7, 2, 5, 1, 6, 0, 4, 3]


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def batch(rows):
    mapping = torch.arange(1, SLOTS, dtype=torch.int32).reshape(REQUESTS, CONTEXT)
    n = min(rows, REQUESTS)
    requests = torch.tensor(ORDER[:n], dtype=torch.int64)
    lengths = [rows // n + int(i < rows % n) for i in range(n)]
    prefixes = [2 + i for i in range(n)]
    row_requests = torch.repeat_interleave(requests, torch.tensor(lengths))
    positions = torch.cat([torch.arange(p, p + l, dtype=torch.int64) for p, l in zip(prefixes, lengths)])
    locations = mapping[row_requests, positions].to(torch.int64)
    return locations, requests, positions, mapping, prefixes, lengths, row_requests


def strided(source):
    storage = torch.empty(source.numel() * 2, dtype=source.dtype, device=DEV)
    view = storage[::2]
    view.copy_(source)
    return view


def build(rt, locations, requests, positions, mapping, prefixes, lengths, sliced=False):
    put = strided if sliced else (lambda t: t.to(DEV))
    return rt.PagedMetadata.from_device(put(locations), put(requests), put(positions), mapping.to(DEV), prefixes,
                                        lengths, SLOTS)


@pytest.mark.parametrize("rows", [1, 7, 33, 137, 1025, 4096])
def test_accepts_and_expands(rt, rows):
    locations, requests, positions, mapping, prefixes, lengths, row_requests = batch(rows)
    if rows in (33, 1025):
        positions = positions.to(torch.int32)
    md = build(rt, locations, requests, positions, mapping, prefixes, lengths, sliced=rows == 137)
    assert md.rows() == rows and md.slots() == SLOTS and md.context() == CONTEXT
    for got, want in ((md.row_locations(), locations), (md.row_requests(), row_requests),
                      (md.rotary_positions(), positions)):
        assert got.dtype == torch.int32 and torch.equal(got.cpu().long(), want.long())
    indices = rt.validated_last_token_indices(md)
    assert indices.dtype == torch.int32 and indices._gaudirt_validated_rows == rows
    assert torch.equal(indices.cpu().long(), torch.cumsum(torch.tensor(lengths), 0) - 1)
    codes, last = oracle.device_metadata_status(locations, requests, positions, mapping.tolist(), prefixes, lengths, SLOTS)
    assert not any(codes) and last == indices.cpu().tolist()
    assert rt._C._take_device_status() == 0


def test_page_size_is_detected_on_the_device(rt):
    """The device form finds the same page granularity as the host form (largest power of two <= 128 whose
    pages are slot-contiguous in every visible range)."""
    assert build(rt, *batch(33)[:6]).page_tokens() == 128             # each request's slots are one run
    for page in (16, 64):
        n_req, context = 3, 256
        gen = torch.Generator().manual_seed(page)
        blocks = torch.randperm(n_req * context // page, generator=gen).view(n_req, context // page)
        mapping = (blocks[:, :, None] * page * 2 + 1 + torch.arange(page)[None, None, :]).reshape(n_req, context)
        mapping = mapping.to(torch.int32)                               # pages start 2 * page apart: never adjacent
        prefixes, lengths = [40, 0, 200], [3, 70, 1]
        requests = torch.tensor([2, 0, 1])
        positions = torch.cat([torch.arange(p, p + l) for p, l in zip(prefixes, lengths)])
        row_requests = torch.repeat_interleave(requests, torch.tensor(lengths))
        locations = mapping[row_requests, positions].long()
        slots = int(mapping.max()) + 1
        md = rt.PagedMetadata.from_device(locations.to(DEV), requests.to(DEV), positions.to(DEV), mapping.to(DEV),
                                          prefixes, lengths, slots)
        host = rt.PagedMetadata(locations, row_requests, positions, mapping, slots)
        assert md.page_tokens() == host.page_tokens() == page
    assert rt._C._take_device_status() == 0


def rejected(rt, values, code):
    want, _ = oracle.device_metadata_status(*[v.tolist() if torch.is_tensor(v) else v for v in values], SLOTS)
    assert code in want
    with pytest.raises(RuntimeError, match=r"invalid scheduler metadata at row \d+, code %d\b" % code) as error:
        build(rt, *values)
    row = int(re.search(r"row (\d+)", str(error.value)).group(1))
    # also for two rows on one slot: the later one is named, whichever of them lost the race on the device
    assert row == next(i for i, c in enumerate(want) if c)
    assert rt._C._take_device_status() == 0                            # raised on the host, nothing left pending


def test_rejections_carry_the_reference_codes(rt):
    locations, requests, positions, mapping, prefixes, lengths, _ = batch(7)
    bad = locations.clone(); bad[0] += 1 << 32
    rejected(rt, (bad, requests, positions, mapping, prefixes, lengths), 1)
    bad = requests.clone(); bad[0] += 1 << 32
    rejected(rt, (locations, bad, positions, mapping, prefixes, lengths), 2)
    bad = positions.clone(); bad[0] += 1 << 32
    rejected(rt, (locations, requests, bad, mapping, prefixes, lengths), 1)
    bad = locations.clone(); bad[0] += 1
    rejected(rt, (bad, requests, positions, mapping, prefixes, lengths), 3)
    bad = mapping.clone(); bad[requests[0], 0] = -1
    rejected(rt, (locations, requests, positions, bad, prefixes, lengths), 6)
    bad = mapping.clone(); bad[requests[1], 0] = locations[0]
    rejected(rt, (locations, requests, positions, bad, prefixes, lengths), 7)
    dup_req = torch.tensor([0, 0], dtype=torch.int64)
    dup_pos = torch.tensor([2, 2], dtype=torch.int64)
    rejected(rt, (mapping[dup_req, dup_pos].to(torch.int64), dup_req, dup_pos, mapping, [2, 2], [1, 1]), 4)
    bad = positions.clone(); bad[3] += 1                                # in range, but not prefix + offset
    bad_locations = locations.clone()
    rejected(rt, (bad_locations, requests, bad, mapping, prefixes, lengths), 5)
    with pytest.raises(RuntimeError, match="sequence lengths"):
        build(rt, locations, requests, positions, mapping, prefixes, [lengths[0] + 1] + lengths[1:])


def test_token_ids_are_range_checked(rt):
    locations, requests, positions, mapping, prefixes, lengths, _ = batch(33)
    tokens = torch.arange(33, dtype=torch.int64) * 7 % 1000
    args = [t.to(DEV) for t in (locations, requests, positions, mapping)]
    md = rt.PagedMetadata.from_device_with_tokens(*args, prefixes, lengths, SLOTS, tokens.to(DEV), 1000)
    assert md.vocabulary() == 1000 and torch.equal(md.token_ids().cpu().long(), tokens)
    bad = tokens.clone(); bad[20] = 1000
    with pytest.raises(RuntimeError, match="token ID outside vocabulary at row 20"):
        rt.PagedMetadata.from_device_with_tokens(*args, prefixes, lengths, SLOTS, bad.to(DEV), 1000)
    assert rt._C._take_device_status() == 0


def test_scheduler_form_flags_instead_of_synchronising(rt):
    locations, requests, positions, mapping, prefixes, lengths, _ = batch(7)
    args = lambda loc: (loc.to(DEV), requests.to(DEV), positions.to(DEV), mapping.to(DEV), prefixes, lengths, SLOTS,
                        None, 0)
    md = rt.PagedMetadata._from_scheduler(*args(locations))
    assert md.rows() == 7 and rt._C._take_device_status() == 0
    bad = locations.clone(); bad[2] = bad[1]                            # duplicate slot: checked even without the table
    rt.PagedMetadata._from_scheduler(*args(bad))                        # does not raise ...
    assert rt._C._take_device_status() == 8                             # ... the status word carries GK_DEV_BAD_METADATA
    assert rt._C._take_device_status() == 0


def test_attention_through_device_metadata_matches_host_metadata(rt):
    """Same step described twice -- host lists and device vectors -- gives bit-identical output."""
    heads, kv_heads, d = 8, 2, 128
    locations, requests, positions, mapping, prefixes, lengths, row_requests = batch(137)
    rows = 137
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(rows, heads * d, generator=gen).bfloat16()
    k = torch.randn(rows, kv_heads * d, generator=gen).bfloat16()
    v = torch.randn(rows, kv_heads * d, generator=gen).bfloat16()
    base_k = torch.randn(SLOTS, kv_heads, d, generator=gen).bfloat16()
    base_v = torch.randn(SLOTS, kv_heads, d, generator=gen).bfloat16()
    outs = []
    for form in ("host", "device"):
        pool = rt._C._allocate_paged_kv(1, SLOTS, kv_heads, d)
        key_pool, value_pool = pool[0, 0].transpose(0, 1), pool[0, 1].transpose(0, 1)
        key_pool.copy_(base_k); value_pool.copy_(base_v)
        if form == "host":
            md = rt.PagedMetadata(locations, row_requests, positions, mapping, SLOTS)
        else:
            md = build(rt, locations, requests, positions, mapping, prefixes, lengths)
        out = torch.ops.gaudirt.paged_attn(q.to(DEV), k.to(DEV), v.to(DEV), key_pool, value_pool, md, d, d ** -0.5)
        outs.append((out.cpu(), pool.cpu()))
    assert torch.equal(outs[0][0].view(torch.int16), outs[1][0].view(torch.int16))
    assert torch.equal(outs[0][1].view(torch.int16), outs[1][1].view(torch.int16))
    assert rt._C._take_device_status() == 0


def test_revalidation_refreshes_the_same_device_tensors_and_can_be_replayed_from_a_graph(rt):
    """`_revalidate_` checks new index vectors of a step of the same shape into the tensors the metadata (and a
    plan, and a captured graph) already refer to: launches only, so it is capturable; a bad vector is reported
    through the status word."""
    locations, requests, positions, mapping, prefixes, lengths, row_requests = batch(33)
    loc_d, req_d, pos_d = locations.to(DEV), requests.to(torch.int32).to(DEV), positions.to(DEV)
    md = rt.PagedMetadata.from_device(loc_d, req_d, pos_d, mapping.to(DEV), prefixes, lengths, SLOTS)
    held = md.row_locations()
    address = held.data_ptr()
    assert torch.equal(held.cpu().long(), locations)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        md._revalidate_(loc_d, req_d, pos_d)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            md._revalidate_(loc_d, req_d, pos_d)
    held.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert md.row_locations().data_ptr() == address and torch.equal(held.cpu().long(), locations)
    assert rt._C._take_device_status() == 0
    # the step's vectors change in place: a slot that is not the table's is reported on the next replay
    loc_d[5] += 1
    graph.replay()
    torch.cuda.synchronize()
    assert rt._C._take_device_status() == 8
    loc_d[5] -= 1
    graph.replay()
    torch.cuda.synchronize()
    assert rt._C._take_device_status() == 0 and torch.equal(held.cpu().long(), locations)
    with pytest.raises(RuntimeError, match="request vector"):
        md._revalidate_(loc_d, req_d.clone(), pos_d)
    host = rt.PagedMetadata(locations, row_requests, positions, mapping, SLOTS)
    with pytest.raises(RuntimeError, match="device-validated"):
        host._revalidate_(loc_d, req_d, pos_d)
