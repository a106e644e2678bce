"""The CPU oracle against fixtures produced by the reference's own CPU code and against the
known-answer vectors the reference's tests carry."""
import os

import numpy as np
import pytest
import torch

import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def load(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


def attention_case(z, name):
    g = lambda k: z[f"{name}/{k}"]
    heads, kv_heads, d = int(g("heads")), int(g("kv_heads")), int(g("head_dim"))
    args = (bf16(g("q")), bf16(g("key_pool")), bf16(g("value_pool")), torch.from_numpy(g("requests")),
            torch.from_numpy(g("positions")), torch.from_numpy(g("mapping")), heads, kv_heads, d, float(g("scale")))
    return g, args


@pytest.mark.parametrize("name", ["gqa4_d64", "gqa8_d128", "mha_d64"])
def test_attention_matches_reference_cpu(name):
    g, args = attention_case(load("attention.npz"), name)
    assert torch.equal(oracle.direct_bf16_pv(*args), torch.from_numpy(g("direct_bf16_pv")))
    for tile in (2, 5, 16, 512):
        assert torch.equal(oracle.tiled_bf16_pv(*args, kv_tile=tile), torch.from_numpy(g(f"tiled_{tile}"))), tile
    u32 = oracle.attend_unrounded(*args, dtype=torch.float32)
    u64 = oracle.attend_unrounded(*args, dtype=torch.float64)
    assert torch.equal(u32, torch.from_numpy(g("unrounded32")))
    assert torch.equal(u64, torch.from_numpy(g("unrounded64")))
    assert torch.equal(oracle.attend_fp64_rounded(*args), torch.from_numpy(g("fp64_bf16")))
    # the gates hold between the reference's own arithmetic variants
    oracle.isolated_errors(oracle.direct_bf16_pv(*args), torch.from_numpy(g("fp64_bf16")),
                           torch.from_numpy(g("tiled_512")))
    oracle.fp32_softmax_gate(oracle.direct_bf16_pv(*args), oracle.attend_fp32_softmax(*args))


@pytest.mark.parametrize("name", ["softcap_swa", "swa_only", "softcap_only"])
def test_softcap_and_window_match_reference_cpu(name):
    z = load("softcap_window.npz")
    g, args = attention_case(z, name)
    got = oracle.attend_fp32_softmax(*args, softcap=float(g("softcap")), window=int(g("window")))
    assert torch.equal(got, bf16(g("out_bf16")).double())


def test_split_kv_combine_matches_tiled_reference():
    """tile_softmax + online_merge + online_finalize chained over arbitrary split points
    reproduce the reference's tiled arithmetic bit for bit when the splits are its tiles."""
    g, args = attention_case(load("attention.npz"), "gqa8_d128")
    positions = args[4]
    for tile in (5, 16):
        cuts = [list(range(0, int(p) + 1, tile)) + [int(p) + 1] for p in positions]
        cuts = [c if c[-1] != c[-2] else c[:-1] for c in cuts]
        got = oracle.split_kv_attend(*args, boundaries=cuts)
        ref = torch.from_numpy(g(f"tiled_{tile}"))
        # numpy and torch use different exp/sum kernels: allow one bf16 ulp on a few elements
        assert float((got - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())
        assert float(((got - ref) != 0).double().mean()) < 0.1


def test_merge_corner_cases():
    ninf = np.float32(-np.inf)
    m, l, o = oracle.online_merge([ninf], [0.0], [[7.0, 7.0]], [1.5], [2.0], [[1.0, 3.0]])
    assert m[0] == 1.5 and l[0] == 2.0 and np.array_equal(o, [[2.0, 6.0]])
    m, l, o = oracle.online_merge([ninf], [0.0], [[7.0]], [ninf], [0.0], [[9.0]])
    assert np.isneginf(m[0]) and l[0] == 0 and o[0, 0] == 0
    assert np.array_equal(oracle.online_finalize([0.0, 2.0], [[5.0], [3.0]]), [[0.0], [1.5]])
    m, l, o = oracle.online_merge([0.0], [2.0], [[0.5]], [0.0], [2.0], [[1.0]], prev_unscaled=True)
    assert l[0] == 4.0 and o[0, 0] == 3.0
    p, m, l = oracle.tile_softmax(np.zeros((1, 2, 4), np.float32), [1, -1], 2, 4, 0, 1.0)
    assert np.array_equal(p[0, 0], [0.5, 0.5, 0, 0]) and l[0, 1] == 0 and np.isneginf(m[0, 1])


def test_bf16_rounding_matches_reference():
    z = load("rounding.npz")
    x = torch.from_numpy(z["x"])
    assert torch.equal(oracle.bf16_from_f64(x), torch.from_numpy(z["direct_bf16"]))
    assert torch.equal(oracle.paged_oracle._round_bf16(x), torch.from_numpy(z["store_boundary64"]))
    assert torch.equal(oracle.paged_oracle._round_bf16(x.float()).double(), torch.from_numpy(z["store_boundary32"]))
    # tests/decoder_cpu_reference_test.py:66-68
    mid = torch.tensor([1 + 2 ** -8 + 2 ** -32], dtype=torch.float64)
    assert oracle.bf16_from_f64(mid).item() == 1 + 2 ** -7
    assert mid.float().bfloat16().double().item() == 1
    with pytest.raises(ValueError):
        oracle.bf16_from_f64(torch.tensor([float("nan")], dtype=torch.float64))


def test_norm_and_rotary_match_reference():
    z = load("norm_rotary.npz")
    x, res, gamma = bf16(z["norm_x"]), bf16(z["norm_res"]), bf16(z["norm_gamma"])
    for tag, dtype in (("32", torch.float32), ("64", torch.float64)):
        y, u = oracle.fused_add_rms_norm(x, res, gamma, float(z["epsilon"]), dtype=dtype)
        assert torch.equal(u, torch.from_numpy(z[f"norm_u_{tag}"]))
        assert torch.equal(y, torch.from_numpy(z[f"norm_y_{tag}"]))
    for tag in ("full", "partial"):
        heads, head_dim, rotary_dim = (int(v) for v in z[f"rot_{tag}_geom"])
        xin, cache, pos = bf16(z[f"rot_{tag}_x"]), bf16(z[f"rot_{tag}_cache"]), torch.from_numpy(z[f"rot_{tag}_pos"])
        for style, neox in (("neox", True), ("gptj", False)):
            for w, dtype in (("32", torch.float32), ("64", torch.float64)):
                got = oracle.rotary_embedding(xin, cache, pos, head_dim, rotary_dim, neox, dtype=dtype)
                assert torch.equal(got, torch.from_numpy(z[f"rot_{tag}_{style}_{w}"])), (tag, style, w)


def test_fused_norm_known_answer_vector():
    """The bit-exact midpoint vector of the reference's tests/fused_norm_midpoint_smoke.py:19-35."""
    def sample(hexs):
        return torch.frombuffer(bytearray.fromhex(hexs), dtype=torch.bfloat16).clone()
    x = sample("f2bf093dbb3f46be3a3f7b3f7a3e25bedb3f193ece3ef43ff73ec5bfdf3d8fbe"
               "42bfa73e5dbf553fa1bf0f3f33bf91bfb3bfef3fa6bfa73c893fb6be9b3f55bd"
               "d4bda0bfe53fe13e7b3fa83f0bbfe03f0f40753d0b3f3b3f05bdb03fe53ecb3f"
               "533fb03fb03f50be443f903e03bedfbd803fb83f7fbf14c0bfbf51beb83e7cbd")
    residual = sample("d1bf93bf14c0ee3e7d3d233f793f903f24bf47bf963ee43e103eccbf913fbe3e"
                      "3cbf08bf903dac3feebfef3bfd3e97bf1b3f243f7e3f97bf3bbf93bfa43ffe3f"
                      "fb3e3abe0000833fd4bec0be8cbea3bf84bf523f00004e3d55bf4b3e133f063f"
                      "253f053f72be4ebe353ef2bf2fbf69bfb6bebb3e133f673f3cbc3f3f18bf943d")
    gamma = sample("6d3f7f3f6d3f663f853f943f923f6d3f5a3f983f853f6c3f813f8b3f653f883f"
                   "813f813f823f6b3f7f3f643f653f723f933f703f913f7a3f8a3f543f683f743f"
                   "873f713f763f793f6d3f503f803f703f883f7d3f8e3f913f723f5f3f6e3f853f"
                   "763f823f893f763f653f803f883f7b3f963f6b3f903f723fa33f8a3f963f6f3f")
    y, u = oracle.fused_add_rms_norm(x[None], residual[None], gamma, 1e-6, dtype=torch.float64)
    assert y[0, 57].item() == 1.1796875
    assert torch.equal(u[0], oracle.bf16_from_f64(x.double() + residual.double()))


def test_tile_indices_known_answer():
    """Expected gather indices of the reference's tests/attention_plan_smoke.py:17-38."""
    requests, context, slots = 2, 32, 4096
    mapping = ((np.arange(requests)[:, None] * 256 + np.arange(context)[None, :]) % slots).astype(np.int32)
    row_requests = np.array([0] * 3 + [1] * 10)
    work = []
    for first_row, visible in ((0, 6), (3, 17)):
        for kind in range(2):
            for head in range(2):
                for key in (0, 64):
                    work.append((first_row, key, int(np.clip(visible - key, 0, 64)), (kind * 2 + head) * slots))
    got = oracle.tile_indices(mapping, row_requests, work, context).reshape(2, 2, 2, 128)
    for block, (request, visible) in enumerate(((0, 6), (1, 17))):
        for kind in range(2):
            for head in range(2):
                want = np.full(128, (kind * 2 + head) * slots, dtype=np.int32)
                want[:visible] += mapping[request, :visible]
                want[64:] = 0
                got_row = got[block, kind, head].copy()
                got_row[64:] -= (kind * 2 + head) * slots       # masked task: base + 0
                got_row[64:] = 0 if (got[block, kind, head, 64:] == (kind * 2 + head) * slots).all() else -1
                assert np.array_equal(got_row, want)


def test_kv_store_bits_and_untouched_slots():
    gen = torch.Generator().manual_seed(5)
    pool = torch.randn(2, 3, 20, 64, generator=gen).to(torch.bfloat16)
    before = pool.clone()
    k = torch.randn(4, 3 * 64, generator=gen).to(torch.bfloat16)
    v = torch.randn(4, 3 * 64, generator=gen).to(torch.bfloat16)
    loc = torch.tensor([7, 0, 19, 3], dtype=torch.int32)
    oracle.kv_store_head_major(pool, k, v, loc)
    kp, vp = oracle.pool_views(pool)
    expect_k, expect_v = oracle.pool_views(before.clone())
    expect_k, expect_v = expect_k.clone(), expect_v.clone()
    expect_k[loc.long()] = k.reshape(4, 3, 64)          # tests/paged_attention_smoke.py:82-84
    expect_v[loc.long()] = v.reshape(4, 3, 64)
    assert torch.equal(kp.view(torch.int16), expect_k.view(torch.int16))
    assert torch.equal(vp.view(torch.int16), expect_v.view(torch.int16))


def test_slot_allocator_known_answers():
    """tests/paged_slots_device_smoke.py:16-45."""
    for page in (16, 64):
        prefixes, lengths = [0, 7, page, 2 * page - 1], [19, 14, 20, 66]
        previous = [-1, 81 * page + 6, 82 * page + page - 1, 83 * page + page - 2]
        pages = [13, 7, 23, 41, 12, 33, 55, 61, 15, 18, 19, 20, 21, 22, 24, 25]
        slots, used = oracle.allocate_paged_slots(previous, pages, prefixes, lengths, page)
        want, taken = [], 0
        for prefix, length, last in zip(prefixes, lengths, previous):
            first_fresh = -(-prefix // page)                 # first page index this request must obtain
            for p in range(prefix, prefix + length):
                if p // page < first_fresh:                  # still inside the partly filled page
                    want.append(last + 1 + p - prefix)
                else:
                    want.append(pages[taken + p // page - first_fresh] * page + p % page)
            taken += max(0, -(-(prefix + length) // page) - first_fresh)
        assert slots == want and used == taken
        rel = [13 * page + 7, 7 * page, 13 * page, 23 * page + page - 1, 7 * page + 3]
        assert oracle.release_paged_slots(rel, page, 512) == [13, 7, 23]
        for bad in (0, 513 * page, 1 << 40):
            with pytest.raises(ValueError, match="outside the KV pool"):
                oracle.release_paged_slots([bad], page, 512)


def test_metadata_rules():
    mapping = np.arange(1, 1 + 3 * 8).reshape(3, 8)
    seqs = oracle.validate_paged_metadata([3, 4, 5, 12], [0, 0, 0, 1], [2, 3, 4, 3], mapping, 64)
    assert seqs == [(0, 3, 2), (3, 1, 3)]
    with pytest.raises(ValueError, match="does not match"):
        oracle.validate_paged_metadata([9], [0], [2], mapping, 64)
    with pytest.raises(ValueError, match="duplicate"):
        oracle.validate_paged_metadata([3, 3], [0, 0], [2, 2], mapping, 64)
    with pytest.raises(ValueError, match="out of range"):
        oracle.validate_paged_metadata([3], [0], [9], mapping, 64)
    holes = mapping.copy(); holes[0, 1] = -1
    with pytest.raises(ValueError, match="missing KV slot"):
        oracle.validate_paged_metadata([3], [0], [2], holes, 64)
    alias = mapping.copy(); alias[1, 0] = 3
    with pytest.raises(ValueError, match="aliases"):
        oracle.validate_paged_metadata([3, 12], [0, 1], [2, 3], alias, 64)


def test_bitmask_and_rank_sum_match_the_reference_functions():
    """`after_attention.npz` holds inputs and outputs of the reference's own `ref_apply_bitmask` and
    `_canonical_rank_sum`; the oracle's restatements reproduce them bit for bit."""
    z = load("after_attention.npz")
    names = sorted({k[len("mask_"):-len("_logits")] for k in z.files if k.startswith("mask_") and k.endswith("_logits")})
    assert len(names) == 7
    for name in names:
        is_bf16 = name.startswith("bf16")
        tensor = (lambda a: bf16(a)) if is_bf16 else (lambda a: torch.from_numpy(a.view(np.float32).copy()))
        raw = (lambda t: t.contiguous().view(torch.int16)) if is_bf16 else (lambda t: t.contiguous().view(torch.int32))
        args = z[f"mask_{name}_args"]
        indices = torch.from_numpy(args[2:].astype(np.int32)) if len(args) > 2 else None
        got = oracle.apply_vocab_bitmask(tensor(z[f"mask_{name}_logits"]), torch.from_numpy(z[f"mask_{name}_mask"]),
                                         indices, int(args[0]), bool(args[1]))
        assert torch.equal(raw(got), raw(tensor(z[f"mask_{name}_out"]))), name
    for world in (1, 2, 4, 8):
        parts = [bf16(row) for row in z[f"sum_{world}_parts"]]
        want = bf16(z[f"sum_{world}_out"])
        assert torch.equal(oracle.canonical_rank_sum(parts).view(torch.int16), want.view(torch.int16)), world
