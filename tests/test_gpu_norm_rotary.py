"""fused_add_rms_norm / rms_norm / rotary on the GPU against the oracle, the reference's fixtures
and its known-answer vector (tests/fused_norm_midpoint_smoke.py, tests/fused_add_rms_fx_smoke.py,
tests/rotary_runtime_smoke.py of the reference)."""
import os

import numpy as np
import pytest
import torch

import oracle
from gaudirt_b200 import abi
from gaudirt_b200 import raw as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def b16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def rel_l2(actual, truth):
    return float((torch.linalg.vector_norm(actual - truth, dim=-1) /
                  torch.linalg.vector_norm(truth, dim=-1).clamp_min(1e-30)).max())


def sample(hexs):
    return torch.frombuffer(bytearray.fromhex(hexs), dtype=torch.bfloat16).clone()


MID_X = ("f2bf093dbb3f46be3a3f7b3f7a3e25bedb3f193ece3ef43ff73ec5bfdf3d8fbe"
         "42bfa73e5dbf553fa1bf0f3f33bf91bfb3bfef3fa6bfa73c893fb6be9b3f55bd"
         "d4bda0bfe53fe13e7b3fa83f0bbfe03f0f40753d0b3f3b3f05bdb03fe53ecb3f"
         "533fb03fb03f50be443f903e03bedfbd803fb83f7fbf14c0bfbf51beb83e7cbd")
MID_R = ("d1bf93bf14c0ee3e7d3d233f793f903f24bf47bf963ee43e103eccbf913fbe3e"
         "3cbf08bf903dac3feebfef3bfd3e97bf1b3f243f7e3f97bf3bbf93bfa43ffe3f"
         "fb3e3abe0000833fd4bec0be8cbea3bf84bf523f00004e3d55bf4b3e133f063f"
         "253f053f72be4ebe353ef2bf2fbf69bfb6bebb3e133f673f3cbc3f3f18bf943d")
MID_G = ("6d3f7f3f6d3f663f853f943f923f6d3f5a3f983f853f6c3f813f8b3f653f883f"
         "813f813f823f6b3f7f3f643f653f723f933f703f913f7a3f8a3f543f683f743f"
         "873f713f763f793f6d3f503f803f703f883f7d3f8e3f913f723f5f3f6e3f853f"
         "763f823f893f763f653f803f883f7b3f963f6b3f903f723fa33f8a3f963f6f3f")


def test_fused_norm_midpoint_known_answer(rt):
    x, residual, gamma = sample(MID_X), sample(MID_R), sample(MID_G)
    boundary = oracle.bf16_from_f64(x.double() + residual.double())
    eps = torch.tensor(1e-6, dtype=torch.float32).item()
    truth = oracle.bf16_from_f64(boundary * torch.rsqrt((boundary * boundary).mean() + eps) * gamma.double())
    assert truth[57] == 1.1796875
    for rows in (1, 137):
        norm, updated = torch.ops.gaudirt.fused_add_rms_norm(x.repeat(rows, 1).to(DEV), residual.repeat(rows, 1).to(DEV),
                                                             gamma.to(DEV), 1e-6)
        plain = torch.ops.gaudirt.rms_norm(updated, gamma.to(DEV), 1e-6)
        assert torch.equal(updated.cpu().double(), boundary.expand(rows, -1))
        assert torch.equal(norm.cpu().double(), truth.expand(rows, -1))
        assert torch.equal(plain.cpu().double(), truth.expand(rows, -1))


def test_norm_reference_fixture(rt):
    z = np.load(os.path.join(GOLDEN, "norm_rotary.npz"))
    x, res, gamma = b16(z["norm_x"]), b16(z["norm_res"]), b16(z["norm_gamma"])
    y, u = torch.ops.gaudirt.fused_add_rms_norm(x.to(DEV), res.to(DEV), gamma.to(DEV), float(z["epsilon"]))
    assert torch.equal(u.cpu().double(), torch.from_numpy(z["norm_u_64"])), "residual boundary is bit-exact"
    assert torch.equal(u.cpu().double(), torch.from_numpy(z["norm_u_32"]))
    truth = torch.from_numpy(z["norm_y_64"])
    floor = rel_l2(torch.from_numpy(z["norm_y_32"]), truth)
    err = rel_l2(y.cpu().double(), truth)
    assert err <= max(3e-3, 2 * floor) and err <= 1e-2                 # the reference's gate
    assert float((y.cpu().double() != truth).double().mean()) < 0.01    # in fact (almost) the fp64 truth itself


@pytest.mark.parametrize("rows,hidden,offset", [(1, 64, 0.0), (17, 64, 0.0), (137, 7168, 0.0), (64, 8192, 1.0),
                                                (1025, 7168, 0.0), (5, 100, 0.5), (3, 8192, 0.0)])
def test_fused_norm_against_oracle(rt, rows, hidden, offset):
    gen = torch.Generator().manual_seed(713 + rows + hidden)
    x, res = (torch.randn(rows, hidden, generator=gen).to(torch.bfloat16) for _ in range(2))
    if offset:
        gamma = (0.02 * torch.randn(hidden, generator=gen)).to(torch.bfloat16)       # config 5: w + 1
    else:
        gamma = (torch.randn(hidden, generator=gen) * 0.1 + 1).to(torch.bfloat16)
    y, u = torch.ops.gaudirt.fused_add_rms_norm(x.to(DEV), res.to(DEV), gamma.to(DEV), 1e-5, offset)
    assert y.shape == x.shape and y.is_contiguous() and u.is_contiguous()
    y64, u64 = oracle.fused_add_rms_norm(x, res, gamma, 1e-5, offset, dtype=torch.float64)
    y32, _ = oracle.fused_add_rms_norm(x, res, gamma, 1e-5, offset, dtype=torch.float32)
    assert torch.equal(u.cpu().double(), u64)
    err, floor = rel_l2(y.cpu().double(), y64), rel_l2(y32, y64)
    assert err <= max(3e-3, 2 * floor) and err <= 1e-2
    assert float((y.cpu().double() != y64).double().mean()) < 1e-3
    plain = torch.ops.gaudirt.rms_norm(u, gamma.to(DEV), 1e-5, offset)
    assert torch.equal(plain.view(torch.int16), y.view(torch.int16))
    # 3-D input and a strided (column-sliced) input take the same arithmetic
    if rows % 2 == 0 and hidden % 8 == 0:
        y3, u3 = torch.ops.gaudirt.fused_add_rms_norm(x.to(DEV).view(2, rows // 2, hidden), res.to(DEV).view(2, rows // 2, hidden),
                                                      gamma.to(DEV), 1e-5, offset)
        assert y3.shape == (2, rows // 2, hidden) and torch.equal(y3.view(rows, hidden).view(torch.int16), y.view(torch.int16))
    wide = torch.zeros(rows, hidden + 3, dtype=torch.bfloat16, device=DEV)
    wide[:, 3:] = x.to(DEV)
    ys, us = torch.ops.gaudirt.fused_add_rms_norm(wide[:, 3:], res.to(DEV), gamma.to(DEV), 1e-5, offset)
    assert torch.equal(ys.view(torch.int16), y.view(torch.int16)) and torch.equal(us.view(torch.int16), u.view(torch.int16))


def test_norm_rejects_bad_arguments(rt):
    x = torch.zeros(7, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="epsilon"):
        torch.ops.gaudirt.fused_add_rms_norm(x, x, w, 0.0)
    with pytest.raises(RuntimeError, match="geometry"):
        torch.ops.gaudirt.rms_norm(x, w[:32], 1e-6)
    with pytest.raises(RuntimeError, match="geometry"):
        torch.ops.gaudirt.rms_norm(torch.zeros(2, 8200, dtype=torch.bfloat16, device=DEV),
                                   torch.ones(8200, dtype=torch.bfloat16, device=DEV), 1e-6)
    empty = torch.ops.gaudirt.rms_norm(x[:0], w, 1e-6)
    assert empty.shape == (0, 64)


def test_rotary_reference_fixture(rt):
    z = np.load(os.path.join(GOLDEN, "norm_rotary.npz"))
    for tag in ("full", "partial"):
        heads, head_dim, rotary_dim = (int(v) for v in z[f"rot_{tag}_geom"])
        xin, cache, pos = b16(z[f"rot_{tag}_x"]), b16(z[f"rot_{tag}_cache"]), torch.from_numpy(z[f"rot_{tag}_pos"])
        for style, neox in (("neox", True), ("gptj", False)):
            q_out, k_out = torch.ops.gaudirt.rotary_embedding_positions(xin.to(DEV), xin.to(DEV), cache.to(DEV), pos.to(DEV),
                                                                        head_dim, rotary_dim, neox)
            truth = torch.from_numpy(z[f"rot_{tag}_{style}_64"])
            assert torch.equal(q_out.cpu().double(), truth), (tag, style)      # exact: fp64 is exact here
            assert torch.equal(k_out.cpu().double(), truth)


@pytest.mark.parametrize("q_heads,k_heads,head_dim,rotary_dim,rows", [(56, 8, 128, 128, 1), (56, 8, 128, 128, 137),
                                                                      (56, 8, 128, 128, 1025), (4, 2, 96, 62, 7),
                                                                      (8, 1, 128, 128, 64)])
@pytest.mark.parametrize("neox", [True, False])
def test_rotary_with_metadata(rt, q_heads, k_heads, head_dim, rotary_dim, rows, neox):
    gen = torch.Generator().manual_seed(1403 + rows)
    n_req, context = 64, 64
    slots = n_req * context + 1
    mapping = torch.arange(1, slots, dtype=torch.int32).reshape(n_req, context)
    requests = torch.arange(rows, dtype=torch.int64) % n_req
    positions = torch.arange(rows, dtype=torch.int64) // n_req + 3
    md = rt.PagedMetadata(mapping[requests, positions].to(torch.int64), requests, positions, mapping, slots)
    cache = torch.randn(context, rotary_dim, generator=gen).to(torch.bfloat16)
    q = torch.randn(rows, q_heads * head_dim, generator=gen).to(torch.bfloat16)
    k = torch.randn(rows, k_heads * head_dim, generator=gen).to(torch.bfloat16)
    if rows == 137:                                      # one-element offset views
        qs = torch.zeros(rows, q.size(1) + 1, dtype=torch.bfloat16, device=DEV); qs[:, 1:] = q.to(DEV)
        ks = torch.zeros(rows, k.size(1) + 1, dtype=torch.bfloat16, device=DEV); ks[:, 1:] = k.to(DEV)
        qd, kd = qs[:, 1:], ks[:, 1:]
    else:
        qd, kd = q.to(DEV), k.to(DEV)
    q_out, k_out = torch.ops.gaudirt.rotary_embedding(qd, kd, cache.to(DEV), md, head_dim, rotary_dim, neox)
    for got, src in ((q_out, q), (k_out, k)):
        assert got.shape == src.shape and got.is_contiguous()
        truth = oracle.rotary_embedding(src, cache, positions, head_dim, rotary_dim, neox, dtype=torch.float64)
        assert torch.equal(got.cpu().double(), truth)
    if rows == 7 and neox:
        with pytest.raises(RuntimeError, match="cache"):
            torch.ops.gaudirt.rotary_embedding(qd, kd, cache[:32].to(DEV), md, head_dim, rotary_dim, neox)
        with pytest.raises(RuntimeError, match="rotary dimension"):
            torch.ops.gaudirt.rotary_embedding(qd, kd, cache.to(DEV), md, head_dim, rotary_dim - 1, neox)


def _hard_rotation_cases(count, seed=20261125):
    """bf16 quadruples (a, b, cos, sin) for which a*cos - b*sin is inexact in fp32 and its fp32
    truncation lies exactly on a bf16 rounding midpoint: rounding that truncation instead of the
    exact value (a double rounding) gives the wrong bf16.  Both signs of the result are collected."""
    rng = np.random.default_rng(seed)

    def random_bf16(n):
        x = (rng.standard_normal(n) * rng.choice([0.01, 0.3, 1.0, 7.0], n)).astype(np.float32)
        u = x.view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).view(np.float32)

    found = [np.empty((0, 4), np.float32)] * 2                       # [non-negative results, negative results]
    while min(len(f) for f in found) < count:
        a, b, c, s = (random_bf16(1 << 20) for _ in range(4))
        exact = a.astype(np.float64) * c - b.astype(np.float64) * s   # exact in binary64
        near = exact.astype(np.float32)
        trunc = np.where(np.abs(near.astype(np.float64)) > np.abs(exact), np.nextafter(near, np.float32(0)), near)
        hard = (trunc.astype(np.float64) != exact) & ((trunc.view(np.uint32) & 0xFFFF) == 0x8000)
        for sign in (0, 1):
            pick = hard & ((exact < 0) == bool(sign))
            found[sign] = np.concatenate([found[sign], np.stack([a, b, c, s], 1)[pick]])
    return np.concatenate([found[0][:count], found[1][:count]])


def test_rotary_rounds_the_exact_value_for_both_signs(rt):
    """Known hard inputs: the rotated element must be the rounding of the exact value, also when the
    result is negative (directed roundings toward zero and toward +inf coincide there)."""
    cases = _hard_rotation_cases(16)                                  # 32 quadruples, 4 per row
    rows = len(cases) // 4
    a, b, c, s = (torch.from_numpy(np.ascontiguousarray(cases[:, i])).view(rows, 4).to(torch.bfloat16) for i in range(4))
    x = torch.cat([a, b], dim=1)                                      # neox pairs (i, i + 4) of one head of width 8
    cache = torch.cat([c, s], dim=1)                                  # row r of the table: cos || sin
    positions = torch.arange(rows, dtype=torch.int32)
    truth = oracle.rotary_embedding(x, cache, positions, 8, 8, True, dtype=torch.float64)
    want_first = oracle.bf16_from_f64(a.double() * c.double() - b.double() * s.double())
    assert torch.equal(truth[:, :4], want_first)
    naive = (a.float() * c.float() - b.float() * s.float()).to(torch.bfloat16).double()   # fp32 then bf16: double rounding
    assert int((naive != want_first).sum()) >= 8, "the cases are meant to break a double rounding"
    q_out, k_out = torch.ops.gaudirt.rotary_embedding_positions(x.to(DEV), x.to(DEV), cache.to(DEV), positions.to(DEV), 8, 8, True)
    assert torch.equal(q_out.cpu().double(), truth) and torch.equal(k_out.cpu().double(), truth)
    wide = torch.cat([x] * 16, dim=1)                                 # 16 heads: the 16-byte vector kernel
    q_out, _ = torch.ops.gaudirt.rotary_embedding_positions(wide.to(DEV), x.to(DEV), cache.to(DEV), positions.to(DEV), 8, 8, True)
    assert torch.equal(q_out.cpu().double(), torch.cat([truth] * 16, dim=1))


def test_rotary_fused_with_kv_store_matches_the_two_kernels():
    gen = torch.Generator().manual_seed(5150)
    rows, q_heads, k_heads, d, slots = 64, 8, 1, 128, 4096
    cache = oracle.rotary_cache(2048, d, 500000.0)
    pos = torch.randint(0, 2048, (rows,), generator=gen).to(torch.int32)
    loc = torch.randperm(slots, generator=gen)[:rows].to(torch.int32)
    q, k, v = (torch.randn(rows, h * d, generator=gen).to(torch.bfloat16).to(DEV) for h in (q_heads, k_heads, k_heads))
    pool_a = torch.randn(2, k_heads, slots, d, generator=gen).to(torch.bfloat16).to(DEV)
    pool_b = pool_a.clone()
    lib, s = abi.lib(), H.stream_ptr()
    q1, k1 = torch.empty_like(q), torch.empty_like(k)
    abi.check(lib.gk_rotary_bf16(q.data_ptr(), k.data_ptr(), q.stride(0), k.stride(0), cache.to(DEV).data_ptr(), 2048,
                                 pos.to(DEV).data_ptr(), rows, q.size(1), k.size(1), d, d, 1, q1.data_ptr(), k1.data_ptr(),
                                 None, s), "rotary")
    H.kv_store(pool_a, k1, v, loc.to(DEV))
    q2 = torch.empty_like(q)
    cache_d, pos_d, loc_d = cache.to(DEV), pos.to(DEV), loc.to(DEV)
    abi.check(lib.gk_rotary_kv_store_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                          cache_d.data_ptr(), 2048, pos_d.data_ptr(), loc_d.data_ptr(), rows, q.size(1),
                                          k.size(1), d, d, 1, q2.data_ptr(), None, pool_b[0].data_ptr(), pool_b[1].data_ptr(),
                                          slots, None, s), "rotary+store")
    torch.cuda.synchronize()
    assert torch.equal(q1.view(torch.int16), q2.view(torch.int16))
    assert torch.equal(pool_a.view(torch.int16), pool_b.view(torch.int16))
    truth = oracle.rotary_embedding(k.cpu(), cache, pos, d, d, True, dtype=torch.float64)
    assert torch.equal(k1.cpu().double(), truth)


def test_rotary_out_of_table_position_is_reported(rt):
    q = torch.ones(2, 64, dtype=torch.bfloat16, device=DEV)
    cache = torch.ones(4, 64, dtype=torch.bfloat16, device=DEV)
    rt._C._take_device_status()
    q_out, _ = torch.ops.gaudirt.rotary_embedding_positions(q, q, cache, torch.tensor([1, 9], device=DEV), 64, 64, True)
    assert rt._C._take_device_status() == 1
    assert torch.equal(q_out[1], q[1])
