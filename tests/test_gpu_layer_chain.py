"""The fused decode layer step as one chain through the operators, at the full per-GPU shape of the
tensor-parallel configuration: fused_add_rms_norm (hidden 8192, eps 1e-5, weight_offset 1.0) -> rotary
(theta 500000, positions = the new token's position) -> head-major KV store -> paged GQA decode with
8 query heads on 1 KV head, batch 64, contexts uniform in [1024, 16384].

Layer order of the reference: tests/frozen_same_geometry_layer_smoke.py:22-37 (norm, rotary, paged
attention with its store).  Each link is held to its own gate: the residual boundary and the rotated
rows bit for bit, the pool bit for bit over every slot, attention within the fp32-softmax tolerance
and the reference's relative-L2 gates.  Both launch sequences are run: rotary, then store + attention;
and rotary fused with the store, then attention alone -- they must agree bit for bit."""
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


def test_fused_decode_layer_step_chain_matches_the_oracle_chain(rt):
    batch, q_heads, kv_heads, d, hidden, theta = 64, 8, 1, 128, 8192, 500000.0
    gen = torch.Generator().manual_seed(20261105)
    ctx = torch.randint(1024, 16385, (batch,), generator=gen)
    blocks = int(((ctx + 127) // 128).sum()) + 8
    case = cases.decode_case(batch, q_heads, kv_heads, d, 128, blocks, ctx, seed=20261105)
    x = torch.randn(batch, hidden, generator=gen).bfloat16()
    residual = torch.randn(batch, hidden, generator=gen).bfloat16()
    gamma = (0.02 * torch.randn(hidden, generator=gen)).bfloat16()                 # applied as 1 + gamma
    cache = oracle.rotary_cache(case.mapping.size(1), d, theta)          # one row per position of the request table

    # ---- oracle chain ------------------------------------------------------------------------
    want_y, want_u = oracle.fused_add_rms_norm(x, residual, gamma, 1e-5, 1.0, dtype=torch.float64)
    want_q = oracle.rotary_embedding(case.q, cache, case.positions, d, d, True, dtype=torch.float64)
    want_k = oracle.rotary_embedding(case.k, cache, case.positions, d, d, True, dtype=torch.float64)
    ref_pool = case.pool.clone()
    oracle.kv_store_head_major(ref_pool, want_k.to(torch.bfloat16), case.v, case.locations)
    kp, vp = oracle.pool_views(ref_pool)
    args = (want_q.to(torch.bfloat16), kp, vp, case.requests, case.positions, case.mapping, q_heads, kv_heads, d, case.scale)
    ref32 = oracle.attend_fp32_softmax(*args)
    ref64 = oracle.attend_fp64_rounded(*args)
    tiled = oracle.tiled_bf16_pv(*args, kv_tile=oracle.KV_TILE)

    # ---- the operators, two launch sequences ---------------------------------------------------
    md = rt.PagedMetadata(case.locations, case.requests, case.positions, case.mapping, case.slots)
    xd, rd, gd, cd = x.to(DEV), residual.to(DEV), gamma.to(DEV), cache.to(DEV)
    qd, kd, vd = case.q.to(DEV), case.k.to(DEV), case.v.to(DEV)
    y, u = torch.ops.gaudirt.fused_add_rms_norm(xd, rd, gd, 1e-5, 1.0)
    assert torch.equal(u.cpu().double(), want_u), "updated residual is a bit-exact boundary"
    assert float((y.cpu().double() != want_y).double().mean()) < 1e-3
    outs = []
    for fused in (False, True):
        pool = case.pool.to(DEV)
        key_pool, value_pool = pool[0].transpose(0, 1), pool[1].transpose(0, 1)
        if fused:
            q_rot = torch.ops.gaudirt._rotary_kv_store(qd, kd, vd, cd, md, key_pool, value_pool, d, d, True)
            out = torch.ops.gaudirt._paged_attn_stored(q_rot, key_pool, value_pool, md, d, case.scale)
        else:
            q_rot, k_rot = torch.ops.gaudirt.rotary_embedding(qd, kd, cd, md, d, d, True)
            assert torch.equal(k_rot.cpu().double(), want_k)
            out = torch.ops.gaudirt.paged_attn(q_rot, k_rot, vd, key_pool, value_pool, md, d, case.scale)
        assert torch.equal(q_rot.cpu().double(), want_q), "rotated rows are rounded once from the exact value"
        assert torch.equal(bits(pool.cpu()), bits(ref_pool)), "whole pool, every slot"
        got = out.cpu().double()
        oracle.fp32_softmax_gate(got, ref32)
        oracle.isolated_errors(got, ref64, tiled)
        outs.append(out)
    assert torch.equal(bits(outs[0]), bits(outs[1]))
    assert rt._C._take_device_status() == 0
