"""o_proj on the tensor cores, the rank-ordered sum and its fusion with the residual-add RMS norm.

The GEMM accumulates in fp32, so it is held against the binary64 product rounded once to bf16 with
an explicit error budget; exact cases (one-hot rows) and the sum kernels are bit-exact."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


def bits(t):
    return t.contiguous().view(torch.int16)


def gemm_gate(got, x, w):
    """|got - exact| <= half a bf16 ulp of the exact value (the final rounding) + the fp32 accumulation
    budget k * 2^-24 * sum|x||w|; and nearly all elements must equal the correctly rounded truth."""
    exact = x.double() @ w.double().t()
    ulp = torch.exp2(torch.floor(torch.log2(exact.abs().clamp_min(1e-30))) - 7)
    budget = 0.5 * ulp * (1 + 2 ** -6) + x.size(1) * 2.0 ** -24 * (x.double().abs() @ w.double().abs().t())
    error = (got.double() - exact).abs()
    assert bool((error <= budget).all()), float((error / budget).max())
    same = (bits(got) == bits(oracle.linear_bf16(x, w))).double().mean()
    assert same > 0.98, float(same)


# shapes chosen to reach every kernel variant: 256-, 128- and 64-wide blocks (the widest needs more output
# blocks than SMs: the last two shapes), one or two accumulators, and K cut over clusters of 1, 2 and 4 CTAs
# (few output blocks and many k-steps give the larger clusters)
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (64, 8192, 1024), (137, 256, 192), (256, 4096, 4096), (129, 128, 128),
                                   (300, 192, 320), (1000, 64, 704), (64, 128, 2048), (200, 256, 1024), (10, 512, 1024),
                                   (256, 8192, 1024), (77, 192, 4096), (256, 8192, 8192), (4001, 2048, 256),
                                   (100, 65536, 64)])
def test_oproj_against_binary64(rt, m, n, k):
    gen = torch.Generator().manual_seed(m * 7 + n + k)
    x = torch.randn(m, k, generator=gen).bfloat16()
    w = (torch.randn(n, k, generator=gen) / k ** 0.5).bfloat16()
    got = torch.ops.gaudirt._oproj(x.to(DEV), w.to(DEV))
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    gemm_gate(got.cpu(), x, w)
    again = torch.ops.gaudirt._oproj(x.to(DEV), w.to(DEV))
    assert torch.equal(bits(got), bits(again))
    assert rt._C._take_device_status() == 0


def test_oproj_one_hot_rows_select_weight_columns_exactly(rt):
    """Size-independent exact case at the TP-1 decode size: a one-hot input row copies a weight column."""
    m, n, k = 256, 8192, 8192
    gen = torch.Generator(device=DEV).manual_seed(3)
    w = torch.randn(n, k, generator=gen, device=DEV).bfloat16()
    pick = torch.randint(0, k, (m,), generator=gen, device=DEV)
    x = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV)
    x[torch.arange(m, device=DEV), pick] = -2.0
    got = torch.ops.gaudirt._oproj(x, w)
    # value comparison: a weight that is exactly zero gives +0 from the accumulator and -0 from -2 * 0
    assert torch.equal(got.float(), -2.0 * w[:, pick].t().float())
    # linear in the input: doubling is exact in bf16
    y = torch.randn(m, k, generator=gen, device=DEV).bfloat16()
    assert torch.equal(torch.ops.gaudirt._oproj(y * 2, w).float(), torch.ops.gaudirt._oproj(y, w).float() * 2)


def test_oproj_strided_operands_and_several_destinations(rt):
    gen = torch.Generator().manual_seed(9)
    wide_x = torch.randn(70, 3 * 256, generator=gen).bfloat16().to(DEV)
    wide_w = torch.randn(128, 2 * 256, generator=gen).bfloat16().to(DEV)
    x, w = wide_x[:, 256:512], wide_w[:, 256:]                      # column slices: row strides 768 and 512
    single = torch.ops.gaudirt._oproj(x, w)
    gemm_gate(single.cpu(), x.cpu(), w.cpu())
    slab = torch.full((3, 70, 200), 7.0, dtype=torch.bfloat16, device=DEV)
    torch.ops.gaudirt._oproj_push(x, w, [slab[i][:, 8:136] for i in range(3)])
    for i in range(3):
        assert torch.equal(bits(slab[i][:, 8:136]), bits(single))
        assert bool((slab[i][:, :8] == 7).all()) and bool((slab[i][:, 136:] == 7).all())   # neighbours untouched
    for bad_x, bad_w, text in ((x[:, :100], w[:, :100], "unsupported"), (x, w[:100], "unsupported"),
                               (x.float(), w, "BF16"), (x, w[:, :128], "BF16")):
        with pytest.raises(RuntimeError, match=text):
            torch.ops.gaudirt._oproj(bad_x, bad_w)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rank_sum_is_the_reference_order(rt, world):
    gen = torch.Generator().manual_seed(7000 + world)
    for count in (128, 384, 1536, 24576, 49152):
        parts = [(torch.randn(count, generator=gen) * 10 ** float(torch.randn((), generator=gen))).bfloat16()
                 for _ in range(world)]
        want = oracle.canonical_rank_sum(parts)
        got = torch.ops.gaudirt._rank_sum([p.to(DEV) for p in parts])
        assert torch.equal(bits(got.cpu()), bits(want))
    if world == 4:                                                   # an order that matters: big + small - big
        parts = [torch.full((8,), v).bfloat16() for v in (256.0, 1.0, 1.0, -256.0)]
        got = torch.ops.gaudirt._rank_sum([p.to(DEV) for p in parts])
        assert got.cpu().tolist() == oracle.canonical_rank_sum(parts).tolist() == [2.0] * 8


@pytest.mark.parametrize("world,rows,hidden", [(2, 5, 64), (8, 64, 8192), (4, 137, 4096)])
def test_rank_sum_fused_into_the_residual_add_norm(rt, world, rows, hidden):
    gen = torch.Generator().manual_seed(world * 100 + rows)
    parts = [torch.randn(rows, hidden, generator=gen).bfloat16() for _ in range(world)]
    residual = torch.randn(rows, hidden, generator=gen).bfloat16()
    gamma = (1 + 0.02 * torch.randn(hidden, generator=gen)).bfloat16()
    x = oracle.canonical_rank_sum(parts)
    want_y, want_u = oracle.fused_add_rms_norm(x, residual, gamma, 1e-5, 1.0, dtype=torch.float64)
    slab = torch.stack(parts).to(DEV)
    y, u = torch.ops.gaudirt._rank_sum_add_rms_norm(list(slab.unbind(0)), residual.to(DEV), gamma.to(DEV), 1e-5, 1.0)
    assert torch.equal(u.cpu().double(), want_u)                      # the updated residual is bit-exact
    assert float((y.cpu().double() != want_y).double().mean()) < 1e-3
    # the two-kernel route gives the same bits
    y2, u2 = torch.ops.gaudirt.fused_add_rms_norm(torch.ops.gaudirt._rank_sum(list(slab.unbind(0))), residual.to(DEV),
                                                  gamma.to(DEV), 1e-5, 1.0)
    assert torch.equal(bits(y), bits(y2)) and torch.equal(bits(u), bits(u2))
