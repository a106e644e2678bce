"""After the LM head: vocabulary argmax, grammar bitmask and sampling -- the scenarios of the
reference's device tests (tests/vocabulary_argmax_smoke.py, tests/vocab_bitmask_device_smoke.py,
tests/sampler_vocab_device_smoke.py) against torch's CPU argmax, the oracle's bitmask rule
(bit-exact) and, for sampling, the support and distribution properties the reference checks."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt():
    import gaudirt_b200
    return gaudirt_b200


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax_ties_and_nonfinite_values(rt, dtype):
    gen = torch.Generator().manual_seed(962)
    for width in (1, 3, 127, 128, 129, 4099, 65537, 176131):
        values = torch.randn(8, width, generator=gen).to(dtype)
        values[0].fill_(-float("inf"))
        values[1].fill_(float("inf"))
        values[2].fill_(0)
        values[2, 0] = -0.0
        if width > 1:
            values[3, 0] = float("inf")
            values[3, width // 2] = float("nan")
            values[4, width - 1] = float("nan")
            values[6].fill_(-100)
            values[6, width // 7] = values[6, width - 1] = 100
            values[7, width // 4] = values[7, width - 1] = float("nan")
        got = torch.ops.gaudirt._vocabulary_argmax(values.to(DEV))
        assert got.dtype == torch.int64 and torch.equal(got.cpu(), torch.argmax(values, dim=-1)), (dtype, width)
    wide = torch.randn(5, 300, generator=gen).to(dtype).to(DEV)          # a column slice: strided rows
    assert torch.equal(torch.ops.gaudirt._vocabulary_argmax(wide[:, 7:207]).cpu(), torch.argmax(wide[:, 7:207].cpu(), -1))


def make_bitmask(rows, words, allowed_lists):
    mask = torch.zeros(rows, words, dtype=torch.int32)
    for r, allowed in enumerate(allowed_lists):
        if allowed is None:
            mask[r].fill_(-1)
        else:
            for token in allowed:
                mask[r, token >> 5] |= (1 << (token & 31)) - (1 << 32 if (token & 31) == 31 else 0)
    return mask


def same_bits(a, b):
    return torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bitmask_matches_the_reference_rule(rt, dtype):
    gen = torch.Generator().manual_seed(5)
    apply = torch.ops.gaudirt.apply_token_bitmask_inplace_
    for batch, vocab in ((1, 35), (3, 1025), (13, 49152), (5, 166912)):
        words = (vocab + 31) // 32
        logits = (torch.randn(batch, vocab, generator=gen) * 3).to(dtype)
        allowed = [None if r % 3 == 0 else [0, 31 % vocab, 32 % vocab, vocab - 1] for r in range(batch)]
        mask = make_bitmask(batch, words, allowed)
        want = oracle.apply_vocab_bitmask(logits, mask)
        for mask_in in (mask.to(DEV), mask):                          # device mask, and a host mask uploaded by the op
            device_logits = logits.to(DEV)
            returned = apply(device_logits, mask_in)
            assert returned.data_ptr() == device_logits.data_ptr() and same_bits(device_logits.cpu(), want)
    random_mask = torch.randint(-2 ** 31, 2 ** 31 - 1, (7, 40), generator=gen, dtype=torch.int64).to(torch.int32)
    logits = torch.randn(7, 1271, generator=gen).to(dtype)             # 1271 < 40 * 32: last word partly used
    device_logits = logits.to(DEV)
    apply(device_logits, random_mask.to(DEV))
    assert same_bits(device_logits.cpu(), oracle.apply_vocab_bitmask(logits, random_mask))
    assert rt._C._take_device_status() == 0


def test_bitmask_tail_views_indices_and_errors(rt):
    apply = torch.ops.gaudirt.apply_token_bitmask_inplace_
    for mask_tail in (False, True):
        logits = torch.linspace(-2.0, 2.0, 80).to(torch.bfloat16).reshape(2, 40)
        mask = torch.tensor([[0b101], [-1]], dtype=torch.int32)         # covers 32 of 40 columns
        device_logits = logits.to(DEV)
        apply(device_logits, mask.to(DEV), None, -1, mask_tail)
        assert same_bits(device_logits.cpu(), oracle.apply_vocab_bitmask(logits, mask, mask_tail=mask_tail))
    one_d = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]).to(DEV)
    apply(one_d, torch.tensor([0b10101], dtype=torch.int32))
    assert torch.equal(one_d.cpu(), torch.tensor([1.0, float("-inf"), 3.0, float("-inf"), 5.0]))
    storage = torch.full((3, 192), 77.0, dtype=torch.bfloat16)
    storage[:, :130] = torch.randn(3, 130).to(torch.bfloat16)
    device_storage = storage.clone().to(DEV)
    mask = make_bitmask(3, (130 + 31) // 32, [[1, 65], None, [129]])
    apply(device_storage[:, :130], mask.to(DEV))
    after = device_storage.cpu()
    assert torch.equal(after[:, 130:], storage[:, 130:]), "neighbouring columns were touched"
    assert same_bits(after[:, :130], oracle.apply_vocab_bitmask(storage[:, :130], mask))
    logits = torch.arange(4 * 64, dtype=torch.float32).reshape(4, 64)
    mask = make_bitmask(4, 2, [None, [3], [5, 63], [1]])
    for indices in (torch.tensor([2, 0, 2], dtype=torch.int32), torch.tensor([2, 0, 2]).to(DEV)):
        device_logits = logits.to(DEV)
        apply(device_logits, mask, indices)
        assert torch.equal(device_logits.cpu(), oracle.apply_vocab_bitmask(logits, mask, indices=indices.cpu()))
    with pytest.raises(RuntimeError, match="smaller than vocab_size"):
        apply(torch.zeros(2, 40, dtype=torch.bfloat16, device=DEV), torch.full((2, 1), -1, dtype=torch.int32), None, 40, False)
    with pytest.raises(RuntimeError, match="out of bounds"):
        apply(logits.to(DEV), mask, torch.tensor([4]))
    with pytest.raises(RuntimeError, match="must match logits batch"):
        apply(logits.to(DEV), mask[:3])
    apply(logits.to(DEV), mask, torch.tensor([9]).to(DEV))             # a bad index on the device is skipped and flagged
    assert rt._C._take_device_status() == 8 and rt._C._take_device_status() == 0


def scenario(vocab, dtype):
    logits = torch.full((8, vocab), -20.0, dtype=dtype)
    logits[0, 5], logits[0, 17] = 4.0, 9.0                             # greedy
    logits[1, 3] = logits[1, 100] = 7.0                                # tied greedy: lowest index
    logits[2, 11] = logits[2, 22] = 10.0                               # top_k = 2 -> {11, 22}
    logits[2, 33] = 9.0
    logits[3, 42], logits[3, 43] = 12.0, 2.0                           # top_p = 0.5 with a dominant token
    logits[4, 77], logits[4, 78] = 10.0, 8.0                           # min_p = 0.5 leaves only 77
    logits[5, 0] = logits[5, 9] = float("nan")                         # NaN is never selected
    logits[5, 51] = 5.0
    logits[6, :8] = torch.linspace(1.0, 2.0, 8).to(dtype)
    logits[7, :8] = torch.linspace(2.0, 1.0, 8).to(dtype)
    temps = torch.tensor([0.0, 0.0, 1.0, 1.0, 1.0, 0.0, 0.9, 1.2])
    top_ps = torch.tensor([1.0, 1.0, 1.0, 0.5, 1.0, 1.0, 0.95, 1.0])
    top_ks = torch.tensor([vocab, vocab, 2, vocab, vocab, vocab, 6, 4], dtype=torch.int32)
    min_ps = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.5, 0.0, 0.0, 0.1])
    return logits, temps, top_ps, top_ks, min_ps


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("vocab", [127, 4099, 131072])
def test_sampler_scenarios_of_the_reference(rt, dtype, vocab):
    sample = torch.ops.gaudirt.sample_from_logits
    logits, temps, top_ps, top_ks, min_ps = scenario(vocab, dtype)
    args = [t.to(DEV) for t in (logits, temps, top_ps, top_ks, min_ps)]
    seeds = torch.full((8,), 1234567, dtype=torch.int64, device=DEV)
    positions = torch.arange(8, dtype=torch.int64, device=DEV)
    first = sample(*args, seeds, positions, True).cpu()
    assert first.dtype == torch.int32 and torch.equal(first, sample(*args, seeds, positions, True).cpu())
    assert first[0] == 17 and first[1] == 3 and first[2] in (11, 22) and first[3] == 42 and first[4] == 77 and first[5] == 51
    assert 2 <= first[6] < 8 and 0 <= first[7] < 4
    supports = [set(oracle.sampling_support(logits[r], float(temps[r]), float(top_ps[r]), int(top_ks[r]), float(min_ps[r]))[0]
                    .tolist()) for r in range(8)]
    assert supports[2] == {11, 22} and supports[4] == {77} and supports[6] == set(range(2, 8)) and supports[7] == set(range(4))
    seen = [set() for _ in range(8)]
    for step in range(40):
        tokens = sample(*args, seeds, positions + (step + 1) * 10, True).cpu().tolist()
        for r, token in enumerate(tokens):
            assert token in supports[r], (r, token)
            seen[r].add(token)
    assert seen[2] == {11, 22} and len(seen[6]) >= 4 and len(seen[7]) >= 3   # draws do move with the position


def test_sampler_distribution_and_parameter_shapes(rt):
    sample = torch.ops.gaudirt.sample_from_logits
    vocab, batch = 512, 64
    weights = torch.tensor([3.0, 2.2, 1.5, 0.8, 0.2])
    row = torch.full((vocab,), -50.0)
    row[:5] = weights
    logits = row.expand(batch, vocab).contiguous().to(DEV)
    ones, zeros = torch.ones(1, device=DEV), torch.zeros(batch, 1, device=DEV)    # broadcast and [batch, 1] forms
    counts = torch.zeros(5)
    for r in range(32):
        seeds = torch.full((batch,), 9000 + r, dtype=torch.int64, device=DEV)
        tokens = sample(logits, ones, ones, torch.tensor([vocab], dtype=torch.int32), zeros, seeds,
                        torch.arange(batch, dtype=torch.int32, device=DEV), True).cpu()
        assert bool(((tokens >= 0) & (tokens < 5)).all())
        counts += torch.bincount(tokens.long(), minlength=5).float()
    tvd = 0.5 * float((counts / counts.sum() - torch.softmax(weights, -1)).abs().sum())
    assert tvd < 0.035, tvd
    # unseeded calls differ from call to call, seeds without positions are accepted
    a = sample(logits, ones, ones, torch.tensor([vocab], dtype=torch.int32), zeros).cpu()
    b = sample(logits, ones, ones, torch.tensor([vocab], dtype=torch.int32), zeros).cpu()
    assert not torch.equal(a, b) and bool((a < 5).all())
    sample(logits, ones, ones, torch.tensor([vocab], dtype=torch.int32), zeros, torch.arange(batch, device=DEV))
    with pytest.raises(RuntimeError, match="unexpected dtype for top_ks"):
        sample(logits, ones, ones, torch.tensor([vocab]), zeros)
    with pytest.raises(RuntimeError, match="invalid shape for temperatures"):
        sample(logits, torch.ones(3, device=DEV), ones, torch.tensor([vocab], dtype=torch.int32), zeros)


def test_sampler_support_on_random_rows_and_with_a_grammar_mask(rt):
    sample = torch.ops.gaudirt.sample_from_logits
    gen = torch.Generator().manual_seed(77)
    batch, vocab = 24, 50257
    logits = (torch.randn(batch, vocab, generator=gen) * 2.5).to(torch.bfloat16)
    temps = torch.rand(batch, generator=gen) * 1.5 + 0.3
    top_ps = torch.tensor([1.0, 0.9, 0.5] * 8)
    # 50 / 5 / 1 are found among the bf16 values just below the maximum; vocab - 7 and 30000 lie far down, where the
    # kernel has to take its general selection path
    top_ks = torch.tensor([vocab, 50, 5, 1, vocab - 7, 30000] * 4, dtype=torch.int32)
    min_ps = torch.tensor([0.0, 0.02] * 12)
    args = [t.to(DEV) for t in (logits, temps, top_ps, top_ks, min_ps)]
    # random logits leave every threshold far (in fp32 terms) from the nearest weight, so the binary64 support is exact
    supports = [set(oracle.sampling_support(logits[r], float(temps[r]), float(top_ps[r]), int(top_ks[r]), float(min_ps[r]))[0]
                    .tolist()) for r in range(batch)]
    assert all(1 <= len(supports[r]) <= 3 for r in range(3, batch, 6))   # top_k = 1 (ties at the top stay)
    seeds = torch.arange(batch, dtype=torch.int64, device=DEV) * 7919
    for step in range(25):
        tokens = sample(*args, seeds, torch.full((batch,), step, dtype=torch.int64, device=DEV), True).cpu().tolist()
        for r, token in enumerate(tokens):
            assert token in supports[r], (r, token, step)
    masked = torch.full((4, 1025), 5.0, dtype=torch.bfloat16).to(DEV)
    torch.ops.gaudirt.apply_token_bitmask_inplace_(masked, make_bitmask(4, 33, [[17], [1024], [31, 32], None]).to(DEV))
    tokens = sample(masked, torch.tensor([0.0, 0.8, 1.0, 0.0]), torch.tensor([1.0, 0.9, 0.95, 1.0]),
                    torch.full((4,), 1025, dtype=torch.int32), torch.zeros(4), torch.full((4,), 42), torch.arange(4), True).cpu()
    assert tokens[0] == 17 and tokens[1] == 1024 and tokens[2] in (31, 32) and tokens[3] == 0
