"""CPU restatement of the reference's paged KV-store + paged-attention arithmetic.

Test infrastructure (see the package docstring).  All citations are
``path:line`` inside the reference project (tracycam/GaudiRT).

Conventions shared by every function below
------------------------------------------
* ``pool``            combined KV pool ``[2, kv_heads, slots, head_dim]`` bf16
                      (``src/bridge/paged_kv_pool.cpp:15-41``); ``pool[0]`` holds keys.
* ``key_pool`` view   ``pool[0].transpose(0, 1)`` -> ``[slots, kv_heads, head_dim]``
                      (``tests/paged_attention_smoke.py:70-72``).
* ``mapping``         int ``[requests, context]``; ``mapping[r, p]`` is the slot that holds
                      position ``p`` of request ``r`` (``src/bridge/paged_metadata.cpp:104-140``).
* a block table is that same function sampled once per block:
  ``slot(seq, p) = block_table[seq, p // block] * block + p % block``
  (page rule of ``tests/paged_attention_generalized_smoke.py:148``).
"""
from __future__ import annotations

import math

import numpy as np
import torch

__all__ = [
    "KV_TILE", "bf16_from_f64", "kv_store_head_major", "pool_views", "mapping_from_block_tables",
    "attend_unrounded", "attend_fp32_softmax", "attend_fp64_rounded", "direct_bf16_pv", "tiled_bf16_pv",
    "isolated_errors", "fp32_softmax_gate", "tile_indices", "tile_softmax", "online_merge",
    "online_finalize", "split_kv_attend", "rms_norm", "fused_add_rms_norm", "rotary_embedding",
    "rotary_cache", "validate_paged_metadata", "allocate_paged_slots", "release_paged_slots",
    "device_metadata_status", "gather_dim_last", "linear_bf16", "canonical_rank_sum", "apply_vocab_bitmask",
    "sampling_support",
]

# KV tile of the reference's multi-tile path (src/bridge/paged_metadata.hpp:15, exposed to
# the independent references through _C._paged_attn_kv_tile, generic_private_use1.cpp).
KV_TILE = 512


# --------------------------------------------------------------------------------------
# rounding
# --------------------------------------------------------------------------------------
def bf16_from_f64(values: torch.Tensor) -> torch.Tensor:
    """Round binary64 straight to bf16 (nearest, ties to even) and return it as float64.

    Same contract as ``tests/fp64_reference.py:7-31`` (no intermediate fp32 rounding, so a
    value like ``1 + 2**-8 + 2**-32`` goes up, ``tests/decoder_cpu_reference_test.py:66-68``);
    written with frexp/rint instead of bit fields.  Non-finite input is an error there and here.
    """
    data = np.asarray(values.detach().cpu().numpy(), dtype=np.float64)
    if not np.isfinite(data).all():
        raise ValueError("nonfinite FP64 reference")
    mag = np.abs(data)
    _, exponent = np.frexp(mag)                     # mag = m * 2**exponent, m in [0.5, 1)
    # bf16 keeps 8 significant bits; below 2**-126 the spacing is fixed at 2**-133.
    quantum_exp = np.maximum(exponent - 8, -133)
    rounded = np.ldexp(np.rint(np.ldexp(mag, -quantum_exp)), quantum_exp)
    rounded = np.where(rounded >= 2.0 ** 128, np.inf, rounded)
    return torch.from_numpy(np.copysign(rounded, data)).reshape(values.shape)


def _round_bf16(x: torch.Tensor) -> torch.Tensor:
    """The rounding each arithmetic width uses at a bf16 boundary (decoder_cpu_reference.py:54-56)."""
    if x.dtype == torch.float64:
        return bf16_from_f64(x)
    return x.to(torch.bfloat16).to(x.dtype)


# --------------------------------------------------------------------------------------
# pool + KV store
# --------------------------------------------------------------------------------------
def pool_views(pool_layer: torch.Tensor):
    """``[2, kv_heads, slots, d]`` -> the two ``[slots, kv_heads, d]`` strided views the op takes."""
    assert pool_layer.dim() == 4 and pool_layer.size(0) == 2
    return pool_layer[0].transpose(0, 1), pool_layer[1].transpose(0, 1)


def kv_store_head_major(pool_layer: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                        locations: torch.Tensor) -> None:
    """gk_kv_store_head_major_bf16_v1, in place on ``pool_layer [2, kv_heads, slots, d]``.

    ``pool[(h*slots + loc[r])*d ...] = K[r, h*d ...]`` and the same for V at head index
    ``kv_heads + h`` (CPU statement: ``tests/multitile_paged_attention_unit_test.cpp:455-478``;
    operator-level audit ``tests/paged_attention_smoke.py:82-87``).  A pure 16-bit copy: the
    payload is never interpreted, every other slot keeps its bits.  Rows are applied in order.
    """
    _, kv_heads, slots, d = pool_layer.shape
    rows = key.size(0)
    assert key.shape == (rows, kv_heads * d) and value.shape == key.shape
    loc = locations.to(torch.int64).reshape(rows)
    assert int(loc.min()) >= 0 and int(loc.max()) < slots
    bits = pool_layer.view(torch.int16)
    kb = key.contiguous().view(torch.int16).reshape(rows, kv_heads, d)
    vb = value.contiguous().view(torch.int16).reshape(rows, kv_heads, d)
    for r in range(rows):        # sequential: a later duplicate slot wins, as in the reference loop
        bits[0, :, loc[r]] = kb[r]
        bits[1, :, loc[r]] = vb[r]


def mapping_from_block_tables(block_tables: torch.Tensor, block: int, context: int) -> torch.Tensor:
    """Tabulate ``slot(seq, p)`` for ``p < context`` from ``block_tables [seqs, blocks]`` (int32)."""
    pos = torch.arange(context, dtype=torch.int64)
    table = block_tables.to(torch.int64)
    return (table[:, pos // block] * block + pos % block).to(torch.int32)


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
def _row_operands(row, query, key_pool, value_pool, requests, positions, mapping, heads, kv_heads,
                  head_dim, window, dtype):
    pos = int(positions[row])
    left = 0 if window <= 0 else max(0, pos - window + 1)
    slots = mapping[int(requests[row]), left:pos + 1].to(torch.int64)
    assert slots.numel() > 0
    head_of = torch.arange(heads) // (heads // kv_heads)
    q = query[row].reshape(heads, head_dim).to(dtype)
    k = key_pool[slots].to(dtype)[:, head_of]
    v = value_pool[slots].to(dtype)[:, head_of]
    return q, k, v


def _scores(q, k, scale, softcap):
    s = torch.einsum("hd,thd->ht", q, k) * scale
    if softcap > 0.0:
        s = softcap * torch.tanh(s / softcap)
    return s


def attend_unrounded(query, key_pool, value_pool, requests, positions, mapping, heads, kv_heads,
                     head_dim, scale, softcap=0.0, window=-1, dtype=torch.float32):
    """Exact-softmax attention in ``dtype`` without any bf16 boundary: ``[rows, heads*d]``.

    Restates ``expected_unrounded`` (``tests/paged_attention_smoke.py:38-49``): each row attends
    to ``mapping[request, :position+1]``, query head ``h`` reads KV head ``h // group``; with the
    softcap ``c*tanh(s/c)`` and sliding window ``[pos-window+1, pos]`` of
    ``tests/paged_attention_generalized_smoke.py:16-37``.  ``scale`` is used as given (callers
    pass the fp32-rounded scale, ``paged_attention_smoke.py:24``).
    """
    assert heads % kv_heads == 0
    out = []
    for row in range(query.size(0)):
        q, k, v = _row_operands(row, query, key_pool, value_pool, requests, positions, mapping,
                                heads, kv_heads, head_dim, window, dtype)
        p = torch.softmax(_scores(q, k, scale, softcap), dim=-1)
        out.append(torch.einsum("ht,thd->hd", p, v).reshape(-1))
    return torch.stack(out)


def attend_fp32_softmax(*args, **kwargs):
    """fp32 softmax, fp32 accumulation, one bf16 rounding of the result; returned as float64."""
    return attend_unrounded(*args, dtype=torch.float32, **kwargs).to(torch.bfloat16).double()


def attend_fp64_rounded(*args, **kwargs):
    """Binary64 attention rounded straight to bf16 (``paged_attention_smoke.py:52-55``)."""
    return bf16_from_f64(attend_unrounded(*args, dtype=torch.float64, **kwargs))


def direct_bf16_pv(query, key_pool, value_pool, requests, positions, mapping, heads, kv_heads,
                   head_dim, scale, softcap=0.0, window=-1):
    """Single-tile device arithmetic: fp32 scores/softmax, probabilities rounded to bf16, fp32 PV.

    Restates ``tests/paged_attention_reference.py:6-20`` (the rounding of P before the second
    product is the ``fused_recipe`` boundary, ``src/bridge/paged_attention.cpp:101-121``).
    """
    out = []
    for row in range(query.size(0)):
        q, k, v = _row_operands(row, query, key_pool, value_pool, requests, positions, mapping,
                                heads, kv_heads, head_dim, window, torch.float32)
        p = torch.softmax(_scores(q, k, scale, softcap), dim=-1).to(torch.bfloat16).float()
        out.append(torch.einsum("ht,thd->hd", p, v).reshape(-1))
    return torch.stack(out).to(torch.bfloat16).double()


def tiled_bf16_pv(query, key_pool, value_pool, requests, positions, mapping, heads, kv_heads,
                  head_dim, scale, kv_tile=KV_TILE, softcap=0.0, window=-1):
    """Multi-tile device arithmetic (``tests/paged_attention_reference.py:23-58``).

    Per ``kv_tile`` keys: in-tile softmax normalised and rounded to bf16, fp32 ``o_t = P_t V_t``,
    then the running ``(m, l, o)`` merge of ``gk_attn_online_merge_f32_v1`` where the first
    tile's output is carried scaled by its sum, and a final division by ``l``.
    """
    assert kv_tile > 0
    out = []
    for row in range(query.size(0)):
        q, k, v = _row_operands(row, query, key_pool, value_pool, requests, positions, mapping,
                                heads, kv_heads, head_dim, window, torch.float32)
        m_run = l_run = o_run = None
        for first in range(0, k.size(0), kv_tile):
            # scores are formed tile by tile, as the device does (a whole-row product sliced
            # afterwards can differ in the last fp32 bit)
            st = _scores(q, k[first:first + kv_tile], scale, softcap)
            m_t = st.amax(dim=-1)
            e_t = torch.exp(st - m_t[:, None])
            l_t = e_t.sum(dim=-1)
            p_t = (e_t / l_t[:, None]).to(torch.bfloat16).float()
            o_t = torch.einsum("ht,thd->hd", p_t, v[first:first + kv_tile])
            if m_run is None:
                m_run, l_run, o_run = m_t, l_t, o_t * l_t[:, None]
                continue
            m_new = torch.maximum(m_run, m_t)
            a, b = torch.exp(m_run - m_new), torch.exp(m_t - m_new)
            o_run = o_run * a[:, None] + o_t * (b * l_t)[:, None]
            l_run = l_run * a + l_t * b
            m_run = m_new
        out.append((o_run / l_run[:, None]).reshape(-1))
    return torch.stack(out).to(torch.bfloat16).double()


def isolated_errors(actual, fp64, tiled, gate64=1e-2, gate_tiled=5e-3):
    """The reference's operator gate (``tests/paged_attention_reference.py:60-69``).

    Worst row-relative L2 error against the fp64->bf16 truth (<= 1e-2) and against the tiled
    bf16-PV arithmetic (<= 5e-3); every operand must be finite.  Returns both errors.
    """
    assert actual.shape == fp64.shape == tiled.shape and actual.ndim >= 2
    mats = [t.double().reshape(t.size(0), -1) for t in (actual, fp64, tiled)]
    assert all(bool(torch.isfinite(m).all()) for m in mats)
    a, t64, tt = mats

    def worst(ref):
        return float((torch.linalg.vector_norm(a - ref, dim=-1) /
                      torch.linalg.vector_norm(ref, dim=-1).clamp_min(1e-30)).max())

    e64, et = worst(t64), worst(tt)
    assert e64 <= gate64 and et <= gate_tiled, (e64, et)
    return e64, et


def fp32_softmax_gate(actual, ref32, max_abs=2e-2, mean_abs=2e-3):
    """Attention acceptance gate of this build: max-abs <= 2e-2 and mean-abs <= 2e-3 against the
    fp32-softmax / fp32-accumulate result."""
    diff = (actual.double() - ref32.double()).abs()
    assert bool(torch.isfinite(actual.double()).all())
    worst, mean = float(diff.max()), float(diff.mean())
    assert worst <= max_abs and mean <= mean_abs, (worst, mean)
    return worst, mean


# --------------------------------------------------------------------------------------
# the device kernels of the multi-tile path, one by one (unit-test interpreter semantics)
# --------------------------------------------------------------------------------------
def tile_indices(mapping, requests, work, context):
    """gk_attn_tile_indices_i32_v1 (``tests/multitile_paged_attention_unit_test.cpp:431-454``).

    ``work [tasks, 4] = (first_row, first_key, lanes, base)`` ->
    ``out[t, l] = base + (mapping[requests[first_row]*context + first_key + l] if l < lanes else 0)``.
    """
    flat = np.asarray(mapping, dtype=np.int64).reshape(-1)
    req = np.asarray(requests, dtype=np.int64)
    work = np.asarray(work, dtype=np.int64).reshape(-1, 4)
    out = np.zeros((work.shape[0], 64), dtype=np.int32)
    lane = np.arange(64)
    for t, (first_row, first_key, lanes, base) in enumerate(work):
        live = lane < lanes
        src = req[first_row] * context + first_key + lane[live]
        out[t, live] = flat[src]
        out[t] += base
    return out


def tile_softmax(scores, positions, valid_rows, valid_keys, key_start, scale):
    """gk_attn_tile_softmax_bf16_v1 (``multitile_paged_attention_unit_test.cpp:628-683``).

    ``scores [heads, rows, keys]`` fp32.  Row ``r`` sees keys ``k <= min(pos[r]-key_start,
    valid_keys-1)``; returns ``(P bf16-rounded float32, m, l)``; a fully masked or invalid row
    gives ``m=-inf, l=0, P=0``.
    """
    s = np.asarray(scores, dtype=np.float32)
    heads, rows, keys = s.shape
    p = np.zeros_like(s)
    m = np.full((heads, rows), -np.inf, dtype=np.float32)
    l = np.zeros((heads, rows), dtype=np.float32)
    for r in range(min(rows, valid_rows)):
        last = min(int(positions[r]) - key_start, valid_keys - 1)
        if last < 0:
            continue
        z = s[:, r, :last + 1] * np.float32(scale)
        m[:, r] = z.max(axis=-1)
        e = np.exp(z - m[:, r, None], dtype=np.float32)
        l[:, r] = e.sum(axis=-1, dtype=np.float32)
        p[:, r, :last + 1] = e / l[:, r, None]
    p = torch.from_numpy(p).to(torch.bfloat16).float().numpy()
    return p, m, l


def online_merge(m0, l0, o0, m1, l1, o1, prev_unscaled=False):
    """gk_attn_online_merge_f32_v1 (``multitile_paged_attention_unit_test.cpp:684-722``).

    Sides with ``l == 0`` contribute nothing; with ``prev_unscaled`` the left output is still
    normalised inside its tile and is weighted by ``a*l0`` instead of ``a``.
    """
    m0, l0, m1, l1 = (np.asarray(x, dtype=np.float32) for x in (m0, l0, m1, l1))
    o0, o1 = np.asarray(o0, dtype=np.float32), np.asarray(o1, dtype=np.float32)
    v0 = np.where(l0 > 0, m0, -np.inf)
    v1 = np.where(l1 > 0, m1, -np.inf)
    m = np.maximum(v0, v1)
    origin = np.where(np.isinf(m), np.float32(0), m)
    with np.errstate(invalid="ignore", over="ignore"):
        a = np.where(l0 > 0, np.exp(m0 - origin, dtype=np.float32), np.float32(0))
        b = np.where(l1 > 0, np.exp(m1 - origin, dtype=np.float32), np.float32(0))
    wa = a * l0 if prev_unscaled else a
    wb = b * l1
    return m.astype(np.float32), (a * l0 + b * l1).astype(np.float32), wa[..., None] * o0 + wb[..., None] * o1


def online_finalize(l, o):
    """gk_attn_online_finalize_bf16_v1 (``multitile_paged_attention_unit_test.cpp:723-738``):
    ``bf16(o / l)``, zero where ``l == 0``; returned as float32 holding bf16 values."""
    l = np.asarray(l, dtype=np.float32)
    inv = np.where(l > 0, np.float32(1) / np.where(l > 0, l, np.float32(1)), np.float32(0))
    out = np.asarray(o, dtype=np.float32) * inv[..., None]
    return torch.from_numpy(out).to(torch.bfloat16).float().numpy()


def split_kv_attend(query, key_pool, value_pool, requests, positions, mapping, heads, kv_heads,
                    head_dim, scale, boundaries):
    """Split-KV attention built only from ``tile_softmax`` / ``online_merge`` / ``online_finalize``.

    ``boundaries[row]`` lists the split points ``[0, b1, ..., ctx]`` of that row's keys.  This is
    the combine the CUDA split-KV schedule must reproduce within tolerance; it is exact about
    the corner cases (empty splits, ``l == 0``).
    """
    rows = query.size(0)
    out = np.zeros((rows, heads * head_dim), dtype=np.float32)
    for row in range(rows):
        q, k, v = _row_operands(row, query, key_pool, value_pool, requests, positions, mapping,
                                heads, kv_heads, head_dim, -1, torch.float32)
        raw = torch.einsum("hd,thd->ht", q, k).numpy()[:, None, :]          # [heads, 1, keys]
        cuts = list(boundaries[row])
        state = None
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            width = max(hi - lo, 1)
            tile = np.zeros((heads, 1, width), dtype=np.float32)
            tile[:, :, :hi - lo] = raw[:, :, lo:hi]
            p, m, l = tile_softmax(tile, [int(positions[row])], 1, hi - lo, lo, scale)
            o = np.einsum("ht,thd->hd", p[:, 0, :hi - lo], v[lo:hi].numpy())[:, None, :]
            if state is None:
                state, unscaled = (m, l, o), True
            else:
                state, unscaled = online_merge(*state, m, l, o, prev_unscaled=unscaled), False
        m, l, o = state
        if unscaled:                      # a single split: o is already normalised in-tile
            o = o * l[..., None]
        out[row] = online_finalize(l, o).reshape(-1)
    return torch.from_numpy(out).double()


# --------------------------------------------------------------------------------------
# front of a decode layer: fused residual-add RMS norm, rotary
# --------------------------------------------------------------------------------------
def rms_norm(x, weight, epsilon, weight_offset=0.0, dtype=torch.float32):
    """gk_rms_norm_bf16_v1: ``bf16(x * rsqrt(mean(x^2) + eps) * (w + offset))``.

    Arithmetic of ``tests/fused_add_rms_fx_smoke.py:26-33`` (epsilon taken at fp32 precision).
    ``weight_offset`` is added to the weight before the product: no reference test pins a
    non-zero offset, the Gemma convention is assumed.
    """
    eps = float(torch.tensor(epsilon, dtype=torch.float32))
    xd = x.to(dtype)
    w = weight.to(dtype) + weight_offset
    y = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps) * w
    return _round_bf16(y).double()


def fused_add_rms_norm(x, residual, weight, epsilon, weight_offset=0.0, dtype=torch.float32):
    """gk_fused_add_rms_norm_bf16_v1 -> ``(norm, updated_residual)`` as float64.

    ``u = bf16(x + residual)`` is a real bf16 boundary (bit-exact in the reference,
    ``tests/fused_add_rms_fx_smoke.py:49-50``), the norm is then taken of ``u``
    (``tests/fused_norm_midpoint_smoke.py:32-35``).
    """
    u = _round_bf16(x.to(dtype) + residual.to(dtype))
    return rms_norm(u, weight, epsilon, weight_offset, dtype), u.double()


def rotary_cache(positions: int, rotary_dim: int, theta: float) -> torch.Tensor:
    """``[positions, rotary_dim]`` bf16 table ``cos || sin`` of ``pos * theta**(-2i/rotary_dim)``."""
    inv = theta ** (-torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cat((ang.cos(), ang.sin()), dim=-1).to(torch.float32).to(torch.bfloat16)


def rotary_embedding(x, cache, positions, head_dim, rotary_dim, is_neox, dtype=torch.float32):
    """gk_rotary_bf16_v1 on one of q/k (``tests/rotary_runtime_smoke.py:28-40``).

    ``cache[pos] = cos || sin`` (bf16); neox pairs element ``i`` with ``i + rotary_dim/2``,
    otherwise pairs are interleaved; each product-sum is rounded once to bf16; elements past
    ``rotary_dim`` are copied.
    """
    rows = x.size(0)
    v = x.to(dtype).reshape(rows, -1, head_dim)
    table = cache.to(dtype)[positions.to(torch.int64)]
    cos, sin = table[:, None, :rotary_dim // 2], table[:, None, rotary_dim // 2:]
    rot, rest = v[..., :rotary_dim], v[..., rotary_dim:]
    if is_neox:
        a, b = rot[..., :rotary_dim // 2], rot[..., rotary_dim // 2:]
    else:
        a, b = rot[..., 0::2], rot[..., 1::2]
    first = _round_bf16(a * cos - b * sin).to(dtype)
    second = _round_bf16(b * cos + a * sin).to(dtype)
    if is_neox:
        rot = torch.cat((first, second), dim=-1)
    else:
        rot = torch.stack((first, second), dim=-1).flatten(-2)
    return torch.cat((rot, rest), dim=-1).reshape(x.shape).double()


# --------------------------------------------------------------------------------------
# host-side metadata rules
# --------------------------------------------------------------------------------------
def validate_paged_metadata(locations, requests, positions, mapping, slots):
    """Host checks of the ``PagedMetadata`` constructor (``src/bridge/paged_metadata.cpp:82-140``).

    Returns the sequences ``[(row, length, prefix)]`` (maximal runs of one request with
    consecutive positions) or raises ``ValueError`` with the reference's message.
    """
    loc = [int(v) for v in locations]
    req = [int(v) for v in requests]
    pos = [int(v) for v in positions]
    table = np.asarray(mapping, dtype=np.int64)
    if not (len(loc) == len(req) == len(pos)) or table.ndim != 2:
        raise ValueError("GaudiRT: invalid paged metadata ranks or row counts")
    n_req, context = table.shape
    if len(loc) == 0 or slots <= 0 or n_req == 0 or context == 0:
        raise ValueError("GaudiRT: paged metadata dimensions outside supported range")
    if ((table < -1) | (table >= slots)).any():
        raise ValueError("GaudiRT: request-to-token slot is out of range")
    targets, sequences, reach = {}, [], [-1] * n_req
    for i, (s, r, p) in enumerate(zip(loc, req, pos)):
        if not (0 <= s < slots and 0 <= r < n_req and 0 <= p < context):
            raise ValueError("GaudiRT: paged metadata index is out of range")
        if table[r, p] != s:
            raise ValueError("GaudiRT: output slot does not match request-to-token mapping")
        if s in targets:
            raise ValueError("GaudiRT: duplicate output KV slot")
        targets[s] = (r, p)
        if i and req[i - 1] == r and pos[i - 1] + 1 == p:
            row, length, prefix = sequences[-1]
            sequences[-1] = (row, length + 1, prefix)
        else:
            sequences.append((i, 1, p))
        reach[r] = max(reach[r], p)
    for r in range(n_req):
        for p in range(reach[r] + 1):
            s = int(table[r, p])
            if s < 0:
                raise ValueError("GaudiRT: missing KV slot in a visible prefix")
            if s in targets and targets[s] != (r, p):
                raise ValueError("GaudiRT: output KV slot aliases another visible prefix position")
    return sequences


def allocate_paged_slots(last_slots, free_pages, prefixes, lengths, page_size):
    """Slot allocation rule (``src/bridge/paged_slot_allocator.cpp:91-151``; expected values in
    ``tests/paged_slots_device_smoke.py:22-29``): finish the partly filled last page after
    ``last_slots[i]`` first, then take fresh pages in order.  Returns ``(slots, pages_used)``."""
    out, used = [], 0
    for last, prefix, length in zip(last_slots, prefixes, lengths):
        tail = min(length, (-prefix) % page_size)
        out.extend(int(last) + 1 + i for i in range(tail))
        fresh = length - tail
        out.extend(int(free_pages[used + i // page_size]) * page_size + i % page_size
                   for i in range(fresh))
        used += -(-fresh // page_size)
    return out, used


def release_paged_slots(slots, page_size, max_pages):
    """Slots -> pages, first occurrence order, duplicates dropped
    (``src/bridge/paged_slot_allocator.cpp:153-190``, ``tests/paged_slots_device_smoke.py:34-45``)."""
    seen, pages = set(), []
    for s in slots:
        s = int(s)
        if s <= 0 or s >= max_pages * page_size:
            raise ValueError("GaudiRT: released slot is outside the KV pool")
        page = s // page_size
        if page not in seen:
            seen.add(page)
            pages.append(page)
    return pages


def device_metadata_status(locations, batch_requests, positions, mapping, prefixes, lengths, slots,
                           check_table=True):
    """Row codes of the device-input metadata form (``src/bridge/paged_metadata.cpp:176-430``; the
    validating kernel itself is not part of the reference tree, so the numbering is pinned by what
    ``tests/paged_device_metadata_smoke.py:130-150`` observes -- 1 out-of-range slot or position,
    2 out-of-range request, 3 slot differs from the table, 4 duplicate slot, 6 bad visible table
    entry, 7 cached prefix aliases a slot written this step -- and 5, position not equal to
    prefix + offset, is this build's own number for the one rule the test does not exercise).
    Returns ``(codes per row, last row index per sequence)``; a duplicate is charged to the later
    row, 6 and 7 to the first row of the sequence."""
    n_req, context = len(mapping), len(mapping[0])
    codes, last, written, row = [], [], set(), 0
    firsts = []
    for b, (prefix, length) in enumerate(zip(prefixes, lengths)):
        firsts.append(row)
        request = int(batch_requests[b])
        for i in range(length):
            slot, position = int(locations[row]), int(positions[row])
            if not (0 <= slot < slots and 0 <= position < context):
                code = 1
            elif not 0 <= request < n_req:
                code = 2
            elif position != prefix + i:
                code = 5
            elif check_table and int(mapping[request][position]) != slot:
                code = 3
            elif slot in written:
                code = 4
            else:
                code = 0
                written.add(slot)
            codes.append(code)
            row += 1
        last.append(row - 1)
    if check_table:
        for b, (prefix, length) in enumerate(zip(prefixes, lengths)):
            request = int(batch_requests[b])
            if not 0 <= request < n_req:
                continue
            worst = 0
            for p in range(prefix + length):
                slot = int(mapping[request][p])
                if not 0 <= slot < slots:
                    worst = 6
                    break
                if p < prefix and slot in written:
                    worst = worst or 7
            if worst and codes[firsts[b]] == 0:
                codes[firsts[b]] = worst
    return codes, last


def gather_dim_last(shards):
    """AllGatherDimLast (``src/bridge/segmented_runner.cpp:170-191``): rank-major concatenation of
    ``[B, cols]`` shards along the last dimension."""
    return torch.cat(list(shards), dim=-1)


def linear_bf16(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``bf16(x @ weight.T)`` with the product evaluated in binary64 and rounded once: the truth an
    fp32-accumulating tensor-core GEMM is held against (it may differ in the last bf16 bit where the
    fp32 sum lands on the other side of a rounding boundary)."""
    exact = x.double() @ weight.double().t()
    return bf16_from_f64(exact).to(torch.bfloat16)


def canonical_rank_sum(tensors):
    """The reference's all-reduce result (``tests/tp4_gather_reduce_smoke.py:16-20``, device rule
    ``src/bridge/communicator.cpp:373-417``): fp32 accumulator seeded with rank 0, the other ranks
    added in rank order with one fp32 rounding each, one final rounding to the input dtype."""
    total = None
    for part in tensors:
        total = part.to(torch.float32) if total is None else total + part.to(torch.float32)
    return total.to(tensors[0].dtype)


def apply_vocab_bitmask(logits, bitmask, indices=None, vocab_size=-1, mask_tail=False):
    """Grammar bitmask (rule of ``tests/vocab_bitmask_device_smoke.py:14-33``): in every listed row,
    column ``c < active`` becomes ``-inf`` when bit ``c & 31`` of word ``c >> 5`` of the row's mask is
    clear, columns ``>= active`` become ``-inf`` only with ``mask_tail``; ``active`` is the smaller of
    the mask's bit count and ``vocab_size`` (the logits width when negative).  Returns a new tensor."""
    out = logits.clone()
    work = out.view(1, -1) if out.dim() == 1 else out
    masks = bitmask.view(1, -1) if bitmask.dim() == 1 else bitmask
    cols = work.size(1)
    active = min(cols if vocab_size < 0 else vocab_size, masks.size(1) * 32)
    column = torch.arange(cols)
    rows = range(work.size(0)) if indices is None else sorted({int(i) for i in indices.reshape(-1).tolist()})
    for r in rows:
        words = masks[r].to(torch.int64) & 0xFFFFFFFF
        allowed = (words[(column.clamp(max=max(active, 1) - 1)) >> 5] >> (column & 31)) & 1
        banned = torch.where(column < active, allowed == 0, torch.full((cols,), bool(mask_tail)))
        work[r, banned] = float("-inf")
    return out


def sampling_support(row, temperature, top_p, top_k, min_p, nan_to_neg_inf=True):
    """Tokens a draw may return for one row under this build's sampling rule (the reference's
    sampling kernel is not in its tree; its test, ``tests/sampler_vocab_device_smoke.py:24-88``,
    pins the support in a few scenarios and the distribution, not the algorithm): with
    ``w = exp((x - max) / temperature)``, keep ``w >=`` the ``top_k``-th largest, of those the
    smallest high-``w`` set (ties kept) whose mass reaches ``top_p`` of theirs, and ``w >= min_p``.
    ``temperature <= 0`` gives the argmax, lowest index first.  Returns ``(indices, probabilities)``
    in binary64; thresholds closer than a few fp32 ulps to a weight are the caller's to avoid."""
    x = row.double().clone()
    if nan_to_neg_inf:
        x[torch.isnan(x)] = float("-inf")
    if not temperature > 0:
        return torch.tensor([int(torch.argmax(x))]), torch.tensor([1.0], dtype=torch.float64)
    w = torch.exp((x - x.max()) / temperature)
    keep = torch.ones_like(w, dtype=torch.bool)
    if 1 <= top_k < w.numel():
        keep &= w >= torch.sort(w, descending=True).values[top_k - 1]
    if top_p < 1.0:
        order = torch.argsort(torch.where(keep, w, torch.zeros_like(w)), descending=True)
        sorted_w = torch.where(keep, w, torch.zeros_like(w))[order]
        need = top_p * sorted_w.sum()
        reached = int(torch.nonzero(torch.cumsum(sorted_w, 0) >= need)[0])
        keep &= w >= sorted_w[reached]
    if min_p > 0:
        keep &= w >= min_p
    indices = torch.nonzero(keep).reshape(-1)
    return indices, w[indices] / w[indices].sum()
