"""Thin ctypes driver of the raw C ABI: host metadata and schedules through the library's host
entry points, kernel launches on torch CUDA tensors.  Used by the parity tests and by the
benchmark's kernel-only timing pass; the operator layer (torch.ops.gaudirt.*) does not go
through here."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import abi


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def validate(locations, requests, positions, mapping, slots):
    loc, req, pos = (np.ascontiguousarray(np.asarray(x), dtype=np.int32) for x in (locations, requests, positions))
    table = np.ascontiguousarray(np.asarray(mapping), dtype=np.int32)
    seq = np.zeros((len(loc), 4), dtype=np.int32)
    n_seq, page = C.c_int64(0), C.c_int32(0)
    status = abi.lib().gk_paged_metadata_validate(_ptr(loc), _ptr(req), _ptr(pos), len(loc), _ptr(table),
                                                  table.shape[0], table.shape[1], slots, _ptr(seq),
                                                  C.byref(n_seq), C.byref(page))
    abi.check(status, "gk_paged_metadata_validate")
    return seq[: n_seq.value].copy(), page.value


def plan(seq, q_heads, kv_heads, head_dim, window=-1, sm_count=148, split_tokens=0):
    seq = np.ascontiguousarray(seq, dtype=np.int32).reshape(-1, 4)
    n_work, n_comb, entries = C.c_int64(0), C.c_int64(0), C.c_int64(0)
    lib = abi.lib()
    args = (_ptr(seq), len(seq), q_heads, kv_heads, head_dim, window, sm_count, split_tokens)
    abi.check(lib.gk_attention_plan_build(*args, None, 0, C.byref(n_work), None, 0, C.byref(n_comb),
                                          C.byref(entries)), "gk_attention_plan_build(count)")
    work = np.zeros((n_work.value, 8), dtype=np.int32)
    comb = np.zeros((max(n_comb.value, 1), 4), dtype=np.int32)
    abi.check(lib.gk_attention_plan_build(*args, _ptr(work), len(work), C.byref(n_work), _ptr(comb), len(comb),
                                          C.byref(n_comb), C.byref(entries)), "gk_attention_plan_build")
    return work, comb[: n_comb.value].copy(), entries.value


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def kv_store(pool_layer, key, value, locations, status=None):
    """pool_layer: cuda bf16 [2, kv_heads, slots, d]; key/value: cuda bf16 [rows, kv_heads*d] (any row stride)."""
    _, kv_heads, slots, d = pool_layer.shape
    assert key.stride(1) == 1 and value.stride(1) == 1 and locations.dtype == torch.int32
    st = abi.lib().gk_kv_store_head_major_bf16(
        key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), locations.data_ptr(), key.size(0),
        pool_layer[0].data_ptr(), pool_layer[1].data_ptr(), slots, kv_heads, d,
        status.data_ptr() if status is not None else None, stream_ptr())
    abi.check(st, "gk_kv_store_head_major_bf16")


def paged_attn(query, pool_layer, table, page_tokens, work, combine, entries, q_heads, scale,
               softcap=0.0, window=-1, status=None, entry_stride=1, table_rows=None, fused_combine=False):
    """Launch attention (+ combine) for a prepared schedule; returns the bf16 output tensor.  With
    `fused_combine` the attention kernel merges the splits itself (no combine launch)."""
    _, kv_heads, slots, d = pool_layer.shape
    dev = query.device
    out = torch.empty((query.size(0), q_heads * d), dtype=torch.bfloat16, device=dev)
    work_d = torch.from_numpy(work).to(dev)
    part_ml = torch.empty(max(entries, 1) * 2, dtype=torch.float32, device=dev)
    part_o = torch.empty(max(entries, 1) * d, dtype=torch.float32, device=dev)
    lib = abi.lib()
    if fused_combine:
        counters = torch.zeros(query.size(0) * kv_heads, dtype=torch.int32, device=dev)
        outs = (C.c_void_p * 1)(out.data_ptr())
        st = lib.gk_paged_attn_multi_bf16(
            query.data_ptr(), query.stride(0), pool_layer[0].data_ptr(), pool_layer[1].data_ptr(), slots,
            table.data_ptr(), table.stride(0), entry_stride, page_tokens,
            table_rows.data_ptr() if table_rows is not None else None, work_d.data_ptr(), work.shape[0], outs, 1,
            out.stride(0), part_ml.data_ptr(), part_o.data_ptr(), counters.data_ptr(), scale, softcap, window, q_heads,
            kv_heads, d, status.data_ptr() if status is not None else None, stream_ptr())
        abi.check(st, "gk_paged_attn_multi_bf16")
        torch.cuda.current_stream().synchronize()
        assert int(counters.abs().sum()) == 0, "split counters must return to zero"
        return out
    st = lib.gk_paged_attn_bf16(
        query.data_ptr(), query.stride(0), pool_layer[0].data_ptr(), pool_layer[1].data_ptr(), slots,
        table.data_ptr(), table.stride(0), entry_stride, page_tokens,
        table_rows.data_ptr() if table_rows is not None else None, work_d.data_ptr(), work.shape[0], out.data_ptr(),
        out.stride(0), part_ml.data_ptr(), part_o.data_ptr(), scale, softcap, window, q_heads, kv_heads, d,
        status.data_ptr() if status is not None else None, stream_ptr())
    abi.check(st, "gk_paged_attn_bf16")
    if len(combine):
        comb_d = torch.from_numpy(combine).to(dev)
        st = lib.gk_paged_attn_combine_bf16(part_ml.data_ptr(), part_o.data_ptr(), comb_d.data_ptr(), len(combine),
                                            out.data_ptr(), out.stride(0), q_heads, d, stream_ptr())
        abi.check(st, "gk_paged_attn_combine_bf16")
    torch.cuda.current_stream().synchronize()
    return out


def prefill_plan(seq, q_heads, kv_heads, window=-1, min_rows=0):
    """Tensor-core work records for the multi-row sequences, and the sequences left for `plan`."""
    seq = np.ascontiguousarray(seq, dtype=np.int32).reshape(-1, 4)
    n_work, n_rest = C.c_int64(0), C.c_int64(0)
    lib = abi.lib()
    abi.check(lib.gk_prefill_plan_build(_ptr(seq), len(seq), q_heads, kv_heads, window, min_rows, None, 0,
                                        C.byref(n_work), None, C.byref(n_rest)), "gk_prefill_plan_build(count)")
    work = np.zeros((max(n_work.value, 1), 8), dtype=np.int32)
    rest = np.zeros((max(n_rest.value, 1), 4), dtype=np.int32)
    abi.check(lib.gk_prefill_plan_build(_ptr(seq), len(seq), q_heads, kv_heads, window, min_rows, _ptr(work), len(work),
                                        C.byref(n_work), _ptr(rest), C.byref(n_rest)), "gk_prefill_plan_build")
    return work[: n_work.value].copy(), rest[: n_rest.value].copy()


def paged_prefill_tc(query, pool_layer, table, page_tokens, work, out, q_heads, scale, softcap=0.0, window=-1,
                     status=None, entry_stride=1, table_rows=None):
    """Launch the tensor-core prefill kernel for prepared work records, writing rows of `out`."""
    _, kv_heads, slots, d = pool_layer.shape
    work_d = torch.from_numpy(np.ascontiguousarray(work)).to(query.device)
    st = abi.lib().gk_paged_prefill_tc_bf16(
        query.data_ptr(), query.stride(0), pool_layer[0].data_ptr(), pool_layer[1].data_ptr(), slots,
        table.data_ptr(), table.stride(0), entry_stride, page_tokens,
        table_rows.data_ptr() if table_rows is not None else None, work_d.data_ptr(), len(work), out.data_ptr(),
        out.stride(0), scale, softcap, window, q_heads, kv_heads, d,
        status.data_ptr() if status is not None else None, stream_ptr())
    abi.check(st, "gk_paged_prefill_tc_bf16")
    torch.cuda.current_stream().synchronize()
    return out
