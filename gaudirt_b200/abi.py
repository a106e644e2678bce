"""ctypes binding of the C ABI declared in ``include/gaudirt_b200.h``.

The library is loaded from ``gaudirt_b200/lib``; a missing library is an error (there is no
Python or CPU stand-in for any entry point).
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

i32p, i64p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_float)
vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float

# name -> (restype, argtypes); one entry per declaration in include/gaudirt_b200.h
PROTOTYPES = {
    "gk_status_string": (C.c_char_p, [i32]),
    "gk_abi_version": (i32, []),
    "gk_last_cuda_error": (i32, []),
    "gk_paged_kv_pool_bytes": (i32, [i64, i64, i64, i64, C.POINTER(C.c_uint64)]),
    "gk_paged_metadata_validate": (i32, [vp, vp, vp, i64, vp, i64, i64, i64, vp, i64p, i32p]),
    "gk_metadata_error": (C.c_char_p, []),
    "gk_attention_plan_build": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, vp, i64, i64p, vp, i64, i64p, i64p]),
    "gk_kv_store_head_major_bf16": (i32, [vp, vp, i64, i64, vp, i64, vp, vp, i64, i32, i32, vp, vp]),
    "gk_paged_attn_bf16": (i32, [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp, i64, vp, vp, f32, f32, i32,
                                 i32, i32, i32, vp, vp]),
    "gk_paged_attn_combine_bf16": (i32, [vp, vp, vp, i64, vp, i64, i32, i32, vp]),
    "gk_set_attention_form": (i32, [i32]),
    "gk_set_programmatic_launch": (i32, [i32]),
    "gk_prefill_plan_build": (i32, [vp, i64, i32, i32, i32, i32, vp, i64, i64p, vp, i64p]),
    "gk_paged_prefill_tc_bf16": (i32, [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp, i64, f32, f32, i32,
                                       i32, i32, i32, vp, vp]),
    "gk_paged_prefill_tc_multi_bf16": (i32, [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp, i32, i64, f32, f32,
                                             i32, i32, i32, i32, vp, vp]),
    "gk_paged_attn_store_multi_bf16": (i32, [vp, i64, vp, vp, i64, i64, vp, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp,
                                             i32, i64, vp, vp, vp, f32, f32, i32, i32, i32, i32, vp, vp]),
    "gk_paged_attn_multi_bf16": (i32, [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp, i32, i64, vp, vp, vp, f32,
                                       f32, i32, i32, i32, i32, vp, vp]),
    "gk_paged_attn_combine_multi_bf16": (i32, [vp, vp, vp, i64, vp, i32, i64, i32, i32, vp]),
    "gk_peer_barrier": (i32, [vp, i32, i32, i32, i64, vp, vp]),
    "gk_peer_barrier_counted": (i32, [vp, i32, i32, vp, i64, vp, vp]),
    "gk_rms_norm_bf16": (i32, [vp, vp, f32, f32, i64, i64, i64, vp, vp]),
    "gk_fused_add_rms_norm_bf16": (i32, [vp, vp, vp, f32, f32, i64, i64, i64, i64, vp, vp, vp]),
    "gk_rotary_bf16": (i32, [vp, vp, i64, i64, vp, i64, vp, i64, i64, i64, i32, i32, i32, vp, vp, vp, vp]),
    "gk_rotary_kv_store_bf16": (i32, [vp, vp, vp, i64, i64, i64, vp, i64, vp, vp, i64, i64, i64, i32, i32, i32,
                                      vp, vp, vp, vp, i64, vp, vp]),
    "gk_paged_slots_layout": (i32, [vp, vp, i64, i64, i64, vp, i64p, i64p]),
    "gk_paged_slots_allocate": (i32, [vp, vp, vp, i64, i64, i64, vp, vp, i64, i64, i64, vp, vp, vp, vp]),
    "gk_paged_slots_release_workspace_bytes": (i32, [i64, i64, C.POINTER(C.c_uint64)]),
    "gk_paged_slots_release": (i32, [vp, i64, i64, i64, vp, vp, vp, vp]),
    "gk_advance_decode_lengths": (i32, [vp, vp, i64, vp, vp, vp]),
    "gk_paged_metadata_device_workspace_bytes": (i32, [i64, C.POINTER(C.c_uint64)]),
    "gk_paged_metadata_device_validate": (i32, [vp, vp, vp, vp, i32, i64, vp, i64, i64, i64, i64, vp, i64, i64, vp,
                                                vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "gk_oproj_bf16": (i32, [vp, i64, vp, i64, i64, i64, i64, vp, i32, i64, vp, vp]),
    "gk_rank_sum_bf16": (i32, [vp, i32, i64, vp, vp]),
    "gk_rank_sum_add_rms_norm_bf16": (i32, [vp, i32, i64, vp, vp, f32, f32, i64, i64, i64, vp, vp, vp]),
    "gk_vocab_argmax": (i32, [vp, i32, i64, i64, i64, vp, vp]),
    "gk_apply_vocab_bitmask": (i32, [vp, i32, i64, i64, i64, vp, i64, i64, vp, i64, i64, i32, vp, vp]),
    "gk_sample_vocab": (i32, [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, vp, i32, C.c_uint64, i32, vp, vp]),
    "gk_paged_attn_static_scratch_bf16": (i32, [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, i64, vp, i64, i64,
                                                vp, i64, f32, f32, i32, i32, i32, i32, vp, vp]),
}

_lib = None


def library_path() -> str:
    return _build.ABI_SO


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python gaudirt_b200/build.py` (needs nvcc, sm_100a)")
        handle = C.CDLL(path)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class GkError(RuntimeError):
    def __init__(self, status: int, where: str):
        text = lib().gk_status_string(status).decode()
        if status == 5:
            text = lib().gk_metadata_error().decode()
        elif status == 3:
            text += f" (cudaError {lib().gk_last_cuda_error()})"
        super().__init__(f"{where}: {text}")
        self.status = status


def check(status: int, where: str) -> None:
    if status != 0:
        raise GkError(status, where)
