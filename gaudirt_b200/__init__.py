"""B200-native paged KV-store / paged-attention path behind the GaudiRT operator surface.

Importing the package loads the two in-tree native libraries (``python gaudirt_b200/build.py``
makes them) and exposes the reference's Python-visible names for this path:

* ``torch.ops.gaudirt.paged_attn`` / ``_paged_attn_validated`` and
  ``torch.classes.gaudirt.PagedMetadata`` (reference: ``src/bridge/generic_private_use1.cpp:430-489``);
* ``gaudirt_b200._C._allocate_paged_kv`` / ``_C._paged_attn_kv_tile`` / ``_C._allocate_paged_slots`` /
  ``_C._release_paged_slots`` (reference: the ``gaudirt._C`` bindings of the same names) and
  ``torch.ops.gaudirt._advance_decode_lengths``;
* fake-tensor registrations with the reference's shape contracts (``python/gaudirt/__init__.py:136-153``).

There is no CPU or pure-PyTorch fallback: a missing library is an import error.
"""
from __future__ import annotations

import os
import types

import torch

from . import abi, build

__all__ = ["abi", "build", "_C", "PagedMetadata", "synchronize", "validated_last_token_indices"]

if not os.path.exists(build.OPS_SO):
    raise ImportError(f"{build.OPS_SO} is missing: run `python gaudirt_b200/build.py` (needs nvcc and g++)")
abi.lib()
torch.ops.load_library(build.OPS_SO)

PagedMetadata = torch.classes.gaudirt.PagedMetadata

_C = types.SimpleNamespace(
    _allocate_paged_kv=lambda layers, slots, heads, head_dim: torch.ops.gaudirt._allocate_paged_kv(
        layers, slots, heads, head_dim),
    _paged_attn_kv_tile=lambda rows: int(torch.ops.gaudirt._paged_attn_kv_tile(rows)),
    _take_device_status=lambda: int(torch.ops.gaudirt._take_device_status()),
    _allocate_paged_slots=lambda last_slots, free_pages, prefixes, lengths, page_size:
        torch.ops.gaudirt._allocate_paged_slots(last_slots, free_pages, prefixes, lengths, page_size),
    _allocate_paged_slots_into=lambda last_slots, free_pages, prefixes, lengths, page_size, mapping, batch_requests:
        torch.ops.gaudirt._allocate_paged_slots_into(last_slots, free_pages, prefixes, lengths, page_size, mapping,
                                                     batch_requests),
    _release_paged_slots=lambda slots, page_size, max_pages:
        torch.ops.gaudirt._release_paged_slots(slots, page_size, max_pages),
)


def validated_last_token_indices(metadata) -> torch.Tensor:
    """Row index of the last token of every sequence of a device-validated batch (int32), tagged with
    the row count it was validated for (reference: ``python/gaudirt/__init__.py``, used by
    ``tests/paged_device_metadata_smoke.py:85-89``)."""
    indices = metadata.last_token_indices()
    indices._gaudirt_validated_rows = metadata.rows()
    return indices


def synchronize() -> None:
    torch.cuda.synchronize()


@torch.library.register_fake("gaudirt::paged_attn")
def _fake_paged_attn(query, key, value, key_pool, value_pool, metadata, head_dim, scale,
                     softcap=0.0, sliding_window=-1):
    torch._check(key.shape[0] == query.shape[0])
    torch._check(value.shape[0] == query.shape[0])
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.register_fake("gaudirt::_paged_attn_validated")
def _fake_paged_attn_validated(query, key, value, key_pool, value_pool, locations, requests, positions,
                               mapping, header, head_dim, scale, softcap=0.0, sliding_window=-1):
    torch._check(key.shape[0] == query.shape[0])
    torch._check(value.shape[0] == query.shape[0])
    torch._check(locations.shape[0] == query.shape[0])
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.register_fake("gaudirt::_paged_attn_stored")
def _fake_paged_attn_stored(query, key_pool, value_pool, metadata, head_dim, scale, softcap=0.0, sliding_window=-1):
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.register_fake("gaudirt::_rotary_kv_store")
def _fake_rotary_kv_store(query, key, value, cache, metadata, key_pool, value_pool, head_dim, rotary_dim, is_neox):
    torch._check(key.shape[0] == query.shape[0])
    torch._check(value.shape[0] == query.shape[0])
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.register_fake("gaudirt::rms_norm")
def _fake_rms_norm(input, weight, epsilon, weight_offset=0.0):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake("gaudirt::fused_add_rms_norm")
def _fake_fused_add_rms_norm(input, residual, weight, epsilon, weight_offset=0.0):
    if input.ndim >= 1 and residual.ndim >= 1:
        torch._check(residual.shape[0] == input.shape[0])
    return (torch.empty_like(input, memory_format=torch.contiguous_format),
            torch.empty_like(residual, memory_format=torch.contiguous_format))


@torch.library.register_fake("gaudirt::rotary_embedding")
def _fake_rotary_embedding(query, key, cache, metadata, head_dim, rotary_dim, is_neox):
    torch._check(key.shape[0] == query.shape[0])
    return (torch.empty_like(query, memory_format=torch.contiguous_format),
            torch.empty_like(key, memory_format=torch.contiguous_format))


@torch.library.register_fake("gaudirt::rotary_embedding_positions")
def _fake_rotary_embedding_positions(query, key, cache, positions, head_dim, rotary_dim, is_neox):
    torch._check(key.shape[0] == query.shape[0])
    torch._check(positions.shape[0] == query.shape[0])
    return (torch.empty_like(query, memory_format=torch.contiguous_format),
            torch.empty_like(key, memory_format=torch.contiguous_format))


@torch.library.register_fake("gaudirt::_rotary_embedding_validated")
def _fake_rotary_embedding_validated(query, key, cache, positions, header, context, head_dim, rotary_dim, is_neox):
    torch._check(key.shape[0] == query.shape[0])
    torch._check(positions.shape[0] == query.shape[0])
    return (torch.empty_like(query, memory_format=torch.contiguous_format),
            torch.empty_like(key, memory_format=torch.contiguous_format))
