"""``load_*`` getters with the names and return shape of the reference's ``cda/kernels_cuda/hmma_loader.py:27-59``.

There each getter imports a prebuilt pybind11 module and callers use its native function as an attribute
(``mod.cda_decode_full_hmma_v3(...)``, ``encode_mod.cda_paged_encode_fused(...)``).  Here every getter returns a small
namespace whose attribute of the same name forwards, argument for argument, to ``libcda_b200.so``; all variants
(k4v4 / k4v2, group size 4 / 8) come from the one library.
"""
from __future__ import annotations

from functools import lru_cache
from types import SimpleNamespace

import torch

from .. import ops


class PrebuiltMissing(ImportError):
    """Same role as ``cda._prebuilt_loader.PrebuiltMissing`` (cda/_prebuilt_loader.py:41-53)."""


def _check_rotation(rot: torch.Tensor) -> None:
    """The kernels apply the Sylvester-Hadamard rotation by butterflies; a rotation matrix argument is accepted for
    signature compatibility and only its shape is checked (a value check would need a device read)."""
    if rot is not None and tuple(rot.shape) != (ops.HEAD_DIM, ops.HEAD_DIM):
        raise ValueError("rotation must be (128, 128)")


def _decode_native(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, rot_fp32, rot_fp16, out, group_size, block_size,
                   tile_N, max_seq_len, scale):
    """Positional signature of ``cda_decode_full_hmma_v3`` (cda/kernels_cuda/wrappers.py:115-124).  ``tile_N`` is the
    reference kernel's split granularity; this library plans its own splits, so the value is ignored."""
    _check_rotation(rot_fp32)
    _check_rotation(rot_fp16)
    H_kv = kv_cache.shape[-2]
    if Q.shape[1] != H_kv * int(group_size):
        raise ValueError(f"H_q={Q.shape[1]} != H_kv*group_size={H_kv * int(group_size)}")
    ops.decode(Q, kv_cache, block_table, seq_lens, out, cb_K=cb_K, cb_V=cb_V, block_size=int(block_size),
               scale=float(scale), max_seq_len=int(max_seq_len))


def _encode_native(K, V, slot_mapping, flat_cache, cb_K, cb_V):
    """``cda_paged_encode_fused`` (cda/kernels_cuda/wrappers.py:153-156)."""
    ops.paged_encode(K, V, slot_mapping, flat_cache, cb_K, cb_V)


def _loader_native(kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, max_seq_len):
    """``cda_fa2_paged_cache_to_dense_rotated`` (cda/kernels_cuda/fa2_cda.py:86-95); returns ``(k_rot, v_rot)``."""
    return ops.cache_to_dense_rotated(kv_cache, block_table, seq_lens, cb_K=cb_K, cb_V=cb_V, block_size=int(block_size),
                                      max_seq_len=int(max_seq_len))


def _hadamard_native(x, y, scale):
    """``hadamard128_fp16`` (cda/kernels_cuda/fa2_cda.py:50-53)."""
    ops.hadamard128(x, out=y, scale=float(scale))


def _varlen_native(Q, k_rot, v_rot, out, cu_q, cu_k, seqused_k, max_q, max_k, scale):
    """``cda_fa2_varlen_fwd_hadamard`` (cda/kernels_cuda/fa2_cda.py:170-181)."""
    ops.varlen_fwd_hadamard(Q, k_rot, v_rot, out, cu_q, cu_k, seqused_k, int(max_q), int(max_k), float(scale))


@lru_cache(maxsize=8)
def load_decode_hmma(k4v2: bool = False, group_size: int = 4):
    if group_size not in (4, 8):
        raise ValueError(f"group_size must be 4 or 8 (got {group_size})")
    return SimpleNamespace(cda_decode_full_hmma_v3=_decode_native, k4v2=bool(k4v2), group_size=int(group_size))


@lru_cache(maxsize=2)
def load_paged_encode_fused():
    return SimpleNamespace(cda_paged_encode_fused=_encode_native)


@lru_cache(maxsize=4)
def load_kv_cache_update(k4v2: bool = False):
    """The reference names ``_v1_kv_update_k4v{2,4}`` here but ships neither (cda/kernels_cuda/hmma_loader.py:41-43);
    selecting it fails the same way."""
    name = "_v1_kv_update_k4v2" if k4v2 else "_v1_kv_update_k4v4"
    raise PrebuiltMissing(f"kernel '{name}' does not exist; cache updates go through paged_encode_fused_cuda")


@lru_cache(maxsize=4)
def load_fa2_cda_loader(k4v2: bool = False):
    return SimpleNamespace(cda_fa2_paged_cache_to_dense_rotated=_loader_native, k4v2=bool(k4v2))


@lru_cache(maxsize=1)
def load_fa2_cda_hadamard():
    return SimpleNamespace(hadamard128_fp16=_hadamard_native)


@lru_cache(maxsize=1)
def load_fa2_cda_varlen_fused():
    return SimpleNamespace(cda_fa2_varlen_fwd_hadamard=_varlen_native)


__all__ = [
    "load_decode_hmma",
    "load_paged_encode_fused",
    "load_kv_cache_update",
    "load_fa2_cda_loader",
    "load_fa2_cda_hadamard",
    "load_fa2_cda_varlen_fused",
    "PrebuiltMissing",
]
