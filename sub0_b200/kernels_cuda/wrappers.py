"""Decode and paged-encode wrappers with the signatures of the reference's ``cda/kernels_cuda/wrappers.py``.

* :func:`decode_hmma_v1`          -- wrappers.py:79-124
* :func:`paged_encode_fused_cuda` -- wrappers.py:127-156

Differences a caller can observe: the split-KV scratch is a caller-visible workspace (optional ``workspace=``, else a
per-device cache that only grows and refuses to grow during a stream capture -- see ``sub0_b200.ops``) instead of an
allocation inside the kernel call; 2-bit codebooks (4 levels) select the low-bit slot layouts; GQA groups of 1..8 are
accepted.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from .. import ops
from .hmma_loader import load_decode_hmma, load_paged_encode_fused


def _choose_splits(max_seq_len: int, *, B: int = 1, H_kv: int = 8, device_idx: int = 0) -> int:
    """Counterpart of ``_choose_tile_n`` (wrappers.py:41-76): the number of partial results per output row the decode
    kernel will produce.  The kernel cuts the concatenation of all sequences' keys into equal chunks, one CTA (all KV
    heads of the chunk) per SM, never below 128 tokens per chunk; a sequence is merged from as many partials as chunks
    it touches.  There is no 256-split cap."""
    return ops.plan_splits(B, H_kv, max_seq_len, device_idx)


def decode_hmma_v1(
    Q_fp16: Tensor,           # (B, H_q, D) fp16 -- UNROTATED
    kv_cache: Tensor,         # (num_total_slots, H_kv, slot_bytes) uint8
    block_table: Tensor,      # (B, max_blocks) int32
    seq_lens: Tensor,         # (B,) int32 -- full seq_len (past + 1)
    output: Tensor,           # (B, H_q, D) fp16 -- written in place
    *,
    cb_K: Tensor,
    cb_V: Tensor,
    rotation_fp32: Optional[Tensor] = None,
    rotation_fp16: Optional[Tensor] = None,
    group_size: int,
    block_size: int,
    scale: Optional[float] = None,
    max_seq_len: Optional[int] = None,
    workspace: Optional[Tensor] = None,
    num_splits: int = 0,
) -> None:
    """Single-query GQA decode over the paged compressed cache, output written in place."""
    B, H_q, D = Q_fp16.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if max_seq_len is None:
        max_seq_len = int(seq_lens.max().item())
    if output.dtype != torch.float16:
        raise ValueError("decode_hmma_v1 requires fp16 output buffer")
    load_decode_hmma(k4v2=cb_V.numel() == 4, group_size=group_size if group_size in (4, 8) else 4)
    H_kv = kv_cache.shape[-2]
    if H_q != H_kv * int(group_size):
        raise ValueError(f"H_q={H_q} != H_kv*group_size={H_kv * int(group_size)}")
    ops.decode(Q_fp16, kv_cache, block_table, seq_lens, output, cb_K=cb_K, cb_V=cb_V, block_size=block_size,
               scale=scale, max_seq_len=max_seq_len, num_splits=num_splits, workspace=workspace)


def paged_encode_fused_cuda(
    K: Tensor,                      # (T, H_kv, D=128) fp16, UN-rotated
    V: Tensor,
    slot_mapping: Tensor,           # (T,) int32
    flat_cache: Tensor,             # (num_slots, H_kv, slot_w) uint8
    *,
    cb_K: Tensor,                   # (16,) fp32 (or (4,) for 2-bit K)
    cb_V: Tensor,
) -> None:
    """Fused Hadamard rotation + L2 normalisation + nearest-level quantisation + paged scatter (one kernel)."""
    if K.dtype != torch.float16 or V.dtype != torch.float16:
        raise TypeError("K, V must be fp16")
    if flat_cache.dtype != torch.uint8:
        raise TypeError("flat_cache must be uint8")
    if K.shape[-1] != 128:
        raise ValueError(f"D must be 128, got {K.shape[-1]}")
    load_paged_encode_fused().cda_paged_encode_fused(K, V, slot_mapping, flat_cache, cb_K, cb_V)


__all__ = [
    "decode_hmma_v1",
    "paged_encode_fused_cuda",
]
