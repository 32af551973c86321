"""Prefill wrappers with the signatures of the reference's ``cda/kernels_cuda/fa2_cda.py``.

* :func:`paged_cache_to_dense_rotated`     -- fa2_cda.py:64-95
* :func:`fa2_cda_prefill_varlen_v1`        -- fa2_cda.py:98-230
* :func:`fa2_cda_prefill_rawkv_varlen_v1`  -- fa2_cda.py:305-377
* :func:`fa2_raw_prefill_varlen_v1`        -- fa2_cda.py:380-462

The reference's default prefill is two kernels with a dense fp16 K/V round trip through HBM (loader, then attention).
Here ``fa2_cda_prefill_varlen_v1`` runs ONE kernel that decodes K/V tiles from the paged cache inside the attention
loop; the dense loader is still available (and is what ``return_dense_kv=True`` returns).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from .. import ops


def _hadamard_or_matmul(x: Tensor, rotation_fp32: Optional[Tensor] = None, *, out: Optional[Tensor] = None) -> Tensor:
    """fa2_cda.py:36-61 -- always the butterfly kernel here (fp16, contiguous, last dim 128)."""
    x = x if x.dtype == torch.float16 else x.to(torch.float16)
    return ops.hadamard128(x.contiguous(), out=out)


def paged_cache_to_dense_rotated(
    kv_cache: Tensor,
    block_table: Tensor,
    seq_lens: Tensor,
    *,
    cb_K: Tensor,
    cb_V: Tensor,
    block_size: int,
    max_seq_len: int,
    k4v2: bool = False,
) -> tuple[Tensor, Tensor]:
    """Dense rotated-frame fp16 K/V, each ``(B * max_seq_len, H_kv, 128)``; rows beyond ``seq_lens[b]`` are zero."""
    if k4v2 and cb_V.numel() != 4:
        raise ValueError("k4v2=True needs a 4-level V codebook")
    return ops.cache_to_dense_rotated(kv_cache, block_table, seq_lens, cb_K=cb_K, cb_V=cb_V, block_size=int(block_size),
                                      max_seq_len=int(max_seq_len))


def fa2_cda_prefill_varlen_v1(
    Q_fp16: Tensor,           # (T, H_q, D) fp16, unrotated
    kv_cache: Tensor,         # (num_slots, H_kv, slot_w) uint8
    block_table: Tensor,      # (B, max_blocks) int32
    cu_seqlens_q: Tensor,     # (B+1,) int32
    seq_lens: Tensor,         # (B,) int32, full key lengths
    output: Tensor,           # (T, H_q, D) fp16, written in place
    *,
    cb_K: Tensor,
    cb_V: Tensor,
    rotation_fp32: Optional[Tensor] = None,
    group_size: int,
    block_size: int,
    max_query_len: int,
    max_seq_len: int,
    scale: Optional[float] = None,
    causal: bool = True,
    k4v2: bool = False,
    return_dense_kv: bool = False,
    fuse_fa2_epilogue: bool = False,
) -> tuple[Tensor, Tensor] | None:
    """Causal variable-length prefill over the compressed cache (query i of a chunk of length q_len sees keys
    ``k <= seq_len - q_len + i``).  ``fuse_fa2_epilogue`` is accepted for compatibility; rotation of Q and the inverse
    rotation of the output are always fused into the attention kernel."""
    if Q_fp16.dim() != 3:
        raise ValueError("Q_fp16 must be (T, H_q, D)")
    if output.shape != Q_fp16.shape:
        raise ValueError("output shape must match Q_fp16")
    if output.dtype != torch.float16:
        raise ValueError("output must be fp16")
    Q_in = Q_fp16.to(torch.float16) if Q_fp16.dtype != torch.float16 else Q_fp16
    T, H_q, D = Q_in.shape
    B = int(cu_seqlens_q.numel()) - 1
    if B <= 0:
        return None
    if H_q % group_size != 0:
        raise ValueError("H_q must be divisible by group_size")
    if not causal:
        raise NotImplementedError("the fused CDA prefill kernel is causal-only")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ops.prefill_varlen(Q_in, kv_cache, block_table, cu_seqlens_q, seq_lens, output, cb_K=cb_K, cb_V=cb_V,
                       block_size=int(block_size), max_query_len=int(max_query_len), max_seq_len=int(max_seq_len),
                       scale=float(scale))
    if return_dense_kv:
        return paged_cache_to_dense_rotated(kv_cache, block_table, seq_lens, cb_K=cb_K, cb_V=cb_V,
                                            block_size=block_size, max_seq_len=max_seq_len, k4v2=k4v2)
    return None


def fa2_cda_prefill_rawkv_varlen_v1(
    Q_fp16: Tensor,           # (T, H_q, D) fp16, unrotated
    K_fp16: Tensor,           # (T, H_kv, D) fp16, fresh uncompressed K
    V_fp16: Tensor,           # (T, H_kv, D) fp16, fresh uncompressed V
    cu_seqlens_q: Tensor,     # (B+1,) int32
    seq_lens: Tensor,         # (B,) int32, key lengths (== query lengths: no compressed past)
    output: Tensor,           # (T, H_q, D) fp16, written in place
    *,
    rotation_fp32: Optional[Tensor] = None,
    group_size: int,
    max_query_len: int,
    max_seq_len: int,
    scale: Optional[float] = None,
    causal: bool = True,
) -> None:
    """No-past prefill on raw K/V: rotate K and V with the butterfly kernel, then the fused attention kernel on the
    dense rows (ragged layout: sequence b's keys are rows ``cu_seqlens_q[b] ..``)."""
    if Q_fp16.dim() != 3:
        raise ValueError("Q_fp16 must be (T, H_q, D)")
    if K_fp16.dim() != 3 or V_fp16.dim() != 3:
        raise ValueError("K_fp16 and V_fp16 must be (T, H_kv, D)")
    if K_fp16.shape != V_fp16.shape:
        raise ValueError("K_fp16 and V_fp16 shapes must match")
    if output.shape != Q_fp16.shape:
        raise ValueError("output shape must match Q_fp16")
    if output.dtype != torch.float16:
        raise ValueError("output must be fp16")
    if not causal:
        raise NotImplementedError("fa2_cda_prefill_rawkv_varlen_v1 is causal-only")
    T, H_q, D = Q_fp16.shape
    if K_fp16.shape[0] != T:
        raise ValueError("raw K/V must have the same token count as Q")
    if K_fp16.shape[2] != D:
        raise ValueError("Q/K/V head dimensions must match")
    if H_q != K_fp16.shape[1] * int(group_size):
        raise ValueError("H_q must equal H_kv * group_size")
    if int(cu_seqlens_q.numel()) - 1 <= 0:
        return
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    Q_in = Q_fp16.to(torch.float16) if Q_fp16.dtype != torch.float16 else Q_fp16
    k_rot = _hadamard_or_matmul(K_fp16)
    v_rot = _hadamard_or_matmul(V_fp16)
    ops.varlen_fwd_hadamard(Q_in, k_rot, v_rot, output, cu_seqlens_q, cu_seqlens_q, seq_lens, int(max_query_len),
                            int(max_seq_len), float(scale))


def fa2_raw_prefill_varlen_v1(
    Q_fp16: Tensor,
    K_fp16: Tensor,
    V_fp16: Tensor,
    cu_seqlens_q: Tensor,
    output: Tensor,
    *,
    group_size: int,
    max_query_len: int,
    scale: Optional[float] = None,
    causal: bool = True,
) -> None:
    """No-past prefill over raw Q/K/V.  The reference hands this case to a stock FlashAttention call because the
    rotation is orthonormal and cancels; this build keeps a single attention kernel and computes the same result in the
    rotated frame (rotate K/V, fused Q rotation, inverse rotation of the output)."""
    if not causal:
        raise NotImplementedError("fa2_raw_prefill_varlen_v1 is causal-only")
    cu = cu_seqlens_q.to(torch.int32) if cu_seqlens_q.dtype != torch.int32 else cu_seqlens_q
    seq = (cu[1:] - cu[:-1]).contiguous()
    fa2_cda_prefill_rawkv_varlen_v1(Q_fp16, K_fp16, V_fp16, cu, seq, output, group_size=group_size,
                                    max_query_len=max_query_len, max_seq_len=max_query_len, scale=scale, causal=True)


__all__ = [
    "fa2_cda_prefill_rawkv_varlen_v1",
    "fa2_cda_prefill_varlen_v1",
    "fa2_raw_prefill_varlen_v1",
    "paged_cache_to_dense_rotated",
]
