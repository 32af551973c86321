"""Class-(a) baseline: materialise fp16 K/V from the compressed representation, then run a dense varlen attention.

Mirrors the public functions of the reference's ``cda/kernels_vllm_fa2_fork/interface.py`` (``dequantize_compressed_kv``
``:138-162``, ``flash_attn_varlen_func`` ``:165-258``, ``flash_attn_varlen_compressed_kv_func`` ``:261-329``): same names,
argument order and errors.  Everything works in the rotated frame, as there.  The dequantisation is this package's CUDA
kernel (``cda_b200_dequantize_rows``); the dense attention body is the ``flash_attn`` library -- this path exists to be
compared *against*, it is not the product.  The reference's fused variant
(``flash_attn_varlen_compressed_kv_fused_func``) has no counterpart here: the fused product path is the paged prefill
kernel (``sub0_b200.kernels_cuda.fa2_cda.fa2_cda_prefill_varlen_v1``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .._lib import check, lib

HEAD_DIM = 128


def _flatten_compressed_kv(idx: torch.Tensor, norm: torch.Tensor, *, name: str):
    if idx.dim() == 3:
        if norm.dim() != 2:
            raise ValueError(f"{name}_norm must be (total_k, H_kv) for 3D idx")
        return idx.contiguous(), norm.contiguous()
    if idx.dim() == 4:
        if norm.dim() != 3:
            raise ValueError(f"{name}_norm must be (B, H_kv, N) for 4D idx")
        if idx.shape[:3] != norm.shape:
            raise ValueError(f"{name}_idx and {name}_norm shape mismatch")
        # (B, H_kv, N, bytes) -> token-major (B * N, H_kv, bytes), the order varlen attention expects
        return (idx.permute(0, 2, 1, 3).reshape(-1, idx.shape[1], idx.shape[3]).contiguous(),
                norm.permute(0, 2, 1).reshape(-1, norm.shape[1]).contiguous())
    raise ValueError(f"{name}_idx must be 3D or 4D, got {idx.dim()}D")


def _dequantize(idx: torch.Tensor, norm: torch.Tensor, cb: torch.Tensor) -> torch.Tensor:
    if not idx.is_cuda or idx.dtype != torch.uint8:
        raise TypeError("indices must be a uint8 CUDA tensor")
    levels = cb.numel()
    if levels not in (16, 4):
        raise ValueError("codebook must have 16 or 4 levels")
    bits = 4 if levels == 16 else 2
    if idx.shape[-1] != 16 * bits:
        raise ValueError(f"{bits}-bit indices must be {16 * bits} bytes per row, got {idx.shape[-1]}")
    norm = norm.to(device=idx.device, dtype=torch.float32).contiguous()
    cb = cb.to(device=idx.device, dtype=torch.float32).contiguous()
    rows = idx.numel() // idx.shape[-1]
    out = torch.empty(*idx.shape[:-1], HEAD_DIM, dtype=torch.float16, device=idx.device)
    check(lib.cda_b200_dequantize_rows(idx.data_ptr(), norm.data_ptr(), cb.data_ptr(), out.data_ptr(), rows, bits,
                                       torch.cuda.current_stream(idx.device).cuda_stream))
    return out


def dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cb_k, cb_v):
    """Rotated-frame fp16 K and V, ``(total_k, H_kv, 128)`` each, from packed indices and norms."""
    k_idx_flat, k_norm_flat = _flatten_compressed_kv(k_idx, k_norm, name="k")
    v_idx_flat, v_norm_flat = _flatten_compressed_kv(v_idx, v_norm, name="v")
    if k_idx_flat.shape[:2] != v_idx_flat.shape[:2]:
        raise ValueError("K/V idx shape mismatch after flattening")
    if k_norm_flat.shape != v_norm_flat.shape:
        raise ValueError("K/V norm shape mismatch after flattening")
    return _dequantize(k_idx_flat, k_norm_flat, cb_k), _dequantize(v_idx_flat, v_norm_flat, cb_v)


def flash_attn_varlen_func(q, k, v, max_seqlen_q: int, cu_seqlens_q, max_seqlen_k: int, cu_seqlens_k, *, out=None,
                           dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False,
                           window_size: Optional[Sequence[int]] = None, softcap: float = 0.0, alibi_slopes=None,
                           return_softmax_lse: bool = False, num_splits: int = 0):
    """Dense varlen attention (library kernel)."""
    if dropout_p != 0.0:
        raise NotImplementedError("inference-only")
    from flash_attn import flash_attn_varlen_func as _fa

    res = _fa(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), dropout_p=0.0,
              softmax_scale=softmax_scale, causal=causal, window_size=tuple(window_size) if window_size else (-1, -1),
              softcap=softcap, alibi_slopes=alibi_slopes, return_attn_probs=return_softmax_lse)
    o, lse = (res[0], res[1]) if return_softmax_lse else (res, None)
    if out is not None:
        out.copy_(o)
        o = out
    return (o, lse) if return_softmax_lse else o


def flash_attn_varlen_compressed_kv_func(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, max_seqlen_q: int, cu_seqlens_q,
                                         max_seqlen_k: int, cu_seqlens_k, *, out=None, dropout_p: float = 0.0,
                                         softmax_scale: Optional[float] = None, causal: bool = False,
                                         window_size: Optional[Sequence[int]] = None, softcap: float = 0.0, alibi_slopes=None,
                                         return_softmax_lse: bool = False, num_splits: int = 0):
    """Compressed-KV attention through the dense body: dequantise into fp16 scratch, then :func:`flash_attn_varlen_func`.
    Inputs (``q`` included) are in the rotated frame."""
    if dropout_p != 0.0:
        raise NotImplementedError("compressed-KV adapter is inference-only")
    k, v = dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cb_k, cb_v)
    return flash_attn_varlen_func(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, out=out,
                                  softmax_scale=softmax_scale, causal=causal, window_size=window_size, softcap=softcap,
                                  alibi_slopes=alibi_slopes, return_softmax_lse=return_softmax_lse, num_splits=num_splits)


def flash_attn_varlen_compressed_kv_fused_func(*args, **kwargs):
    raise NotImplementedError("the fused compressed-KV path of this package is the paged prefill kernel: "
                              "sub0_b200.kernels_cuda.fa2_cda.fa2_cda_prefill_varlen_v1")
