"""Class-(a) baseline: materialise fp16 K/V from the compressed representation, then run a dense varlen attention.

Mirrors the public functions of the reference's ``cda/kernels_vllm_fa2_fork/interface.py`` (``dequantize_compressed_kv``
``:138-162``, ``flash_attn_varlen_func`` ``:165-258``, ``flash_attn_varlen_compressed_kv_func`` ``:261-329``): same names,
argument order and errors.  Everything works in the rotated frame, as there.  The dequantisation is this package's CUDA
kernel (``cda_b200_dequantize_rows``); the dense attention body is the ``flash_attn`` library -- this path exists to be
compared *against*, it is not the product.  The reference's fused variant
(``flash_attn_varlen_compressed_kv_fused_func``, ``:332-470``) is served by the paged prefill kernel of this package: the
separate index / norm tensors are packed into slots and the rotated-frame query and result are passed through the
(self-inverse) Hadamard transform around it.
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


def _slot_cache(k_idx, k_norm, v_idx, v_norm):
    """(rows, H_kv, slot_bytes) uint8 slots [K idx | V idx | fp32 K norm | fp32 V norm | pad] from separate index and
    norm tensors of shape (rows, H_kv, bytes) / (rows, H_kv)."""
    rows, H_kv = k_idx.shape[0], k_idx.shape[1]
    width = (k_idx.shape[-1] + v_idx.shape[-1] + 8 + 15) // 16 * 16
    cache = torch.zeros(rows, H_kv, width, dtype=torch.uint8, device=k_idx.device)
    kb, vb = k_idx.shape[-1], v_idx.shape[-1]
    cache[..., :kb] = k_idx
    cache[..., kb:kb + vb] = v_idx
    cache[..., kb + vb:kb + vb + 4] = k_norm.to(torch.float32).contiguous().view(torch.uint8).view(rows, H_kv, 4)
    cache[..., kb + vb + 4:kb + vb + 8] = v_norm.to(torch.float32).contiguous().view(torch.uint8).view(rows, H_kv, 4)
    return cache


def flash_attn_varlen_compressed_kv_fused_func(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, max_seqlen_q: int, cu_seqlens_q,
                                               max_seqlen_k: int, cu_seqlens_k=None, *, seqused_k=None, block_table=None,
                                               out=None, dropout_p: float = 0.0, softmax_scale: Optional[float] = None,
                                               causal: bool = False, window_size: Optional[Sequence[int]] = None,
                                               softcap: float = 0.0, alibi_slopes=None, return_softmax_lse: bool = False,
                                               num_splits: int = 0, gqa_decode_swap: Optional[bool] = None,
                                               uniform_codebook: bool = False):
    """Compressed-KV attention without fp16 K/V scratch (reference: ``interface.py:332-470``, same arguments and checks),
    on this package's fused paged prefill kernel.  Everything is in the rotated frame, as there: the kernel rotates its
    queries and un-rotates its output, so ``q`` is un-rotated first and the result rotated back (the transform is its own
    inverse).  Supported slice: fp16, D = 128, bottom-right aligned causal masking (``causal=True``, or single-token
    queries, for which the mask is empty), no window / softcap / ALiBi / LSE.  Flattened K/V (``cu_seqlens_k``) or a paged
    cache (``block_table`` + ``seqused_k``; block size a multiple of 16)."""
    from .. import ops
    if dropout_p != 0.0:
        raise NotImplementedError("compressed-KV fused path is inference-only")
    if block_table is not None and seqused_k is None:
        raise ValueError("seqused_k must be provided when block_table is provided")
    if cu_seqlens_k is None and seqused_k is None:
        raise ValueError("cu_seqlens_k or seqused_k must be provided")
    if (window_size is not None and tuple(window_size) != (-1, -1)) or softcap != 0.0 or alibi_slopes is not None:
        raise NotImplementedError("sliding window, softcap and ALiBi are not supported by the fused path")
    if return_softmax_lse:
        raise NotImplementedError("the fused path does not return the log-sum-exp")
    if not causal and int(max_seqlen_q) > 1:
        raise NotImplementedError("the fused path masks causally (bottom-right aligned); non-causal needs single-token queries")
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM or q.dtype != torch.float16:
        raise ValueError("q must be (total_q, H_q, 128) fp16")
    dev = q.device
    B = int(cu_seqlens_q.numel() - 1)
    if block_table is not None:
        if k_idx.dim() != 4 or v_idx.dim() != 4:
            raise ValueError("paged k_idx/v_idx must be (num_blocks, block_size, H_kv, D/2)")
        if k_norm.dim() != 3 or v_norm.dim() != 3:
            raise ValueError("paged k_norm/v_norm must be (num_blocks, block_size, H_kv)")
        if k_idx.shape != v_idx.shape:
            raise ValueError("K/V idx shape mismatch")
        if k_norm.shape != v_norm.shape or k_norm.shape != k_idx.shape[:3]:
            raise ValueError("K/V idx/norm shape mismatch")
        nb, bs, H_kv = k_idx.shape[:3]
        cache = _slot_cache(k_idx.reshape(nb * bs, H_kv, -1), k_norm.reshape(nb * bs, H_kv),
                            v_idx.reshape(nb * bs, H_kv, -1), v_norm.reshape(nb * bs, H_kv))
        bt, seq = block_table.to(torch.int32), seqused_k.to(torch.int32)
    else:
        ki, kn = _flatten_compressed_kv(k_idx, k_norm, name="k")
        vi, vn = _flatten_compressed_kv(v_idx, v_norm, name="v")
        if ki.shape[:2] != vi.shape[:2]:
            raise ValueError("K/V idx shape mismatch after flattening")
        if kn.shape != vn.shape:
            raise ValueError("K/V norm shape mismatch after flattening")
        if cu_seqlens_k is None:
            raise ValueError("flattened K/V need cu_seqlens_k")
        # every sequence gets its own run of 16-slot blocks in a fresh cache
        bs, H_kv = 16, ki.shape[1]
        cu_k = cu_seqlens_k.to(torch.int64).cpu()
        lens = (cu_k[1:] - cu_k[:-1]).tolist()
        blocks = [-(-n // bs) for n in lens]
        starts = [0]
        for nblk in blocks:
            starts.append(starts[-1] + nblk)
        dst = torch.cat([torch.arange(n, dtype=torch.int64) + starts[b] * bs for b, n in enumerate(lens)]) if lens else torch.zeros(0, dtype=torch.int64)
        src = torch.cat([torch.arange(n, dtype=torch.int64) + int(cu_k[b]) for b, n in enumerate(lens)]) if lens else dst
        flat = _slot_cache(ki, kn, vi, vn)
        cache = torch.zeros(max(starts[-1], 1) * bs, H_kv, flat.shape[-1], dtype=torch.uint8, device=dev)
        cache[dst.to(dev)] = flat[src.to(dev)]
        bt = torch.zeros(B, max(max(blocks, default=1), 1), dtype=torch.int32)
        for b, nblk in enumerate(blocks):
            bt[b, :nblk] = torch.arange(starts[b], starts[b] + nblk, dtype=torch.int32)
        bt = bt.to(dev)
        seq = torch.tensor(lens, dtype=torch.int32, device=dev) if seqused_k is None else seqused_k.to(torch.int32)
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else float(softmax_scale)
    res = torch.empty_like(q) if out is None else out
    q_model = ops.hadamard128(q.contiguous())
    o_model = torch.empty_like(q_model)
    ops.prefill_varlen(q_model, cache, bt, cu_seqlens_q.to(torch.int32), seq, o_model, cb_K=cb_k, cb_V=cb_v, block_size=bs,
                       max_query_len=int(max_seqlen_q), max_seq_len=int(max_seqlen_k), scale=scale)
    if res.is_contiguous():
        ops.hadamard128(o_model, out=res)
    else:
        res.copy_(ops.hadamard128(o_model))
    return res
