"""``torch.ops._cda_vllm_fa2_fork_C`` -- the operator namespace the reference's compiled extension registers
(``cda/kernels_vllm_fa2_fork/interface.py:9, 58-111``), provided by this package's functions: ``dequantize_compressed_kv``,
``varlen_fwd``, ``varlen_fwd_compressed_kv`` and ``varlen_fwd_compressed_kv_fused`` with the positional argument lists the
reference's wrappers pass (``interface.py:154-161, 234-257, 304-328, 433-460``).  Every operator returns ``(out,
softmax_lse)`` like the native one; ``softmax_lse`` is an empty tensor where the path does not produce it.

Importing this module registers the namespace once per process (``register()`` is idempotent)."""
from __future__ import annotations

import torch

NAMESPACE = "_cda_vllm_fa2_fork_C"
_LIB = None


def _window(left: int, right: int):
    return None if (left, right) == (-1, -1) else (left, right)


def _no_lse(q: torch.Tensor) -> torch.Tensor:
    return torch.empty(0, dtype=torch.float32, device=q.device)


def _dequantize(k_idx, k_norm, v_idx, v_norm, cb_k, cb_v):
    from .interface import dequantize_compressed_kv
    return dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cb_k, cb_v)


def _varlen_fwd(q, k, v, out, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table, alibi_slopes, max_seqlen_q,
                max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_left, window_right, softcap,
                return_softmax, num_splits, gen):
    from .interface import flash_attn_varlen_func
    if block_table is not None or seqused_k is not None or leftpad_k is not None:
        raise NotImplementedError("varlen_fwd: the dense comparison body takes flattened K/V (no block table)")
    o, lse = flash_attn_varlen_func(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, out=out,
                                    dropout_p=p_dropout, softmax_scale=softmax_scale, causal=is_causal,
                                    window_size=_window(window_left, window_right), softcap=softcap,
                                    alibi_slopes=alibi_slopes, return_softmax_lse=True, num_splits=num_splits)
    return o, lse


def _varlen_fwd_compressed_kv(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, out, cu_seqlens_q, cu_seqlens_k, alibi_slopes,
                              max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_left,
                              window_right, softcap, return_softmax, num_splits, gen):
    from .interface import flash_attn_varlen_compressed_kv_func
    o, lse = flash_attn_varlen_compressed_kv_func(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, max_seqlen_q, cu_seqlens_q,
                                                  max_seqlen_k, cu_seqlens_k, out=out, dropout_p=p_dropout,
                                                  softmax_scale=softmax_scale, causal=is_causal,
                                                  window_size=_window(window_left, window_right), softcap=softcap,
                                                  alibi_slopes=alibi_slopes, return_softmax_lse=True, num_splits=num_splits)
    return o, lse


def _varlen_fwd_compressed_kv_fused(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, out, cu_seqlens_q, cu_seqlens_k, seqused_k,
                                    block_table, alibi_slopes, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale,
                                    zero_tensors, is_causal, window_left, window_right, softcap, return_softmax, num_splits,
                                    uniform_codebook, gen):
    from .interface import flash_attn_varlen_compressed_kv_fused_func
    o = flash_attn_varlen_compressed_kv_fused_func(q, k_idx, k_norm, v_idx, v_norm, cb_k, cb_v, max_seqlen_q, cu_seqlens_q,
                                                   max_seqlen_k, cu_seqlens_k, seqused_k=seqused_k, block_table=block_table,
                                                   out=out, dropout_p=p_dropout, softmax_scale=softmax_scale,
                                                   causal=is_causal, window_size=_window(window_left, window_right),
                                                   softcap=softcap, alibi_slopes=alibi_slopes, return_softmax_lse=False,
                                                   num_splits=num_splits, uniform_codebook=uniform_codebook)
    return o, _no_lse(q)


_SCHEMAS = {
    "dequantize_compressed_kv": ("(Tensor k_idx, Tensor k_norm, Tensor v_idx, Tensor v_norm, Tensor cb_k, Tensor cb_v) -> (Tensor, Tensor)",
                                 _dequantize),
    "varlen_fwd": ("(Tensor q, Tensor k, Tensor v, Tensor(a!)? out, Tensor cu_seqlens_q, Tensor cu_seqlens_k, Tensor? seqused_k, "
                   "Tensor? leftpad_k, Tensor? block_table, Tensor? alibi_slopes, int max_seqlen_q, int max_seqlen_k, float p_dropout, "
                   "float softmax_scale, bool zero_tensors, bool is_causal, int window_size_left, int window_size_right, float softcap, "
                   "bool return_softmax, int num_splits, Generator? gen) -> (Tensor, Tensor)", _varlen_fwd),
    "varlen_fwd_compressed_kv": ("(Tensor q, Tensor k_idx, Tensor k_norm, Tensor v_idx, Tensor v_norm, Tensor cb_k, Tensor cb_v, "
                                 "Tensor(a!)? out, Tensor cu_seqlens_q, Tensor cu_seqlens_k, Tensor? alibi_slopes, int max_seqlen_q, "
                                 "int max_seqlen_k, float p_dropout, float softmax_scale, bool zero_tensors, bool is_causal, "
                                 "int window_size_left, int window_size_right, float softcap, bool return_softmax, int num_splits, "
                                 "Generator? gen) -> (Tensor, Tensor)", _varlen_fwd_compressed_kv),
    "varlen_fwd_compressed_kv_fused": ("(Tensor q, Tensor k_idx, Tensor k_norm, Tensor v_idx, Tensor v_norm, Tensor cb_k, Tensor cb_v, "
                                       "Tensor(a!)? out, Tensor cu_seqlens_q, Tensor? cu_seqlens_k, Tensor? seqused_k, Tensor? block_table, "
                                       "Tensor? alibi_slopes, int max_seqlen_q, int max_seqlen_k, float p_dropout, float softmax_scale, "
                                       "bool zero_tensors, bool is_causal, int window_size_left, int window_size_right, float softcap, "
                                       "bool return_softmax, int num_splits, bool uniform_codebook, Generator? gen) -> (Tensor, Tensor)",
                                       _varlen_fwd_compressed_kv_fused),
}


def register() -> None:
    """Define the namespace and its CUDA implementations (once per process)."""
    global _LIB
    if _LIB is not None:
        return
    ns = getattr(torch.ops, NAMESPACE, None)
    if ns is not None and hasattr(ns, "varlen_fwd"):
        _LIB = False                        # another extension (the reference's own) already owns the namespace
        return
    lib = torch.library.Library(NAMESPACE, "DEF")
    for name, (schema, fn) in _SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, fn, "CUDA")
    _LIB = lib


register()
