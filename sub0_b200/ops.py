"""Torch-tensor front end of the C ABI: checks dtype / device / contiguity, finds the current CUDA stream, owns the
grow-only decode workspace, and calls ``libcda_b200.so``.  PyTorch is used for device memory and streams only.

All functions enqueue on ``torch.cuda.current_stream()`` and never synchronise, so they may be captured in a CUDA
graph.  The split-KV workspace is either passed in (``workspace=``) or taken from a per-device cache that only grows;
growing it frees the old buffer, so the cache refuses to grow while a stream capture is in progress (size it first with
:func:`reserve_workspace` or by one eager call at the largest shape) -- a graph captured earlier keeps the pointer it
was captured with.  The cache assumes one stream per device: calls on different streams that share it would race.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib

HEAD_DIM = 128


def slot_bytes(k_bits: int = 4, v_bits: int = 4) -> int:
    rc = lib.cda_b200_slot_bytes(k_bits, v_bits)
    if rc < 0:
        check(rc)
    return rc


def _bits_of(cb: Tensor, what: str) -> int:
    n = cb.numel()
    if n == 16:
        return 4
    if n == 4:
        return 2
    raise ValueError(f"{what} must have 16 or 4 levels, got {n}")


def _cuda(t: Tensor, name: str, dtype: Optional[torch.dtype] = None) -> Tensor:
    if not isinstance(t, Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (sub0_b200 has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t


def _cb(cb: Tensor, dev: torch.device) -> Tensor:
    if cb.device != dev or cb.dtype != torch.float32 or not cb.is_contiguous():
        cb = cb.to(device=dev, dtype=torch.float32).contiguous()
    return cb


def _i32(t: Tensor) -> Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _flat_cache(kv_cache: Tensor) -> Tensor:
    """Accept (num_slots, H_kv, W) or (num_blocks, block_size, H_kv, W); uint8 or the fp16-typed view vLLM allocates."""
    c = kv_cache
    if c.dtype != torch.uint8:
        if c.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("kv_cache must be uint8 (or a 16-bit typed view of the same bytes)")
        c = c.view(torch.uint8)
    if c.dim() == 4:
        c = c.view(c.shape[0] * c.shape[1], c.shape[2], c.shape[3])
    if c.dim() != 3 or not c.is_contiguous():
        raise ValueError("kv_cache must be contiguous (num_slots, H_kv, slot_bytes)")
    return c


# ---- encode -----------------------------------------------------------------------------------------------------------

def paged_encode(K: Tensor, V: Tensor, slot_mapping: Tensor, flat_cache: Tensor, cb_K: Tensor, cb_V: Tensor) -> None:
    _cuda(K, "K"), _cuda(V, "V")
    if K.dtype != torch.float16 or V.dtype != torch.float16:
        raise TypeError("K, V must be fp16")
    if K.shape != V.shape or K.dim() != 3:
        raise ValueError("K and V must both be (T, H_kv, 128)")
    if K.shape[-1] != HEAD_DIM:
        raise ValueError(f"D must be 128, got {K.shape[-1]}")
    if flat_cache.dtype != torch.uint8:
        raise TypeError("flat_cache must be uint8")
    cache = _flat_cache(_cuda(flat_cache, "flat_cache"))
    kb, vb = _bits_of(cb_K, "cb_K"), _bits_of(cb_V, "cb_V")
    T, H = K.shape[0], K.shape[1]
    if cache.shape[1] != H:
        raise ValueError(f"cache has {cache.shape[1]} KV heads, K has {H}")
    if slot_mapping.numel() < T:
        raise ValueError("slot_mapping shorter than the token count")
    K, V = K.contiguous(), V.contiguous()
    sm = _i32(_cuda(slot_mapping, "slot_mapping")).contiguous()
    cbk, cbv = _cb(cb_K, K.device), _cb(cb_V, K.device)
    check(lib.cda_b200_paged_encode(K.data_ptr(), V.data_ptr(), sm.data_ptr(), cache.data_ptr(), cbk.data_ptr(),
                                    cbv.data_ptr(), T, H, cache.shape[0], cache.shape[2], kb, vb, _stream(K.device)))


def quantize_rotated(x_rot: Tensor, cb: Tensor):
    """(idx (rows, 16*bits) uint8, norm (rows) fp32) of rotated fp32 rows -- the encoder's index selection alone."""
    _cuda(x_rot, "x_rot", torch.float32)
    if x_rot.shape[-1] != HEAD_DIM:
        raise ValueError("last dim must be 128")
    bits = _bits_of(cb, "cb")
    x = x_rot.contiguous().view(-1, HEAD_DIM)
    idx = torch.empty(x.shape[0], 16 * bits, dtype=torch.uint8, device=x.device)
    norm = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    c = _cb(cb, x.device)
    check(lib.cda_b200_quantize_rotated(x.data_ptr(), x.shape[0], c.data_ptr(), bits, idx.data_ptr(), norm.data_ptr(),
                                        _stream(x.device)))
    return idx.view(*x_rot.shape[:-1], 16 * bits), norm.view(x_rot.shape[:-1])


def hadamard128(x: Tensor, out: Optional[Tensor] = None, scale: Optional[float] = None) -> Tensor:
    _cuda(x, "x", torch.float16)
    if x.shape[-1] != HEAD_DIM or not x.is_contiguous():
        raise ValueError("x must be contiguous (..., 128)")
    y = torch.empty_like(x) if out is None else out
    if y.shape != x.shape or y.dtype != torch.float16 or not y.is_contiguous() or not y.is_cuda:
        raise ValueError("out must be a contiguous fp16 CUDA tensor shaped like x")
    s = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
    check(lib.cda_b200_hadamard128(x.data_ptr(), y.data_ptr(), x.numel() // HEAD_DIM, s, _stream(x.device)))
    return y


# ---- decode -----------------------------------------------------------------------------------------------------------

_WORKSPACES: dict = {}


def decode_workspace_bytes(B: int, H_q: int, H_kv: int, max_seq_len: int, num_splits: int = 0, device: int = -1) -> int:
    return int(lib.cda_b200_decode_workspace_bytes(B, H_q, H_kv, max_seq_len, num_splits, device))


def plan_splits(B: int, H_kv: int, max_seq_len: int, device: int = -1) -> int:
    rc = lib.cda_b200_decode_plan_splits(B, H_kv, max_seq_len, device)
    if rc < 0:
        check(rc)
    return rc


def new_workspace(nbytes: int, device: torch.device) -> Tensor:
    """A zero-filled workspace (the first 256 bytes hold a device status word that must start at zero)."""
    return torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _workspace(need: int, dev: torch.device, given: Optional[Tensor]) -> Tensor:
    if given is not None:
        _cuda(given, "workspace", torch.uint8)
        if given.numel() < need:
            raise ValueError(f"workspace has {given.numel()} bytes, need {need}")
        return given
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"the cached decode workspace must grow to {need} bytes during a stream capture; call "
                               "ops.reserve_workspace() (or run the largest shape once) before capturing, or pass workspace=")
        ws = new_workspace(need, dev)
        _WORKSPACES[key] = ws
    return ws


def reserve_workspace(nbytes: int, device: Optional[torch.device] = None) -> Tensor:
    """Grow the cached per-device workspace to at least ``nbytes`` now (e.g. for the largest batch and context a server
    will see), so that later calls -- including captured ones -- never reallocate it."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return _workspace(int(nbytes), dev, None)


def workspace_status(workspace: Optional[Tensor] = None, device: Optional[torch.device] = None) -> int:
    """Read the device status word (synchronises).  Bit 0: a block-table entry was outside the cache."""
    if workspace is None:
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        workspace = _WORKSPACES.get((dev.type, dev.index if dev.index is not None else torch.cuda.current_device()))
        if workspace is None:
            return 0
    return int(workspace[:4].view(torch.int32).item())


class _DecodeArgs:
    __slots__ = ("Q", "cache", "bt", "sl", "cbk", "cbv", "B", "Hq", "Hkv", "bs", "kb", "vb", "scale", "max_len")


def _decode_args(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, scale, max_seq_len) -> _DecodeArgs:
    a = _DecodeArgs()
    _cuda(Q, "Q")
    if Q.dim() != 3 or Q.shape[-1] != HEAD_DIM:
        raise ValueError("Q must be (B, H_q, 128)")
    a.Q = (Q if Q.dtype == torch.float16 else Q.to(torch.float16)).contiguous()
    a.cache = _flat_cache(_cuda(kv_cache, "kv_cache"))
    a.bt = _i32(_cuda(block_table, "block_table")).contiguous()
    a.sl = _i32(_cuda(seq_lens, "seq_lens")).contiguous()
    a.kb, a.vb = _bits_of(cb_K, "cb_K"), _bits_of(cb_V, "cb_V")
    a.cbk, a.cbv = _cb(cb_K, Q.device), _cb(cb_V, Q.device)
    a.B, a.Hq = Q.shape[0], Q.shape[1]
    a.Hkv = a.cache.shape[1]
    a.bs = int(block_size)
    if a.bt.dim() != 2 or a.bt.shape[0] < a.B or a.sl.numel() < a.B:
        raise ValueError("block_table must be (B, max_blocks) and seq_lens (B,)")
    a.scale = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
    a.max_len = int(seq_lens.max().item()) if max_seq_len is None else int(max_seq_len)
    return a


def decode(Q: Tensor, kv_cache: Tensor, block_table: Tensor, seq_lens: Tensor, output: Tensor, *, cb_K: Tensor,
           cb_V: Tensor, block_size: int, scale: Optional[float] = None, max_seq_len: Optional[int] = None,
           num_splits: int = 0, workspace: Optional[Tensor] = None, lse: Optional[Tensor] = None) -> None:
    """``lse``: optional (B, H_q) fp32 buffer that receives the natural-log log-sum-exp of the scaled scores."""
    a = _decode_args(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, scale, max_seq_len)
    if output.dtype != torch.float16:
        raise ValueError("decode requires an fp16 output buffer")
    if not output.is_cuda or output.shape != Q.shape or not output.is_contiguous():
        raise ValueError("output must be a contiguous CUDA tensor shaped like Q")
    if lse is not None and (lse.dtype != torch.float32 or not lse.is_cuda or not lse.is_contiguous()
                            or lse.numel() != a.B * a.Hq):
        raise ValueError("lse must be a contiguous fp32 CUDA tensor of B * H_q elements")
    if a.B == 0:
        return
    need = decode_workspace_bytes(a.B, a.Hq, a.Hkv, a.max_len, num_splits)
    ws = _workspace(need, Q.device, workspace)
    if lse is None:
        check(lib.cda_b200_decode(a.Q.data_ptr(), a.cache.data_ptr(), a.bt.data_ptr(), a.sl.data_ptr(), a.cbk.data_ptr(),
                                  a.cbv.data_ptr(), output.data_ptr(), ws.data_ptr(), ws.numel(), a.B, a.Hq, a.Hkv, a.bs,
                                  a.bt.shape[1], a.max_len, a.cache.shape[0], a.cache.shape[2], a.kb, a.vb, a.scale,
                                  num_splits, _stream(Q.device)))
    else:
        check(lib.cda_b200_decode_lse(a.Q.data_ptr(), a.cache.data_ptr(), a.bt.data_ptr(), a.sl.data_ptr(),
                                      a.cbk.data_ptr(), a.cbv.data_ptr(), output.data_ptr(), lse.data_ptr(), ws.data_ptr(),
                                      ws.numel(), a.B, a.Hq, a.Hkv, a.bs, a.bt.shape[1], a.max_len, a.cache.shape[0],
                                      a.cache.shape[2], a.kb, a.vb, a.scale, num_splits, _stream(Q.device)))


def decode_partial(Q: Tensor, kv_cache: Tensor, block_table: Tensor, seq_lens: Tensor, *, cb_K: Tensor, cb_V: Tensor,
                   block_size: int, scale: Optional[float] = None, max_seq_len: Optional[int] = None,
                   num_splits: int = 0, workspace: Optional[Tensor] = None, out: Optional[Tensor] = None) -> Tensor:
    """Rotated-frame partial of the keys held in this cache, packed as (B, H_q, 130) fp32: 128 un-normalised O values,
    then m (natural-log domain), then l.  One tensor so that a sequence-sharded rank sends a single message; the merge
    kernel writes the packed rows directly (two launches in all)."""
    a = _decode_args(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, scale, max_seq_len)
    need = decode_workspace_bytes(a.B, a.Hq, a.Hkv, a.max_len, num_splits)
    ws = _workspace(need, Q.device, workspace)
    if out is None:
        packed = torch.empty(a.B, a.Hq, HEAD_DIM + 2, dtype=torch.float32, device=Q.device)
    else:
        packed = out
        if (packed.dtype != torch.float32 or not packed.is_cuda or not packed.is_contiguous()
                or packed.numel() != a.B * a.Hq * (HEAD_DIM + 2)):
            raise ValueError("out must be a contiguous fp32 CUDA tensor of B * H_q * 130 elements")
    if a.B:
        check(lib.cda_b200_decode_partial_packed(a.Q.data_ptr(), a.cache.data_ptr(), a.bt.data_ptr(), a.sl.data_ptr(),
                                                 a.cbk.data_ptr(), a.cbv.data_ptr(), packed.data_ptr(), ws.data_ptr(),
                                                 ws.numel(), a.B, a.Hq, a.Hkv, a.bs, a.bt.shape[1], a.max_len,
                                                 a.cache.shape[0], a.cache.shape[2], a.kb, a.vb, a.scale, num_splits,
                                                 _stream(Q.device)))
    return packed


def decode_exchange_bytes(B: int, H_q: int, world: int) -> int:
    """Bytes of one rank's exchange buffer for :func:`decode_exchange`."""
    return int(lib.cda_b200_decode_exchange_bytes(B, H_q, world))


def decode_exchange(Q: Tensor, kv_cache: Tensor, block_table: Tensor, seq_lens: Tensor, output: Tensor, *, cb_K: Tensor,
                    cb_V: Tensor, block_size: int, peer_pointers: Tensor, counters: Tensor, rank: int, world: int,
                    scale: Optional[float] = None, max_seq_len: Optional[int] = None, num_splits: int = 0,
                    wait_ms: int = 1000, workspace: Optional[Tensor] = None) -> None:
    """Sequence-sharded decode step with the exchange inside the merge kernel: this rank's keys are in ``kv_cache``, ``Q``
    is the same on every rank, ``output`` (B, H_q, 128) fp16 is the merged result on every rank.  ``peer_pointers``:
    int64 CUDA tensor of ``world`` device addresses (every rank's exchange buffer, see
    :class:`sub0_b200.sharding.PeerExchange`), ``counters``: two zeroed int64 on this device."""
    a = _decode_args(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, scale, max_seq_len)
    if output.dtype != torch.float16 or output.shape != Q.shape or not output.is_contiguous() or not output.is_cuda:
        raise ValueError("output must be a contiguous fp16 CUDA tensor shaped like Q")
    if peer_pointers.dtype != torch.int64 or not peer_pointers.is_cuda or peer_pointers.numel() != world:
        raise ValueError("peer_pointers must be an int64 CUDA tensor with one address per rank")
    if counters.dtype != torch.int64 or not counters.is_cuda or counters.numel() < 2:
        raise ValueError("counters must be an int64 CUDA tensor of two elements")
    need = decode_workspace_bytes(a.B, a.Hq, a.Hkv, a.max_len, num_splits)
    ws = _workspace(need, Q.device, workspace)
    check(lib.cda_b200_decode_exchange(a.Q.data_ptr(), a.cache.data_ptr(), a.bt.data_ptr(), a.sl.data_ptr(), a.cbk.data_ptr(),
                                       a.cbv.data_ptr(), output.data_ptr(), ws.data_ptr(), ws.numel(), peer_pointers.data_ptr(),
                                       counters.data_ptr(), rank, world, wait_ms, a.B, a.Hq, a.Hkv, a.bs, a.bt.shape[1],
                                       a.max_len, a.cache.shape[0], a.cache.shape[2], a.kb, a.vb, a.scale, num_splits,
                                       _stream(Q.device)))


def merge_partials(packed: Tensor, output: Tensor, *, unrotate: bool = True) -> None:
    """Merge (S, ..., 130) packed partials (see :func:`decode_partial`) into fp16 ``output`` (..., 128)."""
    _cuda(packed, "packed", torch.float32)
    if packed.shape[-1] != HEAD_DIM + 2 or packed.dim() < 2:
        raise ValueError("packed partials must be (S, ..., 130)")
    if output.dtype != torch.float16 or not output.is_cuda or not output.is_contiguous():
        raise ValueError("output must be a contiguous fp16 CUDA tensor")
    S = packed.shape[0]
    R = packed[0].numel() // (HEAD_DIM + 2)
    if output.numel() != R * HEAD_DIM:
        raise ValueError("output does not match the number of partial rows")
    flat = packed.contiguous()
    check(lib.cda_b200_merge_partials_packed(flat.data_ptr(), S, R, output.data_ptr(), 1 if unrotate else 0,
                                             _stream(packed.device)))


def decode_scalar(Q: Tensor, kv_cache: Tensor, block_table: Tensor, seq_lens: Tensor, output: Tensor, *, cb_K: Tensor,
                  cb_V: Tensor, block_size: int, scale: Optional[float] = None) -> None:
    """Slow device-side cross-check of :func:`decode` (no tensor cores, no splitting)."""
    a = _decode_args(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, block_size, scale, 0)
    if output.dtype != torch.float16 or output.shape != Q.shape or not output.is_contiguous():
        raise ValueError("output must be contiguous fp16 shaped like Q")
    check(lib.cda_b200_decode_scalar(a.Q.data_ptr(), a.cache.data_ptr(), a.bt.data_ptr(), a.sl.data_ptr(),
                                     a.cbk.data_ptr(), a.cbv.data_ptr(), output.data_ptr(), a.B, a.Hq, a.Hkv, a.bs,
                                     a.bt.shape[1], a.cache.shape[0], a.cache.shape[2], a.kb, a.vb, a.scale,
                                     _stream(Q.device)))


# ---- prefill ----------------------------------------------------------------------------------------------------------

def cache_to_dense_rotated(kv_cache: Tensor, block_table: Tensor, seq_lens: Tensor, *, cb_K: Tensor, cb_V: Tensor,
                           block_size: int, max_seq_len: int):
    cache = _flat_cache(_cuda(kv_cache, "kv_cache"))
    bt = _i32(_cuda(block_table, "block_table")).contiguous()
    sl = _i32(_cuda(seq_lens, "seq_lens")).contiguous()
    kb, vb = _bits_of(cb_K, "cb_K"), _bits_of(cb_V, "cb_V")
    dev = cache.device
    cbk, cbv = _cb(cb_K, dev), _cb(cb_V, dev)
    B, H = bt.shape[0], cache.shape[1]
    k = torch.empty(B * int(max_seq_len), H, HEAD_DIM, dtype=torch.float16, device=dev)
    v = torch.empty_like(k)
    check(lib.cda_b200_cache_to_dense_rotated(cache.data_ptr(), bt.data_ptr(), sl.data_ptr(), cbk.data_ptr(),
                                              cbv.data_ptr(), k.data_ptr(), v.data_ptr(), B, H, int(block_size),
                                              bt.shape[1], int(max_seq_len), cache.shape[0], cache.shape[2], kb, vb,
                                              _stream(dev)))
    return k, v


def prefill_varlen(Q: Tensor, kv_cache: Tensor, block_table: Tensor, cu_seqlens_q: Tensor, seq_lens: Tensor,
                   output: Tensor, *, cb_K: Tensor, cb_V: Tensor, block_size: int, max_query_len: int, max_seq_len: int,
                   scale: Optional[float] = None) -> None:
    _cuda(Q, "Q", torch.float16)
    if Q.dim() != 3 or Q.shape[-1] != HEAD_DIM:
        raise ValueError("Q must be (T, H_q, 128)")
    if output.shape != Q.shape or output.dtype != torch.float16 or not output.is_contiguous() or not output.is_cuda:
        raise ValueError("output must be a contiguous fp16 CUDA tensor shaped like Q")
    cache = _flat_cache(_cuda(kv_cache, "kv_cache"))
    bt = _i32(_cuda(block_table, "block_table")).contiguous()
    cu = _i32(_cuda(cu_seqlens_q, "cu_seqlens_q")).contiguous()
    sl = _i32(_cuda(seq_lens, "seq_lens")).contiguous()
    kb, vb = _bits_of(cb_K, "cb_K"), _bits_of(cb_V, "cb_V")
    cbk, cbv = _cb(cb_K, Q.device), _cb(cb_V, Q.device)
    Qc = Q.contiguous()
    s = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
    check(lib.cda_b200_prefill_varlen(Qc.data_ptr(), cache.data_ptr(), bt.data_ptr(), cu.data_ptr(), sl.data_ptr(),
                                      cbk.data_ptr(), cbv.data_ptr(), output.data_ptr(), Q.shape[0], cu.numel() - 1,
                                      Q.shape[1], cache.shape[1], int(block_size), bt.shape[1], int(max_query_len),
                                      int(max_seq_len), cache.shape[0], cache.shape[2], kb, vb, s, _stream(Q.device)))


def prefill_fault() -> bool:
    """True if a CTA of the paged prefill kernel gave up on one of its bounded waits on the current device since the
    last :func:`prefill_clear_status` (its rows of the output were then left unwritten, and later prefill launches
    return at once).  Synchronises the device."""
    rc = lib.cda_b200_prefill_fault()
    if rc < 0:
        check(rc)
    return rc != 0


PREFILL_BAD_BLOCK, PREFILL_WAIT_GAVE_UP, PREFILL_QLEN_EXCEEDS_SEQLEN = 1, 4, 8


def prefill_status() -> int:
    """Sticky status bits of the paged prefill kernel on the current device (``PREFILL_*``).  Synchronises the device."""
    rc = lib.cda_b200_prefill_status()
    if rc < 0:
        check(rc)
    return rc


def prefill_clear_status() -> None:
    check(lib.cda_b200_prefill_clear_status())


def prefill_debug(wait_limit_us: int = 0, withhold_first_k_arrive: bool = False) -> None:
    """Diagnostic knobs of the following prefill launches (see ``cda_b200_prefill_debug``); call with no arguments to
    restore the defaults."""
    check(lib.cda_b200_prefill_debug(int(wait_limit_us), 1 if withhold_first_k_arrive else 0))


def varlen_fwd_hadamard(Q: Tensor, k_rot: Tensor, v_rot: Tensor, output: Tensor, cu_seqlens_q: Tensor,
                        cu_seqlens_k: Tensor, seqused_k: Tensor, max_query_len: int, max_seq_len: int,
                        scale: float, *, mma_sync: bool = False) -> None:
    """Causal varlen attention over dense rotated-frame K/V on the tcgen05 kernel; ``mma_sync=True`` runs the independent
    mma.sync implementation instead (a cross-check)."""
    _cuda(Q, "Q", torch.float16), _cuda(k_rot, "k_rot", torch.float16), _cuda(v_rot, "v_rot", torch.float16)
    if Q.dim() != 3 or Q.shape[-1] != HEAD_DIM or k_rot.dim() != 3 or k_rot.shape != v_rot.shape:
        raise ValueError("Q must be (T, H_q, 128); k_rot, v_rot (rows, H_kv, 128)")
    if output.shape != Q.shape or output.dtype != torch.float16 or not output.is_contiguous():
        raise ValueError("output must be contiguous fp16 shaped like Q")
    Qc, kc, vc = Q.contiguous(), k_rot.contiguous(), v_rot.contiguous()
    cq, ck, su = (_i32(t).contiguous() for t in (cu_seqlens_q, cu_seqlens_k, seqused_k))
    fn = lib.cda_b200_varlen_fwd_hadamard_mma if mma_sync else lib.cda_b200_varlen_fwd_hadamard
    check(fn(Qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), output.data_ptr(), cq.data_ptr(), ck.data_ptr(), su.data_ptr(),
             Q.shape[0], cq.numel() - 1, Q.shape[1], k_rot.shape[1], int(max_query_len), int(max_seq_len), float(scale),
             _stream(Q.device)))
