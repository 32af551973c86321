"""CPU oracle for compressed-domain attention (CDA).

TEST INFRASTRUCTURE ONLY.  This module is the checker, never the product: it may be imported
by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.  Nothing under ``sub0_b200/`` imports it, and the product path raises when
its CUDA library is missing instead of falling back to this code.

It restates, in plain torch-on-CPU, the rotated-frame algorithm that the reference project
declares to be the correctness definition of its (closed) CUDA kernels:

* ``cda/algorithm/compression.py`` -- Hadamard rotation, scalar codebooks, encode / decode, packing;
* ``cda/algorithm/attention.py``   -- fp32 GQA attention on decoded K/V, split-KV partials, merge.

Each function cites the reference lines it follows.  Parity is pinned by golden vectors that were
produced by running the reference's own Python in the build container
(``tests/golden/make_golden.py`` -> ``tests/golden/*.npz``); ``tests/test_oracle_golden.py`` checks
this file against them.  The arithmetic deliberately uses the same torch primitives as the
reference (``bucketize``, fp32 ``matmul``, ``softmax``) so that, on one machine, results are
identical bit for bit.

In addition to the reference's functions this file defines the paged slot layout codec
(``pack_slots`` / ``unpack_slots``), which the reference only implements inside its closed encode
kernel; the byte layout follows ``cda/kernels_cuda/vllm_integration/cda_attn_v2.py:20-27,51-60``.
"""
from __future__ import annotations

import math
from typing import NamedTuple, Optional, Sequence

import torch
from torch import Tensor

HEAD_DIM = 128
NORM_FLOOR = 1e-12          # compression.py:328


# ----------------------------------------------------------------------------------------------
# Rotation (compression.py:43-57, 287-296)
# ----------------------------------------------------------------------------------------------

def sylvester_hadamard(d: int = HEAD_DIM) -> Tensor:
    """Orthonormal Sylvester-Hadamard matrix, natural (Kronecker) order: entry (i, j) is
    ``(-1)**popcount(i & j) / sqrt(d)``.  Built by the same doubling recursion and the same final
    division as compression.py:52-56 so the fp32 entries are identical."""
    if d <= 0 or d & (d - 1):
        raise ValueError(f"d must be a positive power of two, got {d}")
    h = torch.ones(1, 1, dtype=torch.float32)
    while h.shape[0] < d:
        top = torch.cat([h, h], dim=1)
        bot = torch.cat([h, -h], dim=1)
        h = torch.cat([top, bot], dim=0)
    return h / (d ** 0.5)


def rotate(x: Tensor, rot: Tensor) -> Tensor:
    """``x @ rot`` in fp32, cast back to ``x``'s dtype (compression.py:287-291)."""
    return torch.matmul(x.float(), rot).to(x.dtype)


def unrotate(x: Tensor, rot: Tensor) -> Tensor:
    """``x @ rot.T`` in fp32, cast back (compression.py:293-296)."""
    return torch.matmul(x.float(), rot.t()).to(x.dtype)


# ----------------------------------------------------------------------------------------------
# Codebooks (compression.py:75-155)
# ----------------------------------------------------------------------------------------------

def uniform_levels(levels: int) -> Tensor:
    """Bin centres of ``levels`` equal bins on [-1, 1] (compression.py:75-83)."""
    edges = torch.linspace(-1.0, 1.0, levels + 1, dtype=torch.float32)
    return ((edges[:-1] + edges[1:]) * 0.5).contiguous()


def lloyd_max_levels(levels: int, samples: Tensor, *, iters: int = 50, tol: float = 1e-7) -> Tensor:
    """Lloyd iteration from the uniform start; a level whose cell is empty keeps its value
    (compression.py:116-155).  Output sorted ascending."""
    samples = samples.flatten()
    cb = uniform_levels(levels).to(samples.dtype)
    for _ in range(iters):
        owner = (samples[:, None] - cb[None, :]).pow(2).argmin(dim=1)
        nxt = cb.clone()
        for c in range(levels):
            sel = owner == c
            if bool(sel.any()):
                nxt[c] = samples[sel].mean()
        moved = float((nxt - cb).abs().max())
        cb = nxt
        if moved < tol:
            break
    return cb.sort().values.contiguous()


def default_codebook(levels: int, d: int = HEAD_DIM, *, seed: int = 0xCDA,
                     n_samples: int = 100_000) -> Tensor:
    """The reference's default ("lloyd_beta") table: Lloyd-Max on the first coordinate of
    ``n_samples`` seeded Gaussian vectors projected to the unit sphere, CPU generator
    (compression.py:86-113)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(n_samples, d, dtype=torch.float32, generator=g)
    unit = x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    return lloyd_max_levels(levels, unit[:, 0])


# ----------------------------------------------------------------------------------------------
# Index packing (compression.py:163-188, 375-397)
# ----------------------------------------------------------------------------------------------

def bits_for_levels(levels: int) -> int:
    if levels == 16:
        return 4
    if levels == 4:
        return 2
    raise ValueError(f"codebook must have 4 or 16 levels, got {levels}")


def pack_indices(idx: Tensor, bits: int) -> Tensor:
    """MSB-first packing: 4-bit -> byte j = idx[2j] << 4 | idx[2j+1];
    2-bit -> byte j = idx[4j] << 6 | idx[4j+1] << 4 | idx[4j+2] << 2 | idx[4j+3]."""
    idx = idx.to(torch.uint8)
    per = 8 // bits
    if idx.shape[-1] % per:
        raise ValueError("last dim not divisible by values-per-byte")
    grouped = idx.reshape(*idx.shape[:-1], idx.shape[-1] // per, per)
    out = torch.zeros(grouped.shape[:-1], dtype=torch.uint8)
    for k in range(per):
        out |= grouped[..., k] << (bits * (per - 1 - k))
    return out.contiguous()


def unpack_indices(packed: Tensor, bits: int) -> Tensor:
    per = 8 // bits
    mask = (1 << bits) - 1
    parts = [(packed >> (bits * (per - 1 - k))) & mask for k in range(per)]
    return torch.stack(parts, dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * per).contiguous()


# ----------------------------------------------------------------------------------------------
# Encode / decode of rows (compression.py:298-361)
# ----------------------------------------------------------------------------------------------

class Slot(NamedTuple):
    """Encoded rows: ``idx`` (..., 128 * bits / 8) uint8 and ``norm`` (...) fp32
    (compression.py:196-205)."""
    idx: Tensor
    norm: Tensor


def nearest_level(x_unit: Tensor, cb: Tensor) -> Tensor:
    """Nearest entry of the sorted table ``cb`` (compression.py:298-313): ``upper`` = number of
    entries strictly below x (``bucketize``), clamped to the last index; ``lower`` = the entry
    before it; ``upper`` wins only when strictly closer, so an exact midpoint goes down."""
    levels = cb.numel()
    upper = torch.bucketize(x_unit.contiguous(), cb).clamp_(0, levels - 1)
    lower = (upper - 1).clamp_(min=0)
    take_upper = (cb[upper] - x_unit).abs() < (x_unit - cb[lower]).abs()
    return torch.where(take_upper, upper, lower).to(torch.uint8)


def quantize_rotated(x_rot: Tensor, cb: Tensor, *, norm: Optional[Tensor] = None) -> Slot:
    """Steps 2-5 of encode on an already rotated fp32 row (compression.py:328-335).  ``norm`` may be
    supplied (e.g. the norm a kernel computed) so that index parity can be tested on identical
    fp32 quotients."""
    x_rot = x_rot.float()
    if norm is None:
        norm = x_rot.norm(dim=-1).clamp_min(NORM_FLOOR)
    unit = (x_rot / norm.unsqueeze(-1)).clamp_(-1.0, 1.0)
    idx = nearest_level(unit, cb)
    return Slot(pack_indices(idx, bits_for_levels(cb.numel())), norm.contiguous())


def encode(x: Tensor, cb: Tensor, rot: Optional[Tensor] = None) -> Slot:
    """Rotate (result rounded to ``x``'s dtype), normalise, pick levels, pack
    (compression.py:315-335)."""
    if x.shape[-1] != HEAD_DIM and rot is None:
        raise ValueError("last dim must be 128")
    rot = sylvester_hadamard(x.shape[-1]) if rot is None else rot
    return quantize_rotated(rotate(x, rot).float(), cb)


def decode_rotated(slot: Slot, cb: Tensor, *, dtype: torch.dtype = torch.float16) -> Tensor:
    """``cb[idx] * norm`` in fp32, then cast -- values stay in the rotated frame
    (compression.py:337-360 with ``rotated=True``)."""
    idx = unpack_indices(slot.idx, bits_for_levels(cb.numel()))
    return (cb[idx.long()] * slot.norm.unsqueeze(-1)).to(dtype)


# ----------------------------------------------------------------------------------------------
# Attention (attention.py:46-93, 190-272, 306-482)
# ----------------------------------------------------------------------------------------------

def _allowed(m_q: int, m_k: int, q_offset: int) -> Tensor:
    """Lower-right causal rule: query row q sees keys 0..q+q_offset (attention.py:46-57)."""
    q = torch.arange(m_q).unsqueeze(1) + q_offset
    return torch.arange(m_k).unsqueeze(0) <= q


def _scores(Q: Tensor, K: Tensor, group: int, scale: Optional[float], causal: bool,
            q_offset: int) -> Tensor:
    B, Hq, Mq, D = Q.shape
    Hkv, Mk = K.shape[1], K.shape[2]
    if Hq != Hkv * group:
        raise ValueError(f"H_q={Hq} != H_kv*group={Hkv * group}")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    s = torch.einsum("bhgmd,bhkd->bhgmk", Q.float().view(B, Hkv, group, Mq, D), K.float()) * scale
    if causal:
        s = s.masked_fill(~_allowed(Mq, Mk, q_offset), float("-inf"))
    return s


def gqa_attention(Q: Tensor, K: Tensor, V: Tensor, *, group: int, scale: Optional[float] = None,
                  causal: bool = False, q_offset: int = 0) -> Tensor:
    """fp32 softmax attention; query head h reads KV head h // group; fp16 result
    (attention.py:60-93)."""
    B, Hq, Mq, D = Q.shape
    p = torch.softmax(_scores(Q, K, group, scale, causal, q_offset), dim=-1)
    o = torch.einsum("bhgmk,bhkd->bhgmd", p, V.float())
    return o.reshape(B, Hq, Mq, D).to(torch.float16)


def gqa_partial(Q: Tensor, K: Tensor, V: Tensor, *, group: int, scale: Optional[float] = None,
                causal: bool = False, q_offset: int = 0):
    """Split-KV contract (attention.py:190-236): ``m`` row max, ``l = sum exp(s - m)``,
    ``O = sum exp(s - m) V`` un-normalised, all fp32; NaNs from all-masked rows become 0."""
    B, Hq, Mq, D = Q.shape
    s = _scores(Q, K, group, scale, causal, q_offset)
    m = s.max(dim=-1).values
    p = torch.exp(s - m.unsqueeze(-1))
    p = torch.where(p.isnan(), torch.zeros_like(p), p)
    o = torch.einsum("bhgmk,bhkd->bhgmd", p, V.float())
    return o.reshape(B, Hq, Mq, D), m.reshape(B, Hq, Mq), p.sum(dim=-1).reshape(B, Hq, Mq)


def merge_partials(parts: Sequence) -> Tensor:
    """Log-sum-exp merge of (O, m, l) partials over disjoint key ranges (attention.py:239-272)."""
    if not parts:
        raise ValueError("no partials to merge")
    O = torch.stack([p[0] for p in parts])
    m = torch.stack([p[1] for p in parts])
    l = torch.stack([p[2] for p in parts])
    if len(parts) == 1:
        return (O[0] / l[0].unsqueeze(-1).clamp_min(1e-30)).to(torch.float16)
    top = m.max(dim=0).values
    w = (m - top.unsqueeze(0)).exp()
    w = torch.where(w.isnan(), torch.zeros_like(w), w)
    denom = (l * w).sum(dim=0)
    num = (O * w.unsqueeze(-1)).sum(dim=0)
    return (num / denom.unsqueeze(-1).clamp_min(1e-30)).to(torch.float16)


def _window(slot: Slot, start: int, end: Optional[int]) -> Slot:
    n = slot.norm.shape[-1]
    end = n if end is None else end
    if not 0 <= start <= end <= n:
        raise ValueError(f"invalid key window [{start}, {end}) for length {n}")
    return Slot(slot.idx[..., start:end, :].contiguous(), slot.norm[..., start:end].contiguous())


def cda_attention_rotated(Q_rot: Tensor, K_slot: Slot, V_slot: Slot, *, cb_K: Tensor, cb_V: Tensor,
                          group: int, scale: Optional[float] = None, causal: bool = False,
                          q_offset: int = 0, key_start: int = 0,
                          key_end: Optional[int] = None) -> Tensor:
    """Decode K/V of the key window to fp16 in the rotated frame and attend; output stays rotated
    (attention.py:306-346)."""
    K = decode_rotated(_window(K_slot, key_start, key_end), cb_K)
    V = decode_rotated(_window(V_slot, key_start, key_end), cb_V)
    off = q_offset - key_start if causal else q_offset
    return gqa_attention(Q_rot, K, V, group=group, scale=scale, causal=causal, q_offset=off)


def cda_partial_rotated(Q_rot: Tensor, K_slot: Slot, V_slot: Slot, *, cb_K: Tensor, cb_V: Tensor,
                        group: int, scale: Optional[float] = None, causal: bool = False,
                        q_offset: int = 0, key_start: int = 0, key_end: Optional[int] = None):
    """(O, m, l) of one key window (attention.py:349-384)."""
    K = decode_rotated(_window(K_slot, key_start, key_end), cb_K)
    V = decode_rotated(_window(V_slot, key_start, key_end), cb_V)
    off = q_offset - key_start if causal else q_offset
    return gqa_partial(Q_rot, K, V, group=group, scale=scale, causal=causal, q_offset=off)


def cda_attention_split(Q_rot: Tensor, K_slot: Slot, V_slot: Slot, *, cb_K: Tensor, cb_V: Tensor,
                        group: int, k_splits: int, scale: Optional[float] = None,
                        causal: bool = False, q_offset: int = 0) -> Tensor:
    """Equal-chunk split + merge (attention.py:387-423)."""
    if k_splits < 1:
        raise ValueError("k_splits must be >= 1")
    n = K_slot.norm.shape[-1]
    if n <= 0:
        raise ValueError("need at least one key")
    chunk = -(-n // k_splits)
    return merge_partials([
        cda_partial_rotated(Q_rot, K_slot, V_slot, cb_K=cb_K, cb_V=cb_V, group=group, scale=scale,
                            causal=causal, q_offset=q_offset, key_start=s, key_end=min(s + chunk, n))
        for s in range(0, n, chunk)])


def cda_attention(Q: Tensor, K_slot: Slot, V_slot: Slot, *, cb_K: Tensor, cb_V: Tensor, group: int,
                  scale: Optional[float] = None, causal: bool = False, q_offset: int = 0,
                  rot: Optional[Tensor] = None) -> Tensor:
    """The decode / prefill oracle (attention.py:426-482): rotate Q (rounded to fp16), attend over
    decoded K/V in the rotated frame, rotate the fp16 result back, fp16 out.
    Shapes: Q (B, H_q, M_q, 128); slots indexed (B, H_kv, M_k, ...)."""
    rot = sylvester_hadamard(Q.shape[-1]) if rot is None else rot
    o_rot = cda_attention_rotated(rotate(Q, rot), K_slot, V_slot, cb_K=cb_K, cb_V=cb_V, group=group,
                                  scale=scale, causal=causal, q_offset=q_offset)
    return unrotate(o_rot, rot).to(torch.float16)


def uniform16_scores(Q_rot: Tensor, K_slot: Slot, *, group: int, scale: Optional[float] = None) -> Tensor:
    """QK scores from integer codes for the 16-level uniform table, where
    ``K[k, d] = norm[k] * (code / 8 - 15 / 16)`` (attention.py:101-155); an independent check."""
    B, Hq, Mq, D = Q_rot.shape
    Hkv = K_slot.idx.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    codes = unpack_indices(K_slot.idx, 4).float()
    Qg = Q_rot.float().view(B, Hkv, group, Mq, D)
    dot = torch.einsum("bhgmd,bhkd->bhgmk", Qg, codes)
    tot = Qg.sum(dim=-1).unsqueeze(-1)
    return K_slot.norm.float()[:, :, None, None, :] * (dot * 0.125 - tot * 0.9375) * scale


# ----------------------------------------------------------------------------------------------
# Paged slot layout (cda_attn_v2.py:20-27, 51-60; the byte order the closed encode kernel writes,
# wrappers.py:136-142)
# ----------------------------------------------------------------------------------------------

def slot_payload_bytes(k_bits: int, v_bits: int) -> int:
    """K indices | V indices | fp32 K norm | fp32 V norm."""
    return HEAD_DIM * k_bits // 8 + HEAD_DIM * v_bits // 8 + 8


def slot_bytes(k_bits: int, v_bits: int) -> int:
    """Payload rounded up to 16 B so every slot starts on a 16-byte boundary
    (cda_attn_v2.py:53-58): 144 for k4v4, 112 for k4v2, 80 for k2v2."""
    return (slot_payload_bytes(k_bits, v_bits) + 15) // 16 * 16


def pack_slots(flat_cache: Tensor, slot_mapping: Tensor, K_slot: Slot, V_slot: Slot,
               k_bits: int = 4, v_bits: int = 4) -> None:
    """Scatter encoded tokens into ``flat_cache`` (num_slots, H_kv, slot_w) uint8.  ``K_slot.idx`` is
    (T, H_kv, 128*k_bits/8) and ``K_slot.norm`` (T, H_kv); entries of ``slot_mapping`` below zero
    are skipped.  Pad bytes are not written."""
    kb, vb = HEAD_DIM * k_bits // 8, HEAD_DIM * v_bits // 8
    keep = slot_mapping >= 0
    dst = slot_mapping[keep].long()
    flat_cache[dst, :, 0:kb] = K_slot.idx[keep]
    flat_cache[dst, :, kb:kb + vb] = V_slot.idx[keep]
    flat_cache[dst, :, kb + vb:kb + vb + 4] = K_slot.norm[keep].contiguous().view(torch.uint8).reshape(
        -1, K_slot.norm.shape[1], 4)
    flat_cache[dst, :, kb + vb + 4:kb + vb + 8] = V_slot.norm[keep].contiguous().view(torch.uint8).reshape(
        -1, V_slot.norm.shape[1], 4)


def unpack_slots(flat_cache: Tensor, slots: Tensor, k_bits: int = 4, v_bits: int = 4):
    """Inverse of :func:`pack_slots` for the slot ids in ``slots`` (T,): returns
    ``(K_slot, V_slot)`` with leading shape (T, H_kv)."""
    kb, vb = HEAD_DIM * k_bits // 8, HEAD_DIM * v_bits // 8
    rows = flat_cache[slots.long()]
    kn = rows[:, :, kb + vb:kb + vb + 4].contiguous().view(torch.float32).squeeze(-1)
    vn = rows[:, :, kb + vb + 4:kb + vb + 8].contiguous().view(torch.float32).squeeze(-1)
    return Slot(rows[:, :, 0:kb].contiguous(), kn), Slot(rows[:, :, kb:kb + vb].contiguous(), vn)


def slots_of_sequence(block_table_row: Tensor, seq_len: int, block_size: int) -> Tensor:
    """Slot id of token n: ``block_table[n // block_size] * block_size + n % block_size``."""
    n = torch.arange(seq_len)
    return block_table_row.long()[n // block_size] * block_size + n % block_size


def gather_sequence(flat_cache: Tensor, block_table_row: Tensor, seq_len: int, block_size: int,
                    k_bits: int = 4, v_bits: int = 4):
    """Slots of one sequence as (1, H_kv, N, ...) tensors ready for :func:`cda_attention`."""
    K, V = unpack_slots(flat_cache, slots_of_sequence(block_table_row, seq_len, block_size), k_bits, v_bits)
    tr = lambda s: Slot(s.idx.permute(1, 0, 2).unsqueeze(0).contiguous(),
                        s.norm.permute(1, 0).unsqueeze(0).contiguous())
    return tr(K), tr(V)


def paged_decode(Q: Tensor, flat_cache: Tensor, block_table: Tensor, seq_lens: Tensor, *, cb_K: Tensor,
                 cb_V: Tensor, group: int, block_size: int, scale: Optional[float] = None,
                 k_bits: int = 4, v_bits: int = 4) -> Tensor:
    """What ``decode_hmma_v1`` (wrappers.py:79-124) must produce: per sequence b, the oracle
    :func:`cda_attention` over that sequence's slots.  Q, result: (B, H_q, 128) fp16."""
    outs = []
    for b in range(Q.shape[0]):
        n = int(seq_lens[b])
        if n == 0:
            outs.append(torch.zeros_like(Q[b]))
            continue
        Ks, Vs = gather_sequence(flat_cache, block_table[b], n, block_size, k_bits, v_bits)
        o = cda_attention(Q[b].unsqueeze(0).unsqueeze(2), Ks, Vs, cb_K=cb_K, cb_V=cb_V, group=group, scale=scale)
        outs.append(o[0, :, 0])
    return torch.stack(outs)


def paged_prefill(Q: Tensor, flat_cache: Tensor, block_table: Tensor, cu_seqlens_q: Tensor,
                  seq_lens: Tensor, *, cb_K: Tensor, cb_V: Tensor, group: int, block_size: int,
                  scale: Optional[float] = None, k_bits: int = 4, v_bits: int = 4) -> Tensor:
    """What ``fa2_cda_prefill_varlen_v1`` (fa2_cda.py:98-230) must produce: causal attention of each
    sequence's query chunk against all of its cached keys, bottom-right aligned
    (``q_offset = seq_len - q_len``, fa2_cda.py:121-125).  Q, result: (T, H_q, 128) fp16."""
    out = torch.zeros_like(Q)
    for b in range(cu_seqlens_q.numel() - 1):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        n = int(seq_lens[b])
        if q1 == q0 or n == 0:
            continue
        Ks, Vs = gather_sequence(flat_cache, block_table[b], n, block_size, k_bits, v_bits)
        q = Q[q0:q1].permute(1, 0, 2).unsqueeze(0)
        o = cda_attention(q, Ks, Vs, cb_K=cb_K, cb_V=cb_V, group=group, scale=scale, causal=True,
                          q_offset=n - (q1 - q0))
        out[q0:q1] = o[0].permute(1, 0, 2)
    return out


def dense_rotated(flat_cache: Tensor, block_table: Tensor, seq_lens: Tensor, *, cb_K: Tensor, cb_V: Tensor,
                  block_size: int, max_seq_len: int, k_bits: int = 4, v_bits: int = 4):
    """What ``paged_cache_to_dense_rotated`` (fa2_cda.py:64-95) must produce: decoded rotated-frame fp16
    K and V, (B * max_seq_len, H_kv, 128), rows at or beyond ``seq_lens[b]`` zero."""
    B, Hkv = block_table.shape[0], flat_cache.shape[1]
    k = torch.zeros(B * max_seq_len, Hkv, HEAD_DIM, dtype=torch.float16)
    v = torch.zeros_like(k)
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            continue
        Ks, Vs = unpack_slots(flat_cache, slots_of_sequence(block_table[b], n, block_size), k_bits, v_bits)
        k[b * max_seq_len:b * max_seq_len + n] = decode_rotated(Ks, cb_K)
        v[b * max_seq_len:b * max_seq_len + n] = decode_rotated(Vs, cb_V)
    return k, v
