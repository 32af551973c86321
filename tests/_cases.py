"""Seeded synthetic cases shared by the CPU and GPU tests: paged caches built with the CPU oracle's encoder."""
from __future__ import annotations

import torch

from oracle import cda_oracle as O

OUTLIER_CHANNELS = (3, 37, 64, 101)


def codebooks():
    return {4: O.default_codebook(16), 2: O.default_codebook(4)}


_CB = None


def cb_for(bits: int) -> torch.Tensor:
    global _CB
    if _CB is None:
        _CB = codebooks()
    return _CB[bits]


def rows(gen, *shape, outliers=False, scale=1.0):
    x = torch.randn(*shape, 128, generator=gen) * scale
    if outliers:
        x[..., list(OUTLIER_CHANNELS)] *= 8.0
    return x.to(torch.float16)


def paged_case(lens, *, H_kv=2, group=4, k_bits=4, v_bits=4, block_size=16, seed=0, shuffle=True, poison=0xFF,
               extra_blocks=3):
    """Build a paged cache holding sequences of the given lengths.  Returns a dict of CPU tensors:
    Q (B,H_q,128) fp16, cache (slots,H_kv,W) uint8, block_table (B,max_blocks) int32, seq_lens (B) int32, cb_K, cb_V, and
    the raw K/V rows per sequence.  Unused slots and pad bytes are filled with ``poison``."""
    gen = torch.Generator().manual_seed(seed)
    B = len(lens)
    nblk = [-(-n // block_size) for n in lens]
    total = sum(nblk) + extra_blocks
    order = torch.randperm(total, generator=gen) if shuffle else torch.arange(total)
    W = O.slot_bytes(k_bits, v_bits)
    cache = torch.full((total * block_size, H_kv, W), poison, dtype=torch.uint8)
    bt = torch.zeros(B, max(max(nblk), 1), dtype=torch.int32)
    cbk, cbv = cb_for(k_bits), cb_for(v_bits)
    raw, used = [], 0
    for b, n in enumerate(lens):
        k = rows(gen, n, H_kv, outliers=True)
        v = rows(gen, n, H_kv)
        bt[b, :nblk[b]] = order[used:used + nblk[b]].to(torch.int32)
        used += nblk[b]
        if n:
            slots = O.slots_of_sequence(bt[b], n, block_size).to(torch.int32)
            O.pack_slots(cache, slots, O.encode(k, cbk), O.encode(v, cbv), k_bits, v_bits)
        raw.append((k, v))
    Q = rows(gen, B, H_kv * group)
    return dict(Q=Q, cache=cache, block_table=bt, seq_lens=torch.tensor(lens, dtype=torch.int32), cb_K=cbk, cb_V=cbv,
                raw=raw, H_kv=H_kv, group=group, k_bits=k_bits, v_bits=v_bits, block_size=block_size)


def oracle_decode(case):
    return O.paged_decode(case["Q"], case["cache"], case["block_table"], case["seq_lens"], cb_K=case["cb_K"],
                          cb_V=case["cb_V"], group=case["group"], block_size=case["block_size"],
                          k_bits=case["k_bits"], v_bits=case["v_bits"])


def close(got: torch.Tensor, want: torch.Tensor, rtol=2e-3, atol=1e-3):
    """(ok, worst violation ratio, cosine).  Tolerance is the one the task states for fp16 attention outputs:
    |got - want| <= atol + rtol * |want|."""
    g, w = got.float().cpu(), want.float().cpu()
    err = (g - w).abs()
    bound = atol + rtol * w.abs()
    ratio = float((err / bound).max()) if err.numel() else 0.0
    cos = float(torch.nn.functional.cosine_similarity(g.flatten(), w.flatten(), dim=0)) if err.numel() else 1.0
    return ratio <= 1.0, ratio, cos
