"""Seeded synthetic decode workloads built on the GPU with this package's own encoder.

Stand-in for real model activations: Q, K, V ~ N(0, 1) in fp16, with four fixed K channels scaled x8 ("outlier
channels", the same four for every KV head), encoded into a paged cache whose block table is a seeded random
permutation of the pages.  Sequence b's tensors depend only on (seed, b), never on how KV heads are sharded, so a
head-sharded run sees exactly the slices of the single-GPU data.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from . import ops
from .codebook import default_codebook

OUTLIER_CHANNELS = (3, 37, 64, 101)
HEAD_DIM = 128


@dataclass
class DecodeWorkload:
    Q: Tensor              # (B, H_q_local, 128) fp16
    cache: Tensor          # (slots, H_kv_local, slot_bytes) uint8
    block_table: Tensor    # (B, blocks_per_seq) int32
    seq_lens: Tensor       # (B,) int32
    cb_K: Tensor
    cb_V: Tensor
    group: int
    block_size: int
    k_bits: int
    v_bits: int
    N: int

    @property
    def B(self) -> int:
        return self.Q.shape[0]

    @property
    def H_kv(self) -> int:
        return self.cache.shape[1]

    def algorithmic_bytes(self) -> int:
        """Bytes one decode call must move: payload of every visited slot (indices + two fp32 norms, pad excluded),
        Q in and out (fp16), the block-table entries and sequence lengths."""
        payload = 16 * self.k_bits + 16 * self.v_bits + 8
        B, Hq = self.Q.shape[0], self.Q.shape[1]
        blocks = -(-self.N // self.block_size)
        return B * self.H_kv * self.N * payload + B * Hq * HEAD_DIM * 2 * 2 + B * blocks * 4 + B * 4


def sequence_tensors(seed: int, b: int, N: int, H_kv: int, group: int, device) -> tuple[Tensor, Tensor, Tensor]:
    """(q (H_q,128), K (N,H_kv,128), V (N,H_kv,128)) fp16 of sequence b (all KV heads)."""
    gen = torch.Generator(device=device).manual_seed(seed + 1_000_003 * (b + 1))
    q = torch.randn(H_kv * group, HEAD_DIM, generator=gen, device=device, dtype=torch.float32).to(torch.float16)
    K = torch.randn(N, H_kv, HEAD_DIM, generator=gen, device=device, dtype=torch.float32)
    K[..., list(OUTLIER_CHANNELS)] *= 8.0
    V = torch.randn(N, H_kv, HEAD_DIM, generator=gen, device=device, dtype=torch.float32)
    return q, K.to(torch.float16), V.to(torch.float16)


def build_decode_workload(B: int, N: int, *, H_kv: int = 8, group: int = 4, k_bits: int = 4, v_bits: int = 4,
                          block_size: int = 16, seed: int | None = None, device="cuda", head_lo: int = 0,
                          head_hi: int | None = None, shuffle_pages: bool = True) -> DecodeWorkload:
    """Encode B sequences of N tokens into a fresh paged cache holding KV heads [head_lo, head_hi) only."""
    device = torch.device(device)
    head_hi = H_kv if head_hi is None else head_hi
    hl = head_hi - head_lo
    seed = 0xCDA + N + 97 * B if seed is None else seed
    blocks = -(-N // block_size)
    W = ops.slot_bytes(k_bits, v_bits)
    cache = torch.zeros(B * blocks * block_size, hl, W, dtype=torch.uint8, device=device)
    pg = torch.Generator().manual_seed(seed)
    order = torch.randperm(B * blocks, generator=pg) if shuffle_pages else torch.arange(B * blocks)
    bt = order.view(B, blocks).to(torch.int32).to(device)
    cbk = default_codebook(16 if k_bits == 4 else 4, device=device)
    cbv = default_codebook(16 if v_bits == 4 else 4, device=device)
    Q = torch.empty(B, hl * group, HEAD_DIM, dtype=torch.float16, device=device)
    pos = torch.arange(N, device=device)
    for b in range(B):
        q, K, V = sequence_tensors(seed, b, N, H_kv, group, device)
        Q[b] = q[head_lo * group:head_hi * group]
        slots = (bt[b].long()[pos // block_size] * block_size + pos % block_size).to(torch.int32)
        ops.paged_encode(K[:, head_lo:head_hi].contiguous(), V[:, head_lo:head_hi].contiguous(), slots, cache, cbk, cbv)
    return DecodeWorkload(Q=Q, cache=cache, block_table=bt, seq_lens=torch.full((B,), N, dtype=torch.int32, device=device),
                          cb_K=cbk, cb_V=cbv, group=group, block_size=block_size, k_bits=k_bits, v_bits=v_bits, N=N)
