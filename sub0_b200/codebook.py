"""Host-side tables for compressed-domain attention: the Hadamard rotation matrix and the scalar codebooks.

These are set-up-time utilities (the reference builds them once per process in Python too,
``cda/algorithm/compression.py:43-155``); kernels take the codebook as an input tensor and apply the rotation by
butterflies, so nothing here is on the hot path.
"""
from __future__ import annotations

import torch
from torch import Tensor

HEAD_DIM = 128

# Default tables of the reference (Lloyd-Max on the first coordinate of 100 000 seeded unit vectors, CPU generator,
# seed 0xCDA), as IEEE-754 bit patterns so that they do not depend on this machine's random-number stream.
_DEFAULT_16 = (0xbf700000, 0xbf500000, 0xbf300000, 0xbf100000, 0xbe401459, 0xbdf4d0d9, 0xbd8ead6c, 0xbcdadd51,
               0x3c4ec2dc, 0x3d546849, 0x3dbfc3a0, 0x3e117705, 0x3e560388, 0x3f300000, 0x3f500000, 0x3f700000)
_DEFAULT_4 = (0xbf400000, 0xbd8fba69, 0x3d91f2a4, 0x3f400000)


def hadamard_matrix(d: int = HEAD_DIM, *, dtype: torch.dtype = torch.float32, device=None) -> Tensor:
    """Orthonormal Sylvester-Hadamard matrix in natural order: ``H[i, j] = (-1)**popcount(i & j) / sqrt(d)``."""
    if d <= 0 or d & (d - 1):
        raise ValueError(f"d must be a positive power of two, got {d}")
    i = torch.arange(d)
    bits = i[:, None] & i[None, :]
    parity = torch.zeros_like(bits)
    while bool(bits.any()):
        parity ^= bits & 1
        bits >>= 1
    return ((1 - 2 * parity).to(torch.float32) / (d ** 0.5)).to(dtype=dtype, device=device)


def uniform_codebook(levels: int, *, device=None) -> Tensor:
    """Centres of ``levels`` equal bins on [-1, 1]."""
    edges = torch.linspace(-1.0, 1.0, levels + 1, dtype=torch.float32)
    return ((edges[:-1] + edges[1:]) * 0.5).contiguous().to(device)


def lloyd_max_codebook(levels: int, samples: Tensor, *, iters: int = 50, tol: float = 1e-7) -> Tensor:
    """Lloyd iteration from the uniform start; empty cells keep their level; sorted ascending."""
    samples = samples.flatten().float().cpu()
    cb = uniform_codebook(levels)
    for _ in range(iters):
        owner = (samples[:, None] - cb[None, :]).abs().argmin(dim=1)
        sums = torch.zeros(levels).index_add_(0, owner, samples)
        cnt = torch.zeros(levels).index_add_(0, owner, torch.ones_like(samples))
        nxt = torch.where(cnt > 0, sums / cnt.clamp_min(1), cb)
        moved = float((nxt - cb).abs().max())
        cb = nxt
        if moved < tol:
            break
    return cb.sort().values.contiguous()


def default_codebook(levels: int, *, device=None) -> Tensor:
    """The reference's default table for 16 (4-bit) or 4 (2-bit) levels, bit for bit."""
    if levels == 16:
        raw = _DEFAULT_16
    elif levels == 4:
        raw = _DEFAULT_4
    else:
        raise ValueError(f"levels must be 4 or 16 (got {levels})")
    return torch.tensor(raw, dtype=torch.int64).to(torch.int32).view(torch.float32).clone().to(device)
