"""A CPU model of the arithmetic of the tcgen05 prefill kernel (test infrastructure).

The oracle follows the reference: K and V rows are decoded to fp16(level * norm) and everything else is fp32.  The
kernel's K and V tiles hold exactly those rows; it differs from the oracle in one documented place, which this model
restates, so that a GPU test can hold the kernel to the model as well as to the oracle:

  Probabilities are exp2(score - m) with m the largest score among the row's first 128 keys, rounded to fp16 for the
  P V product (later tiles move the reference by whole powers of two only, which does not change the rounding); the row
  sum adds the unrounded values.

The normalised rotated-frame row is rounded to fp16 and rotated back exactly as in the reference."""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import cda_oracle as O

LOG2E = 1.4426950408889634


def round_mantissa_to_fp16(x: torch.Tensor) -> torch.Tensor:
    """fp32 values rounded (nearest even) to the 11 significant bits of fp16, without fp16's exponent range."""
    bits = x.contiguous().view(torch.int32)
    bits = (bits + 0x0FFF + ((bits >> 13) & 1)) & ~0x1FFF
    return bits.view(torch.float32)


def paged_prefill_model(Q, flat_cache, block_table, cu_seqlens_q, seq_lens, *, cb_K, cb_V, group, block_size,
                        k_bits=4, v_bits=4, scale=None):
    """Same call as ``oracle.cda_oracle.paged_prefill``; the result the kernel's arithmetic gives."""
    rot = O.sylvester_hadamard()
    scale = 1.0 / math.sqrt(Q.shape[-1]) if scale is None else scale
    out = torch.zeros_like(Q)
    for b in range(cu_seqlens_q.numel() - 1):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        n = int(seq_lens[b])
        if q1 == q0 or n == 0:
            continue
        Ks, Vs = O.gather_sequence(flat_cache, block_table[b], n, block_size, k_bits, v_bits)
        k_rows, v_rows = O.decode_rotated(Ks, cb_K).float(), O.decode_rotated(Vs, cb_V).float()   # (1, H_kv, n, 128)
        q = O.rotate(Q[q0:q1].permute(1, 0, 2).unsqueeze(0), rot)                                # fp16 (1, H_q, Mq, 128)
        Hkv, Mq = k_rows.shape[1], q1 - q0
        s = torch.einsum("bhgmd,bhkd->bhgmk", q.float().view(1, Hkv, group, Mq, 128), k_rows)
        x = s * np.float32(scale * LOG2E)
        allowed = O._allowed(Mq, n, n - Mq)
        x = x.masked_fill(~allowed, float("-inf"))
        m = x[..., :128].max(dim=-1, keepdim=True).values      # the first tile always holds key 0, which every row sees
        p = torch.exp2(x - m)
        l = p.sum(dim=-1, keepdim=True)
        o = torch.einsum("bhgmk,bhkd->bhgmd", round_mantissa_to_fp16(p), v_rows) / l
        o16 = o.reshape(1, Hkv * group, Mq, 128).to(torch.float16)
        out[q0:q1] = O.unrotate(o16, rot).to(torch.float16)[0].permute(1, 0, 2)
    return out
