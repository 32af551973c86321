"""A CPU model of the roundings the tcgen05 prefill kernel makes on top of the reference algorithm (test infrastructure).

The oracle follows the reference: K and V rows are decoded to fp16(level * norm) and everything else is fp32.  The kernel
differs in four documented places, and this model restates exactly those, so that a GPU test can hold the kernel to a
bound several times tighter than the path's stated tolerance against the model -- a wrong tile, mask or scale shows up
there even where the comparison with the oracle would still be inside its (wider) bound:

  1. K tile entries of a 2-bit side are fp16(level / alpha_k) -- no norm inside; the score is multiplied by
     norm_k * scale * log2(e) * alpha_k in fp32.  (A 4-bit side holds the reference's own rows, fp16(level * norm).)
  2. V tile entries of a 2-bit side are fp16 arithmetic on fp16(level / alpha_v): e * hi + fp16(e * lo) with
     hi = fp16(norm_v), lo = fp16(norm_v - hi), one rounding at the end; alpha_v multiplies the final normalisation.
     (A 4-bit side: the reference's own rows.)
  3. Probabilities are exp2(score - m) with m the largest score among the row's first 128 keys, rounded to fp16 for the
     P V product (later tiles move the reference by whole powers of two only, which does not change the rounding); the
     row sum adds the unrounded values.
  4. alpha = 1 for 16-level tables; for 4-level tables it is the first of 512 candidates 1 + i / 8192 whose worst
     |alpha * fp16(level / alpha) - level| is smallest.
The normalised rotated-frame row is rounded to fp16 and rotated back exactly as in the reference."""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import cda_oracle as O

LOG2E = 1.4426950408889634


def table_scale(cb: torch.Tensor) -> float:
    """Item 4 above (``find_table_scales`` of the CUDA sources), in the kernel's fp32 arithmetic."""
    if cb.numel() != 4:
        return 1.0
    lv = cb.to(torch.float32).numpy()
    best, arg = np.float32(3.0e38), 0
    for i in range(512):
        alpha = np.float32(1.0) + np.float32(i) * np.float32(1.0 / 8192.0)
        inv = np.float32(1.0) / alpha
        tv = (lv * inv).astype(np.float16).astype(np.float64)
        err = np.abs((np.float64(alpha) * tv - lv.astype(np.float64)).astype(np.float32)).max()   # fmaf: one rounding
        if err < best:
            best, arg = err, i
    return float(np.float32(1.0) + np.float32(arg) * np.float32(1.0 / 8192.0))


def round_mantissa_to_fp16(x: torch.Tensor) -> torch.Tensor:
    """fp32 values rounded (nearest even) to the 11 significant bits of fp16, without fp16's exponent range."""
    bits = x.contiguous().view(torch.int32)
    bits = (bits + 0x0FFF + ((bits >> 13) & 1)) & ~0x1FFF
    return bits.view(torch.float32)


def kernel_tiles(slot_k, slot_v, cb_K, cb_V, k_bits, v_bits):
    """K tile rows (fp32 tensor of fp16 values), the per-key score factor without the softmax scale, alpha_k, the V rows as
    the producers store them (fp32 tensor of fp16 values) and alpha_v for the final normalisation."""
    if k_bits == 4:
        k_rows, k_factor, ak = O.decode_rotated(slot_k, cb_K).float(), torch.ones_like(slot_k.norm.float()), 1.0
    else:
        ak = table_scale(cb_K)
        ki = O.unpack_indices(slot_k.idx, k_bits).long()
        k_rows, k_factor = (cb_K.float() * np.float32(1.0 / np.float32(ak))).half().float()[ki], slot_k.norm.float()
    if v_bits == 4:
        return k_rows, k_factor, ak, O.decode_rotated(slot_v, cb_V).float(), 1.0
    av = table_scale(cb_V)
    vi = O.unpack_indices(slot_v.idx, v_bits).long()
    v_lev = (cb_V.float() * np.float32(1.0 / np.float32(av))).half().float()[vi]
    n = slot_v.norm.float().unsqueeze(-1)
    hi = n.half().float()
    lo = (n - hi).half().float()
    t = (v_lev * lo).half().float()
    v_rows = (v_lev.double() * hi.double() + t.double()).half().float()          # fma.rn.f16x2: one rounding
    return k_rows, k_factor, ak, v_rows, av


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
        k_lev, k_norm, ak, v_rows, av = kernel_tiles(Ks, Vs, cb_K, cb_V, k_bits, v_bits)       # (1, H_kv, n, 128)
        q = O.rotate(Q[q0:q1].permute(1, 0, 2).unsqueeze(0), rot)                                # fp16 (1, H_q, Mq, 128)
        Hkv, Mq = k_lev.shape[1], q1 - q0
        s = torch.einsum("bhgmd,bhkd->bhgmk", q.float().view(1, Hkv, group, Mq, 128), k_lev)
        kscale = np.float32(np.float32(scale * LOG2E) * np.float32(ak))
        kn = (k_norm * kscale).view(1, Hkv, 1, 1, n)
        x = s * kn
        allowed = O._allowed(Mq, n, n - Mq)
        x = x.masked_fill(~allowed, float("-inf"))
        m = x[..., :128].max(dim=-1, keepdim=True).values      # the first tile always holds key 0, which every row sees
        p = torch.exp2(x - m)
        l = p.sum(dim=-1, keepdim=True)
        o = torch.einsum("bhgmk,bhkd->bhgmd", round_mantissa_to_fp16(p), v_rows) * (np.float32(av) / l)
        o16 = o.reshape(1, Hkv * group, Mq, 128).to(torch.float16)
        out[q0:q1] = O.unrotate(o16, rot).to(torch.float16)[0].permute(1, 0, 2)
    return out
