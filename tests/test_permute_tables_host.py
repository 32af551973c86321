"""Host check of the byte-permute selection the prefill producers use to expand codes into exact fp16 rows.

The CUDA code (``expand_quad_exact`` / ``expand_quad_exact2`` in ``sub0_b200/csrc/prefill_umma.cu``) keeps a key's decoded
values ``fp16(level * norm)`` as byte planes in registers and picks them with ``prmt.b32``.  The selectors and the order
of the spread steps are restated here with a numpy ``prmt`` and run over random code words: the 8 (or 16) coordinates a
32-bit word of codes expands to must be the reference's ``Compressor.decode`` of those codes (compression.py:163-188,
:337-361, :375-397), in order."""
import numpy as np
import torch

from oracle import cda_oracle as O


def prmt(a: int, b: int, c: int) -> int:
    """PTX ``prmt.b32`` in its default mode: selector nibble k picks byte (nibble & 7) of {b, a}; with bit 3 set the byte's
    sign bit is replicated instead of the byte being copied.  Only c[15:0] is read."""
    src = [(a >> (8 * i)) & 0xFF for i in range(4)] + [(b >> (8 * i)) & 0xFF for i in range(4)]
    out = 0
    for k in range(4):
        sel = (c >> (4 * k)) & 0xF
        byte = src[sel & 7]
        if sel & 8:
            byte = 0xFF if byte & 0x80 else 0x00
        out |= byte << (8 * k)
    return out


def planes(values_fp16: np.ndarray):
    """Byte planes of 4 fp16 values: (low bytes, high bytes), value i in byte i."""
    bits = values_fp16.view(np.uint16).astype(np.uint32)
    h0, h1 = int(bits[0] | (bits[1] << 16)), int(bits[2] | (bits[3] << 16))
    return prmt(h0, h1, 0x6420), prmt(h0, h1, 0x7531)


def halves(word: int):
    return np.array([word & 0xFFFF, word >> 16], dtype=np.uint16).view(np.float16)


def expand_word_4bit(x: int, t16: np.ndarray) -> np.ndarray:
    lo = [planes(t16[4 * k:4 * k + 4])[0] for k in range(4)]
    hi = [planes(t16[4 * k:4 * k + 4])[1] for k in range(4)]
    m, y = x & 0x77777777, x & 0x88888888
    a = (y << 4) & 0xFFFFFFFF
    out = []
    for h in range(2):
        sel = (m >> 16) if h else m
        upper = prmt(a, y, 0xFBEA if h else 0xD9C8)
        la, lb = prmt(lo[0], lo[1], sel), prmt(lo[2], lo[3], sel)
        ha, hb = prmt(hi[0], hi[1], sel), prmt(hi[2], hi[3], sel)
        l = (lb & upper) | (la & ~upper & 0xFFFFFFFF)
        hh = (hb & upper) | (ha & ~upper & 0xFFFFFFFF)
        out += [halves(prmt(l, hh, 0x4051)), halves(prmt(l, hh, 0x6273))]
    return np.concatenate(out)


def expand_halfword_2bit(s: int, t16: np.ndarray) -> np.ndarray:
    lo, hi = planes(t16)
    s = (s | (s << 8)) & 0x00FF00FF
    s = (s | (s << 4)) & 0x0F0F0F0F
    s = (s | (s << 2)) & 0x33333333
    l0, h0 = prmt(lo, lo, s), prmt(hi, hi, s)
    l1, h1 = prmt(lo, lo, s >> 16), prmt(hi, hi, s >> 16)
    return np.concatenate([halves(prmt(l0, h0, 0x6273)), halves(prmt(l0, h0, 0x4051)),
                           halves(prmt(l1, h1, 0x6273)), halves(prmt(l1, h1, 0x4051))])


def reference_rows(code_bytes: np.ndarray, cb: torch.Tensor, norm: float, bits: int) -> np.ndarray:
    slot = O.Slot(torch.from_numpy(code_bytes.copy())[None], torch.tensor([norm], dtype=torch.float32))
    idx = O.unpack_indices(slot.idx, bits).long()
    return (cb.float()[idx] * slot.norm.unsqueeze(-1)).to(torch.float16)[0].numpy()


def test_four_bit_codes_select_the_reference_rows():
    rng = np.random.default_rng(4)
    cb = O.default_codebook(16)
    for norm in (1.0, 0.37, 23.5, 1e-12):
        t16 = (cb.float() * torch.tensor(norm, dtype=torch.float32)).to(torch.float16).numpy()
        for _ in range(200):
            code_bytes = rng.integers(0, 256, 4, dtype=np.uint8)
            x = int(code_bytes.view(np.uint32)[0])
            want = reference_rows(code_bytes, cb, norm, 4)
            assert np.array_equal(expand_word_4bit(x, t16).view(np.uint16), want.view(np.uint16))


def test_two_bit_codes_select_the_reference_rows():
    rng = np.random.default_rng(2)
    cb = O.default_codebook(4)
    for norm in (1.0, 0.37, 23.5):
        t16 = (cb.float() * torch.tensor(norm, dtype=torch.float32)).to(torch.float16).numpy()
        for _ in range(200):
            code_bytes = rng.integers(0, 256, 2, dtype=np.uint8)
            s = int(code_bytes.view(np.uint16)[0])
            want = reference_rows(code_bytes, cb, norm, 2)
            assert np.array_equal(expand_halfword_2bit(s, t16).view(np.uint16), want.view(np.uint16))
