"""Generate the golden vectors under ``tests/golden/`` by running the REFERENCE project's own Python
(``cda.algorithm.compression`` / ``cda.algorithm.attention``) on CPU.

The reference tree is only needed to (re)generate; the ``.npz`` files are committed and the tests read
them alone.  Usage (from the repository root; ``CDA_REFERENCE`` is the path of the reference checkout)::

    CDA_REFERENCE=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

All inputs are seeded; the reference has no fixtures of its own, so these files are the pin.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

REF = os.environ.get("CDA_REFERENCE")
if not REF:
    raise SystemExit("set CDA_REFERENCE to the path of the reference checkout")
sys.path.insert(0, REF)
from cda.algorithm import attention as ref_attn          # noqa: E402
from cda.algorithm import compression as ref_comp        # noqa: E402

OUT = Path(__file__).resolve().parent
OUTLIER_CHANNELS = (3, 37, 64, 101)


def npy(t):
    return t.detach().cpu().numpy()


def synth_rows(gen, *shape, outliers=True):
    x = torch.randn(*shape, 128, generator=gen)
    if outliers:
        x[..., list(OUTLIER_CHANNELS)] *= 8.0
    return x.to(torch.float16)


def main():
    torch.set_num_threads(1)
    cmp16 = ref_comp.Compressor(128, num_levels=16)
    cmp4 = ref_comp.Compressor(128, num_levels=4)
    cmpu = ref_comp.Compressor(128, num_levels=16, codebook_mode="uniform")

    # 1. tables ------------------------------------------------------------------------------
    H = ref_comp.hadamard_matrix(128)
    np.savez_compressed(OUT / "tables.npz", cb16=npy(cmp16.codebook), cb4=npy(cmp4.codebook),
             cb16_uniform=npy(cmpu.codebook), hadamard_row1=npy(H[1]), hadamard_row2=npy(H[2]),
             hadamard_row77=npy(H[77]))

    # 2. encode ------------------------------------------------------------------------------
    g = torch.Generator().manual_seed(0xCDA + 1)
    x = synth_rows(g, 96)
    x[5] = 0                                   # norm floor path
    x[6] = (x[6].float() * 1e-4).to(torch.float16)
    x[7, :] = 0
    x[7, 9] = 1.0                              # rotated row of equal magnitudes
    x_rot = cmp16.rotate(x)
    e16 = cmp16.encode(x)
    e4 = cmp4.encode(x)
    eu = cmpu.encode(x)
    np.savez_compressed(OUT / "encode.npz", x=npy(x), x_rot=npy(x_rot), idx16=npy(e16.idx), norm16=npy(e16.norm),
             idx4=npy(e4.idx), norm4=npy(e4.norm), idx16_uniform=npy(eu.idx),
             dec16_rot=npy(cmp16.decode(e16, rotated=True)), dec4_rot=npy(cmp4.decode(e4, rotated=True)),
             dec16=npy(cmp16.decode(e16)))

    # 3. quantize known answers --------------------------------------------------------------
    cb = cmp16.codebook
    mids = (cb[:-1] + cb[1:]) * 0.5
    probe = torch.cat([torch.tensor([-1.0, 1.0, 0.0, -0.0]), cb, mids,
                       torch.nextafter(mids, torch.tensor(2.0)), torch.nextafter(mids, torch.tensor(-2.0))])
    np.savez_compressed(OUT / "quantize.npz", probe=npy(probe), idx16=npy(cmp16.quantize_unit(probe.clone())),
             idx4=npy(cmp4.quantize_unit(probe.clone())), idx16_uniform=npy(cmpu.quantize_unit(probe.clone())))

    # 4. decode attention, g=4, k4v4 ----------------------------------------------------------
    def attn_case(name, seed, B, Hkv, grp, Mq, N, ck, cv, *, causal=False, q_offset=0, window=None, splits=3):
        gg = torch.Generator().manual_seed(seed)
        Q = torch.randn(B, Hkv * grp, Mq, 128, generator=gg).to(torch.float16)
        K = synth_rows(gg, B, Hkv, N)
        V = synth_rows(gg, B, Hkv, N, outliers=False)
        Ks, Vs = ck.encode(K), cv.encode(V)
        out = ref_attn.attention_compressed(Q, Ks, Vs, cmp_K=ck, cmp_V=cv, group_size=grp,
                                            causal=causal, q_offset=q_offset)
        Q_rot = ck.rotate(Q)
        out_rot = ref_attn.attention_compressed_rotated_reference(
            Q_rot, Ks, Vs, cmp_K=ck, cmp_V=cv, group_size=grp, causal=causal, q_offset=q_offset)
        ws, we = window if window else (0, N)
        O, m, l = ref_attn.attention_compressed_partial_reference(
            Q_rot, Ks, Vs, cmp_K=ck, cmp_V=cv, group_size=grp, causal=causal, q_offset=q_offset,
            key_start=ws, key_end=we)
        split = ref_attn.attention_compressed_split_reference(
            Q_rot, Ks, Vs, cmp_K=ck, cmp_V=cv, group_size=grp, k_splits=splits, causal=causal,
            q_offset=q_offset)
        np.savez_compressed(OUT / f"{name}.npz", Q=npy(Q), K_idx=npy(Ks.idx), K_norm=npy(Ks.norm),
                 V_idx=npy(Vs.idx), V_norm=npy(Vs.norm), cb_K=npy(ck.codebook), cb_V=npy(cv.codebook),
                 out=npy(out), Q_rot=npy(Q_rot), out_rot=npy(out_rot), part_O=npy(O), part_m=npy(m),
                 part_l=npy(l), split_out=npy(split),
                 meta=np.array([B, Hkv, grp, Mq, N, int(causal), q_offset, ws, we, splits], dtype=np.int64))

    attn_case("decode_g4_k4v4", 0xCDA + 11, 2, 2, 4, 1, 77, cmp16, cmp16, window=(16, 50))
    attn_case("decode_g8_k4v2", 0xCDA + 12, 1, 2, 8, 1, 40, cmp16, cmp4, window=(0, 17), splits=4)
    attn_case("decode_g4_k2v2", 0xCDA + 13, 1, 1, 4, 1, 33, cmp4, cmp4, window=(5, 33), splits=2)
    attn_case("prefill_g4_k4v4", 0xCDA + 14, 1, 2, 4, 19, 45, cmp16, cmp16, causal=True, q_offset=26,
              window=(16, 45))

    # 5. integer-code score identity on the uniform table ------------------------------------
    gg = torch.Generator().manual_seed(0xCDA + 15)
    Q = torch.randn(1, 4, 1, 128, generator=gg).to(torch.float16)
    K = synth_rows(gg, 1, 1, 24)
    Ks = cmpu.encode(K)
    s = ref_attn.qk_scores_uniform_4bit_without_k_decode(cmpu.rotate(Q), Ks, group_size=4)
    np.savez_compressed(OUT / "uniform_scores.npz", Q_rot=npy(cmpu.rotate(Q)), K_idx=npy(Ks.idx), K_norm=npy(Ks.norm),
             scores=npy(s))
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
