"""The CPU oracle (``oracle/cda_oracle.py``) against golden vectors produced by the reference's own
Python (``tests/golden/make_golden.py``), plus the known answers that follow from the reference source.

Integer results (indices, packed bytes) must match exactly whenever the floating-point inputs are
identical; end-to-end paths that pass through an fp32 matmul or reduction (whose summation order may
differ between CPUs) are compared within stated tolerances.
"""
import math

import numpy as np
import pytest
import torch

from oracle import cda_oracle as O

T = torch.from_numpy


def slot(idx, norm):
    return O.Slot(T(idx), T(norm))


# ---- tables -----------------------------------------------------------------------------------

def test_default_codebooks_match_reference(golden):
    g = golden("tables")
    assert torch.equal(O.default_codebook(16), T(g["cb16"]))
    assert torch.equal(O.default_codebook(4), T(g["cb4"]))
    assert torch.equal(O.uniform_levels(16), T(g["cb16_uniform"]))


def test_default_codebook_known_values(golden):
    """Hex values obtained by running the reference (seed 0xCDA, CPU generator)."""
    want16 = "bf700000 bf500000 bf300000 bf100000 be401459 bdf4d0d9 bd8ead6c bcdadd51 " \
             "3c4ec2dc 3d546849 3dbfc3a0 3e117705 3e560388 3f300000 3f500000 3f700000"
    want4 = "bf400000 bd8fba69 3d91f2a4 3f400000"
    g = golden("tables")
    assert [f"{v:08x}" for v in g["cb16"].view(np.uint32)] == want16.split()
    assert [f"{v:08x}" for v in g["cb4"].view(np.uint32)] == want4.split()


def test_uniform_levels_closed_form():
    assert torch.equal(O.uniform_levels(16), torch.arange(-15, 16, 2, dtype=torch.float32) / 16)


def test_hadamard_properties(golden):
    g = golden("tables")
    H = O.sylvester_hadamard(128)
    assert torch.equal(H, H.t())
    assert float((H @ H.t() - torch.eye(128)).abs().max()) < 1e-6
    assert float(H[0, 0]) == pytest.approx(1 / math.sqrt(128), rel=1e-7)
    for r in (1, 2, 77):
        assert torch.equal(H[r], T(g[f"hadamard_row{r}"]))
    i = torch.arange(128)
    sign = 1 - 2 * torch.tensor([[bin(int(a & b)).count("1") & 1 for b in i] for a in i])
    assert torch.equal(torch.sign(H).long(), sign)
    with pytest.raises(ValueError):
        O.sylvester_hadamard(96)


# ---- packing ----------------------------------------------------------------------------------

def test_pack_known_bytes_and_round_trip():
    idx = torch.arange(128) % 16
    p = O.pack_indices(idx, 4)
    assert p.shape == (64,) and int(p[0]) == 0x01 and int(p[1]) == 0x23
    assert torch.equal(O.unpack_indices(p, 4), idx.to(torch.uint8))
    idx2 = torch.arange(128) % 4
    p2 = O.pack_indices(idx2, 2)
    assert p2.shape == (32,) and int(p2[0]) == 0x1B
    assert torch.equal(O.unpack_indices(p2, 2), idx2.to(torch.uint8))
    g = torch.Generator().manual_seed(3)
    r = torch.randint(0, 16, (5, 7, 128), generator=g)
    assert torch.equal(O.unpack_indices(O.pack_indices(r, 4), 4), r.to(torch.uint8))


# ---- quantise ---------------------------------------------------------------------------------

def test_quantize_probe_matches_reference(golden):
    g, t = golden("quantize"), golden("tables")
    probe = T(g["probe"])
    assert torch.equal(O.nearest_level(probe, T(t["cb16"])), T(g["idx16"]))
    assert torch.equal(O.nearest_level(probe, T(t["cb4"])), T(g["idx4"]))
    assert torch.equal(O.nearest_level(probe, T(t["cb16_uniform"])), T(g["idx16_uniform"]))


def test_quantize_edges(golden):
    cb = T(golden("tables")["cb16"])
    assert int(O.nearest_level(torch.tensor([-1.0]), cb)) == 0
    assert int(O.nearest_level(torch.tensor([1.0]), cb)) == 15
    assert torch.equal(O.nearest_level(cb.clone(), cb), torch.arange(16, dtype=torch.uint8))
    u = O.uniform_levels(16)
    mid = (u[4] + u[5]) / 2                        # exactly representable: tie goes down
    assert int(O.nearest_level(mid.reshape(1), u)) == 4


# ---- encode / decode --------------------------------------------------------------------------

@pytest.mark.parametrize("levels,key", [(16, "16"), (4, "4")])
def test_quantize_rotated_exact_given_reference_inputs(golden, levels, key):
    """Indices are bit-exact when the fp32 quotient is the same: feed the stored rotated rows and
    the stored norms."""
    g, t = golden("encode"), golden("tables")
    cb = T(t[f"cb{levels}"])
    s = O.quantize_rotated(T(g["x_rot"]).float(), cb, norm=T(g[f"norm{key}"]))
    assert torch.equal(s.idx, T(g[f"idx{key}"]))


def test_encode_end_to_end(golden):
    g, t = golden("encode"), golden("tables")
    x = T(g["x"])
    for levels, key in ((16, "16"), (4, "4")):
        s = O.encode(x, T(t[f"cb{levels}"]))
        ref_idx, ref_norm = T(g[f"idx{key}"]), T(g[f"norm{key}"])
        assert s.idx.shape == ref_idx.shape
        # matmul / norm summation order is CPU dependent: allow 2 ulp on norms, 1e-4 index flips
        ulp = torch.abs(ref_norm) * 2 ** -23
        assert bool(((s.norm - ref_norm).abs() <= 2 * ulp + 1e-30).all())
        bits = 4 if levels == 16 else 2
        flips = (O.unpack_indices(s.idx, bits) != O.unpack_indices(ref_idx, bits)).float().mean()
        assert float(flips) <= 1e-4
    assert float(T(g["norm16"])[5]) == pytest.approx(1e-12)        # zero row hits the floor
    su = O.encode(x, T(t["cb16_uniform"]))
    assert float((O.unpack_indices(su.idx, 4) != O.unpack_indices(T(g["idx16_uniform"]), 4)).float().mean()) <= 1e-4


def test_decode_rotated_exact(golden):
    g, t = golden("encode"), golden("tables")
    d16 = O.decode_rotated(slot(g["idx16"], g["norm16"]), T(t["cb16"]))
    d4 = O.decode_rotated(slot(g["idx4"], g["norm4"]), T(t["cb4"]))
    assert torch.equal(d16, T(g["dec16_rot"]))
    assert torch.equal(d4, T(g["dec4_rot"]))
    d32 = O.decode_rotated(slot(g["idx16"], g["norm16"]), T(t["cb16"]), dtype=torch.float32)
    back = O.unrotate(d32, O.sylvester_hadamard()).to(torch.float16)      # compression.py:361
    torch.testing.assert_close(back.float(), T(g["dec16"]).float(), rtol=1e-3, atol=1e-3)


# ---- attention --------------------------------------------------------------------------------

CASES = ["decode_g4_k4v4", "decode_g8_k4v2", "decode_g4_k2v2", "prefill_g4_k4v4"]


@pytest.mark.parametrize("name", CASES)
def test_attention_matches_reference(golden, name):
    g = golden(name)
    B, Hkv, grp, Mq, N, causal, q_off, ws, we, splits = (int(v) for v in g["meta"])
    Ks, Vs = slot(g["K_idx"], g["K_norm"]), slot(g["V_idx"], g["V_norm"])
    kw = dict(cb_K=T(g["cb_K"]), cb_V=T(g["cb_V"]), group=grp, causal=bool(causal), q_offset=q_off)
    Q, Q_rot = T(g["Q"]), T(g["Q_rot"])
    tol = dict(rtol=2e-3, atol=1e-3)
    assert float((O.rotate(Q, O.sylvester_hadamard()).float() - Q_rot.float()).abs().max()) <= 2e-3
    out_rot = O.cda_attention_rotated(Q_rot, Ks, Vs, **kw)
    torch.testing.assert_close(out_rot.float(), T(g["out_rot"]).float(), **tol)
    out = O.cda_attention(Q, Ks, Vs, **kw)
    torch.testing.assert_close(out.float(), T(g["out"]).float(), **tol)
    Op, m, l = O.cda_partial_rotated(Q_rot, Ks, Vs, key_start=ws, key_end=we, **kw)
    torch.testing.assert_close(m, T(g["part_m"]), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(l, T(g["part_l"]), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(Op, T(g["part_O"]), rtol=1e-4, atol=1e-5)
    sp = O.cda_attention_split(Q_rot, Ks, Vs, k_splits=splits, **kw)
    torch.testing.assert_close(sp.float(), T(g["split_out"]).float(), **tol)


@pytest.mark.parametrize("splits", [1, 2, 5, 77])
def test_split_equals_unsplit(golden, splits):
    g = golden("decode_g4_k4v4")
    Ks, Vs = slot(g["K_idx"], g["K_norm"]), slot(g["V_idx"], g["V_norm"])
    kw = dict(cb_K=T(g["cb_K"]), cb_V=T(g["cb_V"]), group=4)
    full = O.cda_attention_rotated(T(g["Q_rot"]), Ks, Vs, **kw)
    sp = O.cda_attention_split(T(g["Q_rot"]), Ks, Vs, k_splits=splits, **kw)
    torch.testing.assert_close(sp.float(), full.float(), rtol=2e-3, atol=1e-3)


def test_merge_handles_empty_partial():
    """A partial over an empty / fully masked range has m = -inf, l = 0 and must not poison the merge."""
    o = torch.ones(1, 1, 1, 128)
    good = (o * 3.0, torch.zeros(1, 1, 1), torch.full((1, 1, 1), 3.0))
    empty = (torch.zeros(1, 1, 1, 128), torch.full((1, 1, 1), float("-inf")), torch.zeros(1, 1, 1))
    out = O.merge_partials([good, empty])
    assert torch.equal(out, torch.ones(1, 1, 1, 128, dtype=torch.float16))
    both = O.merge_partials([empty, empty])
    assert not bool(both.isnan().any())


def test_uniform_integer_score_identity(golden):
    g, t = golden("uniform_scores"), golden("tables")
    Ks = slot(g["K_idx"], g["K_norm"])
    s = O.uniform16_scores(T(g["Q_rot"]), Ks, group=4)
    torch.testing.assert_close(s, T(g["scores"]), rtol=1e-5, atol=1e-6)
    # and it agrees with scores from decoded fp32 keys
    K = O.decode_rotated(Ks, T(t["cb16_uniform"]), dtype=torch.float32)
    direct = torch.einsum("bhgmd,bhkd->bhgmk", T(g["Q_rot"]).float().view(1, 1, 4, 1, 128), K) / math.sqrt(128)
    torch.testing.assert_close(s, direct, rtol=1e-4, atol=1e-4)


# ---- paged layout -----------------------------------------------------------------------------

def test_slot_sizes():
    assert (O.slot_payload_bytes(4, 4), O.slot_bytes(4, 4)) == (136, 144)
    assert (O.slot_payload_bytes(4, 2), O.slot_bytes(4, 2)) == (104, 112)
    assert (O.slot_payload_bytes(2, 2), O.slot_bytes(2, 2)) == (72, 80)


@pytest.mark.parametrize("kb,vb", [(4, 4), (4, 2), (2, 2)])
def test_paged_round_trip_and_decode(golden, kb, vb):
    t = golden("tables")
    cbs = {4: T(t["cb16"]), 2: T(t["cb4"])}
    gen = torch.Generator().manual_seed(17)
    B, Hkv, grp, bs = 3, 2, 4, 16
    lens = [1, 17, 40]
    nblk = sum(-(-n // bs) for n in lens)
    perm = torch.randperm(nblk + 2, generator=gen)
    bt = torch.full((B, 3), -1, dtype=torch.int32)
    cache = torch.full(((nblk + 2) * bs, Hkv, O.slot_bytes(kb, vb)), 0xA5, dtype=torch.uint8)
    used = 0
    per_seq = []
    for b, n in enumerate(lens):
        k = torch.randn(n, Hkv, 128, generator=gen).to(torch.float16)
        v = torch.randn(n, Hkv, 128, generator=gen).to(torch.float16)
        nb = -(-n // bs)
        bt[b, :nb] = perm[used:used + nb].to(torch.int32)
        used += nb
        slots = O.slots_of_sequence(bt[b], n, bs)
        Ks, Vs = O.encode(k, cbs[kb]), O.encode(v, cbs[vb])
        O.pack_slots(cache, slots.to(torch.int32), Ks, Vs, kb, vb)
        K2, V2 = O.unpack_slots(cache, slots, kb, vb)
        assert torch.equal(K2.idx, Ks.idx) and torch.equal(V2.norm, Vs.norm)
        per_seq.append((Ks, Vs))
    pay = O.slot_payload_bytes(kb, vb)
    assert bool((cache[:, :, pay:] == 0xA5).all())                 # pad bytes untouched
    Q = torch.randn(B, Hkv * grp, 128, generator=gen).to(torch.float16)
    out = O.paged_decode(Q, cache, bt, torch.tensor(lens), cb_K=cbs[kb], cb_V=cbs[vb], group=grp,
                         block_size=bs, k_bits=kb, v_bits=vb)
    for b, (Ks, Vs) in enumerate(per_seq):
        tr = lambda s: O.Slot(s.idx.permute(1, 0, 2).unsqueeze(0), s.norm.permute(1, 0).unsqueeze(0))
        want = O.cda_attention(Q[b][None, :, None, :], tr(Ks), tr(Vs), cb_K=cbs[kb], cb_V=cbs[vb], group=grp)
        assert torch.equal(out[b], want[0, :, 0])
