"""The "dequantise, then dense attention" comparison path (reference: cda/kernels_vllm_fa2_fork/interface.py:138-329):
the dequantisation is bit-exact against Compressor.decode; the composed attention agrees with the oracle's rotated-frame
attention (the dense body is a library kernel, checked with a looser tolerance)."""
import pytest
import torch

from oracle import cda_oracle as O
from tests import _cases as Cs

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("bits", [4, 2])
def test_dequantize_rows_bit_exact(bits):
    from sub0_b200.kernels_vllm_fa2_fork.interface import dequantize_compressed_kv
    gen = torch.Generator().manual_seed(bits)
    cb = Cs.cb_for(bits)
    k = Cs.rows(gen, 2, 3, 37, outliers=True)          # (B, H_kv, N, 128)
    v = Cs.rows(gen, 2, 3, 37)
    ks, vs = O.encode(k, cb), O.encode(v, cb)
    kd, vd = dequantize_compressed_kv(ks.idx.to(DEV), ks.norm.to(DEV), vs.idx.to(DEV), vs.norm.to(DEV), cb.to(DEV), cb.to(DEV))
    want_k = O.decode_rotated(ks, cb).permute(0, 2, 1, 3).reshape(-1, 3, 128)
    want_v = O.decode_rotated(vs, cb).permute(0, 2, 1, 3).reshape(-1, 3, 128)
    assert kd.shape == (2 * 37, 3, 128) and torch.equal(kd.cpu(), want_k) and torch.equal(vd.cpu(), want_v)


def test_compressed_kv_attention_through_dense_body():
    pytest.importorskip("flash_attn")
    from sub0_b200.kernels_vllm_fa2_fork.interface import flash_attn_varlen_compressed_kv_func
    gen = torch.Generator().manual_seed(11)
    cb = Cs.cb_for(4)
    lens, H_kv, group = [70, 33], 2, 4
    qs, ks_, vs_, want = [], [], [], []
    for n in lens:
        k = Cs.rows(gen, 1, H_kv, n, outliers=True)
        v = Cs.rows(gen, 1, H_kv, n)
        q_rot = Cs.rows(gen, 1, H_kv * group, n)                        # queries, already in the rotated frame
        ke, ve = O.encode(k, cb), O.encode(v, cb)
        kd, vd = O.decode_rotated(ke, cb), O.decode_rotated(ve, cb)      # (1, H_kv, n, 128) fp16
        want.append(O.gqa_attention(q_rot, kd, vd, group=group, causal=True)[0].transpose(0, 1))   # (n, H_q, 128)
        qs.append(q_rot[0].transpose(0, 1)); ks_.append(ke); vs_.append(ve)
    q = torch.cat(qs).contiguous().to(DEV)
    k_idx = torch.cat([e.idx[0].transpose(0, 1) for e in ks_]).contiguous().to(DEV)      # (total_k, H_kv, 64)
    v_idx = torch.cat([e.idx[0].transpose(0, 1) for e in vs_]).contiguous().to(DEV)
    k_norm = torch.cat([e.norm[0].transpose(0, 1) for e in ks_]).contiguous().to(DEV)
    v_norm = torch.cat([e.norm[0].transpose(0, 1) for e in vs_]).contiguous().to(DEV)
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen_compressed_kv_func(q, k_idx, k_norm, v_idx, v_norm, cb.to(DEV), cb.to(DEV), max(lens), cu, max(lens), cu,
                                               softmax_scale=128 ** -0.5, causal=True)
    err = (out.float().cpu() - torch.cat(want).float()).abs().max().item()
    assert err < 5e-3, err
