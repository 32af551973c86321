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


def test_fused_compressed_kv_attention_flat_and_paged():
    """The fused comparator (reference interface.py:332-470) on the paged prefill kernel: flattened varlen K/V and a paged
    cache, against the oracle's rotated-frame causal attention."""
    from sub0_b200.kernels_vllm_fa2_fork.interface import flash_attn_varlen_compressed_kv_fused_func
    gen = torch.Generator().manual_seed(12)
    cb = Cs.cb_for(4)
    lens, H_kv, group = [70, 33], 2, 4
    qs, ks_, vs_, want = [], [], [], []
    for n in lens:
        k = Cs.rows(gen, 1, H_kv, n, outliers=True)
        v = Cs.rows(gen, 1, H_kv, n)
        q_rot = Cs.rows(gen, 1, H_kv * group, n)
        ke, ve = O.encode(k, cb), O.encode(v, cb)
        kd, vd = O.decode_rotated(ke, cb), O.decode_rotated(ve, cb)
        want.append(O.gqa_attention(q_rot, kd, vd, group=group, causal=True)[0].transpose(0, 1))
        qs.append(q_rot[0].transpose(0, 1)); ks_.append(ke); vs_.append(ve)
    q = torch.cat(qs).contiguous().to(DEV)
    k_idx = torch.cat([e.idx[0].transpose(0, 1) for e in ks_]).contiguous().to(DEV)
    v_idx = torch.cat([e.idx[0].transpose(0, 1) for e in vs_]).contiguous().to(DEV)
    k_norm = torch.cat([e.norm[0].transpose(0, 1) for e in ks_]).contiguous().to(DEV)
    v_norm = torch.cat([e.norm[0].transpose(0, 1) for e in vs_]).contiguous().to(DEV)
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen_compressed_kv_fused_func(q, k_idx, k_norm, v_idx, v_norm, cb.to(DEV), cb.to(DEV), max(lens), cu,
                                                     max(lens), cu, softmax_scale=128 ** -0.5, causal=True)
    torch.cuda.synchronize()
    err = (out.float().cpu() - torch.cat(want).float()).abs().max().item()
    assert err < 5e-3, err
    # the same keys as a paged cache: 16-slot blocks in reverse order
    bs = 16
    nblk = [-(-n // bs) for n in lens]
    total = sum(nblk)
    pk_idx = torch.zeros(total, bs, H_kv, 64, dtype=torch.uint8); pv_idx = torch.zeros_like(pk_idx)
    pk_norm = torch.ones(total, bs, H_kv); pv_norm = torch.ones(total, bs, H_kv)
    bt = torch.zeros(2, max(nblk), dtype=torch.int32)
    ids = list(range(total))[::-1]
    at = 0
    for b, n in enumerate(lens):
        for j in range(nblk[b]):
            blk = ids[at]; at += 1
            bt[b, j] = blk
            m = min(bs, n - j * bs)
            pk_idx[blk, :m] = ks_[b].idx[0].transpose(0, 1)[j * bs:j * bs + m]
            pv_idx[blk, :m] = vs_[b].idx[0].transpose(0, 1)[j * bs:j * bs + m]
            pk_norm[blk, :m] = ks_[b].norm[0].transpose(0, 1)[j * bs:j * bs + m]
            pv_norm[blk, :m] = vs_[b].norm[0].transpose(0, 1)[j * bs:j * bs + m]
    out2 = flash_attn_varlen_compressed_kv_fused_func(q, pk_idx.to(DEV), pk_norm.to(DEV), pv_idx.to(DEV), pv_norm.to(DEV),
                                                      cb.to(DEV), cb.to(DEV), max(lens), cu, max(lens),
                                                      seqused_k=torch.tensor(lens, dtype=torch.int32, device=DEV),
                                                      block_table=bt.to(DEV), softmax_scale=128 ** -0.5, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    with pytest.raises(NotImplementedError):
        flash_attn_varlen_compressed_kv_fused_func(q, k_idx, k_norm, v_idx, v_norm, cb.to(DEV), cb.to(DEV), max(lens), cu,
                                                   max(lens), cu, causal=False)


def test_operator_namespace_calls_match_the_functions():
    """torch.ops._cda_vllm_fa2_fork_C.* with the positional argument lists of the reference's wrappers
    (interface.py:154-161, 433-460) give what the package's functions give."""
    import sub0_b200.kernels_vllm_fa2_fork._ops  # noqa: F401  (registers the namespace)
    from sub0_b200.kernels_vllm_fa2_fork.interface import dequantize_compressed_kv, flash_attn_varlen_compressed_kv_fused_func
    ns = torch.ops._cda_vllm_fa2_fork_C
    gen = torch.Generator().manual_seed(13)
    cb = Cs.cb_for(4)
    n, H_kv, group = 90, 2, 4
    ke, ve = O.encode(Cs.rows(gen, 1, H_kv, n, outliers=True), cb), O.encode(Cs.rows(gen, 1, H_kv, n), cb)
    k_idx, v_idx = ke.idx[0].transpose(0, 1).contiguous().to(DEV), ve.idx[0].transpose(0, 1).contiguous().to(DEV)
    k_norm, v_norm = ke.norm[0].transpose(0, 1).contiguous().to(DEV), ve.norm[0].transpose(0, 1).contiguous().to(DEV)
    cbd = cb.to(DEV)
    kd, vd = ns.dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cbd, cbd)
    kd2, vd2 = dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cbd, cbd)
    assert torch.equal(kd, kd2) and torch.equal(vd, vd2)
    q = Cs.rows(gen, 1, H_kv * group, n)[0].transpose(0, 1).contiguous().to(DEV)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    out, lse = ns.varlen_fwd_compressed_kv_fused(q, k_idx, k_norm, v_idx, v_norm, cbd, cbd, None, cu, cu, None, None, None, n, n,
                                                 0.0, 128 ** -0.5, False, True, -1, -1, 0.0, False, 0, False, None)
    want = flash_attn_varlen_compressed_kv_fused_func(q, k_idx, k_norm, v_idx, v_norm, cbd, cbd, n, cu, n, cu,
                                                      softmax_scale=128 ** -0.5, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(out, want) and lse.numel() == 0
