"""CPU-only checks of the drop-in boundary: the C-ABI library loads, exports every symbol that include/cda_b200.h
declares, rejects bad arguments with the right status before touching a GPU, and the Python wrappers keep the
reference's signatures and error behaviour.  No kernel is launched here."""
import ctypes as C
import inspect
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from sub0_b200 import build
    build.build()
    from sub0_b200 import _lib
    return _lib


def declared_functions():
    text = (ROOT / "include" / "cda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cda_b200_\w+)\s*\(", text)))


def test_header_symbols_all_exported(lib):
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib.lib, n), f"{n} declared in the header but not exported"
    assert sorted(lib.PROTOTYPES) == names


def test_version_and_slot_bytes(lib):
    assert lib.lib.cda_b200_version() == 1
    assert lib.lib.cda_b200_slot_bytes(4, 4) == 144
    assert lib.lib.cda_b200_slot_bytes(4, 2) == 112
    assert lib.lib.cda_b200_slot_bytes(2, 2) == 80
    assert lib.lib.cda_b200_slot_bytes(3, 4) == lib.CDA_ERR_UNSUPPORTED
    assert "2 or 4" in lib.last_error()


def test_status_codes_without_gpu(lib):
    L = lib.lib
    buf = (C.c_char * 4096)()
    p = C.addressof(buf)
    al = (p + 15) // 16 * 16
    # encode
    assert L.cda_b200_paged_encode(al, al, al, al, al, al, -1, 8, 16, 144, 4, 4, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_paged_encode(al, al, al, al, al, al, 1, 8, 16, 136, 4, 4, None) == lib.CDA_ERR_BAD_SHAPE
    assert L.cda_b200_paged_encode(al, al, al, al, al, al, 1, 8, 16, 144, 8, 4, None) == lib.CDA_ERR_UNSUPPORTED
    assert L.cda_b200_paged_encode(al + 2, al, al, al, al, al, 1, 8, 16, 144, 4, 4, None) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_paged_encode(None, al, al, al, al, al, 1, 8, 16, 144, 4, 4, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_paged_encode(al, al, al, al, al, al, 0, 8, 16, 144, 4, 4, None) == lib.CDA_OK   # nothing to do
    # decode
    def dec(**kw):
        a = dict(Q=al, cache=al, bt=al, sl=al, cbk=al, cbv=al, out=al, ws=al, wsb=1 << 20, B=1, Hq=32, Hkv=8, bs=16,
                 stride=4, maxlen=64, slots=64, sw=144, kb=4, vb=4, scale=0.1, splits=0)
        a.update(kw)
        return L.cda_b200_decode(a["Q"], a["cache"], a["bt"], a["sl"], a["cbk"], a["cbv"], a["out"], a["ws"], a["wsb"],
                                 a["B"], a["Hq"], a["Hkv"], a["bs"], a["stride"], a["maxlen"], a["slots"], a["sw"],
                                 a["kb"], a["vb"], a["scale"], a["splits"], None)
    assert dec(Hq=30) == lib.CDA_ERR_BAD_SHAPE           # H_q not a multiple of H_kv
    assert dec(Hq=128) == lib.CDA_ERR_UNSUPPORTED        # group 16
    assert dec(bs=24) == lib.CDA_ERR_BAD_SHAPE           # block size not a multiple of 16
    assert dec(sw=136) == lib.CDA_ERR_BAD_SHAPE          # slot width must be the padded 144
    assert dec(stride=2) == lib.CDA_ERR_BAD_SHAPE        # block table row too short for max_seq_len
    assert dec(Q=al + 8) == lib.CDA_ERR_BAD_ALIGN
    assert dec(maxlen=(1 << 30) + 1, stride=1 << 28) == lib.CDA_ERR_N_TOO_LARGE
    assert dec(wsb=16) == lib.CDA_ERR_WORKSPACE
    assert "workspace" in lib.last_error()
    assert dec(ws=None) == lib.CDA_ERR_WORKSPACE
    assert dec(B=0) == lib.CDA_OK
    # merge / hadamard / prefill
    assert L.cda_b200_merge_partials(al, al, al, 0, 4, al, 1, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_hadamard128(al + 2, al, 4, 1.0, None) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_hadamard128(al, al, 0, 1.0, None) == lib.CDA_OK
    assert L.cda_b200_prefill_varlen(al, al, al, al, al, al, al, al, 8, 1, 30, 8, 16, 4, 8, 64, 64, 144, 4, 4, 0.1,
                                     None) == lib.CDA_ERR_BAD_SHAPE
    assert L.cda_b200_prefill_varlen(al, al, al, al, al, al, al, al, 8, 1, 32, 8, 48 + 1, 4, 8, 64, 64, 144, 4, 4, 0.1,
                                     None) == lib.CDA_ERR_BAD_SHAPE
    assert L.cda_b200_cache_to_dense_rotated(al, al, al, al, al, al, al, 1, 8, 16, 4, 64, 64, 100, 4, 4,
                                             None) == lib.CDA_ERR_BAD_SHAPE
    # alignment contracts: the tcgen05 prefill kernel moves Q / out in 16-byte pieces, the scalar decode and the dense
    # loader store 8 bytes at a time -- a misaligned pointer is refused before any launch
    pf = lambda q, o: L.cda_b200_prefill_varlen(q, al, al, al, al, al, al, o, 8, 1, 32, 8, 16, 4, 8, 64, 64, 144, 4, 4, 0.1, None)
    assert pf(al + 8, al) == lib.CDA_ERR_BAD_ALIGN
    assert pf(al, al + 8) == lib.CDA_ERR_BAD_ALIGN
    assert "16-byte" in lib.last_error()
    assert L.cda_b200_decode_scalar(al, al, al, al, al, al, al + 4, 1, 32, 8, 16, 4, 64, 144, 4, 4, 0.1,
                                    None) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_cache_to_dense_rotated(al, al, al, al, al, al + 4, al, 1, 8, 16, 4, 64, 64, 144, 4, 4,
                                             None) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_cache_to_dense_rotated(al, al, al, al, al, al, al + 4, 1, 8, 16, 4, 64, 64, 144, 4, 4,
                                             None) == lib.CDA_ERR_BAD_ALIGN
    # packed partials and log-sum-exp variants share the decode validation
    assert L.cda_b200_decode_partial_packed(al, al, al, al, al, al, al + 4, al, 1 << 20, 1, 32, 8, 16, 4, 64, 64, 144, 4, 4,
                                            0.1, 0, None) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_decode_partial_packed(al, al, al, al, al, al, None, al, 1 << 20, 1, 32, 8, 16, 4, 64, 64, 144, 4, 4,
                                            0.1, 0, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_decode_lse(al, al, al, al, al, al, al, None, al, 1 << 20, 1, 32, 8, 16, 4, 64, 64, 144, 4, 4, 0.1, 0,
                                 None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_merge_partials_packed(al, 0, 4, al, 1, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_merge_partials_packed(al + 4, 2, 4, al, 1, None) == lib.CDA_ERR_BAD_ALIGN
    # the exchange form of the sequence-sharded decode: sizes and argument checks (nothing is launched)
    assert L.cda_b200_decode_exchange_bytes(1, 64, 8) == 2 * 8 * 64 * 132 * 4
    assert L.cda_b200_decode_exchange_bytes(0, 64, 8) == 0
    ex = lambda **kw: L.cda_b200_decode_exchange(al, al, al, al, al, al, kw.get("out", al), al, 1 << 20, kw.get("peers", al),
                                                 kw.get("counters", al), kw.get("rank", 0), kw.get("world", 2), kw.get("wait_ms", 100),
                                                 kw.get("B", 1), 32, 8, 16, 4, 64, 64, 144, 4, 4, 0.1, 0, None)
    assert ex(world=0) == lib.CDA_ERR_BAD_ARG and ex(rank=2) == lib.CDA_ERR_BAD_ARG and ex(world=33) == lib.CDA_ERR_BAD_ARG
    assert ex(peers=None) == lib.CDA_ERR_BAD_ARG and ex(counters=None) == lib.CDA_ERR_BAD_ARG and ex(B=0) == lib.CDA_ERR_BAD_ARG
    assert ex(wait_ms=0) == lib.CDA_ERR_BAD_ARG and ex(wait_ms=60000) == lib.CDA_ERR_BAD_ARG
    assert ex(out=al + 4) == lib.CDA_ERR_BAD_ALIGN and ex(counters=al + 4) == lib.CDA_ERR_BAD_ALIGN
    assert L.cda_b200_exchange_export(None, al) == lib.CDA_ERR_BAD_ARG and L.cda_b200_exchange_import(al, None) == lib.CDA_ERR_BAD_ARG
    assert L.cda_b200_exchange_free(None) == lib.CDA_OK and L.cda_b200_exchange_close(None) == lib.CDA_OK
    assert L.cda_b200_prefill_debug(0, 0) == lib.CDA_OK


def test_split_planning_properties(lib):
    L = lib.lib
    for B, Hkv, n in [(32, 8, 65536), (1, 8, 65536), (1, 8, 4096), (4, 8, 16384), (64, 8, 32768), (1, 8, 1 << 20),
                      (1, 1, 131072), (7, 2, 999), (1, 8, 1)]:
        s = L.cda_b200_decode_plan_splits(B, Hkv, n, -1)
        assert 1 <= s <= max(1, -(-n // 16))
        ws = L.cda_b200_decode_workspace_bytes(B, Hkv * 4, Hkv, n, 0, -1)
        assert ws == 256 + s * B * Hkv * 4 * 130 * 4       # one partial row of 128 + 2 floats per split and query head
        assert L.cda_b200_decode_workspace_bytes(B, Hkv * 4, Hkv, n, 3, -1) <= 256 + 3 * B * Hkv * 4 * 520
    # the line of all sequences' 16-token groups is cut into 148 equal chunks (one per SM): 32 x 4096 groups -> chunks of
    # 886 groups, and a sequence of 4096 groups touches at most 6 of them
    assert L.cda_b200_decode_plan_splits(32, 8, 65536, -1) == 6
    assert L.cda_b200_decode_plan_splits(4, 8, 65536, -1) == 37       # 148 = 4 x 37: equal ranges inside each sequence
    assert L.cda_b200_decode_plan_splits(32, 8, 4096, -1) == 6        # 148 chunks over a line with a gap behind every sequence
    # an odd number of partial rows (13 sequences x 3 query heads x 1 or 3 parts): the (m, l) pairs are padded to a
    # multiple of 16 bytes so that the O rows behind them stay 16-byte aligned
    for parts in (1, 3):
        rows = parts * 13 * 3
        assert L.cda_b200_decode_workspace_bytes(13, 3, 3, 5000, parts, -1) == 256 + (rows * 8 + 8) + rows * 512
    assert L.cda_b200_decode_plan_splits(37, 8, 4096, -1) == 4        # 37 x 4 = 148: equal ranges inside each sequence
    assert L.cda_b200_decode_plan_splits(1, 8, 4096, -1) == 32        # never below 128 tokens per chunk
    assert L.cda_b200_decode_plan_splits(0, 8, 16, -1) == lib.CDA_ERR_BAD_ARG


def test_wrapper_signatures_match_reference():
    """Parameter names and order of the public wrappers (reference: cda/kernels_cuda/wrappers.py:79-94, 127-135;
    fa2_cda.py:64-74, 98-118)."""
    from sub0_b200.kernels_cuda import fa2_cda, hmma_loader, wrappers
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(wrappers.decode_hmma_v1)[:13] == ["Q_fp16", "kv_cache", "block_table", "seq_lens", "output", "cb_K", "cb_V",
                                                 "rotation_fp32", "rotation_fp16", "group_size", "block_size", "scale",
                                                 "max_seq_len"]
    assert sig(wrappers.paged_encode_fused_cuda) == ["K", "V", "slot_mapping", "flat_cache", "cb_K", "cb_V"]
    assert sig(fa2_cda.paged_cache_to_dense_rotated) == ["kv_cache", "block_table", "seq_lens", "cb_K", "cb_V", "block_size",
                                                         "max_seq_len", "k4v2"]
    assert sig(fa2_cda.fa2_cda_prefill_varlen_v1) == ["Q_fp16", "kv_cache", "block_table", "cu_seqlens_q", "seq_lens", "output",
                                                      "cb_K", "cb_V", "rotation_fp32", "group_size", "block_size",
                                                      "max_query_len", "max_seq_len", "scale", "causal", "k4v2",
                                                      "return_dense_kv", "fuse_fa2_epilogue"]
    assert hasattr(hmma_loader.load_decode_hmma(False, 4), "cda_decode_full_hmma_v3")
    assert hasattr(hmma_loader.load_paged_encode_fused(), "cda_paged_encode_fused")
    assert hasattr(hmma_loader.load_fa2_cda_loader(False), "cda_fa2_paged_cache_to_dense_rotated")
    assert hasattr(hmma_loader.load_fa2_cda_hadamard(), "hadamard128_fp16")
    assert hasattr(hmma_loader.load_fa2_cda_varlen_fused(), "cda_fa2_varlen_fwd_hadamard")
    with pytest.raises(ValueError):
        hmma_loader.load_decode_hmma(False, 3)
    with pytest.raises(ImportError):
        hmma_loader.load_kv_cache_update(False)


def test_wrappers_reject_cpu_and_bad_dtypes():
    """Same exception types as the reference wrappers (wrappers.py:112-113, 143-148); CPU tensors are refused -- there
    is no fallback path."""
    from sub0_b200.kernels_cuda import wrappers
    K = torch.zeros(2, 8, 128, dtype=torch.float32)
    cache = torch.zeros(32, 8, 144, dtype=torch.uint8)
    cb = torch.zeros(16)
    sm = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(TypeError):
        wrappers.paged_encode_fused_cuda(K, K, sm, cache, cb_K=cb, cb_V=cb)
    with pytest.raises(TypeError):
        wrappers.paged_encode_fused_cuda(K.half(), K.half(), sm, cache.float(), cb_K=cb, cb_V=cb)
    with pytest.raises(ValueError):
        wrappers.paged_encode_fused_cuda(K.half()[..., :64], K.half()[..., :64], sm, cache, cb_K=cb, cb_V=cb)
    with pytest.raises(ValueError, match="CUDA"):
        wrappers.paged_encode_fused_cuda(K.half(), K.half(), sm, cache, cb_K=cb, cb_V=cb)
    Q = torch.zeros(1, 32, 128, dtype=torch.float16)
    with pytest.raises(ValueError):
        wrappers.decode_hmma_v1(Q, cache, sm.view(1, 2), sm[:1], Q.float(), cb_K=cb, cb_V=cb, group_size=4, block_size=16,
                                max_seq_len=4)
    with pytest.raises(ValueError, match="CUDA"):
        wrappers.decode_hmma_v1(Q, cache, sm.view(1, 2), sm[:1], Q.clone(), cb_K=cb, cb_V=cb, group_size=4, block_size=16,
                                max_seq_len=4)


def test_codebook_module_matches_golden(golden):
    from sub0_b200 import codebook
    t = golden("tables")
    assert torch.equal(codebook.default_codebook(16), torch.from_numpy(t["cb16"]))
    assert torch.equal(codebook.default_codebook(4), torch.from_numpy(t["cb4"]))
    assert torch.equal(codebook.uniform_codebook(16), torch.from_numpy(t["cb16_uniform"]))
    H = codebook.hadamard_matrix(128)
    for r in (1, 2, 77):
        assert torch.equal(H[r], torch.from_numpy(t[f"hadamard_row{r}"]))
    g = torch.Generator().manual_seed(0xCDA)
    x = torch.randn(100_000, 128, generator=g)
    samples = (x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12))[:, 0]
    torch.testing.assert_close(codebook.lloyd_max_codebook(16, samples), torch.from_numpy(t["cb16"]), rtol=1e-5, atol=1e-6)
