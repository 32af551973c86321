"""GPU parity of the vLLM backend implementation class: cache update and forward for decode, ragged prefill and a mixed
batch, through the same calls vLLM makes (reference: cda_attn_v2.py:655-864), against the CPU oracle."""
import types

import pytest
import torch

from oracle import cda_oracle as O
from tests import _cases as Cs
from tests.test_gpu_prefill import assert_close, prefill_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def vllm_cache(case):
    """The oracle-built byte cache as vLLM would hold it: (num_blocks, block_size, H_kv, 72) typed fp16."""
    slots, hkv, w = case["cache"].shape
    bs = case["block_size"]
    return case["cache"].view(slots // bs, bs, hkv, w).contiguous().to(DEV).view(torch.float16)


def metadata(Metadata, q_lens, case, slot_mapping=None):
    cu = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(q_lens).cumsum(0)
    nd = sum(1 for q in q_lens if q == 1) if max(q_lens) > 1 else len(q_lens)
    n = int(cu[-1])
    return Metadata(num_actual_tokens=n, num_reqs=len(q_lens), max_query_len=max(q_lens), max_seq_len=int(case["seq_lens"].max()),
                    query_start_loc=cu.to(DEV), seq_lens=case["seq_lens"].to(DEV), block_table=case["block_table"].to(DEV),
                    slot_mapping=slot_mapping if slot_mapping is not None else torch.zeros(n, dtype=torch.int64, device=DEV),
                    num_decodes=nd, num_prefills=len(q_lens) - nd, num_decode_tokens=nd, num_prefill_tokens=n - nd), cu


def test_cache_update_then_decode_matches_oracle():
    from sub0_b200.vllm_integration.cda_attn_v2 import get_backend_classes
    Backend, Impl, _, Metadata = get_backend_classes()
    lens = [70, 33, 129, 16]
    case = Cs.paged_case(lens, H_kv=2, group=4, seed=5)
    impl = Impl(8, 128, 128 ** -0.5, num_kv_heads=2)
    nb = case["cache"].shape[0] // 16
    kv = torch.zeros(Backend.get_kv_cache_shape(nb, 16, 2, 128), dtype=torch.float16, device=DEV)
    # write every token of every sequence through the backend's own cache update
    keys = torch.cat([k for k, _ in case["raw"]]).to(DEV)
    vals = torch.cat([v for _, v in case["raw"]]).to(DEV)
    slots = torch.cat([O.slots_of_sequence(case["block_table"][b], n, 16) for b, n in enumerate(lens)]).to(DEV)
    impl.do_kv_cache_update(None, keys, vals, kv, slots)
    md, _ = metadata(Metadata, [1] * len(lens), case, slots[: len(lens)])
    out = torch.full((len(lens), 8 * 128), float("nan"), dtype=torch.float16, device=DEV)
    res = impl.forward(None, case["Q"].to(DEV).view(len(lens), -1), None, None, kv, md, output=out)
    torch.cuda.synchronize()
    assert res is out
    assert_close(out.view(len(lens), 8, 128).cpu(), Cs.oracle_decode(case), "vllm decode")


def test_ragged_prefill_and_mixed_batch():
    from sub0_b200.vllm_integration.cda_attn_v2 import get_backend_classes
    _, Impl, _, Metadata = get_backend_classes()
    impl = Impl(8, 128, 128 ** -0.5, num_kv_heads=2)
    # decodes first (q_len 1), then a chunk with a compressed past and a full prompt
    lens, q_lens = [200, 90, 300, 130], [1, 1, 45, 130]
    case = Cs.paged_case(lens, H_kv=2, group=4, seed=17)
    Q, cu = prefill_inputs(case, q_lens, 3)
    want = O.paged_prefill(Q, case["cache"], case["block_table"], cu, case["seq_lens"], cb_K=case["cb_K"], cb_V=case["cb_V"],
                           group=4, block_size=16)
    kv = vllm_cache(case)
    md, _ = metadata(Metadata, q_lens, case)
    n = Q.shape[0]
    out = torch.full((n + 3, 8 * 128), float("nan"), dtype=torch.float16, device=DEV)      # padded like a CUDA-graph batch
    qpad = torch.zeros(n + 3, 8 * 128, dtype=torch.float16, device=DEV)
    qpad[:n] = Q.to(DEV).view(n, -1)
    impl.forward(None, qpad, None, None, kv, md, output=out)
    torch.cuda.synchronize()
    assert_close(out[:n].view(n, 8, 128).cpu(), want, "vllm mixed")
    assert bool(out[n:].isnan().all())                   # rows past num_actual_tokens are not touched

    # prefill only, counts left at zero on purpose: forward recounts them from query_start_loc
    lens2, q2 = [77, 260], [77, 100]
    case2 = Cs.paged_case(lens2, H_kv=2, group=4, seed=23)
    Q2, cu2 = prefill_inputs(case2, q2, 4)
    want2 = O.paged_prefill(Q2, case2["cache"], case2["block_table"], cu2, case2["seq_lens"], cb_K=case2["cb_K"], cb_V=case2["cb_V"],
                            group=4, block_size=16)
    md2, _ = metadata(Metadata, q2, case2)
    md2.num_decodes = md2.num_prefills = md2.num_decode_tokens = md2.num_prefill_tokens = 0
    out2 = torch.empty(Q2.shape[0], 8 * 128, dtype=torch.float16, device=DEV)
    impl.forward(None, Q2.to(DEV).view(Q2.shape[0], -1), None, None, vllm_cache(case2), md2, output=out2)
    torch.cuda.synchronize()
    assert_close(out2.view(-1, 8, 128).cpu(), want2, "vllm prefill")
