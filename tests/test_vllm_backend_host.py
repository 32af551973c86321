"""Host logic of the vLLM backend (no GPU): class surface, batch splitting, cache views, page-size patch.
Reference: cda/kernels_cuda/vllm_integration/cda_attn_v2.py:443-653, :1707-1756."""
import types

import pytest
import torch

from sub0_b200.vllm_integration import cda_attn_v2 as V


def test_split_counts():
    f = V.split_counts_from_query_start
    assert f(torch.tensor([0, 1, 2, 3]), 3, 3, 1) == (3, 0, 3, 0)
    assert f(torch.tensor([0, 1, 2, 10, 30]), 4, 30, 20) == (2, 2, 2, 28)
    assert f(torch.tensor([0, 7, 20]), 2, 20, 13) == (0, 2, 0, 20)
    assert f(torch.tensor([0]), 0, 0, 0) == (0, 0, 0, 0)
    assert f([0, 1, 5], 2, 5, 4) == (1, 1, 1, 4)


def test_cache_view():
    c = torch.zeros(3, 16, 8, 72, dtype=torch.float16)
    u = V.as_uint8_cache(c)
    assert u.shape == (3, 16, 8, 144) and u.dtype == torch.uint8 and u.data_ptr() == c.data_ptr()
    assert V.as_uint8_cache(u) is u
    with pytest.raises(ValueError):
        V.as_uint8_cache(torch.zeros(3, 16, 8, 256, dtype=torch.float16))
    with pytest.raises(ValueError):
        V.as_uint8_cache(torch.zeros(3, 16, 8, 100, dtype=torch.uint8))


def test_class_surface():
    Backend, Impl, Builder, Metadata = V.get_backend_classes()
    assert Backend.accept_output_buffer is True and Backend.forward_includes_kv_cache_update is False
    assert Backend.supported_dtypes == [torch.float16] and Backend.supported_kv_cache_dtypes == ["auto", "uint8"]
    assert Backend.get_impl_cls() is Impl and Backend.get_builder_cls() is Builder
    assert Backend.get_supported_head_sizes() == [128]
    sizes = Backend.get_supported_kernel_block_sizes()
    assert len(sizes) == 1 and int(getattr(sizes[0], "base", sizes[0])) == 16
    assert Backend.get_kv_cache_shape(10, 16, 8, 128) == (10, 16, 8, 72)
    with pytest.raises(ValueError):
        Backend.get_kv_cache_shape(10, 16, 8, 64)
    assert Builder.reorder_batch_threshold == 1
    assert Impl.can_return_lse_for_decode is True          # the reference leaves it False (cda_attn_v2.py:621)
    impl = Impl(32, 128, 0.088, num_kv_heads=8)
    assert impl.group_size == 4
    for bad in (dict(alibi_slopes=[1.0]), dict(sliding_window=128), dict(attn_type="encoder"), dict(num_kv_heads=16)):
        kw = dict(num_kv_heads=8)
        kw.update(bad)
        with pytest.raises(NotImplementedError):
            Impl(32, 128, 0.088, **kw)
    with pytest.raises(ValueError):
        impl.forward(None, torch.zeros(1, 32, 128), None, None, torch.zeros(0), None, output=None)
    out = torch.ones(2, 32 * 128)
    assert impl.forward(None, torch.zeros(2, 32 * 128), None, None, torch.zeros(0), None, output=out).abs().sum() == 0
    src = torch.arange(4 * 2 * 1 * 72, dtype=torch.float16).view(4, 2, 1, 72)
    dst = torch.zeros_like(src)
    Backend.swap_blocks(src, dst, torch.tensor([[1, 3]]))
    assert torch.equal(dst[3], src[1])
    Backend.copy_blocks([dst], torch.tensor([[3, 0]]))
    assert torch.equal(dst[0], src[1])


def test_builder_counts_and_dcp_lengths():
    _, _, Builder, _ = V.get_backend_classes()
    b = Builder()
    c = types.SimpleNamespace(num_actual_tokens=30, num_reqs=4, max_query_len=20, max_seq_len=100,
                              query_start_loc=torch.tensor([0, 1, 2, 10, 30]), query_start_loc_cpu=torch.tensor([0, 1, 2, 10, 30]),
                              seq_lens=torch.tensor([50, 60, 70, 100]), block_table_tensor=torch.zeros(4, 7, dtype=torch.int32),
                              slot_mapping=torch.zeros(30, dtype=torch.int64), causal=True, dcp_local_seq_lens=torch.tensor([25, 30, 35, 50]),
                              is_prefilling=None)
    md = b.build(0, c)
    assert (md.num_decodes, md.num_prefills, md.num_decode_tokens, md.num_prefill_tokens) == (2, 2, 2, 28)
    assert md.dcp_world_size == 1 and torch.equal(md.seq_lens, c.seq_lens)
    b.dcp_world_size, b.dcp_rank = 2, 1
    md = b.build(0, c)
    assert md.dcp_world_size == 2 and md.dcp_rank == 1 and torch.equal(md.seq_lens, c.dcp_local_seq_lens)


def test_memory_saving_patch_and_registration():
    kvi = pytest.importorskip("vllm.v1.kv_cache_interface")
    V.enable_cda_memory_saving()
    V.enable_cda_memory_saving()                      # idempotent
    assert kvi.AttentionSpec._cda_v2_patched is True
    spec = kvi.FullAttentionSpec(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.float16)
    assert spec.real_page_size_bytes == 16 * 8 * 144
    from sub0_b200 import vllm_plugin
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    vllm_plugin.register_cda_v2()
    assert AttentionBackendEnum.CUSTOM.get_class().__name__ == "CDAv2AttentionBackend"


def test_step_timing_hooks(monkeypatch, tmp_path):
    """CDA_V2_TIME_STEPS=1 brackets backend calls (reference ``_time_call``, cda_attn_v2.py:264-292); off by default."""
    from sub0_b200.vllm_integration import cda_attn_v2 as M
    M._STEP_TIMINGS.clear()
    assert M._time_call("x", lambda: 7) == 7 and not M._STEP_TIMINGS
    monkeypatch.setenv("CDA_V2_TIME_STEPS", "1")
    monkeypatch.setenv("CDA_V2_TIME_STEPS_OUT", str(tmp_path / "t"))
    assert M._time_call("forward_decode", lambda: 8) == 8
    M._time_call("forward_decode", lambda: None)
    summ = M.step_timing_summary()
    assert summ["forward_decode"]["calls"] == 2 and summ["forward_decode"]["cpu_ms_mean"] >= 0
    M._dump_step_timings()
    import json, os
    data = json.loads((tmp_path / f"t.{os.getpid()}.json").read_text())
    assert data["summary"]["forward_decode"]["calls"] == 2
    M._STEP_TIMINGS.clear()
