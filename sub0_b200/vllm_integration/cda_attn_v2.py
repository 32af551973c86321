"""vLLM attention backend ``cda_v2`` over the B200 kernels of this package.

Mirrors the reference backend ``cda/kernels_cuda/vllm_integration/cda_attn_v2.py`` (classes ``:443-864``, entry
points ``:1707-1756``): same class names, methods, class attributes, argument meaning and error behaviour, but every
device computation goes through :mod:`sub0_b200.kernels_cuda` (``paged_encode_fused_cuda``, ``decode_hmma_v1``,
``fa2_cda_prefill_varlen_v1``) and :mod:`sub0_b200.ops` (partial decode + merge for decode context parallelism).

What differs from the reference, on purpose:

* one prefill route: the fused kernel handles full prompts, chunked prefill with a compressed past and ragged
  batches alike (``q_offset = seq_len - q_len`` per request), so there is no backend switch and no "uniform chunk"
  restriction (reference ``:817-851``);
* decode context parallelism is implemented (the reference raises ``NotImplementedError``, ``:1697-1701``): every
  rank attends over its own key shard with the partial kernel, the ``(O, m, l)`` rows are all-gathered over vLLM's
  DCP group and merged locally;
* the backend registers in vLLM's ``CUSTOM`` slot (stock vLLM has no ``CDA`` member).

The module imports without vLLM (stand-in base classes), which is how the CPU tests exercise the host logic.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

HEAD_DIM = 128
DATA_BYTES_PER_TOKEN = HEAD_DIM + 8                               # k4v4 payload: 64 + 64 + 4 + 4
BYTES_PER_TOKEN = (DATA_BYTES_PER_TOKEN + 15) // 16 * 16          # 144: slots start on 16-byte boundaries
SLOT_FP16_ELEMS_COMPACT = BYTES_PER_TOKEN // 2                    # 72 fp16 elements per slot (compact allocation)
SLOT_FP16_ELEMS_DEFAULT = 2 * HEAD_DIM                            # 256 fp16 elements (vLLM's un-patched K+V page)


def as_uint8_cache(kv_cache: torch.Tensor) -> torch.Tensor:
    """View vLLM's fp16-typed cache ``(num_blocks, block_size, H_kv, 72)`` as bytes ``(..., 144)``
    (reference ``_as_uint8_cache``, ``:63-78``).  The un-patched 256-element page is refused: its slots would be
    512 bytes apart, which the kernels' 144-byte layout does not describe."""
    if kv_cache.dtype == torch.uint8:
        if kv_cache.dim() != 4 or kv_cache.shape[-1] != BYTES_PER_TOKEN:
            raise ValueError(f"CDA cache must be (num_blocks, block_size, H_kv, {BYTES_PER_TOKEN}) uint8, got {tuple(kv_cache.shape)}")
        return kv_cache
    if kv_cache.dim() != 4 or kv_cache.element_size() != 2:
        raise ValueError(f"CDA cache must be a 4-D 16-bit or uint8 tensor, got {tuple(kv_cache.shape)} {kv_cache.dtype}")
    nb, bs, hkv, last = kv_cache.shape
    if last != SLOT_FP16_ELEMS_COMPACT:
        raise ValueError(f"unexpected CDA cache last dim {last} (expected {SLOT_FP16_ELEMS_COMPACT}; call "
                         "enable_cda_memory_saving() before the engine allocates the cache)")
    return kv_cache.view(torch.uint8).view(nb, bs, hkv, BYTES_PER_TOKEN)


def enable_cda_memory_saving() -> None:
    """Make vLLM size KV pages for 144-byte slots (reference ``:84-106``): patches ``real_page_size_bytes`` of the
    attention specs.  Idempotent; call before the engine allocates the cache."""
    from vllm.v1 import kv_cache_interface as kvi

    if getattr(kvi.AttentionSpec, "_cda_v2_patched", False):
        return

    def _real_page_size_bytes(self):
        return self.block_size * self.num_kv_heads * BYTES_PER_TOKEN

    prop = property(_real_page_size_bytes)
    for name in ("AttentionSpec", "FullAttentionSpec", "ChunkedLocalAttentionSpec", "SlidingWindowSpec"):
        cls = getattr(kvi, name, None)
        if cls is not None and "real_page_size_bytes" in cls.__dict__:
            cls.real_page_size_bytes = prop
    kvi.AttentionSpec._cda_v2_patched = True


def split_counts_from_query_start(query_start_loc, num_reqs: int, num_actual_tokens: int, max_query_len: int):
    """``(num_decodes, num_prefills, num_decode_tokens, num_prefill_tokens)`` of a batch that vLLM ordered decodes
    first (reference ``_split_counts_from_query_start``, ``:352-383``): the decodes are the leading requests with one
    query token.  Reads ``query_start_loc`` on the host."""
    if num_reqs == 0:
        return 0, 0, 0, 0
    if max_query_len <= 1:
        return num_reqs, 0, num_actual_tokens, 0
    qs = query_start_loc[: num_reqs + 1].tolist() if hasattr(query_start_loc, "tolist") else list(query_start_loc)[: num_reqs + 1]
    num_decodes = 0
    while num_decodes < num_reqs and qs[num_decodes + 1] - qs[num_decodes] == 1:
        num_decodes += 1
    num_decode_tokens = int(qs[num_decodes]) - int(qs[0]) if num_decodes else 0
    return num_decodes, num_reqs - num_decodes, num_decode_tokens, num_actual_tokens - num_decode_tokens


# ---- optional per-call timing (CDA_V2_TIME_STEPS=1) -----------------------------------------------------------------------
# Same switch and output location as the reference's ``_time_call`` (``:115-296``): with CDA_V2_TIME_STEPS=1 every
# backend call (cache update, decode, prefill, DCP decode) is bracketed by a host timer and -- outside stream capture -- a
# pair of CUDA events; ``step_timing_summary()`` resolves the events, and the summary is written as JSON to
# ``$CDA_V2_TIME_STEPS_OUT`` (default /tmp/cda_v2_step_timings) + ``.<pid>.json`` when the process exits.
_STEP_TIMINGS: dict = {}


def _time_steps_enabled() -> bool:
    import os
    return os.environ.get("CDA_V2_TIME_STEPS") == "1"


def _time_call(label: str, fn):
    """Run ``fn()``; when step timing is on, record its host time and (if the stream is not capturing) device time."""
    if not _time_steps_enabled():
        return fn()
    import time
    events = None
    if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
        events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        events[0].record()
    t0 = time.perf_counter()
    try:
        return fn()
    finally:
        cpu_ms = (time.perf_counter() - t0) * 1e3
        if events is not None:
            events[1].record()
        if not _STEP_TIMINGS:
            import atexit
            atexit.register(_dump_step_timings)
        _STEP_TIMINGS.setdefault(label, []).append((cpu_ms, events))


def step_timing_summary() -> dict:
    """``{label: {calls, cpu_ms_mean, gpu_ms_mean, gpu_calls}}`` of the calls timed so far (synchronises the device)."""
    if torch.cuda.is_available() and any(ev is not None for recs in _STEP_TIMINGS.values() for _, ev in recs):
        torch.cuda.synchronize()
    out = {}
    for label, recs in _STEP_TIMINGS.items():
        gpu = [ev[0].elapsed_time(ev[1]) for _, ev in recs if ev is not None]
        out[label] = {"calls": len(recs), "cpu_ms_mean": sum(c for c, _ in recs) / len(recs),
                      "gpu_ms_mean": (sum(gpu) / len(gpu)) if gpu else None, "gpu_calls": len(gpu)}
    return out


def _dump_step_timings() -> None:
    import json
    import os
    try:
        path = os.environ.get("CDA_V2_TIME_STEPS_OUT", "/tmp/cda_v2_step_timings") + f".{os.getpid()}.json"
        with open(path, "w") as f:
            json.dump({"pid": os.getpid(), "summary": step_timing_summary()}, f, indent=2)
    except Exception:
        pass


_CODEBOOKS: dict = {}


def get_codebooks(device: torch.device):
    """The reference's default 16-level codebook for K and V on ``device`` (``_get_compressors``, ``:109-131``);
    cached per device.  Replace with :func:`set_codebooks` for a calibrated table."""
    key = (device.type, device.index)
    if key not in _CODEBOOKS:
        from .. import codebook

        cb = codebook.default_codebook(16).to(device)
        _CODEBOOKS[key] = (cb, cb)
    return _CODEBOOKS[key]


def set_codebooks(device: torch.device, cb_K: torch.Tensor, cb_V: torch.Tensor) -> None:
    _CODEBOOKS[(device.type, device.index)] = (cb_K.to(device=device, dtype=torch.float32).contiguous(),
                                              cb_V.to(device=device, dtype=torch.float32).contiguous())


def _vllm_bases():
    try:
        from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata,
                                               AttentionMetadataBuilder, AttentionType, MultipleOf)
        return AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata, AttentionMetadataBuilder, AttentionType, MultipleOf, True
    except ModuleNotFoundError:
        class _Generic:
            def __init__(self, *a, **k):
                pass

            def __class_getitem__(cls, item):
                return cls

        class AttentionBackend:
            pass

        class AttentionImpl(_Generic):
            pass

        class AttentionMetadata:
            pass

        class AttentionMetadataBuilder(_Generic):
            pass

        class AttentionType:
            DECODER = "decoder"

        class AttentionCGSupport:
            UNIFORM_BATCH = "uniform_batch"

        class MultipleOf(int):
            pass

        return AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata, AttentionMetadataBuilder, AttentionType, MultipleOf, False


_CLASSES = None


def get_backend_classes():
    """``(Backend, Impl, MetadataBuilder, Metadata)``, built on first use (reference ``get_backend_classes``, ``:1749-1756``)."""
    global _CLASSES
    if _CLASSES is None:
        _CLASSES = _build_backend_classes()
    return _CLASSES


def _build_backend_classes():
    (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata, AttentionMetadataBuilder, AttentionType,
     MultipleOf, have_vllm) = _vllm_bases()

    @dataclass
    class CDAv2AttentionMetadata(AttentionMetadata):
        """Per-step metadata (reference ``:443-463``).  With decode context parallelism ``seq_lens`` are the lengths of
        this rank's key shard."""
        num_actual_tokens: int
        num_reqs: int
        max_query_len: int
        max_seq_len: int
        query_start_loc: torch.Tensor
        seq_lens: torch.Tensor
        block_table: torch.Tensor
        slot_mapping: torch.Tensor
        causal: bool = True
        dcp_world_size: int = 1
        dcp_rank: int = 0
        num_prefill_tokens: int = 0
        num_decode_tokens: int = 0
        num_prefills: int = 0
        num_decodes: int = 0

    class CDAv2AttentionMetadataBuilder(AttentionMetadataBuilder[CDAv2AttentionMetadata]):
        _cudagraph_support: ClassVar = AttentionCGSupport.UNIFORM_BATCH
        reorder_batch_threshold: Optional[int] = 1          # decodes first, so one boundary splits the batch

        @classmethod
        def get_cudagraph_support(cls, vllm_config=None, kv_cache_spec=None):
            return cls._cudagraph_support

        def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None) -> None:
            if have_vllm and vllm_config is not None:
                super().__init__(kv_cache_spec, layer_names, vllm_config, device)
            self.dcp_world_size, self.dcp_rank = 1, 0
            try:
                from vllm.distributed.parallel_state import get_dcp_group

                self.dcp_world_size = get_dcp_group().world_size
                self.dcp_rank = get_dcp_group().rank_in_group
            except Exception:                                # not initialised: no context parallelism
                pass

        def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False) -> CDAv2AttentionMetadata:
            c = common_attn_metadata
            counts = None
            if have_vllm:
                try:
                    from vllm.v1.attention.backends.utils import split_decodes_and_prefills

                    counts = split_decodes_and_prefills(c, decode_threshold=1)
                except Exception:
                    counts = None
            if counts is None:
                qsl = getattr(c, "query_start_loc_cpu", None)
                counts = split_counts_from_query_start(qsl if qsl is not None else c.query_start_loc, c.num_reqs,
                                                       c.num_actual_tokens, c.max_query_len)
            num_decodes, num_prefills, num_decode_tokens, num_prefill_tokens = counts
            seq_lens = c.seq_lens
            if self.dcp_world_size > 1 and getattr(c, "dcp_local_seq_lens", None) is not None:
                seq_lens = c.dcp_local_seq_lens
            return CDAv2AttentionMetadata(
                num_actual_tokens=c.num_actual_tokens, num_reqs=c.num_reqs, max_query_len=c.max_query_len,
                max_seq_len=c.max_seq_len, query_start_loc=c.query_start_loc, seq_lens=seq_lens,
                block_table=c.block_table_tensor, slot_mapping=c.slot_mapping, causal=getattr(c, "causal", True),
                dcp_world_size=self.dcp_world_size, dcp_rank=self.dcp_rank, num_prefill_tokens=num_prefill_tokens,
                num_decode_tokens=num_decode_tokens, num_prefills=num_prefills, num_decodes=num_decodes)

    class CDAv2AttentionBackend(AttentionBackend):
        accept_output_buffer: bool = True
        supported_dtypes: ClassVar[list] = [torch.float16]
        supported_kv_cache_dtypes: ClassVar[list] = ["auto", "uint8"]
        forward_includes_kv_cache_update: bool = False

        @staticmethod
        def get_supported_kernel_block_sizes() -> list:
            return [MultipleOf(16)]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM" if have_vllm else "CDA"

        @staticmethod
        def get_impl_cls():
            return CDAv2AttentionImpl

        @staticmethod
        def get_builder_cls():
            return CDAv2AttentionMetadataBuilder

        @staticmethod
        def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                               cache_dtype_str: str = "auto") -> tuple:
            if head_size != HEAD_DIM:
                raise ValueError(f"CDA backend supports head_size={HEAD_DIM} only. Got head_size={head_size}.")
            if have_vllm:
                enable_cda_memory_saving()
            return (num_blocks, block_size, num_kv_heads, SLOT_FP16_ELEMS_COMPACT)

        @classmethod
        def get_supported_head_sizes(cls) -> list:
            return [HEAD_DIM]

        @staticmethod
        def swap_blocks(src_kv_cache: torch.Tensor, dst_kv_cache: torch.Tensor, src_to_dst: torch.Tensor) -> None:
            dst_kv_cache[src_to_dst[:, 1]] = src_kv_cache[src_to_dst[:, 0]]

        @staticmethod
        def copy_blocks(kv_caches: list, src_to_dists: torch.Tensor) -> None:
            for kv_cache in kv_caches:
                kv_cache[src_to_dists[:, 1]] = kv_cache[src_to_dists[:, 0]]

    class CDAv2AttentionImpl(AttentionImpl[CDAv2AttentionMetadata]):
        # The reference leaves this False (``:621``): its decode kernel cannot hand out the log-sum-exp.  Here the merge
        # kernel writes it on request (``forward_decode_with_lse``), and the DCP path exchanges (O, m, l) itself.
        can_return_lse_for_decode: bool = True

        def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                     alibi_slopes: Optional[list] = None, sliding_window: Optional[int] = None, kv_cache_dtype: str = "auto",
                     logits_soft_cap: Optional[float] = None, attn_type: str = AttentionType.DECODER,
                     kv_sharing_target_layer_name: Optional[str] = None) -> None:
            self.num_heads = num_heads
            self.head_size = head_size
            self.scale = float(scale)
            self.num_kv_heads = num_kv_heads or num_heads
            self.group_size = self.num_heads // self.num_kv_heads
            self.attn_type = attn_type
            if head_size != HEAD_DIM:
                raise NotImplementedError(f"CDA backend supports head_size={HEAD_DIM} only, got {head_size}.")
            if alibi_slopes is not None:
                raise NotImplementedError("CDA backend does not support ALiBi.")
            if sliding_window is not None:
                raise NotImplementedError("CDA backend does not support sliding window.")
            if attn_type not in (AttentionType.DECODER,):
                raise NotImplementedError(f"CDA backend is DECODER-only, got {attn_type}.")
            if self.group_size not in (4, 8):
                raise NotImplementedError(f"CDA supports group_size in {{4, 8}}. Got group_size={self.group_size}.")

        # -- cache update ------------------------------------------------------------------------------------------
        def do_kv_cache_update(self, layer, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                               slot_mapping: torch.Tensor) -> None:
            if kv_cache.numel() == 0:
                return
            from ..kernels_cuda.wrappers import paged_encode_fused_cuda

            cache = as_uint8_cache(kv_cache)
            nb, bs, hkv, w = cache.shape
            cb_K, cb_V = get_codebooks(cache.device)
            n = slot_mapping.shape[0]
            _time_call("do_kv_cache_update", lambda: paged_encode_fused_cuda(
                key[:n], value[:n], slot_mapping, cache.view(nb * bs, hkv, w), cb_K=cb_K, cb_V=cb_V))

        # -- attention ---------------------------------------------------------------------------------------------
        def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                    attn_metadata, output: Optional[torch.Tensor] = None, output_scale: Optional[torch.Tensor] = None,
                    output_block_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
            if output is None:
                raise ValueError("CDA backend requires an output buffer.")
            if output_scale is not None or output_block_scale is not None:
                raise NotImplementedError("CDA backend does not support fused output quantization.")
            if attn_metadata is None:                        # profiling run
                return output.fill_(0)
            md = attn_metadata
            cache = as_uint8_cache(kv_cache)
            n = md.num_actual_tokens
            q = query[:n].view(n, self.num_heads, HEAD_DIM)
            out = output[:n].view(n, self.num_heads, HEAD_DIM)
            if md.dcp_world_size > 1:
                if md.max_query_len > 1:
                    raise NotImplementedError("CDA decode context parallelism covers decode steps only.")
                _time_call("forward_decode_dcp", lambda: self._forward_decode_dcp(q, cache, out, md))
                return output
            if md.max_query_len <= 1:
                _time_call("forward_decode", lambda: self._forward_decode(q, cache, out, md.block_table, md.seq_lens, md.max_seq_len))
                return output
            nd, npf, nd_tok, np_tok = md.num_decodes, md.num_prefills, md.num_decode_tokens, md.num_prefill_tokens
            if nd + npf != md.num_reqs or nd_tok + np_tok != n:      # metadata built elsewhere: recount
                nd, npf, nd_tok, np_tok = split_counts_from_query_start(md.query_start_loc, md.num_reqs, n, md.max_query_len)
            if nd_tok > 0:                                   # decodes come first in the batch
                _time_call("forward_decode", lambda: self._forward_decode(q[:nd_tok], cache, out[:nd_tok], md.block_table[:nd],
                                                                          md.seq_lens[:nd], md.max_seq_len))
            if np_tok > 0:
                cu = md.query_start_loc[nd: nd + npf + 1]
                if nd_tok:
                    cu = cu - nd_tok
                _time_call("forward_prefill", lambda: self._forward_prefill(
                    q[nd_tok: nd_tok + np_tok], cache, out[nd_tok: nd_tok + np_tok], md.block_table[nd: nd + npf], cu,
                    md.seq_lens[nd: nd + npf], md.max_query_len, md.max_seq_len))
            return output

        def _flat(self, cache: torch.Tensor):
            nb, bs, hkv, w = cache.shape
            return cache.view(nb * bs, hkv, w), bs

        def _forward_decode(self, q, cache, out, block_table, seq_lens, max_seq_len) -> None:
            from ..kernels_cuda.wrappers import decode_hmma_v1

            flat, bs = self._flat(cache)
            cb_K, cb_V = get_codebooks(cache.device)
            dst = out if out.is_contiguous() else torch.empty_like(q)
            decode_hmma_v1(q.contiguous(), flat, block_table, seq_lens, dst, cb_K=cb_K, cb_V=cb_V, group_size=self.group_size,
                           block_size=bs, scale=self.scale, max_seq_len=int(max_seq_len))
            if dst is not out:
                out.copy_(dst)

        def forward_decode_with_lse(self, query: torch.Tensor, kv_cache: torch.Tensor, attn_metadata):
            """Decode step that also returns the log-sum-exp of the scaled scores: ``(out (n, H, 128) fp16, lse (n, H) fp32,
            natural log)`` -- what ``can_return_lse_for_decode`` promises a caller that corrects the output across ranks
            itself."""
            from .. import ops

            md = attn_metadata
            cache = as_uint8_cache(kv_cache)
            n = md.num_actual_tokens
            q = query[:n].view(n, self.num_heads, HEAD_DIM).contiguous()
            flat, bs = self._flat(cache)
            cb_K, cb_V = get_codebooks(cache.device)
            out = torch.empty_like(q)
            lse = torch.empty(n, self.num_heads, dtype=torch.float32, device=q.device)
            ops.decode(q, flat, md.block_table, md.seq_lens, out, cb_K=cb_K, cb_V=cb_V, block_size=bs, scale=self.scale,
                       max_seq_len=int(md.max_seq_len), lse=lse)
            return out, lse

        def _forward_prefill(self, q, cache, out, block_table, cu_seqlens_q, seq_lens, max_query_len, max_seq_len) -> None:
            from ..kernels_cuda.fa2_cda import fa2_cda_prefill_varlen_v1

            flat, bs = self._flat(cache)
            cb_K, cb_V = get_codebooks(cache.device)
            dst = out if out.is_contiguous() else torch.empty_like(q)
            fa2_cda_prefill_varlen_v1(q.contiguous(), flat, block_table, cu_seqlens_q.to(torch.int32), seq_lens, dst, cb_K=cb_K,
                                      cb_V=cb_V, rotation_fp32=None, group_size=self.group_size, block_size=bs,
                                      max_query_len=int(max_query_len), max_seq_len=int(max_seq_len), scale=self.scale,
                                      causal=True, fuse_fa2_epilogue=True)
            if dst is not out:
                out.copy_(dst)

        def _dcp_exchange(self, q, group):
            """``CDA_V2_DCP_EXCHANGE=peer``: exchange the partial rows inside the merge kernel (peer stores over NVLink)
            instead of the all-gather.  The buffers are built once, collectively, for ``CDA_V2_DCP_MAX_BATCH`` sequences
            (256 by default); a larger batch takes the all-gather."""
            import torch.distributed as dist

            if os.environ.get("CDA_V2_DCP_EXCHANGE", "nccl") != "peer":
                return None
            cap = int(os.environ.get("CDA_V2_DCP_MAX_BATCH", "256"))
            if q.shape[0] > cap:
                return None
            px = getattr(self, "_px", None)
            if px is None:
                from ..sharding import PeerExchange

                heads_all = q.shape[1] * dist.get_world_size(group)
                px = self._px = PeerExchange(cap, heads_all, q.device, group=group)
            return px

        def _forward_decode_dcp(self, q, cache, out, md) -> None:
            """Decode with the keys of every sequence sharded over the DCP group.  The group lies inside the
            tensor-parallel group: its ranks share this rank's KV heads but hold different query heads, so the queries are
            all-gathered along the head axis first; then this rank's ``(O, m, l)`` rows over its own key shard, one
            all-gather, local merge (the split-KV contract of ``attention_partial_reference`` / ``merge_partials``,
            cda/algorithm/attention.py:190-272), and this rank keeps its own heads."""
            from ..sharding import decode_context_parallel

            flat, bs = self._flat(cache)
            cb_K, cb_V = get_codebooks(cache.device)
            group = None
            try:
                from vllm.distributed.parallel_state import get_dcp_group

                group = get_dcp_group().device_group
            except Exception:
                group = None                                 # plain torch.distributed default group (tests)
            dst = out if out.is_contiguous() else torch.empty_like(q)
            decode_context_parallel(q.contiguous(), flat, md.block_table, md.seq_lens, dst, cb_K=cb_K, cb_V=cb_V,
                                    block_size=bs, local_max_seq_len=int(md.max_seq_len), scale=self.scale, group=group,
                                    exchange=self._dcp_exchange(q, group))
            if dst is not out:
                out.copy_(dst)

    return CDAv2AttentionBackend, CDAv2AttentionImpl, CDAv2AttentionMetadataBuilder, CDAv2AttentionMetadata


def register_backend(slot: str = "CUSTOM") -> None:
    """Register the backend classes in vLLM's ``AttentionBackendEnum`` (reference ``register_backend``, ``:1712-1747``).
    Stock vLLM offers the ``CUSTOM`` member for out-of-tree backends; select it with
    ``--attention-backend CUSTOM`` (or ``VLLM_ATTENTION_BACKEND=CUSTOM``)."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    from vllm.v1.attention.backends.registry import register_backend as _register

    member = AttentionBackendEnum[slot]
    _register(member, "sub0_b200.vllm_integration._backend_eager.CDAv2AttentionBackend")
