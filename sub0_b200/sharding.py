"""Multi-GPU decode: one process per GPU (``torch.distributed``), two ways to split the work.

* **KV-head sharding** (:func:`head_shard`): rank r owns a contiguous slice of KV heads and the query heads that read
  them, with its own paged cache ``(slots, H_kv / W, slot_bytes)`` and the full block table.  Heads never interact
  (the reference's tensor-parallel split, ``cda/kernels_cuda/vllm_integration/cda_attn_v2.py:636-640``), so the data
  path has **no collective**; outputs stay head-sharded.
* **Sequence sharding** (:func:`sequence_shard`, :func:`decode_sequence_sharded`): for one very long sequence, rank r
  owns a contiguous, block-aligned range of keys of every head.  Each rank produces the un-normalised partial
  ``(O, m, l)`` of its keys, one all-gather moves ``(B, H_q, 130)`` fp32 per rank, and every rank merges locally --
  the path the reference leaves as ``NotImplementedError`` (``cda_attn_v2.py:1697-1701``) with the contract of
  ``cda/algorithm/attention.py:190-272``.  :class:`PeerExchange` is the same step without a collective library: the
  merge kernel stores its row into every GPU's memory over NVLink and merges what the others stored.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

PARTIAL_WIDTH = 130          # 128 un-normalised outputs, then m (natural log domain), then l


def head_shard(rank: int, world: int, H_kv: int) -> Tuple[int, int]:
    """KV heads [lo, hi) of ``rank``.  ``H_kv`` must divide evenly (8 heads -> world in {1, 2, 4, 8})."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if H_kv % world:
        raise ValueError(f"H_kv={H_kv} does not divide over {world} ranks")
    per = H_kv // world
    return rank * per, (rank + 1) * per


def sequence_shard(rank: int, world: int, seq_len: int, block_size: int) -> Tuple[int, int]:
    """Token range [lo, hi) of ``rank``: contiguous, starting on a block boundary, sizes differing by at most one
    block; ranks past the end get an empty range."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if block_size <= 0 or block_size % 16:
        raise ValueError("block_size must be a positive multiple of 16")
    blocks = -(-seq_len // block_size)
    base, extra = divmod(blocks, world)
    lo_blk = rank * base + min(rank, extra)
    hi_blk = lo_blk + base + (1 if rank < extra else 0)
    return min(lo_blk * block_size, seq_len), min(hi_blk * block_size, seq_len)


def gather_partials(packed: Tensor, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """All-gather packed partials ``(..., 130)`` from every rank into ``(world, ..., 130)`` (one collective)."""
    if packed.shape[-1] != PARTIAL_WIDTH:
        raise ValueError(f"packed partials must end in {PARTIAL_WIDTH} columns")
    packed = packed.contiguous()
    world = dist.get_world_size(group)
    flat = packed.reshape(-1)
    out = torch.empty(world * flat.numel(), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.view((world,) + tuple(packed.shape))


def decode_sequence_sharded(Q: Tensor, local_cache: Tensor, local_block_table: Tensor, local_seq_lens: Tensor,
                            output: Tensor, *, cb_K: Tensor, cb_V: Tensor, block_size: int, local_max_seq_len: int,
                            scale: Optional[float] = None, group: Optional[dist.ProcessGroup] = None,
                            workspace: Optional[Tensor] = None) -> None:
    """Decode one step when every rank holds a different key range of the same sequences.  ``Q`` and ``output`` are
    (B, H_q, 128) fp16; ``local_*`` describe this rank's keys only.

    Precondition: ``Q`` is the SAME tensor on every rank of ``group`` (all query heads, replicated) -- the partial rows
    of different ranks are merged row by row.  When the ranks hold different query heads (tensor parallelism inside the
    group) use :func:`decode_context_parallel`, which exchanges the queries first."""
    from . import ops
    packed = ops.decode_partial(Q, local_cache, local_block_table, local_seq_lens, cb_K=cb_K, cb_V=cb_V,
                                block_size=block_size, scale=scale, max_seq_len=local_max_seq_len, workspace=workspace)
    ops.merge_partials(gather_partials(packed, group), output)


class PeerExchange:
    """Exchange buffers of a sequence-sharded decode group: one buffer per rank, each mapped into every process of the
    node (CUDA IPC handles travel over the process group), so that the merge kernel can store its row straight into the
    other GPUs' memory.  Collective: every rank of ``group`` constructs it with the same ``B`` (the largest batch of a
    call; smaller batches use the front of the buffers, the same size on every rank) and ``H_q``.  The
    buffers live until :meth:`close` (collective as well); keep the object for the lifetime of the decode loop and of
    any CUDA graph captured over :meth:`decode`."""

    def __init__(self, B: int, H_q: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C
        from . import ops
        from ._lib import check, lib
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.B, self.H_q = B, H_q
        self._lib, self._own, self._imported = lib, None, []
        nbytes = ops.decode_exchange_bytes(B, H_q, self.world)
        with torch.cuda.device(device):
            own = C.c_void_p()
            check(lib.cda_b200_exchange_alloc(nbytes, C.byref(own)))
            self._own = own.value
            raw = C.create_string_buffer(64)
            check(lib.cda_b200_exchange_export(self._own, raw))
            handles = [None] * self.world
            dist.all_gather_object(handles, raw.raw, group=group)
            addresses = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    addresses.append(self._own)
                    continue
                ptr = C.c_void_p()
                check(lib.cda_b200_exchange_import(C.create_string_buffer(h, 64), C.byref(ptr)))
                self._imported.append(ptr.value)
                addresses.append(ptr.value)
        self.counters = torch.zeros(2, dtype=torch.int64, device=device)
        self.pointers = torch.tensor(addresses, dtype=torch.int64, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                                  # nobody sends before every mapping exists

    def close(self) -> None:
        """Unmap the other ranks' buffers and free this rank's (after a barrier: nobody may still be sending)."""
        if self._own is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for ptr in self._imported:
            self._lib.cda_b200_exchange_close(ptr)
        self._lib.cda_b200_exchange_free(self._own)
        self._own, self._imported = None, []

    def decode(self, Q: Tensor, local_cache: Tensor, local_block_table: Tensor, local_seq_lens: Tensor, output: Tensor, *,
               cb_K: Tensor, cb_V: Tensor, block_size: int, local_max_seq_len: int, scale: Optional[float] = None,
               workspace: Optional[Tensor] = None, wait_ms: int = 1000) -> None:
        """One decode step: split kernel over the local keys, then ONE kernel that merges, exchanges and merges again
        (see ``cda_b200_decode_exchange``).  Same precondition on ``Q`` as :func:`decode_sequence_sharded`."""
        from . import ops
        if Q.shape[0] > self.B or Q.shape[1] != self.H_q:
            raise ValueError("Q does not match the exchange buffers (at most B sequences, exactly H_q heads)")
        ops.decode_exchange(Q, local_cache, local_block_table, local_seq_lens, output, cb_K=cb_K, cb_V=cb_V,
                            block_size=block_size, peer_pointers=self.pointers, counters=self.counters, rank=self.rank,
                            world=self.world, scale=scale, max_seq_len=local_max_seq_len, wait_ms=wait_ms,
                            workspace=workspace)


def gather_heads(q_local: Tensor, H_kv: int, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """All-gather query heads over ``group``: every rank holds (n, H_kv * g_local, 128) -- its own g_local query heads of
    each of the H_kv KV heads the group shares -- and receives (n, H_kv * world * g_local, 128) ordered
    (KV head, rank, local head), i.e. KV head h again owns a contiguous run of world * g_local query heads."""
    world = dist.get_world_size(group)
    n, h_local, d = q_local.shape
    g_local = h_local // H_kv
    buf = torch.empty((world, n, h_local, d), dtype=q_local.dtype, device=q_local.device)
    dist.all_gather_into_tensor(buf.view(-1), q_local.contiguous().view(-1), group=group)
    return buf.view(world, n, H_kv, g_local, d).permute(1, 2, 0, 3, 4).reshape(n, H_kv * world * g_local, d).contiguous()


def decode_context_parallel(q_local: Tensor, local_cache: Tensor, local_block_table: Tensor, local_seq_lens: Tensor,
                            output_local: Tensor, *, cb_K: Tensor, cb_V: Tensor, block_size: int, local_max_seq_len: int,
                            scale: Optional[float] = None, group: Optional[dist.ProcessGroup] = None,
                            workspace: Optional[Tensor] = None, exchange: Optional["PeerExchange"] = None) -> None:
    """Decode step of a context-parallel group that sits inside a tensor-parallel group: the ranks share the same KV
    heads, each holds its own slice of the query heads of those KV heads and its own part of every sequence's keys.

    1. all-gather the queries along the head axis, so that every rank attends ALL of the group's query heads over its
       own keys (the GQA group seen by the kernel becomes world * g_local, which must stay <= 8);
    2. partial (O, m, l) rows of those heads over the local keys;
    3. one all-gather of the packed partials, local log-sum-exp merge (cda/algorithm/attention.py:239-272);
    4. keep this rank's query heads.
    With ``exchange`` (a :class:`PeerExchange` of the same group, built for ``H_kv * world * g_local`` heads) steps 2 and 3
    are one call: the merge kernel exchanges the rows by peer stores instead of the all-gather.
    ``q_local`` / ``output_local``: (n, H_kv * g_local, 128) fp16."""
    from . import ops
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    H_kv = local_cache.shape[-2]
    n, h_local, d = q_local.shape
    g_local = h_local // H_kv
    if g_local * H_kv != h_local or g_local * world > 8:
        raise NotImplementedError(f"context-parallel decode needs world * local GQA group <= 8 (got {world} x {g_local})")
    q_all = gather_heads(q_local, H_kv, group)
    out_all = torch.empty_like(q_all)
    if exchange is not None:
        exchange.decode(q_all, local_cache, local_block_table, local_seq_lens, out_all, cb_K=cb_K, cb_V=cb_V,
                        block_size=block_size, local_max_seq_len=local_max_seq_len, scale=scale, workspace=workspace)
    else:
        packed = ops.decode_partial(q_all, local_cache, local_block_table, local_seq_lens, cb_K=cb_K, cb_V=cb_V,
                                    block_size=block_size, scale=scale, max_seq_len=local_max_seq_len, workspace=workspace)
        ops.merge_partials(gather_partials(packed, group), out_all)
    output_local.copy_(out_all.view(n, H_kv, world, g_local, d)[:, :, rank].reshape(n, h_local, d))
