"""Two-GPU checks (skipped with fewer than 2 devices): KV-head sharding reproduces the single-GPU output (same kernel,
same bytes, no collective; only the fp32 summation order changes because fewer heads per CTA means more warps per
head), and sequence sharding matches the oracle both as partial -> all-gather -> merge and with the exchange inside the
merge kernel (peer stores)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sub0_b200 import ops
        from sub0_b200.sharding import decode_sequence_sharded, head_shard, sequence_shard
        from sub0_b200.synth import build_decode_workload
        from tests import _cases as Cs
        B, N, H_kv, group = 2, 2048, 8, 4
        # --- head sharding: this rank's heads of the seeded workload vs the same heads cut from the full workload
        lo, hi = head_shard(rank, world, H_kv)
        full = build_decode_workload(B, N, H_kv=H_kv, group=group, device=dev, seed=123)
        mine = build_decode_workload(B, N, H_kv=H_kv, group=group, device=dev, seed=123, head_lo=lo, head_hi=hi)
        out_full = torch.empty_like(full.Q)
        ops.decode(full.Q, full.cache, full.block_table, full.seq_lens, out_full, cb_K=full.cb_K, cb_V=full.cb_V,
                   block_size=16, max_seq_len=N, num_splits=4)
        out_mine = torch.empty_like(mine.Q)
        ops.decode(mine.Q, mine.cache, mine.block_table, mine.seq_lens, out_mine, cb_K=mine.cb_K, cb_V=mine.cb_V,
                   block_size=16, max_seq_len=N, num_splits=4)
        torch.cuda.synchronize()
        same = Cs.close(out_mine.cpu(), out_full[:, lo * group:hi * group].cpu(), atol=2e-4, rtol=1e-3, strict_rows=True)[0]
        # --- sequence sharding: each rank keeps the blocks of its key range only
        case = Cs.paged_case([1000, 333], H_kv=4, group=4, seed=5, shuffle=False, extra_blocks=0)
        want = Cs.oracle_decode(case)
        bt_rows, lens, local_max = [], [], 0
        for b, n in enumerate([1000, 333]):
            t0, t1 = sequence_shard(rank, world, n, 16)
            blocks = case["block_table"][b, t0 // 16:-(-t1 // 16)] if t1 > t0 else case["block_table"][b, :0]
            bt_rows.append(blocks)
            lens.append(t1 - t0)
            local_max = max(local_max, t1 - t0)
        width = max(max(len(r) for r in bt_rows), 1)
        bt = torch.zeros(2, width, dtype=torch.int32)
        for b, r in enumerate(bt_rows):
            bt[b, :len(r)] = r
        out = torch.empty(2, 16, 128, dtype=torch.float16, device=dev)
        decode_sequence_sharded(case["Q"].to(dev), case["cache"].to(dev), bt.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev),
                                out, cb_K=case["cb_K"].to(dev), cb_V=case["cb_V"].to(dev), block_size=16,
                                local_max_seq_len=max(local_max, 1))
        torch.cuda.synchronize()
        ok, ratio, cos = Cs.close(out.cpu(), want)
        # --- the same step with the exchange inside the merge kernel (peer stores, no collective): three calls, so that
        # both parities of the exchange buffers and a re-used parity are exercised; then the status word (bit 3 = a wait
        # for the other rank ran out of time) must be clear
        from sub0_b200.sharding import PeerExchange
        px = PeerExchange(2, 16, dev)
        ws = ops.new_workspace(ops.decode_workspace_bytes(2, 16, 4, max(local_max, 1)), dev)
        for call in range(3):
            out_px = torch.full((2, 16, 128), float("nan"), dtype=torch.float16, device=dev)
            px.decode(case["Q"].to(dev), case["cache"].to(dev), bt.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev),
                      out_px, cb_K=case["cb_K"].to(dev), cb_V=case["cb_V"].to(dev), block_size=16,
                      local_max_seq_len=max(local_max, 1), workspace=ws)
            torch.cuda.synchronize()
            ok_px, ratio_px, _ = Cs.close(out_px.cpu(), want)
            ok, ratio = ok and ok_px, max(ratio, ratio_px)
        ok = ok and ops.workspace_status(ws) == 0 and int(px.counters[0]) == 3
        px.close()
        # --- the vLLM backend's decode-context-parallel path (gathers over the default group).  The DCP group lies inside
        # the tensor-parallel group: both ranks share the two KV heads, each holds FOUR of the eight query heads of every
        # KV head (distinct queries per rank) and its own key range of every sequence.
        from sub0_b200.vllm_integration.cda_attn_v2 import get_backend_classes
        _, Impl, _, Metadata = get_backend_classes()
        case2 = Cs.paged_case([1000, 333], H_kv=2, group=8, seed=6, shuffle=False, extra_blocks=0)
        want2 = Cs.oracle_decode(case2).view(2, 2, world, 4, 128)[:, :, rank].reshape(2, 8, 128)
        q_local = case2["Q"].view(2, 2, world, 4, 128)[:, :, rank].reshape(2, 8 * 128).contiguous()
        bt_rows = []
        for b, n in enumerate([1000, 333]):
            t0, t1 = sequence_shard(rank, world, n, 16)
            bt_rows.append(case2["block_table"][b, t0 // 16:-(-t1 // 16)] if t1 > t0 else case2["block_table"][b, :0])
        bt2 = torch.zeros(2, width, dtype=torch.int32)
        for b, r in enumerate(bt_rows):
            bt2[b, :len(r)] = r
        impl = Impl(8, 128, 128 ** -0.5, num_kv_heads=2)
        slots, hkv, w = case2["cache"].shape
        kv = case2["cache"].view(slots // 16, 16, hkv, w).contiguous().to(dev).view(torch.float16)
        md = Metadata(num_actual_tokens=2, num_reqs=2, max_query_len=1, max_seq_len=max(local_max, 1),
                      query_start_loc=torch.tensor([0, 1, 2], dtype=torch.int32, device=dev),
                      seq_lens=torch.tensor(lens, dtype=torch.int32, device=dev), block_table=bt2.to(dev),
                      slot_mapping=torch.zeros(2, dtype=torch.int64, device=dev), dcp_world_size=world, dcp_rank=rank,
                      num_decodes=2, num_decode_tokens=2)
        out2 = torch.empty(2, 8 * 128, dtype=torch.float16, device=dev)
        impl.forward(None, q_local.to(dev), None, None, kv, md, output=out2)
        torch.cuda.synchronize()
        ok2, ratio2, _ = Cs.close(out2.view(2, 8, 128).cpu(), want2)
        # the same backend call with the exchange inside the merge kernel (opt-in switch), twice
        os.environ["CDA_V2_DCP_EXCHANGE"] = "peer"
        os.environ["CDA_V2_DCP_MAX_BATCH"] = "4"
        for _ in range(2):
            out3 = torch.full((2, 8 * 128), float("nan"), dtype=torch.float16, device=dev)
            impl.forward(None, q_local.to(dev), None, None, kv, md, output=out3)
            torch.cuda.synchronize()
            ok3, ratio3, _ = Cs.close(out3.view(2, 8, 128).cpu(), want2)
            ok2, ratio2 = ok2 and ok3, max(ratio2, ratio3)
        ok2 = ok2 and ops.workspace_status() == 0
        impl._px.close()
        q.put((rank, same, ok and ok2, max(ratio, ratio2)))
    except Exception as exc:
        q.put((rank, False, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_head_and_sequence_sharding_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, same, ok, ratio in sorted(results):
        assert same, f"rank {rank}: head-sharded output differs from the single-GPU slice ({ratio})"
        assert ok, f"rank {rank}: sequence-sharded decode off by {ratio}"
