"""Host logic of the multi-GPU paths on CPU ranks (gloo, world size 2): shard plans, the one all-gather of packed
partials, and that merging shard partials reproduces the unsharded result (checked with the oracle -- no kernel runs)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import cda_oracle as O
from tests import _cases as Cs


def test_shard_plans():
    from sub0_b200.sharding import head_shard, sequence_shard
    assert [head_shard(r, 4, 8) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert head_shard(7, 8, 8) == (7, 8)
    with pytest.raises(ValueError):
        head_shard(0, 3, 8)
    n = 1_048_576
    parts = [sequence_shard(r, 8, n, 16) for r in range(8)]
    assert parts[0][0] == 0 and parts[-1][1] == n and all(parts[i][1] == parts[i + 1][0] for i in range(7))
    assert all(lo % 16 == 0 for lo, _ in parts) and {hi - lo for lo, hi in parts} == {n // 8}
    ragged = [sequence_shard(r, 4, 100, 16) for r in range(4)]          # 7 blocks over 4 ranks
    assert ragged == [(0, 32), (32, 64), (64, 96), (96, 100)]
    assert sequence_shard(3, 4, 20, 16) == (20, 20)                      # nothing left for the last ranks


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sub0_b200.sharding import gather_partials, sequence_shard
        torch.set_num_threads(1)
        n, bs = 200, 16
        case = Cs.paged_case([n], H_kv=2, group=4, seed=77, block_size=bs)        # same seed -> same data on every rank
        want = Cs.oracle_decode(case)
        lo, hi = sequence_shard(rank, world, n, bs)
        Ks, Vs = O.gather_sequence(case["cache"], case["block_table"][0], n, bs)
        Qr = O.rotate(case["Q"][0][None, :, None, :], O.sylvester_hadamard())
        Oo, m, l = O.cda_partial_rotated(Qr, Ks, Vs, cb_K=case["cb_K"], cb_V=case["cb_V"], group=4, key_start=lo, key_end=hi)
        packed = torch.cat([Oo[0, :, 0], m[0, :, 0, None], l[0, :, 0, None]], dim=-1)[None]       # (1, H_q, 130)
        allp = gather_partials(packed)                                                              # (world, 1, H_q, 130)
        assert allp.shape == (world, 1, 8, 130)
        parts = [(allp[r, :, :, None, :128], allp[r, :, :, None, 128], allp[r, :, :, None, 129]) for r in range(world)]
        merged = O.unrotate(O.merge_partials(parts), O.sylvester_hadamard())[:, :, 0]
        ok, ratio, cos = Cs.close(merged, want)
        # query all-gather of the context-parallel path: rank r holds heads (kv j, r, i) of a (kv, rank, local) grid
        from sub0_b200.sharding import gather_heads
        grid = torch.arange(3 * 2 * world * 2 * 128, dtype=torch.float32).view(3, 2, world, 2, 128)   # (n, kv, rank, local, d)
        mine = grid[:, :, rank].reshape(3, 4, 128).contiguous()
        ok = ok and bool(torch.equal(gather_heads(mine, 2), grid.reshape(3, 2 * world * 2, 128)))
        q.put((rank, ok, ratio, bool(torch.equal(allp[rank], packed))))
    except Exception as exc:                      # report instead of leaving the parent waiting
        q.put((rank, False, float("inf"), repr(exc)))
    finally:
        dist.destroy_process_group()


def test_sequence_shard_all_gather_and_merge_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, ratio, own in sorted(results):
        assert ok, f"rank {rank}: merged shards differ from the unsharded oracle (ratio {ratio:.3f}) {own}"
        assert own is True
