"""``cda_b200_decode_static`` -- the decode entry point that brings its own scratch -- against ``cda_b200_decode``.

Some hosts of this library cannot allocate device memory when they call it: an inference runtime that sized its memory
pool at start-up and gave all of it away, a plugin that is only allowed to touch the tensors it is handed, code that
runs while the framework's allocator is locked.  For them the library carries an 8 MiB split-KV scratch of its own.
This test calls the entry point straight through the C ABI, twice in a row with different problems (the second call
finds the first call's leftovers in the shared scratch), and checks each result against the ordinary entry point,
which gets a fresh caller-owned workspace.  It also checks that a problem too large for the built-in scratch is
refused with a message instead of being run.

The file name sorts last on purpose: if this entry point is broken, a run that stops at the first failure has still
executed every other test.
"""
import pytest
import torch

from tests import _cases as Cs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def both_entry_points(case, num_splits):
    from sub0_b200 import _lib, ops
    L = _lib.lib
    d = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    Q, cache, bt, sl = d["Q"].contiguous(), d["cache"], d["block_table"].contiguous(), d["seq_lens"].contiguous()
    cbk, cbv = d["cb_K"].float().contiguous(), d["cb_V"].float().contiguous()
    B, Hq = Q.shape[0], Q.shape[1]
    slots, Hkv, W = cache.shape
    max_len = int(case["seq_lens"].max())
    kb, vb, bs = case["k_bits"], case["v_bits"], case["block_size"]
    scale = 1.0 / 128 ** 0.5
    stream = torch.cuda.current_stream().cuda_stream

    out_static = torch.full_like(Q, float("nan"))
    rc = L.cda_b200_decode_static(Q.data_ptr(), cache.data_ptr(), bt.data_ptr(), sl.data_ptr(), cbk.data_ptr(),
                                  cbv.data_ptr(), out_static.data_ptr(), B, Hq, Hkv, bs, bt.shape[1], max_len, slots, W,
                                  kb, vb, scale, num_splits, stream)
    assert rc == 0, _lib.last_error()

    need = L.cda_b200_decode_workspace_bytes(B, Hq, Hkv, max_len, num_splits, -1)
    ws = ops.new_workspace(need, torch.device(DEV))
    out_ref = torch.full_like(Q, float("nan"))
    rc = L.cda_b200_decode(Q.data_ptr(), cache.data_ptr(), bt.data_ptr(), sl.data_ptr(), cbk.data_ptr(), cbv.data_ptr(),
                           out_ref.data_ptr(), ws.data_ptr(), need, B, Hq, Hkv, bs, bt.shape[1], max_len, slots, W, kb, vb,
                           scale, num_splits, stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out_static.cpu(), out_ref.cpu()


def test_static_scratch_matches_workspace_entry_point_twice():
    # first call: four partials per output row; second call: a different, smaller problem with other bit widths, so
    # every byte it reads from the scratch was either rewritten by it or is skipped
    first = Cs.paged_case([3000, 777, 2048], H_kv=8, group=4, seed=901)
    second = Cs.paged_case([130, 0, 1], H_kv=2, group=8, k_bits=4, v_bits=2, seed=902)
    for case, splits in ((first, 4), (second, 0), (first, 0)):
        got, ref = both_entry_points(case, splits)
        assert not bool(got.isnan().any())
        ok, ratio, cos = Cs.close(got, ref, strict_rows=True)
        assert ok and cos >= 0.9999, f"static scratch vs workspace: worst error/tolerance {ratio:.3f}, cosine {cos:.6f}"
        assert torch.equal(got, ref)          # same plan, same kernels: the two paths should agree bit for bit
        want = Cs.oracle_decode(case)
        ok, ratio, cos = Cs.close(got, want)
        assert ok, f"static scratch vs oracle: worst error/tolerance {ratio:.3f}"


def test_static_scratch_refuses_what_does_not_fit():
    from sub0_b200 import _lib
    L = _lib.lib
    # B * H_q * 520 B > 8 MiB even with a single partial per output row: must be refused before any launch
    B, Hq, Hkv = 4096, 32, 8
    Q = torch.zeros(16, dtype=torch.uint8, device=DEV)          # never dereferenced: the size check comes first
    p = Q.data_ptr()
    rc = L.cda_b200_decode_static(p, p, p, p, p, p, p, B, Hq, Hkv, 16, 4, 64, 64, 144, 4, 4, 0.1, 0,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.CDA_ERR_WORKSPACE
    msg = _lib.last_error()
    assert "scratch" in msg and "cda_b200_decode" in msg
    torch.cuda.synchronize()


def test_static_status_word_reports_a_bad_block_id():
    """The built-in scratch keeps the status word of the last call: clear after a good call, bit 0 up after a call whose
    block table holds an id outside the cache (block 0 is read instead; nothing faults)."""
    import ctypes as C
    from sub0_b200 import _lib
    L = _lib.lib
    case = Cs.paged_case([300, 40], H_kv=2, group=4, seed=903)
    word = C.c_int(-1)
    both_entry_points(case, 0)
    assert L.cda_b200_decode_static_status(C.byref(word)) == 0 and word.value == 0
    bad = dict(case)
    bad["block_table"] = case["block_table"].clone()
    bad["block_table"][0, 1] = 1 << 20
    both_entry_points(bad, 0)
    assert L.cda_b200_decode_static_status(C.byref(word)) == 0 and word.value & 1
    assert L.cda_b200_decode_static_status(None) == _lib.CDA_ERR_BAD_ARG
