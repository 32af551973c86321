"""The operator namespace of the comparison ops (reference: cda/kernels_vllm_fa2_fork/interface.py:9, 58-111): registered
under the reference's name with the argument counts its wrappers pass (interface.py:154-161, 234-257, 304-328, 433-460)."""
import torch


def test_namespace_and_argument_counts():
    import sub0_b200.kernels_vllm_fa2_fork._ops as ops_mod
    ops_mod.register()                                     # idempotent
    ns = getattr(torch.ops, ops_mod.NAMESPACE)
    want = {"dequantize_compressed_kv": 6, "varlen_fwd": 22, "varlen_fwd_compressed_kv": 23, "varlen_fwd_compressed_kv_fused": 26}
    for name, n_args in want.items():
        op = getattr(ns, name)
        schema = op.default._schema
        assert len(schema.arguments) == n_args, (name, len(schema.arguments))
        assert len(schema.returns) == 2
    fused = ns.varlen_fwd_compressed_kv_fused.default._schema
    assert [a.name for a in fused.arguments][7:13] == ["out", "cu_seqlens_q", "cu_seqlens_k", "seqused_k", "block_table", "alibi_slopes"]
