"""The "dequantise, then dense attention" comparison path (reference: cda/kernels_vllm_fa2_fork/interface.py)."""
