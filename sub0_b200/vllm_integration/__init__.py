"""vLLM ``cda_v2`` attention backend on the B200 kernels (see :mod:`sub0_b200.vllm_integration.cda_attn_v2`)."""
