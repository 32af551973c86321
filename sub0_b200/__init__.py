"""sub0_b200 -- compressed-domain attention (CDA) for NVIDIA B200 (sm_100a).

Hand-written CUDA kernels behind a C ABI (``include/cda_b200.h`` -> ``libcda_b200.so``) plus a thin Python layer that
keeps the call surface of the reference project's ``cda.kernels_cuda`` package:

* ``sub0_b200.kernels_cuda.wrappers``     -- ``decode_hmma_v1``, ``paged_encode_fused_cuda``
* ``sub0_b200.kernels_cuda.fa2_cda``      -- ``paged_cache_to_dense_rotated``, ``fa2_cda_prefill_varlen_v1``, raw-KV variants
* ``sub0_b200.kernels_cuda.hmma_loader``  -- ``load_*`` getters returning objects with the reference's native function names
* ``sub0_b200.codebook``                  -- host-side Hadamard matrix and Lloyd-Max / uniform codebooks
* ``sub0_b200.sharding``                  -- KV-head and sequence sharding across GPUs (``torch.distributed``)

There is no CPU or PyTorch fallback: importing ``sub0_b200._lib`` raises if the CUDA library has not been built
(``python -m sub0_b200.build``).
"""

__version__ = "0.1.0"
HEAD_DIM = 128
