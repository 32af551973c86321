"""Counterpart of the reference package ``cda.kernels_cuda`` (cda/kernels_cuda/__init__.py:1-22): the wrapper functions
live in :mod:`.wrappers` and :mod:`.fa2_cda`, the ``load_*`` getters in :mod:`.hmma_loader`."""
from .hmma_loader import (
    load_decode_hmma,
    load_fa2_cda_hadamard,
    load_fa2_cda_loader,
    load_fa2_cda_varlen_fused,
    load_kv_cache_update,
    load_paged_encode_fused,
)

__all__ = [
    "load_decode_hmma",
    "load_fa2_cda_hadamard",
    "load_fa2_cda_loader",
    "load_fa2_cda_varlen_fused",
    "load_kv_cache_update",
    "load_paged_encode_fused",
]
