"""Class-path entry for vLLM's backend registry, which resolves classes by ``module.attribute`` path
(reference ``cda/vllm_integration/_backend_eager.py``): materialises the backend classes at import time."""
from .cda_attn_v2 import get_backend_classes

(CDAv2AttentionBackend, CDAv2AttentionImpl, CDAv2AttentionMetadataBuilder, CDAv2AttentionMetadata) = get_backend_classes()

__all__ = ["CDAv2AttentionBackend", "CDAv2AttentionImpl", "CDAv2AttentionMetadataBuilder", "CDAv2AttentionMetadata"]
