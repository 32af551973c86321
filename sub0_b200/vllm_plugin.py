"""vLLM general-plugin entry point (reference ``cda/vllm_plugin.py:16-29``).

vLLM runs every enabled general plugin at start-up in every worker process, which is what makes the backend visible
inside tensor-parallel workers.  Declare it in the installing project's metadata as

    [project.entry-points."vllm.general_plugins"]
    cda_v2 = "sub0_b200.vllm_plugin:register_cda_v2"

and enable it with ``VLLM_PLUGINS=cda_v2``.  ``CDA_V2_ENABLE_MEMORY_SAVING=1`` additionally shrinks vLLM's KV page to
144-byte slots before the cache is allocated.
"""
from __future__ import annotations

import os


def register_cda_v2() -> None:
    from .vllm_integration.cda_attn_v2 import enable_cda_memory_saving, register_backend

    if os.environ.get("CDA_V2_ENABLE_MEMORY_SAVING") == "1":
        enable_cda_memory_saving()
    register_backend("CUSTOM")
