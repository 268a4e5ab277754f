"""B200-native NAtS attention hot path: role-masked chunked prefill, KV-cache eviction, decode over the compacted cache.

Public surface (names follow the reference project):
    nats_prefill, nats_chunk_attention, nats_attention      functional entry points
    NAtSCache, NAtSChunkLayerCache                           cache protocol
    BaseNAtSChunkAttentionLayer, LlamaNAtSChunkAttentionLayer, GPTNAtSChunkAttentionLayer
The CUDA kernels live in libnats_b200.so (C-ABI in include/nats_b200.h); build it with
``python -m neuralattentionsearch_b200.build``.
"""
from .functional import (HostPrefillPipeline, check_status, nats_attention, nats_chunk_attention, nats_prefill, prefill_attention,  # noqa: F401
                         roles_from_token_states_info)
from .cache import NAtSCache, NAtSChunkLayerCache  # noqa: F401
from .attention import (BaseNAtSChunkAttentionLayer, GPTNAtSChunkAttentionLayer,  # noqa: F401
                        LlamaNAtSChunkAttentionLayer)

__version__ = '0.1.0'
