"""B200-native (sm_100a) attention backend for the streaming Geometric Context Transformer.

Covers the aggregator's hot path only: the paged two-stream KV cache manager, the fused
q/k-norm + RoPE + bf16 page append, tcgen05 paged and dense attention, and the split-KV merge.
Everything computes on the GPU through the C ABI in libgct_b200.so; there is no CPU fallback.
"""
from . import _lib  # noqa: F401
from .cache import B200KVCacheManager  # noqa: F401
from . import ops  # noqa: F401
from .block import B200Attention, B200Block, B200FrameAttention  # noqa: F401
from . import select  # noqa: F401
from .camera import B200CausalAttention, DecodeCache  # noqa: F401

__all__ = ["B200KVCacheManager", "B200Attention", "B200Block", "B200FrameAttention", "B200CausalAttention",
           "DecodeCache", "ops", "select"]
