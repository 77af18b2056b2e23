"""Select the B200 backend next to the reference's `--backend flashinfer` / `--use_sdpa` without editing
the reference's entry scripts.

The reference builds its global blocks from the name `FlashInferBlock` bound in
lingbot_map/aggregator/stream.py:16 (used at :137) and creates the cache manager through a lazy import of
`FlashInferKVCacheManager` (stream.py:208, attention.py:441).  install() rebinds both names before a model
is constructed; the reference's FlashInfer code path then runs on this backend unchanged.  Frame blocks are
built from `Block(attn_class=Attention)` with defaults captured at definition time (base.py:86,
block.py:42), so they are converted after construction with convert_frame_attention().
"""
import os

_saved = {}


def install(frame_attention: bool = True) -> None:
    """Rebind the reference's class names to the B200 implementations.  Call before building GCTStream."""
    import lingbot_map.aggregator.stream as stream_mod
    import lingbot_map.layers.flashinfer_cache as cache_mod
    from .block import B200Block
    from .cache import B200KVCacheManager

    if not _saved:
        _saved.update(manager=cache_mod.FlashInferKVCacheManager, block=stream_mod.FlashInferBlock,
                      init=stream_mod.AggregatorStream.__init__)
    cache_mod.FlashInferKVCacheManager = B200KVCacheManager
    stream_mod.FlashInferBlock = B200Block
    if frame_attention:
        cls = stream_mod.AggregatorStream
        if not getattr(cls, "_b200_wrapped", False):
            orig_init = cls.__init__

            def wrapped_init(self, *args, **kwargs):
                orig_init(self, *args, **kwargs)
                convert_frame_attention(self)

            cls.__init__ = wrapped_init
            cls._b200_wrapped = True


def uninstall() -> None:
    """Undo install(): models built afterwards use the reference's own FlashInfer classes again."""
    if not _saved:
        return
    import lingbot_map.aggregator.stream as stream_mod
    import lingbot_map.layers.flashinfer_cache as cache_mod
    cache_mod.FlashInferKVCacheManager = _saved["manager"]
    stream_mod.FlashInferBlock = _saved["block"]
    stream_mod.AggregatorStream.__init__ = _saved["init"]
    stream_mod.AggregatorStream._b200_wrapped = False
    _saved.clear()


def convert_frame_attention(aggregator) -> int:
    """Turn the `attn` module of every frame block into a B200FrameAttention.  The module keeps its
    parameters and attributes (qkv, q_norm, k_norm, proj, rope, num_heads, head_dim); only forward changes."""
    from .block import B200FrameAttention
    n = 0
    for blk in getattr(aggregator, "frame_blocks", []):
        attn = blk.attn
        if attn.head_dim == 64 and not isinstance(attn, B200FrameAttention):
            attn.__class__ = B200FrameAttention
            n += 1
    return n


def install_from_env() -> bool:
    """install() when LINGBOT_ATTN_BACKEND=b200 is set; returns whether it did."""
    if os.environ.get("LINGBOT_ATTN_BACKEND", "").lower() == "b200":
        install()
        return True
    return False
