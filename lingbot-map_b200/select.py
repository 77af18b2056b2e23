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


def install(frame_attention: bool = True, patch_embed_attention: bool = None, camera_head: bool = None) -> None:
    """Rebind the reference's class names to the B200 implementations.  Call before building GCTStream.

    frame_attention: convert the aggregator's per-frame blocks.  patch_embed_attention: also convert the 24
    attention layers of the DINOv2 patch embed (vision_transformer.py:144-171; plain attention over 1004 tokens,
    no q/k norm, no RoPE); default from LINGBOT_B200_PATCH_EMBED (off unless set to 1).  camera_head: move the
    camera head's one-token-per-frame dict caches (heads/camera_head.py:284-358) onto the append-only device cache
    of camera.py; default from LINGBOT_B200_CAMERA_HEAD (on unless set to 0)."""
    if patch_embed_attention is None:
        patch_embed_attention = os.environ.get("LINGBOT_B200_PATCH_EMBED", "0") == "1"
    if camera_head is None:
        camera_head = os.environ.get("LINGBOT_B200_CAMERA_HEAD", "1") != "0"
    import lingbot_map.aggregator.stream as stream_mod
    import lingbot_map.layers.flashinfer_cache as cache_mod
    from .block import B200Block
    from .cache import B200KVCacheManager

    if not _saved:
        _saved.update(manager=cache_mod.FlashInferKVCacheManager, block=stream_mod.FlashInferBlock,
                      init=stream_mod.AggregatorStream.__init__)
    cache_mod.FlashInferKVCacheManager = _manager_selector(_saved["manager"], B200KVCacheManager)
    stream_mod.FlashInferBlock = B200Block
    if frame_attention:
        cls = stream_mod.AggregatorStream
        if not getattr(cls, "_b200_wrapped", False):
            orig_init = cls.__init__

            def wrapped_init(self, *args, **kwargs):
                orig_init(self, *args, **kwargs)
                convert_frame_attention(self, patch_embed=patch_embed_attention)

            cls.__init__ = wrapped_init
            cls._b200_wrapped = True
    if camera_head:
        import lingbot_map.heads.camera_head as head_mod
        hcls = head_mod.CameraCausalHead
        if not getattr(hcls, "_b200_wrapped", False):
            _saved.setdefault("head_init", hcls.__init__)
            head_init = hcls.__init__

            def wrapped_head_init(self, *args, **kwargs):
                head_init(self, *args, **kwargs)
                from .camera import convert_camera_head
                convert_camera_head(self)

            hcls.__init__ = wrapped_head_init
            hcls._b200_wrapped = True


def _manager_selector(reference_cls, b200_cls):
    """The class bound to the name `FlashInferKVCacheManager` while the backend is installed.  Constructing it gives
    a B200KVCacheManager, except with force_fp32=True (lingbot_map/aggregator/stream.py:227-228, set by
    gct_profile.py:293-296 for --dtype fp32): that is the reference's fp32 gather + SDPA comparison mode
    (flashinfer_cache.py:372-383), which this backend has no arithmetic for, so the reference's own manager is
    returned and B200Block runs the reference's block code on it.  isinstance() against the name accepts both."""

    class _Meta(type):
        def __instancecheck__(cls, obj):
            return isinstance(obj, (reference_cls, b200_cls))

    class FlashInferKVCacheManager(metaclass=_Meta):
        def __new__(cls, *args, **kwargs):
            if kwargs.get("force_fp32", False):
                return reference_cls(*args, **kwargs)
            return b200_cls(*args, **kwargs)

    FlashInferKVCacheManager.__doc__ = "selects B200KVCacheManager, or the reference's manager for force_fp32"
    return FlashInferKVCacheManager


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
    if "head_init" in _saved:
        import lingbot_map.heads.camera_head as head_mod
        head_mod.CameraCausalHead.__init__ = _saved["head_init"]
        head_mod.CameraCausalHead._b200_wrapped = False
    _saved.clear()


def convert_frame_attention(aggregator, patch_embed: bool = False) -> int:
    """Turn the `attn` module of every frame block (and, with patch_embed, of every block of a ViT patch embed)
    into a B200FrameAttention.  The module keeps its parameters and attributes (qkv, q_norm, k_norm, proj, rope,
    num_heads, head_dim); only forward changes."""
    from .block import B200FrameAttention
    blocks = list(getattr(aggregator, "frame_blocks", []))
    if patch_embed:
        blocks += [b for b in getattr(getattr(aggregator, "patch_embed", None), "blocks", []) if hasattr(b, "attn")]
    n = 0
    for blk in blocks:
        attn = blk.attn
        if getattr(attn, "head_dim", 0) == 64 and hasattr(attn, "qkv") and not isinstance(attn, B200FrameAttention):
            attn.__class__ = B200FrameAttention
            n += 1
    return n


def install_from_env() -> bool:
    """install() when LINGBOT_ATTN_BACKEND=b200 is set; returns whether it did."""
    if os.environ.get("LINGBOT_ATTN_BACKEND", "").lower() == "b200":
        install()
        return True
    return False
