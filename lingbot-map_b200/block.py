"""Attention layers and the global block of the streaming Geometric Context Transformer on the B200 backend.

Mirrors, with identical constructor arguments, sub-module names (checkpoints load with the reference's keys:
norm1, attn.qkv, attn.q_norm, attn.k_norm, attn.proj, ls1.gamma, norm2, mlp.fc1, mlp.fc2, ls2.gamma) and
call signatures:

  B200FrameAttention  <->  lingbot_map/layers/attention.py:36-87    Attention (frame blocks, dense SDPA)
  B200Attention       <->  lingbot_map/layers/attention.py:352-556  FlashInferAttention (global, paged cache)
  B200Block           <->  lingbot_map/layers/block.py:151-310      FlashInferBlock

The Linear layers, LayerNorm(dim), LayerScale and the MLP stay PyTorch; q/k LayerNorm(64), RoPE, the bf16 cast,
the K/V page append and all attention math run in the CUDA library.  Inference only (no dropout, no autograd).
"""
from typing import Callable, Optional

import torch
from torch import Tensor, nn

from . import _lib, ops
from .cache import B200KVCacheManager


def _reference_classes():
    """(FlashInferBlock, FlashInferAttention) of the reference package, for the one mode this backend hands back to
    it: a cache manager that is not a B200KVCacheManager (the reference's fp32 gather + SDPA comparison mode)."""
    from lingbot_map.layers.attention import FlashInferAttention
    from lingbot_map.layers.block import FlashInferBlock
    return FlashInferBlock, FlashInferAttention


class LayerScale(nn.Module):
    """x * gamma (lingbot_map/layers/layer_scale.py).  The parameter name `gamma` is fixed by the checkpoint; the
    module is the usual timm / DINOv2 one-liner, restated here so that the block imports without the reference."""

    def __init__(self, dim: int, init_values: float = 1e-5, inplace: bool = False) -> None:
        super().__init__()
        self.inplace = inplace
        self.gamma = nn.Parameter(init_values * torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        return x.mul_(self.gamma) if self.inplace else x * self.gamma


class Mlp(nn.Module):
    """fc1 -> act -> fc2 (lingbot_map/layers/mlp.py); sub-module names fixed by the checkpoint, as above."""

    def __init__(self, in_features: int, hidden_features: Optional[int] = None, out_features: Optional[int] = None,
                 act_layer: Callable[..., nn.Module] = nn.GELU, drop: float = 0.0, bias: bool = True) -> None:
        super().__init__()
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.fc1 = nn.Linear(in_features, hidden_features, bias=bias)
        self.act = act_layer()
        self.fc2 = nn.Linear(hidden_features, out_features, bias=bias)
        self.drop = nn.Dropout(drop)

    def forward(self, x: Tensor) -> Tensor:
        return self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))


def rope_table_from_pos(pos: Tensor, enable_3d_rope: bool, rope=None) -> Tensor:
    """cos/sin table [tokens, 32, 2] fp32 for the CUDA prologue from what the reference passes as `pos`.

    3-D: `pos` is the complex frequency tensor [1, 1, N, 32] of WanRotaryPosEmbed (rope.py:336-433); its real and
    imaginary parts are the cos and sin the reference multiplies with (rope.py:450-451).
    2-D: `pos` holds integer (y, x) positions [B, N, 2] (base.py:416-442); entry 16*axis + j is the angle
    pos_axis * base^(-2j/32) in fp32 as in RotaryPositionEmbedding2D (rope.py:105-119).  All frames of a batch
    share the positions of frame 0."""
    if enable_3d_rope:
        return torch.view_as_real(pos.reshape(-1, pos.shape[-1]).to(torch.complex64)).contiguous()
    base = float(getattr(rope, "base_frequency", 100.0))
    p = pos[0].to(torch.float32)                                            # [N, 2]
    inv = 1.0 / (base ** (torch.arange(0, 32, 2, device=pos.device, dtype=torch.float32) / 32))
    ang = torch.cat([p[:, 0:1] * inv[None], p[:, 1:2] * inv[None]], dim=1)  # [N, 32]: vertical 16 | horizontal 16
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()


class _AttentionBase(nn.Module):
    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = True, proj_bias: bool = True,
                 attn_drop: float = 0.0, proj_drop: float = 0.0, norm_layer: nn.Module = nn.LayerNorm,
                 qk_norm: bool = False, fused_attn: bool = True, rope=None) -> None:
        super().__init__()
        assert dim % num_heads == 0, "dim should be divisible by num_heads"
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        if self.head_dim != 64:
            raise ValueError("the B200 attention kernels are built for head_dim == 64")
        self.scale = self.head_dim ** -0.5
        self.fused_attn = fused_attn
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.q_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.k_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim, bias=proj_bias)
        self.proj_drop = nn.Dropout(proj_drop)
        self.rope = rope

    def _norm_params(self):
        """fp32 copies of the q/k LayerNorm affine parameters (None when qk_norm is off)."""
        if isinstance(self.q_norm, nn.Identity):
            return None, None, None, None
        f = lambda p: p.detach().to(torch.float32).contiguous()
        return f(self.q_norm.weight), f(self.q_norm.bias), f(self.k_norm.weight), f(self.k_norm.bias)

    def _rope_args(self, pos, enable_3d_rope):
        if self.rope is None or pos is None:
            return None, _lib.ROPE_NONE
        return rope_table_from_pos(pos, enable_3d_rope, self.rope), (_lib.ROPE_3D if enable_3d_rope else _lib.ROPE_2D)

    def _qkv_rows(self, x: Tensor) -> Tensor:
        """qkv Linear -> [B*N, 3*C] in fp32 or bf16 (whatever autocast made of it)."""
        B, N, C = x.shape
        qkv = self.qkv(x).reshape(B * N, 3 * C)
        if qkv.dtype not in (torch.float32, torch.bfloat16):
            qkv = qkv.float()
        return qkv

    def _dense(self, x: Tensor, pos, enable_3d_rope: bool, tokens_per_frame: int):
        """q/k norm + RoPE + bf16 + dense attention with the batch entries as independent sequences.
        Returns (attention output [B, N, C] bf16, k [B*N, H, 64], v [B*N, H, 64])."""
        B, N, C = x.shape
        cs, mode = self._rope_args(pos, enable_3d_rope)
        q, k, v = ops.prep_qkv(self._qkv_rows(x), self.num_heads, tokens_per_frame, *self._norm_params(), cs, mode)
        H, D = self.num_heads, self.head_dim
        out = ops.dense_attention(q.view(B, N, H, D), k.view(B, N, H, D), v.view(B, N, H, D))
        return out.view(B, N, C), k, v


class B200FrameAttention(_AttentionBase):
    """Per-frame self-attention (lingbot_map/layers/attention.py:36-87): every batch entry is one frame."""

    def forward(self, x: Tensor, pos=None, num_patches=None, num_special=None, num_frames=None,
                enable_3d_rope=False) -> Tensor:
        out, _, _ = self._dense(x, pos, enable_3d_rope, tokens_per_frame=x.shape[1])
        return self.proj_drop(self.proj(out.to(x.dtype) if x.dtype != torch.bfloat16 else out))


class B200Attention(_AttentionBase):
    """Global attention over the paged KV cache (lingbot_map/layers/attention.py:352-556)."""

    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = True, proj_bias: bool = True,
                 attn_drop: float = 0.0, proj_drop: float = 0.0, norm_layer: nn.Module = nn.LayerNorm,
                 qk_norm: bool = False, fused_attn: bool = True, rope=None, kv_cache_sliding_window: int = 64,
                 kv_cache_scale_frames: int = 8, kv_cache_cross_frame_special: bool = True,
                 kv_cache_include_scale_frames: bool = True, kv_cache_camera_only: bool = False) -> None:
        super().__init__(dim=dim, num_heads=num_heads, qkv_bias=qkv_bias, proj_bias=proj_bias, attn_drop=attn_drop,
                         proj_drop=proj_drop, norm_layer=norm_layer, qk_norm=qk_norm, fused_attn=fused_attn, rope=rope)
        self.kv_cache_sliding_window = kv_cache_sliding_window
        self.kv_cache_scale_frames = kv_cache_scale_frames
        self.kv_cache_cross_frame_special = kv_cache_cross_frame_special
        self.kv_cache_include_scale_frames = kv_cache_include_scale_frames
        self.kv_cache_camera_only = kv_cache_camera_only

    def _evict(self, manager, global_idx, num_register_tokens):
        manager.evict_frames(block_idx=global_idx, scale_frames=self.kv_cache_scale_frames,
                             sliding_window=self.kv_cache_sliding_window,
                             cross_frame_special=self.kv_cache_cross_frame_special,
                             include_scale_frames=self.kv_cache_include_scale_frames,
                             camera_only=self.kv_cache_camera_only, num_register_tokens=num_register_tokens)

    def prepare_qkv(self, x: Tensor, pos=None, enable_3d_rope: bool = False) -> tuple:
        """(q, k, v), each [tokens, H, 64] bf16 - same contract as attention.py:402-426 (B = 1)."""
        if getattr(self, "_reference_manager", False):      # fp32 comparison mode: the reference's own arithmetic
            return _reference_classes()[1].prepare_qkv(self, x, pos=pos, enable_3d_rope=enable_3d_rope)
        cs, mode = self._rope_args(pos, enable_3d_rope)
        return ops.prep_qkv(self._qkv_rows(x), self.num_heads, x.shape[1], *self._norm_params(), cs, mode)

    def stream_frame(self, x: Tensor, pos, enable_3d_rope: bool, manager: B200KVCacheManager, global_idx: int,
                     num_register_tokens: int = 4) -> Tensor:
        """One streaming frame (attention.py:512-552, block.py:245-282): fused norm+RoPE+append, eviction,
        paged attention; a non-keyframe (manager._skip_append) appends temporarily and rolls back."""
        cs, mode = self._rope_args(pos, enable_3d_rope)
        qkv = self._qkv_rows(x)
        if getattr(manager, "_skip_append", False):
            prev_defer = manager._defer_eviction
            manager._defer_eviction = True
            q = manager.append_frame_fused(global_idx, qkv, *self._norm_params(), cs, mode)
            out = manager.compute_attention(global_idx, q)
            manager.rollback_last_frame(global_idx)
            manager._defer_eviction = prev_defer
        else:
            q = manager.append_frame_fused(global_idx, qkv, *self._norm_params(), cs, mode)
            self._evict(manager, global_idx, num_register_tokens)
            out = manager.compute_attention(global_idx, q)
        return out.reshape(x.shape[0], q.shape[0], self.num_heads * self.head_dim)

    def forward(self, x: Tensor, pos=None, num_patches=None, num_special=None, num_frames=None,
                enable_3d_rope=False, kv_cache=None, global_idx=0, num_frame_per_block=1, num_frame_for_scale=-1,
                num_register_tokens=4) -> Tensor:
        B, N, C = x.shape
        if kv_cache is not None and not isinstance(kv_cache, B200KVCacheManager):
            # a manager of the reference's own class (fp32 comparison mode): its attention layer's code on this module
            self._reference_manager = True
            return _reference_classes()[1].forward(
                self, x, pos=pos, num_patches=num_patches, num_special=num_special, num_frames=num_frames,
                enable_3d_rope=enable_3d_rope, kv_cache=kv_cache, global_idx=global_idx,
                num_frame_per_block=num_frame_per_block, num_frame_for_scale=num_frame_for_scale,
                num_register_tokens=num_register_tokens)
        if not isinstance(kv_cache, B200KVCacheManager):
            # batch mode (attention.py:446-465): dense attention over all N tokens of each batch entry
            out, _, _ = self._dense(x, pos, enable_3d_rope, tokens_per_frame=N)
        elif num_frames is not None and num_frames > 1:
            # phase 1 (attention.py:475-511): all scale frames attend to each other, then each frame's K/V
            # is appended to the paged cache
            if B != 1:
                raise ValueError("streaming with a paged cache expects batch size 1")
            tpf = kv_cache.tokens_per_frame
            out, k, v = self._dense(x, pos, enable_3d_rope, tokens_per_frame=N)
            for f in range(num_frames):
                kv_cache.append_frame(global_idx, k[f * tpf:(f + 1) * tpf], v[f * tpf:(f + 1) * tpf])
                self._evict(kv_cache, global_idx, num_register_tokens)
        else:
            out = self.stream_frame(x, pos, enable_3d_rope, kv_cache, global_idx, num_register_tokens)
        if out.dtype != x.dtype and not torch.is_autocast_enabled():
            out = out.to(x.dtype)
        return self.proj_drop(self.proj(out))


class B200Block(nn.Module):
    """Global block (lingbot_map/layers/block.py:151-310): x + ls1(attn(norm1 x)); x + ls2(mlp(norm2 x))."""

    def __init__(self, dim: int, num_heads: int, mlp_ratio: float = 4.0, qkv_bias: bool = True, proj_bias: bool = True,
                 ffn_bias: bool = True, drop: float = 0.0, attn_drop: float = 0.0, init_values=None,
                 drop_path: float = 0.0, act_layer: Callable[..., nn.Module] = nn.GELU,
                 norm_layer: Callable[..., nn.Module] = nn.LayerNorm, ffn_layer: Callable[..., nn.Module] = Mlp,
                 qk_norm: bool = False, rope=None, kv_cache_sliding_window: int = 64, kv_cache_scale_frames: int = 8,
                 kv_cache_cross_frame_special: bool = True, kv_cache_include_scale_frames: bool = True,
                 kv_cache_camera_only: bool = False) -> None:
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = B200Attention(dim=dim, num_heads=num_heads, qk_norm=qk_norm, qkv_bias=qkv_bias, proj_bias=proj_bias,
                                  attn_drop=attn_drop, proj_drop=drop, rope=rope,
                                  kv_cache_sliding_window=kv_cache_sliding_window,
                                  kv_cache_scale_frames=kv_cache_scale_frames,
                                  kv_cache_cross_frame_special=kv_cache_cross_frame_special,
                                  kv_cache_include_scale_frames=kv_cache_include_scale_frames,
                                  kv_cache_camera_only=kv_cache_camera_only)
        self.ls1 = LayerScale(dim, init_values=init_values) if init_values else nn.Identity()
        self.drop_path1 = nn.Identity()
        self.norm2 = norm_layer(dim)
        self.mlp = ffn_layer(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop=drop,
                             bias=ffn_bias)
        self.ls2 = LayerScale(dim, init_values=init_values) if init_values else nn.Identity()
        self.drop_path2 = nn.Identity()
        self.sample_drop_ratio = drop_path

    def attn_pre(self, x: Tensor, pos=None, enable_3d_rope: bool = False) -> tuple:
        """norm1 + prepare_qkv (block.py:217-227): (q, k, v), each [tokens, H, 64].  The reference's compile_model
        rebinds this attribute to a torch.compile'd callable (gct_profile.py:51-56, demo.py:181-186); the streaming
        forward below then goes through it, so that norm1 and the qkv Linear stay inside the caller's compiled
        region (the q/k norm + RoPE kernel is traced as the custom operator gct_b200::prep_qkv).  While it is not
        rebound the forward uses the fused append, which writes K/V straight into their pages."""
        return self.attn.prepare_qkv(self.norm1(x), pos=pos, enable_3d_rope=enable_3d_rope)

    def _stream_through_attn_pre(self, x, pos, enable_3d_rope, manager, global_idx, num_register_tokens):
        """Streaming frame with the caller's (compiled) attn_pre: block.py:245-282 on this backend's manager."""
        q, k, v = self.attn_pre(x, pos=pos, enable_3d_rope=enable_3d_rope)
        if getattr(manager, "_skip_append", False):
            prev_defer = manager._defer_eviction
            manager._defer_eviction = True
            manager.append_frame(global_idx, k, v)
            out = manager.compute_attention(global_idx, q)
            manager.rollback_last_frame(global_idx)
            manager._defer_eviction = prev_defer
        else:
            manager.append_frame(global_idx, k, v)
            self.attn._evict(manager, global_idx, num_register_tokens)
            out = manager.compute_attention(global_idx, q)
        return out.reshape(x.shape[0], q.shape[0], self.attn.num_heads * self.attn.head_dim)

    def forward(self, x: Tensor, pos=None, num_patches=None, num_special=None, num_frames=None, enable_3d_rope=False,
                kv_cache=None, global_idx=0, num_frame_per_block=1, num_frame_for_scale=-1,
                num_register_tokens=4) -> Tensor:
        if kv_cache is not None and not isinstance(kv_cache, B200KVCacheManager):
            # the reference's own manager (force_fp32, its fp32 gather + SDPA comparison mode): run the reference's
            # block code on this module's parameters; nothing of this backend computes in that mode
            self.attn._reference_manager = True
            return _reference_classes()[0].forward(
                self, x, pos=pos, num_patches=num_patches, num_special=num_special, num_frames=num_frames,
                enable_3d_rope=enable_3d_rope, kv_cache=kv_cache, global_idx=global_idx,
                num_frame_per_block=num_frame_per_block, num_frame_for_scale=num_frame_for_scale,
                num_register_tokens=num_register_tokens)
        is_streaming = kv_cache is not None and (num_frames is None or num_frames <= 1)
        if is_streaming:
            if "attn_pre" in self.__dict__:      # rebound by the caller (compile_model): keep its compiled region
                attn_x = self._stream_through_attn_pre(x, pos, enable_3d_rope, kv_cache, global_idx,
                                                       num_register_tokens)
            else:
                attn_x = self.attn.stream_frame(self.norm1(x), pos, enable_3d_rope, kv_cache, global_idx,
                                                num_register_tokens)
            if attn_x.dtype != x.dtype and not torch.is_autocast_enabled():
                attn_x = attn_x.to(x.dtype)
            x = x + self.ls1(self.attn.proj(attn_x))
        else:
            x = x + self.ls1(self.attn(self.norm1(x), pos=pos, num_patches=num_patches, num_special=num_special,
                                       num_frames=num_frames, enable_3d_rope=enable_3d_rope, kv_cache=kv_cache,
                                       global_idx=global_idx, num_frame_per_block=num_frame_per_block,
                                       num_frame_for_scale=num_frame_for_scale,
                                       num_register_tokens=num_register_tokens))
        return self.ffn_residual(x)

    def ffn_residual(self, x: Tensor) -> Tensor:
        return x + self.ls2(self.mlp(self.norm2(x)))
