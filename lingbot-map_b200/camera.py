"""Camera-head attention on an append-only device cache.

The reference's camera head (lingbot_map/heads/camera_head.py:284-358) runs 4 refinement iterations x 4
CameraBlocks per frame on ONE token per frame; each block's CausalAttention (lingbot_map/layers/attention.py:
222-283) keeps its K and V in a dict that grows by torch.cat every frame, clones it for the attention call and
never evicts (the `shape[3] > 1` guard at attention.py:307): 16 caches whose per-frame copy cost grows linearly
with the sequence (about 1 GB moved per frame at 10,000 frames).

B200CausalAttention keeps the same parameters and call signature; in streaming mode (a kv_cache dict is passed)
it stores K/V in preallocated [capacity, H, D] fp32 buffers and calls gct_decode_attention, one kernel that appends
the new rows and computes the attention of the new tokens over all cached + new tokens in fp32.  The batch path
(kv_cache is None: training-style masked attention) stays the reference's own code.  The cache objects live inside
the head's kv_cache dicts, so CameraCausalHead.clean_kv_cache() drops them with the dicts.
"""
import ctypes as C

import torch
from torch import Tensor

from . import _lib
from .cache import _stream_ptr


class DecodeCache:
    """K and V rows of one (refinement iteration, block) pair: [capacity, H, D] fp32, `count` rows valid."""

    def __init__(self, heads: int, head_dim: int, device, capacity: int = 1024):
        self.heads, self.head_dim, self.device = heads, head_dim, torch.device(device)
        self.count = 0
        self.k = torch.zeros(capacity, heads, head_dim, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(capacity, heads, head_dim, dtype=torch.float32, device=self.device)
        need = C.c_size_t()
        _lib.check(_lib.load().gct_decode_workspace_bytes(heads, head_dim, C.byref(need)))
        self.workspace = torch.zeros(need.value, dtype=torch.uint8, device=self.device)

    @property
    def capacity(self) -> int:
        return self.k.shape[0]

    def _grow(self, rows: int) -> None:
        cap = self.capacity
        while cap < rows:
            cap *= 2
        for name in ("k", "v"):
            old = getattr(self, name)
            new = torch.zeros(cap, self.heads, self.head_dim, dtype=torch.float32, device=self.device)
            new[:self.count].copy_(old[:self.count])
            setattr(self, name, new)

    def attend(self, q: Tensor, k_new: Tensor, v_new: Tensor, store: bool) -> Tensor:
        """q, k_new, v_new [n, H, D] fp32: attention of the n new tokens over the cached rows + themselves; with
        `store` the new rows are appended."""
        n = q.shape[0]
        if store and self.count + n > self.capacity:
            self._grow(self.count + n)
        out = torch.empty_like(q)
        lib = _lib.load()
        ws, stream = self.workspace, _stream_ptr(self.device)
        with torch.cuda.device(self.device):
            if n <= 8:
                _lib.check(lib.gct_decode_attention(
                    q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), n, self.k.data_ptr(), self.v.data_ptr(),
                    self.count, self.capacity, 1 if store else 0, self.heads, self.head_dim, out.data_ptr(),
                    ws.data_ptr(), ws.numel(), stream))
            else:
                # a scale phase of more than 8 frames: the kernel takes 8 query tokens per launch.  Each chunk of
                # queries gets its own rows as "new" rows and all other rows (cached + the rest of this call) as the
                # cache; the order of the keys inside a softmax does not matter.  The append is a plain copy.
                for lo in range(0, n, 8):
                    hi = min(lo + 8, n)
                    ok = torch.cat([self.k[:self.count], k_new[:lo], k_new[hi:]])
                    ov = torch.cat([self.v[:self.count], v_new[:lo], v_new[hi:]])
                    qc, kc, vc = q[lo:hi].contiguous(), k_new[lo:hi].contiguous(), v_new[lo:hi].contiguous()
                    _lib.check(lib.gct_decode_attention(
                        qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), hi - lo, ok.data_ptr(), ov.data_ptr(), ok.shape[0],
                        ok.shape[0], 0, self.heads, self.head_dim, out[lo:hi].data_ptr(), ws.data_ptr(), ws.numel(), stream))
                if store:
                    self.k[self.count:self.count + n].copy_(k_new)
                    self.v[self.count:self.count + n].copy_(v_new)
        if store:
            self.count += n
        return out


def _reference_causal_attention():
    from lingbot_map.layers.attention import CausalAttention
    return CausalAttention


class B200CausalAttention(torch.nn.Module):
    """forward() replacement for the reference's CausalAttention (attention.py:143-291).  Instances are made by
    switching the class of an existing CausalAttention module (convert_camera_head), so parameters, attribute
    names and the constructor stay the reference's."""

    def forward(self, x: Tensor, block_mask=None, pos=None, pos_kv=None, frame_seqlen=None, video_mask=None,
                kv_cache=None, current_start=0, current_end=0, global_idx=0, num_frame_per_block=1,
                num_frame_for_scale=-1, enable_3d_rope=False, sliding_window_size=-1, attend_to_scale_frames=False,
                num_random_frames=0, attend_to_special_tokens=False, num_register_tokens=4, is_scale_frames=False,
                **kwargs) -> Tensor:
        B, N, C_ = x.shape
        tokens_per_frame = N // max(num_frame_per_block, 1)
        if (kv_cache is None or not x.is_cuda or B != 1 or tokens_per_frame != 1 or N % max(num_frame_per_block, 1)
                or self.head_dim not in (64, 128)):
            # batch mode, or a cache shape this kernel is not built for: the reference's own code
            return _reference_causal_attention().forward(
                self, x, block_mask=block_mask, pos=pos, pos_kv=pos_kv, frame_seqlen=frame_seqlen,
                video_mask=video_mask, kv_cache=kv_cache, current_start=current_start, current_end=current_end,
                global_idx=global_idx, num_frame_per_block=num_frame_per_block, num_frame_for_scale=num_frame_for_scale,
                enable_3d_rope=enable_3d_rope, sliding_window_size=sliding_window_size,
                attend_to_scale_frames=attend_to_scale_frames, num_random_frames=num_random_frames,
                attend_to_special_tokens=attend_to_special_tokens, num_register_tokens=num_register_tokens,
                is_scale_frames=is_scale_frames, **kwargs)
        from lingbot_map.layers.rope import apply_rotary_emb
        H, D = self.num_heads, self.head_dim
        qkv = self.qkv(x).reshape(B, N, 3, H, D).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)                                            # [1, H, N, D]
        gate = None
        if self.gate_proj is not None:
            gate = self.gate_proj(x).reshape(B, N, H, D)
        q, k = self.q_norm(q), self.k_norm(k)                              # attention.py:223
        if self.rope is not None and not enable_3d_rope:
            q, k = self.rope(q, pos), self.rope(k, pos)
        elif enable_3d_rope and pos is not None:
            q, k = apply_rotary_emb(q, pos), apply_rotary_emb(k, pos)
        key = f"b200_decode_{global_idx}"
        cache = kv_cache.get(key)
        if cache is None:
            cache = kv_cache[key] = DecodeCache(H, D, x.device)
        nhd = lambda t: t[0].permute(1, 0, 2).float().contiguous()          # [N, H, D] fp32
        store = not kv_cache.get("_skip_append", False)                    # attention.py:232-249
        out = cache.attend(nhd(q), nhd(k), nhd(v), store)                  # [N, H, D]
        out = out.to(x.dtype)
        if gate is not None:
            out = out * torch.sigmoid(gate[0])
        out = out.reshape(1, N, H * D)
        return self.proj_drop(self.proj(out))


def convert_camera_head(head) -> int:
    """Switch the attention modules of a CameraCausalHead's trunk (camera_head.py:221-228) to B200CausalAttention.
    Returns how many were converted."""
    n = 0
    for blk in getattr(head, "trunk", []):
        attn = getattr(blk, "attn", None)
        if attn is not None and hasattr(attn, "qkv") and hasattr(attn, "gate_proj") and not isinstance(attn, B200CausalAttention):
            attn.__class__ = B200CausalAttention
            n += 1
    return n
