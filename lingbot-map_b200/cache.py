"""B200KVCacheManager: the two-stream paged KV cache of the streaming Geometric Context Transformer.

Drop-in for the reference's ``FlashInferKVCacheManager`` (lingbot_map/layers/flashinfer_cache.py:55-560):
same constructor arguments, methods, attributes and error behaviour.  Bookkeeping lives in C++ behind the
C ABI (bit-exact page tables and eviction decisions); K/V pages are written by a fused CUDA kernel and
attention over the visible pages runs on the tcgen05 kernel.  There is no CPU compute path.
"""
import ctypes as C
import os
from typing import List, Optional

import torch
from torch import Tensor

from . import _lib


def _dtype_code(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise TypeError(f"unsupported dtype {t.dtype}: the B200 backend takes float32 or bfloat16")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class B200KVCacheManager:
    """Paged KV cache: patch pages (recyclable) + special pages (append-only).

    Args mirror FlashInferKVCacheManager.__init__ (flashinfer_cache.py:75-90).  ``dtype`` float32 is
    stored as bfloat16 like the reference does (:125-127).  ``force_fp32`` (the reference's fp32
    gather+SDPA comparison mode) and ``fa3`` (Hopper-only kernel choice) select code paths this
    backend does not have; ``force_fp32=True`` raises, ``fa3`` is ignored (page size stays exact).
    ``bookkeeping_only=True`` creates the host-side state without any device memory (used for
    dry runs and tests without a GPU); every compute method then raises.
    """

    def __init__(self, num_blocks: int, max_num_frames: int, tokens_per_frame: int, num_heads: int, head_dim: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, num_special_tokens: int = 6,
                 scale_frames: int = 8, sliding_window: int = 64, max_total_frames: int = 2048,
                 force_fp32: bool = False, fa3: bool = False, bookkeeping_only: bool = False,
                 workspace_bytes: int = 128 * 1024 * 1024):
        if force_fp32:
            raise NotImplementedError(
                "force_fp32 (fp32 gather + SDPA) is the reference's comparison mode; the B200 backend computes "
                "attention on bf16 tensor cores only")
        if head_dim != 64:
            raise ValueError("B200 backend supports head_dim == 64 (ViT-L) only")
        self._lib = _lib.load()
        self._handle = C.c_void_p()
        cfg = _lib.MgrConfig(num_blocks, tokens_per_frame, num_heads, head_dim, num_special_tokens,
                             scale_frames, sliding_window, max_total_frames)
        geo = _lib.MgrGeometry()
        rc = self._lib.gct_mgr_create(C.byref(self._handle), C.byref(cfg), C.byref(geo))
        if rc == _lib.ERR_INVALID and tokens_per_frame <= num_special_tokens:
            raise AssertionError(self._lib.gct_last_error().decode())      # flashinfer_cache.py:113-115
        _lib.check(rc)

        self.num_blocks = num_blocks
        self.num_special_tokens = num_special_tokens
        self.patches_per_frame = tokens_per_frame - num_special_tokens
        self.page_size = geo.page_size
        self.scale_frames = scale_frames
        self.sliding_window = sliding_window
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.tokens_per_frame = tokens_per_frame
        self.max_num_frames = max_num_frames
        self.force_fp32 = False
        self.dtype = torch.bfloat16
        self.device = torch.device(device) if device is not None else None
        self.max_patch_pages = geo.max_patch_pages
        self.max_num_pages = geo.max_num_pages
        self._skip_append = False
        self._bound = False
        self.kv_caches: List[Tensor] = []
        self.workspace_buffer: Optional[Tensor] = None

        if not bookkeeping_only:
            if self.device is None or self.device.type != "cuda":
                raise RuntimeError("B200KVCacheManager needs a CUDA device (there is no CPU path)")
            with torch.cuda.device(self.device):
                # pools are zero-initialised: rows past the valid length of the last special page are
                # read (and masked) by the attention kernel and must hold finite values
                self.kv_caches = [torch.zeros(self.max_num_pages, 2, self.page_size, num_heads, head_dim,
                                              dtype=torch.bfloat16, device=self.device) for _ in range(num_blocks)]
                need = C.c_size_t()
                _lib.check(self._lib.gct_mgr_workspace_bytes(self._handle, C.byref(need)))
                self.workspace_buffer = torch.zeros(max(int(workspace_bytes), need.value), dtype=torch.uint8,
                                                    device=self.device)
                pools = (C.c_void_p * num_blocks)(*[t.data_ptr() for t in self.kv_caches])
                _lib.check(self._lib.gct_mgr_bind(self._handle, pools, self.workspace_buffer.data_ptr(),
                                                  self.workspace_buffer.numel()))
            self._bound = True
            if os.environ.get("LINGBOT_B200_BOUNDED_SOFTMAX", "1") == "0":
                self.set_bounded_mode(False)

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            self._lib.gct_mgr_destroy(h)
            self._handle = None

    # ------------------------------------------------------------------ helpers
    def _check(self, rc):
        if rc in (_lib.ERR_POOL_EXHAUSTED, _lib.ERR_UNDERFLOW):
            # the reference signals these with `assert` (flashinfer_cache.py:276-293,489-494,533-537)
            raise AssertionError(self._lib.gct_last_error().decode())
        _lib.check(rc)

    def _require_device(self):
        if not self._bound:
            raise RuntimeError("this manager was created with bookkeeping_only=True: no device memory, no compute")

    def _check_frame_tensor(self, t: Tensor, name: str):
        if t.device != self.device:
            raise ValueError(f"{name} lives on {t.device}, the cache on {self.device}")
        if tuple(t.shape[1:]) != (self.num_heads, self.head_dim):
            raise ValueError(f"{name} must be [tokens, {self.num_heads}, {self.head_dim}], got {tuple(t.shape)}")
        return t if t.is_contiguous() else t.contiguous()

    # ------------------------------------------------------------------ mutation
    def append_frame(self, block_idx: int, k: Tensor, v: Tensor) -> None:
        """Append one frame's K/V ([tokens_per_frame, H, D], specials first) - flashinfer_cache.py:202-227."""
        self._require_device()
        assert k.shape[0] - self.num_special_tokens == self.patches_per_frame, (
            f"block {block_idx}: expected {self.patches_per_frame} patch tokens, "
            f"got {k.shape[0] - self.num_special_tokens} (tokens_per_frame={k.shape[0]})")
        k = self._check_frame_tensor(k, "k")
        v = self._check_frame_tensor(v, "v")
        with torch.cuda.device(self.device):      # the C ABI works on the current device
            self._check(self._lib.gct_mgr_append(self._handle, block_idx, k.data_ptr(), _dtype_code(k),
                                                 v.data_ptr(), _dtype_code(v), _stream_ptr(self.device)))

    def append_frame_bookkeeping(self, block_idx: int) -> None:
        """append_frame without device writes (dry runs; KV-sharded replicas that do not own the page).  Whoever
        fills the pages directly calls rescan_key_norms() afterwards to re-enable the bounded attention mode."""
        self._check(self._lib.gct_mgr_append_bookkeeping(self._handle, block_idx))

    def rescan_key_norms(self, block_idx: Optional[int] = None) -> None:
        """Recompute the per-head maximum key norm of a block (all blocks by default) from its pool, after pages
        were written without going through append_frame / append_frame_fused."""
        self._require_device()
        blocks = range(self.num_blocks) if block_idx is None else [block_idx]
        with torch.cuda.device(self.device):
            for b in blocks:
                self._check(self._lib.gct_mgr_scan_keys(self._handle, b, _stream_ptr(self.device)))

    @property
    def key_norm_max(self) -> Tensor:
        """[num_blocks, H] fp32 view of the per-head maxima of the key 2-norms kept in the workspace header (an upper
        bound over everything written since the last reset; meaningful only while the manager wrote the pages)."""
        self._require_device()
        n = self.num_blocks * self.num_heads
        if 256 + 4 * n > 4096:
            raise RuntimeError("bounded mode is unavailable for this geometry (num_blocks * num_heads > 960)")
        return self.workspace_buffer[256:256 + 4 * n].view(torch.float32).view(self.num_blocks, self.num_heads)

    def set_bounded_mode(self, enable: bool) -> None:
        """Bounded mode (default on) lets the paged attention use |q|*max|k| as a fixed softmax reference when that
        bound is small; off forces the kernel that tracks the running row maximum.  Same softmax either way."""
        self._check(self._lib.gct_mgr_set_bounded_mode(self._handle, 1 if enable else 0))

    def append_frame_fused(self, block_idx: int, qkv: Tensor, q_norm_w, q_norm_b, k_norm_w, k_norm_b,
                           rope_cs: Optional[Tensor], rope_mode: int, q_out: Optional[Tensor] = None) -> Tensor:
        """qkv Linear output [tokens_per_frame, 3*H*D] -> LayerNorm(q,k), RoPE, bf16; K/V go straight into
        their pages, q is returned as [tokens_per_frame, H, D] bf16 (attention.py:413-426 + append_frame)."""
        self._require_device()
        if qkv.dim() != 2 or qkv.shape[0] != self.tokens_per_frame or qkv.shape[1] != 3 * self.num_heads * self.head_dim:
            raise ValueError(f"qkv must be [{self.tokens_per_frame}, {3 * self.num_heads * self.head_dim}]")
        if qkv.stride(1) != 1:
            qkv = qkv.contiguous()
        if q_out is None:
            q_out = torch.empty(self.tokens_per_frame, self.num_heads, self.head_dim, dtype=torch.bfloat16,
                                device=self.device)
        ptr = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_append_fused(
                self._handle, block_idx, qkv.data_ptr(), _dtype_code(qkv), qkv.stride(0), ptr(q_norm_w), ptr(q_norm_b),
                ptr(k_norm_w), ptr(k_norm_b), ptr(rope_cs), rope_mode, q_out.data_ptr(), _stream_ptr(self.device)))
        return q_out

    def evict_frames(self, block_idx: int, scale_frames: int, sliding_window: int, cross_frame_special: bool = True,
                     include_scale_frames: bool = True, camera_only: bool = False, num_register_tokens: int = 4) -> None:
        """Recycle window pages beyond ``sliding_window``; no-op while deferred - flashinfer_cache.py:229-254."""
        self._check(self._lib.gct_mgr_evict(self._handle, block_idx, sliding_window))

    def execute_deferred_eviction(self, block_idx: int, scale_frames: int, sliding_window: int, **kwargs) -> None:
        self._check(self._lib.gct_mgr_exec_deferred(self._handle, block_idx, sliding_window))

    def rollback_last_frame(self, block_idx: int) -> None:
        """Undo the most recent append_frame - flashinfer_cache.py:268-301."""
        self._check(self._lib.gct_mgr_rollback(self._handle, block_idx))

    def reset(self) -> None:
        self._check(self._lib.gct_mgr_reset(self._handle))

    @property
    def _defer_eviction(self) -> bool:
        v = C.c_int()
        self._check(self._lib.gct_mgr_get_defer(self._handle, C.byref(v)))
        return bool(v.value)

    @_defer_eviction.setter
    def _defer_eviction(self, flag: bool):
        self._check(self._lib.gct_mgr_set_defer(self._handle, 1 if flag else 0))

    # ------------------------------------------------------------------ queries
    def _stats(self, block_idx: int):
        out = (C.c_int64 * 6)()
        self._check(self._lib.gct_mgr_stats(self._handle, block_idx, out))
        return list(out)

    def get_cache_stats(self, block_idx: int = 0) -> dict:
        s = self._stats(block_idx)
        return {"frame_count": s[0], "scale_pages": s[1], "live_pages": s[2], "free_pages": s[3],
                "special_tokens": s[4]}

    def build_visible_page_table(self, block_idx: int) -> List[int]:
        n, last = C.c_int(), C.c_int()
        self._check(self._lib.gct_mgr_visible_table(self._handle, block_idx, None, 0, C.byref(n), C.byref(last)))
        buf = (C.c_int32 * max(n.value, 1))()
        self._check(self._lib.gct_mgr_visible_table(self._handle, block_idx, buf, n.value, C.byref(n), C.byref(last)))
        return list(buf[:n.value])

    def compute_last_page_len(self, block_idx: int) -> int:
        n, last = C.c_int(), C.c_int()
        self._check(self._lib.gct_mgr_visible_table(self._handle, block_idx, None, 0, C.byref(n), C.byref(last)))
        return last.value

    def _free_list(self, block_idx: int, which: int) -> List[int]:
        n = C.c_int()
        self._check(self._lib.gct_mgr_free_list(self._handle, block_idx, which, None, 0, C.byref(n)))
        buf = (C.c_int32 * max(n.value, 1))()
        self._check(self._lib.gct_mgr_free_list(self._handle, block_idx, which, buf, n.value, C.byref(n)))
        return list(buf[:n.value])

    # read-only views of the reference's per-block state lists
    @property
    def frame_count(self) -> List[int]:
        return [self._stats(b)[0] for b in range(self.num_blocks)]

    @property
    def special_token_count(self) -> List[int]:
        return [self._stats(b)[4] for b in range(self.num_blocks)]

    @property
    def free_patch_pages(self) -> List[List[int]]:
        return [self._free_list(b, 0) for b in range(self.num_blocks)]

    @property
    def free_special_pages(self) -> List[List[int]]:
        return [self._free_list(b, 1) for b in range(self.num_blocks)]

    def _split_visible(self, b: int):
        vis, s = self.build_visible_page_table(b), self._stats(b)
        return vis[:s[1]], vis[s[1]:s[1] + s[2]], vis[s[1] + s[2]:]

    @property
    def scale_patch_pages(self) -> List[List[int]]:
        return [self._split_visible(b)[0] for b in range(self.num_blocks)]

    @property
    def live_window_patch_pages(self) -> List[List[int]]:
        return [self._split_visible(b)[1] for b in range(self.num_blocks)]

    @property
    def all_special_pages(self) -> List[List[int]]:
        return [self._split_visible(b)[2] for b in range(self.num_blocks)]

    @property
    def num_frames(self) -> int:
        return self._stats(0)[0]

    def _gather_kv(self, block_idx: int):
        """Visible K and V as dense [kv_len, H, D] tensors (flashinfer_cache.py:324-347); debugging aid."""
        self._require_device()
        vis, last = self.build_visible_page_table(block_idx), self.compute_last_page_len(block_idx)
        ks, vs = [], []
        for i, pid in enumerate(vis):
            n = last if i == len(vis) - 1 else self.page_size
            ks.append(self.kv_caches[block_idx][pid, 0, :n])
            vs.append(self.kv_caches[block_idx][pid, 1, :n])
        return torch.cat(ks, dim=0), torch.cat(vs, dim=0)

    # ------------------------------------------------------------------ attention
    def plan(self, page_begin: int = 0, page_end: int = -1) -> None:
        """Snapshot block 0's visible page table for the following compute_attention calls
        (the plan() half of flashinfer_cache.py:385-414).  A sub-range selects a KV shard."""
        self._require_device()
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_plan(self._handle, page_begin, page_end, _stream_ptr(self.device)))

    def compute_attention(self, block_idx: int, q: Tensor, return_lse: bool = False):
        """softmax(q k^T / sqrt(D)) v over the visible pages - flashinfer_cache.py:349-421.
        q [q_len, H, D] (float32 or bfloat16) -> out [q_len, H, D] bfloat16.  Like the reference, the page
        table is planned when block_idx == 0 and reused by the other blocks of the same frame."""
        self._require_device()
        if self._stats(block_idx)[0] == 0:
            return torch.zeros_like(q)                              # :368-370
        q = self._check_frame_tensor(q, "q")
        if block_idx == 0:
            self.plan()
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=self.device)
        lse = torch.empty(q.shape[0], self.num_heads, dtype=torch.float32, device=self.device) if return_lse else None
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_attention(self._handle, block_idx, q.data_ptr(), _dtype_code(q), q.shape[0],
                                                    out.data_ptr(), None if lse is None else lse.data_ptr(),
                                                    _stream_ptr(self.device)))
        return (out, lse) if return_lse else out

    def compute_attention_partial(self, block_idx: int, q: Tensor, out: Optional[Tensor] = None,
                                  lse: Optional[Tensor] = None):
        """Attention over the planned page range only: (out fp32 [q_len,H,D], lse fp32 [q_len,H]) for a
        later log-sum-exp merge across KV shards.  `out` / `lse` may be views of a caller's send buffer."""
        self._require_device()
        q = self._check_frame_tensor(q, "q")
        if out is None:
            out = torch.empty(q.shape, dtype=torch.float32, device=self.device)
        if lse is None:
            lse = torch.empty(q.shape[0], self.num_heads, dtype=torch.float32, device=self.device)
        if not (out.is_contiguous() and lse.is_contiguous() and out.dtype == lse.dtype == torch.float32):
            raise ValueError("out and lse must be contiguous float32 tensors")
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_attention_partial(self._handle, block_idx, q.data_ptr(), _dtype_code(q),
                                                            q.shape[0], out.data_ptr(), lse.data_ptr(),
                                                            _stream_ptr(self.device)))
        return out, lse

    def device_status(self) -> int:
        """Synchronises and returns the kernels' status word (0 = ok); raises if a kernel reported a problem."""
        self._require_device()
        st = C.c_int()
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_device_status(self._handle, _stream_ptr(self.device), C.byref(st)))
        return st.value

    def kernel_timing(self, max_launches: int) -> None:
        """Time every attention-kernel launch with a CUDA-event pair (0 = off); see kernel_time()."""
        self._require_device()
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_kernel_timing(self._handle, max_launches))

    def kernel_time(self):
        """(total milliseconds, launches) of the attention kernel since the last call; synchronises."""
        ms, n = C.c_double(), C.c_int()
        with torch.cuda.device(self.device):
            self._check(self._lib.gct_mgr_kernel_time(self._handle, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    @property
    def launch_count(self) -> int:
        n = C.c_int64()
        self._check(self._lib.gct_mgr_launch_count(self._handle, C.byref(n)))
        return n.value
