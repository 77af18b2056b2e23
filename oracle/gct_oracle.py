"""CPU oracle for the GCT streaming attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy (float64 unless noted), the algorithm of the
reference's streaming attention path so that the CUDA kernels can be checked
against it.  It is imported by the tests, by the smoke check and by the CPU
baseline leg of the benchmark, never by the product path.

Parity status: PINNED.  Every function here is compared against outputs of the
reference implementation itself (fixtures under tests/golden/, produced by
tests/golden/make_goldens.py from the reference's own Python code on CPU):
page tables / eviction traces bit-exactly, floating-point results to fp32
round-off.

Reference locations restated here (paths are relative to the reference repo):
  * paged two-stream KV cache bookkeeping    lingbot_map/layers/flashinfer_cache.py:75-560
  * dense softmax attention                  lingbot_map/layers/attention.py:76 (F.scaled_dot_product_attention)
  * q/k LayerNorm(64)                        lingbot_map/layers/attention.py:58-59,415
  * 2-D RoPE                                 lingbot_map/layers/rope.py:88-198
  * 3-D RoPE table and rotation              lingbot_map/layers/rope.py:293-461
  * prepare_qkv (qkv split, norm, rope, NHD) lingbot_map/layers/attention.py:402-426
  * frame-block positions                    lingbot_map/aggregator/base.py:416-442
"""
from __future__ import annotations

import collections
import math
from typing import List, Optional, Tuple

import numpy as np


# --------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16): round-to-nearest-even on the top 16 bits
# --------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float values to the nearest bfloat16 (ties to even); returns float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    r = ((u + bias) & np.uint32(0xFFFF0000)).astype(np.uint32)
    return r.view(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) of the rounded values."""
    return (bf16_round(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


# --------------------------------------------------------------------------
# Softmax attention (attention.py:76, flashinfer_cache.py:382): non-causal, no mask,
# scale 1/sqrt(D).
# --------------------------------------------------------------------------
def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray,
              scale: Optional[float] = None) -> Tuple[np.ndarray, np.ndarray]:
    """q [nq,H,D], k/v [nkv,H,D] -> (out [nq,H,D], lse [nq,H]) in float64.

    lse is the natural-log-sum-exp of the scaled logits of each (query, head).
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    nq, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = np.empty((nq, H, D), dtype=np.float64)
    lse = np.empty((nq, H), dtype=np.float64)
    for h in range(H):
        s = (q[:, h, :] @ k[:, h, :].T) * scale            # [nq, nkv]
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(axis=1, keepdims=True)
        out[:, h, :] = (p @ v[:, h, :]) / l
        lse[:, h] = (m + np.log(l))[:, 0]
    return out, lse


def merge_partials(outs: List[np.ndarray], lses: List[np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
    """Combine per-split attention results.  outs[i] [nq,H,D] is the softmax-normalised
    output over split i, lses[i] [nq,H] its log-sum-exp.  Returns the result over the
    union of the splits:  O = sum_i e^{lse_i-m} O_i / sum_i e^{lse_i-m}."""
    L = np.stack([np.asarray(x, dtype=np.float64) for x in lses], axis=0)   # [G,nq,H]
    O = np.stack([np.asarray(x, dtype=np.float64) for x in outs], axis=0)   # [G,nq,H,D]
    m = L.max(axis=0)
    w = np.exp(L - m[None])
    den = w.sum(axis=0)
    out = (w[..., None] * O).sum(axis=0) / den[..., None]
    return out, m + np.log(den)


# --------------------------------------------------------------------------
# q/k LayerNorm over head_dim (attention.py:58-59): eps 1e-5, affine
# --------------------------------------------------------------------------
def layernorm_lastdim(x: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(w, np.float64) + np.asarray(b, np.float64)


# --------------------------------------------------------------------------
# 2-D RoPE (rope.py:88-198).  head_dim 64 = [0,32) vertical (y) | [32,64) horizontal (x);
# inside a half, 16 frequencies base^(-2j/32) duplicated to 32, rotate-half pairing (j, j+16).
# The reference builds the cos/sin table in the token dtype with the ANGLE cast to that
# dtype before cos/sin (rope.py:116-119); `table_dtype` reproduces that rounding.
# --------------------------------------------------------------------------
def positions_2d(pph: int, ppw: int, num_special: int) -> np.ndarray:
    """base.py:416-442: specials at (0,0); patch (row,col) at (row+1, col+1).  [P,2] int64."""
    yy, xx = np.meshgrid(np.arange(pph), np.arange(ppw), indexing="ij")
    pos = np.stack([yy.reshape(-1), xx.reshape(-1)], axis=1).astype(np.int64)
    if num_special > 0:
        pos = np.concatenate([np.zeros((num_special, 2), np.int64), pos + 1], axis=0)
    return pos


def rope2d_tables(half_dim: int, n_pos: int, base: float = 100.0,
                  table_dtype: str = "float32") -> Tuple[np.ndarray, np.ndarray]:
    """cos/sin [n_pos, half_dim] as the reference caches them (rope.py:105-120)."""
    exps = np.arange(0, half_dim, 2, dtype=np.float32) / np.float32(half_dim)
    inv = (np.float32(1.0) / (np.float32(base) ** exps)).astype(np.float32)
    ang = np.outer(np.arange(n_pos, dtype=np.float32), inv).astype(np.float32)
    if table_dtype == "bfloat16":
        ang = bf16_round(ang)
    ang = np.concatenate([ang, ang], axis=1)
    c = np.cos(ang).astype(np.float32)
    s = np.sin(ang).astype(np.float32)
    if table_dtype == "bfloat16":
        c, s = bf16_round(c), bf16_round(s)
    return c, s


def rope2d(x: np.ndarray, pos: np.ndarray, base: float = 100.0,
           table_dtype: str = "float32") -> np.ndarray:
    """x [N,H,D] (token-major), pos [N,2] -> rotated x (float64)."""
    x = np.asarray(x, dtype=np.float64)
    N, H, D = x.shape
    half = D // 2
    c, s = rope2d_tables(half, N, base, table_dtype)       # table length = token count (rope.py:187)
    out = np.empty_like(x)
    for axis in (0, 1):
        seg = x[:, :, axis * half:(axis + 1) * half]
        cc = c[pos[:, axis]][:, None, :].astype(np.float64)
        ss = s[pos[:, axis]][:, None, :].astype(np.float64)
        q = half // 2
        rot = np.concatenate([-seg[..., q:], seg[..., :q]], axis=-1)
        out[:, :, axis * half:(axis + 1) * half] = seg * cc + rot * ss
    return out


# --------------------------------------------------------------------------
# 3-D RoPE (rope.py:293-461).  32 complex frequencies per token: m in [0,10) time axis,
# [10,21) height, [21,32) width; theta 10000; table computed in float64.
# Special token i of frame f sits at (f, i, i); patch (r, c) at (f, ns+r, ns+c).
# Rotation acts on interleaved pairs (2m, 2m+1).
# --------------------------------------------------------------------------
FHW_DIM = (20, 22, 22)


def rope3d_angles(f: int, pph: int, ppw: int, num_special: int,
                  fhw_dim=FHW_DIM, theta: float = 10000.0) -> np.ndarray:
    """Angles [P, D/2] float64 for one frame with time index f."""
    def freqs(dim):
        return 1.0 / (theta ** (np.arange(0, dim, 2, dtype=np.float64)[: dim // 2] / dim))
    ft, fh, fw = (freqs(d) for d in fhw_dim)
    rows = []
    for i in range(num_special):
        rows.append(np.concatenate([f * ft, i * fh, i * fw]))
    for r in range(pph):
        for c in range(ppw):
            rows.append(np.concatenate([f * ft, (num_special + r) * fh, (num_special + c) * fw]))
    return np.stack(rows, axis=0)


def apply_rope3d(x: np.ndarray, ang: np.ndarray, cs_dtype: str = "float32") -> np.ndarray:
    """x [N,H,D], ang [N,D/2].  cos/sin are cast to the token dtype first (rope.py:450-451)."""
    x = np.asarray(x, dtype=np.float64)
    c = np.cos(ang)
    s = np.sin(ang)
    if cs_dtype == "float32":
        c, s = c.astype(np.float32).astype(np.float64), s.astype(np.float32).astype(np.float64)
    elif cs_dtype == "bfloat16":
        c, s = bf16_round(c).astype(np.float64), bf16_round(s).astype(np.float64)
    c = c[:, None, :]
    s = s[:, None, :]
    x1 = x[..., 0::2]
    x2 = x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = x1 * c - x2 * s
    out[..., 1::2] = x1 * s + x2 * c
    return out


def prepare_qkv(qkv: np.ndarray, H: int, qw, qb, kw, kb, *, rope: str,
                f: int = 0, pph: int = 0, ppw: int = 0, num_special: int = 0,
                cs_dtype: str = "float32") -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """attention.py:402-426 for one frame.  qkv [N, 3*H*D] is the qkv Linear output; returns
    q, k, v as [N,H,D] float64: LayerNorm on q and k, RoPE ('3d', '2d' or 'none'), v untouched."""
    N = qkv.shape[0]
    D = qkv.shape[1] // (3 * H)
    t = np.asarray(qkv, dtype=np.float64).reshape(N, 3, H, D)
    q, k, v = t[:, 0], t[:, 1], t[:, 2]
    q = layernorm_lastdim(q, qw, qb)
    k = layernorm_lastdim(k, kw, kb)
    if rope == "3d":
        ang = rope3d_angles(f, pph, ppw, num_special)
        q, k = apply_rope3d(q, ang, cs_dtype), apply_rope3d(k, ang, cs_dtype)
    elif rope == "2d":
        pos = positions_2d(pph, ppw, num_special)
        q, k = rope2d(q, pos, table_dtype=cs_dtype), rope2d(k, pos, table_dtype=cs_dtype)
    return q, k, v


# --------------------------------------------------------------------------
# Two-stream paged KV cache (flashinfer_cache.py:75-560)
# --------------------------------------------------------------------------
class PagedCacheOracle:
    """Bookkeeping and storage of the reference's paged KV cache, restated.

    Page pool per block: [max_num_pages, 2, page_size, H, D]; patch page ids [0, max_patch_pages),
    special page ids [max_patch_pages, max_num_pages).  Free lists are LIFO stacks initialised to
    ascending ranges, evicted pages are pushed on top (flashinfer_cache.py:158-166,253-254,496,538).
    """

    def __init__(self, num_blocks: int, tokens_per_frame: int, num_heads: int, head_dim: int,
                 num_special_tokens: int = 6, scale_frames: int = 8, sliding_window: int = 64,
                 max_total_frames: int = 2048, store: bool = True, store_dtype=np.float32):
        self.num_blocks = num_blocks
        self.num_special_tokens = num_special_tokens
        self.patches_per_frame = tokens_per_frame - num_special_tokens
        if self.patches_per_frame <= 0:
            raise AssertionError("tokens_per_frame <= num_special_tokens")
        self.page_size = self.patches_per_frame                     # :100-106 (fa2 branch)
        self.scale_frames = scale_frames
        self.sliding_window = sliding_window
        self.num_heads, self.head_dim = num_heads, head_dim
        self.tokens_per_frame = tokens_per_frame
        self.max_patch_pages = scale_frames + sliding_window + 16   # :132
        self.max_num_pages = self.max_patch_pages + (
            math.ceil(max_total_frames * num_special_tokens / self.page_size) + 16)   # :134-138
        self.store = store
        self.kv = [np.zeros((self.max_num_pages, 2, self.page_size, num_heads, head_dim), store_dtype)
                   for _ in range(num_blocks)] if store else None
        self._defer_eviction = False
        self.reset()

    # -- state ------------------------------------------------------------
    def reset(self):                                                 # :423-432
        nb = self.num_blocks
        self.scale_pages = [collections.deque() for _ in range(nb)]
        self.window_pages = [collections.deque() for _ in range(nb)]
        self.free_patch = [list(range(self.max_patch_pages)) for _ in range(nb)]
        self.special_pages = [[] for _ in range(nb)]
        self.free_special = [list(range(self.max_patch_pages, self.max_num_pages)) for _ in range(nb)]
        self.special_token_count = [0] * nb
        self.frame_count = [0] * nb

    @property
    def num_frames(self):                                            # :557-560
        return self.frame_count[0] if self.frame_count else 0

    # -- mutation ---------------------------------------------------------
    def append_frame(self, b: int, k: Optional[np.ndarray] = None, v: Optional[np.ndarray] = None):
        """:202-227, :474-553.  k, v [tokens_per_frame, H, D], specials first."""
        n, P = self.num_special_tokens, self.page_size
        if not self.free_patch[b]:
            raise AssertionError("patch page pool exhausted")
        page = self.free_patch[b].pop()
        if self.store and k is not None:
            self.kv[b][page, 0, :self.patches_per_frame] = k[n:]
            self.kv[b][page, 1, :self.patches_per_frame] = v[n:]
        if len(self.scale_pages[b]) < self.scale_frames:
            self.scale_pages[b].append(page)
        else:
            self.window_pages[b].append(page)
        remaining, written = n, 0
        while remaining > 0:
            off = self.special_token_count[b] % P
            if off == 0:
                if not self.free_special[b]:
                    raise AssertionError("special page pool exhausted")
                self.special_pages[b].append(self.free_special[b].pop())
            tail = self.special_pages[b][-1]
            w = min(remaining, P - off)
            if self.store and k is not None:
                self.kv[b][tail, 0, off:off + w] = k[written:written + w]
                self.kv[b][tail, 1, off:off + w] = v[written:written + w]
            self.special_token_count[b] += w
            written += w
            remaining -= w
        self.frame_count[b] += 1

    def evict_frames(self, b: int, scale_frames: int = None, sliding_window: int = None, **_):
        """:229-254: no-op while eviction is deferred."""
        if self._defer_eviction:
            return
        self.execute_deferred_eviction(b, scale_frames, sliding_window)

    def execute_deferred_eviction(self, b: int, scale_frames: int = None, sliding_window: int = None, **_):
        sw = self.sliding_window if sliding_window is None else sliding_window       # :256-266
        while len(self.window_pages[b]) > sw:
            self.free_patch[b].append(self.window_pages[b].popleft())

    def rollback_last_frame(self, b: int):                           # :268-301
        if self.frame_count[b] <= 0:
            raise AssertionError("cannot rollback, frame_count is 0")
        if self.frame_count[b] > self.scale_frames:
            page = self.window_pages[b].pop()
        else:
            page = self.scale_pages[b].pop()
        self.free_patch[b].append(page)
        new_count = self.special_token_count[b] - self.num_special_tokens
        if new_count < 0:
            raise AssertionError("special_token_count underflow")
        keep = math.ceil(new_count / self.page_size) if new_count > 0 else 0
        while len(self.special_pages[b]) > keep:
            self.free_special[b].append(self.special_pages[b].pop())
        self.special_token_count[b] = new_count
        self.frame_count[b] -= 1

    # -- queries ----------------------------------------------------------
    def build_visible_page_table(self, b: int) -> List[int]:         # :438-450
        return list(self.scale_pages[b]) + list(self.window_pages[b]) + list(self.special_pages[b])

    def compute_last_page_len(self, b: int) -> int:                  # :452-470
        if not self.special_pages[b]:
            return self.patches_per_frame
        tail = self.special_token_count[b] % self.page_size
        return self.page_size if tail == 0 else tail

    def get_cache_stats(self, b: int = 0) -> dict:                   # :303-322
        return {"frame_count": int(self.frame_count[b]),
                "scale_pages": len(self.scale_pages[b]),
                "live_pages": len(self.window_pages[b]),
                "free_pages": len(self.free_patch[b]),
                "special_tokens": int(self.special_token_count[b])}

    def gather_kv(self, b: int) -> Tuple[np.ndarray, np.ndarray]:    # :324-347
        vis, last = self.build_visible_page_table(b), self.compute_last_page_len(b)
        ks, vs = [], []
        for i, pid in enumerate(vis):
            n = last if i == len(vis) - 1 else self.page_size
            ks.append(self.kv[b][pid, 0, :n])
            vs.append(self.kv[b][pid, 1, :n])
        return np.concatenate(ks, axis=0), np.concatenate(vs, axis=0)

    def compute_attention(self, b: int, q: np.ndarray) -> np.ndarray:    # :349-383
        if self.frame_count[b] == 0:
            return np.zeros_like(np.asarray(q, dtype=np.float64))
        k, v = self.gather_kv(b)
        return attention(q, k, v)[0]

    def snapshot(self, b: int = 0) -> dict:
        """Everything the parity tests compare bit-exactly."""
        return {"visible": self.build_visible_page_table(b),
                "last_page_len": self.compute_last_page_len(b),
                "stats": self.get_cache_stats(b),
                "n_scale": len(self.scale_pages[b]), "n_window": len(self.window_pages[b]),
                "free_patch": list(self.free_patch[b]), "free_special": list(self.free_special[b])}


def kv_len_visible(n_cached: int, patches: int = 999, specials: int = 6,
                   scale: int = 8, window: int = 64) -> int:
    """Visible KV tokens after n_cached keyframes: full frames for scale+window, specials for all."""
    return patches * min(n_cached, scale + window) + specials * n_cached
