"""Stand-alone operators of the B200 backend (thin wrappers over the C ABI): dense attention for the
frame blocks and the phase-1 scale pass, the fused q/k-norm + RoPE + bf16 prologue, RoPE tables and the
log-sum-exp merge of partial attention results.  All of them need a CUDA device.

Dense attention and the prologue are also registered as torch.library custom operators
(`gct_b200::dense_attention`, `gct_b200::prep_qkv`) with shape-only fake implementations: the reference
wraps whole frame blocks and `attn_pre` in torch.compile (demo.py:177-186, gct_profile.py:47-57), and a
custom operator is traced as one opaque node instead of breaking the graph at the ctypes call."""
import ctypes as C
from typing import Optional

import torch
from torch import Tensor

from . import _lib
from .cache import _dtype_code, _stream_ptr

_workspaces = {}


def _workspace(device, nbytes: int) -> Tensor:
    """Per-device scratch (status word + split-KV partials) for calls that have no manager.

    One buffer per device, shared by every stream and thread: two dense-attention calls whose GPU work overlaps in
    time (different streams, or several host threads) race on the split-KV partials and must be serialised by the
    caller.  When the buffer has to grow, the status word a kernel may have set in the old one is carried over, so
    device_status() keeps reporting it."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        new = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        if ws is not None:
            new[:4].copy_(ws[:4])               # stream-ordered after every kernel that used the old buffer
        _workspaces[key] = ws = new
    return ws


def _require_cuda(t: Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the B200 backend has no CPU path")


def dense_attention(q: Tensor, k: Tensor, v: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """softmax(q k^T / 8) v, non-causal (the SDPA call of lingbot_map/layers/attention.py:76,490).

    q [B, Nq, H, 64], k/v [B, Nkv, H, 64] bf16 with arbitrary strides (head_dim contiguous, strides
    multiples of 8 elements) -> [B, Nq, H, 64] bf16 contiguous."""
    if out is None and torch.compiler.is_compiling():
        return torch.ops.gct_b200.dense_attention(q, k, v)      # one opaque node in the traced graph
    return _dense_attention_impl(q, k, v, out)                  # eager: straight to the C ABI


def _dense_attention_impl(q: Tensor, k: Tensor, v: Tensor, out: Optional[Tensor] = None) -> Tensor:
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _require_cuda(t, n)
        if t.dtype != torch.bfloat16 or t.dim() != 4 or t.shape[-1] != 64 or t.stride(-1) != 1:
            raise ValueError(f"{n} must be bf16 [B, N, H, 64] with contiguous head_dim")
    B, Nq, H, _ = q.shape
    Nkv = k.shape[1]
    if k.shape != v.shape or k.shape[0] != B or k.shape[2] != H:
        raise ValueError("k/v shape mismatch")
    if out is None:
        out = torch.empty(B, Nq, H, 64, dtype=torch.bfloat16, device=q.device)
    lib = _lib.load()
    rows = B * Nq * H
    ws = _workspace(q.device, 256 + 8 * rows * (64 * 4 + 4))
    st = lambda t: (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    with torch.cuda.device(q.device):
        _lib.check(lib.gct_attn_dense(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Nq, Nkv, H,
                                      st(q), st(k), st(v), ws.data_ptr(), ws.numel(), _stream_ptr(q.device)))
    return out


def prep_qkv(qkv: Tensor, heads: int, tokens_per_frame: int, q_norm_w, q_norm_b, k_norm_w, k_norm_b,
             rope_cs: Optional[Tensor], rope_mode: int):
    """qkv Linear output [tokens, 3*H*64] -> (q, k, v) bf16 [tokens, H, 64]: LayerNorm(64) on q and k,
    RoPE from the per-token cos/sin table (indexed by token % tokens_per_frame), v cast only
    (lingbot_map/layers/attention.py:67-73)."""
    if torch.compiler.is_compiling():
        return torch.ops.gct_b200.prep_qkv(qkv, heads, tokens_per_frame, q_norm_w, q_norm_b, k_norm_w, k_norm_b, rope_cs,
                                           rope_mode)
    return _prep_qkv_impl(qkv, heads, tokens_per_frame, q_norm_w, q_norm_b, k_norm_w, k_norm_b, rope_cs, rope_mode)


def _prep_qkv_impl(qkv: Tensor, heads: int, tokens_per_frame: int, q_norm_w, q_norm_b, k_norm_w, k_norm_b,
                   rope_cs: Optional[Tensor], rope_mode: int):
    _require_cuda(qkv, "qkv")
    if qkv.dim() != 2 or qkv.shape[1] != 3 * heads * 64:
        raise ValueError("qkv must be [tokens, 3*H*64]")
    if qkv.stride(1) != 1:
        qkv = qkv.contiguous()
    T = qkv.shape[0]
    q, k, v = (torch.empty(T, heads, 64, dtype=torch.bfloat16, device=qkv.device) for _ in range(3))
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().gct_prep_qkv(
            qkv.data_ptr(), _dtype_code(qkv), qkv.stride(0), T, tokens_per_frame, heads, ptr(q_norm_w), ptr(q_norm_b),
            ptr(k_norm_w), ptr(k_norm_b), ptr(rope_cs), rope_mode, q.data_ptr(), k.data_ptr(), v.data_ptr(),
            _stream_ptr(qkv.device)))
    return q, k, v


@torch.library.custom_op("gct_b200::dense_attention", mutates_args=())
def _dense_attention_op(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    return _dense_attention_impl(q, k, v, None)


@_dense_attention_op.register_fake
def _dense_attention_fake(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    return q.new_empty((q.shape[0], q.shape[1], q.shape[2], 64), dtype=torch.bfloat16)


@torch.library.custom_op("gct_b200::prep_qkv", mutates_args=())
def _prep_qkv_op(qkv: Tensor, heads: int, tokens_per_frame: int, q_norm_w: Optional[Tensor], q_norm_b: Optional[Tensor],
                 k_norm_w: Optional[Tensor], k_norm_b: Optional[Tensor], rope_cs: Optional[Tensor],
                 rope_mode: int) -> tuple[Tensor, Tensor, Tensor]:
    return _prep_qkv_impl(qkv, heads, tokens_per_frame, q_norm_w, q_norm_b, k_norm_w, k_norm_b, rope_cs, rope_mode)


@_prep_qkv_op.register_fake
def _prep_qkv_fake(qkv, heads, tokens_per_frame, q_norm_w, q_norm_b, k_norm_w, k_norm_b, rope_cs, rope_mode):
    mk = lambda: qkv.new_empty((qkv.shape[0], heads, 64), dtype=torch.bfloat16)
    return mk(), mk(), mk()


def rope3d_table(frame_index: int, pph: int, ppw: int, num_special: int, device, out: Optional[Tensor] = None) -> Tensor:
    """cos/sin [tokens, 32, 2] fp32 of the 3-D RoPE for one frame (lingbot_map/layers/rope.py:293-433)."""
    n = num_special + pph * ppw
    if out is None:
        out = torch.empty(n, 32, 2, dtype=torch.float32, device=device)
    _require_cuda(out, "out")
    with torch.cuda.device(out.device):
        _lib.check(_lib.load().gct_rope3d_table(frame_index, pph, ppw, num_special, out.data_ptr(), _stream_ptr(out.device)))
    return out


def rope2d_table(pph: int, ppw: int, num_special: int, device, base: float = 100.0) -> Tensor:
    """cos/sin [tokens, 32, 2] fp32 of the frame blocks' 2-D RoPE (lingbot_map/layers/rope.py:88-122)."""
    out = torch.empty(num_special + pph * ppw, 32, 2, dtype=torch.float32, device=device)
    _require_cuda(out, "out")
    with torch.cuda.device(out.device):
        _lib.check(_lib.load().gct_rope2d_table(pph, ppw, num_special, base, out.data_ptr(), _stream_ptr(out.device)))
    return out


def lse_merge(parts: Tensor, lse: Tensor, return_lse: bool = False):
    """parts [G, Nq, H, 64] fp32 (normalised partial outputs), lse [G, Nq, H] fp32 -> [Nq, H, 64] bf16."""
    _require_cuda(parts, "parts")
    G, Nq, H, D = parts.shape
    parts, lse = parts.contiguous(), lse.contiguous()
    out = torch.empty(Nq, H, D, dtype=torch.bfloat16, device=parts.device)
    lo = torch.empty(Nq, H, dtype=torch.float32, device=parts.device) if return_lse else None
    with torch.cuda.device(parts.device):
        _lib.check(_lib.load().gct_lse_merge(parts.data_ptr(), lse.data_ptr(), G, Nq, H, out.data_ptr(),
                                             None if lo is None else lo.data_ptr(), _stream_ptr(parts.device)))
    return (out, lo) if return_lse else out


def device_status(device) -> int:
    """Status word of the manager-less operators on `device` (0 = ok; 1 = a bounded wait timed out,
    2 = an index check failed).  Synchronises the device."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        return 0
    return int(ws[:4].view(torch.int32).item())
