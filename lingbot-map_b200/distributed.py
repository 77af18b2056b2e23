"""One stream over several GPUs: the visible KV pages are sharded across ranks.

The reference is single-GPU (no torch.distributed anywhere); this is the sharding the path offers for one
very long stream.  Every rank runs the same trunk on the same frame, so q, k, v and the cache bookkeeping
(page tables, eviction) are identical and replicated; only the attention over the visible page list is
split.  Rank r attends over a contiguous slice of the list, producing a normalised partial output and
its log-sum-exp; one all-gather per global layer lands every rank's [O | lse] record in local memory and
a local kernel merges them:  O = sum_r e^{lse_r - m} O_r / sum_r e^{lse_r - m}.
No data-path collective is needed for independent streams (one per GPU).
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


def shard_page_range(n_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of the visible page list for `rank`.  All pages but the last hold the same
    number of tokens, so an even split of pages is an even split of work; with fewer pages than ranks the
    trailing ranks get an empty slice."""
    if world <= 0 or not (0 <= rank < world) or n_pages < 0:
        raise ValueError("bad shard arguments")
    return rank * n_pages // world, (rank + 1) * n_pages // world


def record_floats(n_q: int, heads: int, head_dim: int = 64) -> int:
    """Floats in one rank's record: n_q*H*D partial output followed by n_q*H log-sum-exps."""
    return n_q * heads * (head_dim + 1)


def pack_empty_record(buf: torch.Tensor, n_q: int, heads: int, head_dim: int = 64) -> None:
    """Record of a rank that owns no page: zero output, lse = -inf (weight 0 in the merge)."""
    n = n_q * heads * head_dim
    buf[:n].zero_()
    buf[n:].fill_(float("-inf"))


def gather_records(local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather one record per rank into [world, record] (NCCL on GPU tensors, gloo on CPU tensors)."""
    out = torch.empty(world, local.numel(), dtype=local.dtype, device=local.device)
    if world == 1:
        out[0].copy_(local)
    else:
        dist.all_gather_into_tensor(out.view(-1), local.contiguous(), group=group)
    return out


def merge_records_reference(records: torch.Tensor, n_q: int, heads: int, head_dim: int = 64) -> torch.Tensor:
    """The merge in plain PyTorch (any device) - what gct_lse_merge_strided computes; used by CPU tests."""
    n = n_q * heads * head_dim
    o = records[:, :n].reshape(-1, n_q, heads, head_dim).double()
    lse = records[:, n:].reshape(-1, n_q, heads).double()
    m = lse.max(dim=0).values
    w = torch.exp(lse - m)
    return (w[..., None] * o).sum(0) / w.sum(0)[..., None]


def sharded_attention(manager, block_idx: int, q: torch.Tensor, rank: int, world: int, group=None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """compute_attention of one global layer with the visible pages split over `world` ranks.
    Call after the frame's append/evict on every rank; returns [q_len, H, 64] bf16 on every rank."""
    n_q, H, D = q.shape
    if block_idx == 0 or getattr(manager, "_shard_plan", None) is None:
        n_pages = len(manager.build_visible_page_table(0))
        lo, hi = shard_page_range(n_pages, rank, world)
        manager._shard_plan = (lo, hi)
        if hi > lo:
            manager.plan(lo, hi)
    lo, hi = manager._shard_plan
    n = n_q * H * D
    local = torch.empty(record_floats(n_q, H, D), dtype=torch.float32, device=q.device)
    if hi > lo:
        manager.compute_attention_partial(block_idx, q, out=local[:n].view(n_q, H, D), lse=local[n:].view(n_q, H))
    else:
        pack_empty_record(local, n_q, H, D)
    rec = gather_records(local, world, group)
    if out is None:
        out = torch.empty(n_q, H, D, dtype=torch.bfloat16, device=q.device)
    stride = rec.shape[1]
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().gct_lse_merge_strided(
            rec.data_ptr(), rec.data_ptr() + 4 * n, world, n_q, H, stride, stride, out.data_ptr(), None,
            torch.cuda.current_stream(q.device).cuda_stream))
    return out
