"""One stream over several GPUs: the visible KV pages are sharded across ranks.

The reference is single-GPU (no torch.distributed anywhere); this is the sharding the path offers for one
very long stream.  Every rank runs the same trunk on the same frame, so q, k, v and the cache bookkeeping
(page tables, eviction) are identical and replicated; only the attention over the visible page list is
split.  Rank r attends over a contiguous slice of the list, producing a normalised partial output and
its log-sum-exp; the partials are merged as  O = sum_r e^{lse_r - m} O_r / sum_r e^{lse_r - m}.

Two exchanges are offered:

* PeerExchange (default when symmetric memory is available): one CUDA kernel per layer that works on
  peer-mapped buffers over NVLink.  Rows are owned in contiguous slices: every rank stores its partial of the rows
  a peer owns straight into that peer's receive buffer, each rank merges its own row slice and stores the bf16
  rows into every rank's output (gct_mgr_attention_exchange).  No NCCL call on the data path.
* all-gather (fallback): every rank's whole [O | lse] record through one NCCL all-gather per layer, merged
  locally by gct_lse_merge_strided.

No data-path collective is needed for independent streams (one per GPU).
"""
import ctypes as C
import os
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


def row_slice(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of the [n_q * H] output rows that `rank` merges and publishes in the peer exchange."""
    if world <= 0 or not (0 <= rank < world) or rows < 0:
        raise ValueError("bad slice arguments")
    return rank * rows // world, (rank + 1) * rows // world


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


def exchange_host_model(record: torch.Tensor, n_q: int, heads: int, rank: int, world: int, group=None,
                        head_dim: int = 64) -> torch.Tensor:
    """What the peer-exchange kernel does, with host collectives in place of the peer stores (CPU tensors, gloo):
    phase 1 sends to every rank the rows it owns of this rank's record (an all-to-all of row slices), each rank
    merges the `world` partials of its own slice, phase 2 publishes the merged slice to everybody (an all-gather
    of slices of unequal length).  Returns the merged [n_q, heads, head_dim] float64 tensor on every rank."""
    rows = n_q * heads
    n = rows * head_dim
    o = record[:n].reshape(rows, head_dim).double()
    lse = record[n:].reshape(rows).double()
    send = []
    for p in range(world):
        lo, hi = row_slice(rows, p, world)
        send.append(torch.cat([o[lo:hi].reshape(-1), lse[lo:hi]]).contiguous())
    lo, hi = row_slice(rows, rank, world)
    mine = hi - lo
    recv = [torch.empty(mine * (head_dim + 1), dtype=torch.float64) for _ in range(world)]
    if world == 1:
        recv[0].copy_(send[0])
    else:
        # gloo has no all_to_all: one gather per destination rank carries the same slices
        for dst in range(world):
            dist.gather(send[dst], recv if rank == dst else None, dst=dst, group=group)
    po = torch.stack([r[:mine * head_dim].reshape(mine, head_dim) for r in recv])        # [world, mine, D]
    pl = torch.stack([r[mine * head_dim:] for r in recv])                               # [world, mine]
    m = pl.max(dim=0).values
    w = torch.exp(pl - m)
    merged = (w[..., None] * po).sum(0) / w.sum(0)[..., None]
    out = torch.empty(rows, head_dim, dtype=torch.float64)
    for src in range(world):
        slo, shi = row_slice(rows, src, world)
        piece = merged.contiguous() if src == rank else torch.empty(shi - slo, head_dim, dtype=torch.float64)
        if world > 1:
            dist.broadcast(piece, src=src, group=group)
        out[slo:shi] = piece
    return out.reshape(n_q, heads, head_dim)


class PeerExchange:
    """Peer-mapped buffers of the exchange kernel for one process group: a receive buffer, one bf16 output per
    global layer and the flag words, allocated as symmetric memory so that every rank holds addresses of every
    other rank's copies.  One object per (manager, group); all ranks construct it at the same point."""

    def __init__(self, n_q: int, heads: int, num_blocks: int, device, group=None):
        # NVLink multicast objects are not used by this exchange; keep the allocator from binding any
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.n_q, self.heads, self.num_blocks, self.device = n_q, heads, num_blocks, torch.device(device)
        lib = _lib.load()
        rb, fb, sl = C.c_size_t(), C.c_size_t(), C.c_int()
        _lib.check(lib.gct_kv_exchange_sizes(n_q, heads, self.world, C.byref(rb), C.byref(fb), C.byref(sl)))
        self.slice_rows = sl.value
        name = self.group.group_name
        import warnings
        with warnings.catch_warnings():                      # older releases need the call, recent ones deprecate it
            warnings.simplefilter("ignore")
            try:
                symm.enable_symm_mem_for_group(name)
            except Exception:                                # noqa: BLE001
                pass
        self.recv = symm.empty(rb.value // 4, dtype=torch.float32, device=self.device)
        self.out = symm.empty(num_blocks * n_q * heads * 64, dtype=torch.bfloat16, device=self.device)
        self.flags = symm.empty(max(fb.value // 4, 64), dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self.recv.zero_()
        torch.cuda.synchronize(self.device)
        h_recv, h_out, h_flags = (symm.rendezvous(t, name) for t in (self.recv, self.out, self.flags))
        arr = lambda ptrs: (C.c_void_p * self.world)(*[int(p) for p in ptrs])
        self._recv_ptrs, self._flag_ptrs = arr(h_recv.buffer_ptrs), arr(h_flags.buffer_ptrs)
        stride = n_q * heads * 64 * 2
        self._out_ptrs = [arr([int(p) + b * stride for p in h_out.buffer_ptrs]) for b in range(num_blocks)]
        self._handles = (h_recv, h_out, h_flags)
        self.epoch = 0
        dist.barrier(group=self.group)                       # every rank's flags are zero before anybody signals

    def output(self, block_idx: int) -> torch.Tensor:
        n = self.n_q * self.heads * 64
        return self.out[block_idx * n:(block_idx + 1) * n].view(self.n_q, self.heads, 64)

    def attention(self, manager, block_idx: int, q: torch.Tensor, has_pages: bool) -> torch.Tensor:
        """Paged attention over this rank's planned page slice + exchange + merge; returns this layer's output
        [n_q, H, 64] bf16 (a view of the symmetric output buffer, valid until the same layer runs again)."""
        self.epoch += 1
        from .cache import _dtype_code, _stream_ptr
        with torch.cuda.device(self.device):
            manager._check(manager._lib.gct_mgr_attention_exchange(
                manager._handle, block_idx, q.data_ptr(), _dtype_code(q), q.shape[0], self.rank, self.world,
                1 if has_pages else 0, self._recv_ptrs, self._out_ptrs[block_idx], self._flag_ptrs, self.slice_rows,
                self.epoch, _stream_ptr(self.device)))
        return self.output(block_idx)


def make_exchange(manager, group=None) -> Optional[PeerExchange]:
    """A PeerExchange for `manager`, or None when symmetric memory cannot be set up here (the all-gather path is
    used then).  LINGBOT_B200_KV_EXCHANGE=allgather forces the fallback."""
    if os.environ.get("LINGBOT_B200_KV_EXCHANGE", "peer").lower() == "allgather":
        return None
    xchg, err = None, None
    try:
        xchg = PeerExchange(manager.tokens_per_frame, manager.num_heads, manager.num_blocks, manager.device, group)
    except Exception as e:                                   # noqa: BLE001
        err = e
    # every rank must take the same path: one rank without symmetric memory sends all of them to the all-gather
    ok = torch.tensor([1 if xchg is not None else 0], dtype=torch.int32, device=manager.device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        if err is not None:
            import warnings
            warnings.warn(f"peer exchange unavailable ({type(err).__name__}: {err}); using the NCCL all-gather path")
        return None
    return xchg


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
    if world > 1 and not hasattr(manager, "_peer_exchange"):
        manager._peer_exchange = make_exchange(manager, group)
    xchg = getattr(manager, "_peer_exchange", None)
    if xchg is not None and n_q == xchg.n_q and out is None:
        return xchg.attention(manager, block_idx, q, hi > lo)
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
