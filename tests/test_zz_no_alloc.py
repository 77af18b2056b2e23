"""The allocation-free paged-attention entry point against the regular one.

gct_attn_paged_static exists for hosts that may not call cudaMalloc (all device memory already handed to
their own pool, or no tolerance for cudaMalloc's device-wide synchronisation): its scratch is a fixed
array inside the library instead of a caller-provided workspace.  This test calls it through the C ABI,
twice in a row on different cache states, and compares each result with gct_mgr_attention on the same
pages.  The second call would expose scratch contents left behind by the first.  The file name sorts
last so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import lingbot_map_b200 as P
from lingbot_map_b200 import _lib
from oracle import gct_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_attention(m, block, q):
    lib = _lib.load()
    vis = m.build_visible_page_table(block)
    pages = (C.c_int32 * len(vis))(*vis)
    out = torch.empty_like(q)
    status = C.c_int(-1)
    with torch.cuda.device(DEV):
        rc = lib.gct_attn_paged_static(m.kv_caches[block].data_ptr(), m.max_num_pages, m.page_size, m.num_heads,
                                       pages, len(vis), m.compute_last_page_len(block), q.data_ptr(), q.shape[0],
                                       out.data_ptr(), torch.cuda.current_stream(DEV).cuda_stream, C.byref(status))
    _lib.check(rc)
    assert status.value == 0
    return out


def _compare(a, b, tag):
    a64, b64 = a.double().cpu().numpy().ravel(), b.double().cpu().numpy().ravel()
    assert np.isfinite(a64).all(), tag
    cos = float(a64 @ b64 / (np.linalg.norm(a64) * np.linalg.norm(b64)))
    assert float(np.abs(a64 - b64).max()) <= 2e-2 and cos >= 0.9999, f"{tag}: max_abs={np.abs(a64 - b64).max():.3e} cos={cos:.7f}"


def test_static_scratch_matches_workspace_path_twice():
    tpf, H = 306, 2                      # page of 300 tokens, few (head, tile) items -> the KV range is split
    m = P.B200KVCacheManager(2, 48, tpf, H, 64, device=DEV, scale_frames=4, sliding_window=28, max_total_frames=200)
    g = torch.Generator(device=DEV).manual_seed(11)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=g).to(torch.bfloat16)
    for t in range(40):
        for b in range(2):
            m.append_frame(b, rn(tpf, H, 64), rn(tpf, H, 64))
            m.evict_frames(b, 4, 28)
    q1 = rn(200, H, 64)
    ref1 = m.compute_attention(0, q1)                  # plans at block 0
    got1 = _static_attention(m, 0, q1)
    _compare(got1, ref1, "first call")
    # second call: another block, another query length, one more frame in the cache
    for b in range(2):
        m.append_frame(b, rn(tpf, H, 64), rn(tpf, H, 64))
        m.evict_frames(b, 4, 28)
    q2 = rn(tpf, H, 64)
    m.plan()
    ref2 = m.compute_attention(1, q2)
    got2 = _static_attention(m, 1, q2)
    _compare(got2, ref2, "second call")
    # and the first problem once more, after the scratch held the second one's partials
    m2 = _static_attention(m, 0, q1[:130].contiguous())
    _compare(m2, m.compute_attention(0, q1[:130].contiguous()), "third call")
    assert m.device_status() == 0


def _oracle(m, block, q):
    kk, vv = m._gather_kv(block)
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    return torch.from_numpy(O.attention(f64(q), f64(kk), f64(vv))[0])


def test_static_scratch_against_the_oracle_without_allocating():
    """The entry point against the float64 oracle (not only against the workspace path, which runs the same kernels),
    in both of its shapes: a KV range split over CTAs (few heads, long KV: partials in the static array, merged),
    and many heads with a short KV (one pass, bf16 written directly).  No device memory may be allocated by a call:
    the free memory reported by the driver and torch's allocator statistics are unchanged across the second call."""
    g = torch.Generator(device=DEV).manual_seed(5)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=g).to(torch.bfloat16)
    cases = []
    for tpf, H, frames in ((306, 2, 30), (134, 16, 3)):
        m = P.B200KVCacheManager(1, 48, tpf, H, 64, device=DEV, scale_frames=4, sliding_window=28, max_total_frames=200)
        for _ in range(frames):
            m.append_frame(0, rn(tpf, H, 64), rn(tpf, H, 64))
            m.evict_frames(0, 4, 28)
        cases.append((m, rn(tpf, H, 64)))
    for i, (m, q) in enumerate(cases):
        _static_attention(m, 0, q)                     # first call on this device / of this shape
        torch.cuda.synchronize()
        lib = _lib.load()
        vis = m.build_visible_page_table(0)
        pages = (C.c_int32 * len(vis))(*vis)
        out = torch.empty_like(q)
        stats0 = (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV))
        free0, _ = torch.cuda.mem_get_info(DEV)
        status = C.c_int(-1)
        with torch.cuda.device(DEV):
            _lib.check(lib.gct_attn_paged_static(m.kv_caches[0].data_ptr(), m.max_num_pages, m.page_size, m.num_heads,
                                                 pages, len(vis), m.compute_last_page_len(0), q.data_ptr(), q.shape[0],
                                                 out.data_ptr(), torch.cuda.current_stream(DEV).cuda_stream,
                                                 C.byref(status)))
        free1, _ = torch.cuda.mem_get_info(DEV)
        assert status.value == 0
        assert (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV)) == stats0
        # the scratch of one call (page table + partials + log-sum-exps) would be megabytes
        assert free0 - free1 < 256 * 1024, f"device memory shrank by {free0 - free1} bytes across a call"
        _compare(out, _oracle(m, 0, q), f"case {i} vs oracle")


def test_static_scratch_rejects_oversize():
    lib = _lib.load()
    dummy = torch.zeros(16, dtype=torch.bfloat16, device=DEV)
    pages = (C.c_int32 * 1)(0)
    with torch.cuda.device(DEV):
        rc = lib.gct_attn_paged_static(dummy.data_ptr(), 4, 300, 16, pages, 1, 300, dummy.data_ptr(), 1025,
                                       dummy.data_ptr(), 0, None)
    assert rc == _lib.ERR_CAPACITY and b"16384" in lib.gct_last_error()
    big = (C.c_int32 * 5000)(*([0] * 5000))
    with torch.cuda.device(DEV):
        rc = lib.gct_attn_paged_static(dummy.data_ptr(), 4, 300, 2, big, 5000, 300, dummy.data_ptr(), 8,
                                       dummy.data_ptr(), 0, None)
    assert rc == _lib.ERR_CAPACITY and b"4096" in lib.gct_last_error()
