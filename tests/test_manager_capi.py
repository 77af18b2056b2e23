"""Host-side logic of the C-ABI library, no GPU needed: exported symbols, and the cache manager's
bookkeeping bit-exact against traces recorded from the reference's FlashInferKVCacheManager."""
import ctypes
import gzip
import json
import os
import re

import pytest

import lingbot_map_b200 as P
from lingbot_map_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
G = os.path.join(ROOT, "tests", "golden")

with gzip.open(os.path.join(G, "manager_traces.json.gz"), "rt") as f:
    TRACES = json.load(f)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "gct_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(gct_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 25
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/gct_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes prototypes out of sync with the header"
    assert _lib.load().gct_version() == 1


def _mgr(geo, nb=1):
    return P.B200KVCacheManager(nb, geo["scale_frames"] + geo["sliding_window"] + 16, geo["tokens_per_frame"], 1, 64,
                                scale_frames=geo["scale_frames"], sliding_window=geo["sliding_window"],
                                max_total_frames=geo["max_total_frames"], bookkeeping_only=True)


def _snapshot(m, b=0):
    return {"visible": m.build_visible_page_table(b), "last_page_len": m.compute_last_page_len(b),
            "stats": m.get_cache_stats(b), "n_scale": len(m.scale_patch_pages[b]),
            "n_window": len(m.live_window_patch_pages[b]),
            "free_patch": m.free_patch_pages[b], "free_special": m.free_special_pages[b]}


@pytest.mark.parametrize("case", TRACES, ids=[c["name"] for c in TRACES])
def test_manager_trace_bit_exact(case):
    geo = case["geometry"]
    m = _mgr(geo)
    assert (m.page_size, m.max_patch_pages, m.max_num_pages) == (
        geo["page_size"], geo["max_patch_pages"], geo["max_num_pages"])
    snaps = {s["op_index"]: s for s in case["snapshots"]}
    for i, op in enumerate(case["ops"]):
        if op == "append":
            m.append_frame_bookkeeping(0)
        elif op == "evict":
            m.evict_frames(0, geo["scale_frames"], geo["sliding_window"])
        elif op == "defer_on":
            m._defer_eviction = True
        elif op == "defer_off":
            m._defer_eviction = False
        elif op == "exec_deferred":
            m.execute_deferred_eviction(0, geo["scale_frames"], geo["sliding_window"])
        elif op == "rollback":
            m.rollback_last_frame(0)
        elif op == "reset":
            m.reset()
        if i in snaps:
            want = {k: v for k, v in snaps[i].items() if k != "op_index"}
            assert _snapshot(m) == want, f"{case['name']} op {i} ({op})"


def test_sanity_check_known_answers():
    """flashinfer_cache.py:616-631: 2 blocks x 100 frames at 262 tokens."""
    m = P.B200KVCacheManager(2, 88, 262, 16, 64, scale_frames=8, sliding_window=64, max_total_frames=200,
                             bookkeeping_only=True)
    for b in range(2):
        for _ in range(100):
            m.append_frame_bookkeeping(b)
            m.evict_frames(b, scale_frames=8, sliding_window=64)
        assert len(m.scale_patch_pages[b]) == 8 and len(m.live_window_patch_pages[b]) == 64
        assert len(m.all_special_pages[b]) == 3 and m.special_token_count[b] == 600
        assert m.compute_last_page_len(b) == 600 % 256
        vis = m.build_visible_page_table(b)
        assert len(vis) == 75
        assert all(p < m.max_patch_pages for p in vis[:72]) and all(p >= m.max_patch_pages for p in vis[72:])
    m.reset()
    assert m.frame_count[0] == 0 and m.num_frames == 0


def test_blocks_are_independent():
    m = P.B200KVCacheManager(3, 21, 26, 1, 64, scale_frames=2, sliding_window=3, max_total_frames=40,
                             bookkeeping_only=True)
    for _ in range(5):
        m.append_frame_bookkeeping(1)
        m.evict_frames(1, 2, 3)
    assert m.frame_count == [0, 5, 0]
    assert m.build_visible_page_table(0) == [] and len(m.build_visible_page_table(1)) == 7


def test_error_behaviour_matches_reference():
    # tokens_per_frame <= specials: assert in the reference (flashinfer_cache.py:113-115)
    with pytest.raises(AssertionError):
        P.B200KVCacheManager(1, 21, 6, 1, 64, bookkeeping_only=True)
    m = P.B200KVCacheManager(1, 21, 26, 1, 64, scale_frames=2, sliding_window=3, max_total_frames=4,
                             bookkeeping_only=True)
    with pytest.raises(AssertionError, match="cannot rollback"):
        m.rollback_last_frame(0)
    # patch pool: 2 + 3 + 16 = 21 pages; without eviction the 22nd append exhausts it (:489-494)
    m._defer_eviction = True
    for _ in range(21):
        m.append_frame_bookkeeping(0)
    before = _snapshot(m)
    with pytest.raises(AssertionError, match="patch page pool exhausted"):
        m.append_frame_bookkeeping(0)
    assert _snapshot(m) == before            # failed append leaves the state untouched
    # special pool: ceil(4*6/20)+16 = 18 pages of 20 tokens = 60 frames (:533-537)
    m2 = P.B200KVCacheManager(1, 21, 26, 1, 64, scale_frames=2, sliding_window=3, max_total_frames=4,
                              bookkeeping_only=True)
    with pytest.raises(AssertionError, match="special page pool exhausted"):
        for _ in range(61):
            m2.append_frame_bookkeeping(0)
            m2.evict_frames(0, 2, 3)
    assert m2.frame_count[0] == 60
    with pytest.raises(_lib.GctError):
        m2.evict_frames(5, 2, 3)             # block index out of range


def test_compute_needs_device():
    m = P.B200KVCacheManager(1, 21, 26, 1, 64, bookkeeping_only=True)
    import torch
    with pytest.raises(RuntimeError, match="no device memory"):
        m.compute_attention(0, torch.zeros(26, 1, 64))
    with pytest.raises(RuntimeError):
        P.B200KVCacheManager(1, 21, 26, 1, 64, device="cpu")
    with pytest.raises(NotImplementedError):
        P.B200KVCacheManager(1, 21, 26, 1, 64, force_fp32=True, bookkeeping_only=True)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        P.ops.dense_attention(*(torch.zeros(1, 4, 1, 64, dtype=torch.bfloat16) for _ in range(3)))


def test_launch_shape_covers_the_kv_blocks():
    """Host arithmetic of the paged attention launch: every plan covers the KV blocks exactly once with non-empty
    ranges; equal ranges at the benchmark's size, long ranges plus a short one where equal ranges would leave SMs idle
    (one rank's slice of a stream sharded over 4 or 8 GPUs)."""
    import ctypes as C
    lib = _lib.load()

    def shape(n_q, heads, blocks, sms=148, max_splits=16):
        qt, s, ln = C.c_int(), C.c_int(), C.c_int()
        _lib.check(lib.gct_attn_launch_shape(n_q, heads, blocks, sms, max_splits, C.byref(qt), C.byref(s), C.byref(ln)))
        return qt.value, s.value, ln.value

    for n_q in (1, 6, 130, 1005, 8040):
        for heads in (1, 2, 16, 48):
            for blocks in (1, 2, 7, 8, 64, 128, 136, 264, 272, 529, 673, 1057, 1100):
                for max_splits in (1, 4, 16):
                    qt, s, ln = shape(n_q, heads, blocks, max_splits=max_splits)
                    assert qt in (1, 2) and 1 <= s <= min(blocks, max_splits)
                    if ln:
                        rest = blocks - (s - 1) * ln
                        assert s >= 2 and 1 <= rest <= ln
                    else:
                        assert all((i + 1) * blocks // s > i * blocks // s for i in range(s))
    assert shape(1005, 16, 1057) == (2, 9, 0)                     # the 10,000-frame cache on one GPU
    qt, s, ln = shape(1005, 16, 136)                              # 17 of its 133 pages
    assert (qt, s) == (2, 3) and 0 < 136 - 2 * ln < ln
    qt, s, ln = shape(1005, 16, 272)                              # 34 pages
    assert (qt, s) == (2, 3) and 0 < 272 - 2 * ln < ln
    assert shape(1005, 16, 136) == shape(1005, 16, 136)           # the cached plan equals the computed one
    with pytest.raises(Exception):
        _lib.check(lib.gct_attn_launch_shape(0, 16, 8, 148, 16, C.byref(C.c_int()), C.byref(C.c_int()), C.byref(C.c_int())))
