"""Drop-in structure of the host-side mirror, no GPU: parameter names equal the reference's, constructor
signatures accept what the aggregator passes, and (where the reference checkout is importable) the rebinding
makes the reference's own AggregatorStream build B200 blocks with an unchanged state_dict."""
import inspect
import json
import os
import sys

import numpy as np
import pytest
import torch

import lingbot_map_b200 as P

G = os.path.join(os.path.dirname(__file__), "golden")
# a checkout or an installed copy of the reference package: LINGBOT_MAP_REFERENCE, else baseline/_ref of this repository
REF = os.environ.get("LINGBOT_MAP_REFERENCE",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref"))


def test_block_parameter_names_match_reference():
    z = np.load(os.path.join(G, "block_stream_fp32.npz"))
    ref_names = json.loads(bytes(z["param_names_json"]).decode())
    blk = P.B200Block(dim=128, num_heads=2, init_values=0.01, qk_norm=True, rope=object(),
                      kv_cache_sliding_window=3, kv_cache_scale_frames=2)
    assert [n for n, _ in blk.named_parameters()] == ref_names
    for name in ("attn_pre", "ffn_residual"):
        assert callable(getattr(blk, name))
    assert isinstance(blk.attn.proj, torch.nn.Linear)


def test_manager_signature_accepts_aggregator_call():
    """Keyword arguments of the call at lingbot_map/aggregator/stream.py:215-229."""
    sig = inspect.signature(P.B200KVCacheManager.__init__)
    for kw in ("num_blocks", "max_num_frames", "tokens_per_frame", "num_heads", "head_dim", "dtype", "device",
               "num_special_tokens", "scale_frames", "sliding_window", "max_total_frames", "force_fp32", "fa3"):
        assert kw in sig.parameters
    fwd = inspect.signature(P.B200Block.forward)
    for kw in ("x", "pos", "num_patches", "num_special", "num_frames", "enable_3d_rope", "kv_cache", "global_idx",
               "num_frame_per_block", "num_frame_for_scale", "num_register_tokens"):
        assert kw in fwd.parameters      # stream.py:508-520


def test_head_dim_other_than_64_is_rejected():
    with pytest.raises(ValueError):
        P.B200Block(dim=96, num_heads=2)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lingbot_map")), reason="reference checkout not present")
def test_rebinding_builds_b200_blocks_in_reference_aggregator():
    sys.path.insert(0, REF)
    import lingbot_map.aggregator.stream as stream_mod
    import lingbot_map.layers.flashinfer_cache as cache_mod
    saved = (stream_mod.FlashInferBlock, cache_mod.FlashInferKVCacheManager, stream_mod.AggregatorStream.__init__)
    kw = dict(img_size=56, patch_size=14, embed_dim=1024, depth=1, num_heads=16, patch_embed="conv",
              enable_3d_rope=True, max_frame_num=32, kv_cache_sliding_window=3, kv_cache_scale_frames=2)
    try:
        torch.manual_seed(0)
        ref = stream_mod.AggregatorStream(**kw)
        P.select.install()
        torch.manual_seed(0)
        agg = stream_mod.AggregatorStream(**kw)
        assert all(isinstance(b, P.B200Block) for b in agg.global_blocks)
        assert all(isinstance(b.attn, P.B200FrameAttention) for b in agg.frame_blocks)
        assert list(agg.state_dict().keys()) == list(ref.state_dict().keys())
        agg.load_state_dict(ref.state_dict(), strict=True)
        # the name now resolves to a selector: a B200 manager, or the reference's own one for force_fp32
        sel = cache_mod.FlashInferKVCacheManager
        m = sel(num_blocks=1, max_num_frames=21, tokens_per_frame=26, num_heads=2, head_dim=64, dtype=torch.bfloat16,
                device=None, scale_frames=2, sliding_window=3, max_total_frames=40, bookkeeping_only=True)
        assert type(m) is P.B200KVCacheManager and isinstance(m, sel)
    finally:
        stream_mod.FlashInferBlock, cache_mod.FlashInferKVCacheManager, stream_mod.AggregatorStream.__init__ = saved
        stream_mod.AggregatorStream._b200_wrapped = False


def test_manager_selector_hands_fp32_mode_back_to_the_reference_class():
    """force_fp32=True is the reference's fp32 gather + SDPA comparison mode (flashinfer_cache.py:372-383): the
    selector bound by install() returns the reference's manager for it, a B200 manager otherwise, and isinstance()
    against the bound name (attention.py:441-443) accepts both."""
    class FakeReferenceManager:
        def __init__(self, *args, **kwargs):
            self.kwargs = kwargs

    sel = P.select._manager_selector(FakeReferenceManager, P.B200KVCacheManager)
    kw = dict(num_blocks=1, max_num_frames=21, tokens_per_frame=26, num_heads=2, head_dim=64, dtype=torch.float32,
              device=None, scale_frames=2, sliding_window=3, max_total_frames=40)
    ref = sel(force_fp32=True, **kw)
    assert type(ref) is FakeReferenceManager and ref.kwargs["force_fp32"] is True and isinstance(ref, sel)
    ours = sel(force_fp32=False, bookkeeping_only=True, **kw)
    assert type(ours) is P.B200KVCacheManager and isinstance(ours, sel)
    assert not isinstance(object(), sel)
    with pytest.raises(NotImplementedError):          # the B200 manager itself still has no fp32 arithmetic
        P.B200KVCacheManager(force_fp32=True, bookkeeping_only=True, **kw)


def test_block_uses_a_rebound_attn_pre():
    """compile_model rebinds blk.attn_pre on the instance (gct_profile.py:51-56); the streaming forward must then
    route through it.  Checked on CPU with a stand-in manager that records the calls."""
    blk = P.B200Block(dim=128, num_heads=2, qk_norm=True, kv_cache_sliding_window=3, kv_cache_scale_frames=2)
    calls = []

    class Manager(P.B200KVCacheManager):
        def __init__(self):
            pass

        def __del__(self):
            pass
        _skip_append = False

        def append_frame(self, b, k, v):
            calls.append(("append", b, tuple(k.shape)))

        def evict_frames(self, **kw):
            calls.append(("evict", kw["block_idx"], kw["sliding_window"]))

        def compute_attention(self, b, q):
            calls.append(("attend", b))
            return torch.zeros(q.shape, dtype=torch.float32)

    def fake_attn_pre(x, pos=None, enable_3d_rope=False):
        calls.append(("attn_pre",))
        t = torch.zeros(x.shape[1], 2, 64)
        return t, t, t

    blk.attn_pre = fake_attn_pre
    y = blk(torch.zeros(1, 10, 128), pos=None, kv_cache=Manager(), global_idx=3)
    assert y.shape == (1, 10, 128)
    assert calls == [("attn_pre",), ("append", 3, (10, 2, 64)), ("evict", 3, 3), ("attend", 3)]


def test_custom_operators_are_registered_with_fake_implementations():
    """torch.compile of the reference's frame blocks traces the kernels as opaque operators: shapes and dtypes come
    from the fake implementations, no kernel runs."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    assert hasattr(torch.ops.gct_b200, "dense_attention") and hasattr(torch.ops.gct_b200, "prep_qkv")
    with FakeTensorMode():
        q = torch.empty(2, 100, 4, 64, dtype=torch.bfloat16)
        o = torch.ops.gct_b200.dense_attention(q, q, q)
        assert o.shape == (2, 100, 4, 64) and o.dtype == torch.bfloat16
        a, b, c = torch.ops.gct_b200.prep_qkv(torch.empty(200, 768), 4, 100, None, None, None, None, None, 0)
        assert a.shape == b.shape == c.shape == (200, 4, 64) and a.dtype == torch.bfloat16


def test_cpu_tensors_are_rejected_not_computed():
    q = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        P.ops.dense_attention(q, q, q)
    from lingbot_map_b200 import render_ops
    pts = torch.zeros(8, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        render_ops.frustum_cull(pts, torch.eye(3), torch.zeros(3), 1.0, 1.0, 0.0, 0.0, 4, 4, 0.1, 10.0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        render_ops.voxelize_frame(pts, pts, 0.1)


def test_camera_attention_keeps_reference_code_for_batch_mode():
    """B200CausalAttention only takes over the streaming branch on a GPU; without a kv_cache (or on CPU tensors) the
    call goes to the reference's own CausalAttention.forward.  Checked with a stand-in for that class."""
    from lingbot_map_b200 import camera
    seen = {}

    class FakeReference:
        @staticmethod
        def forward(self, x, **kw):
            seen.update(kw)
            return x + 1

    orig = camera._reference_causal_attention
    camera._reference_causal_attention = lambda: FakeReference
    try:
        m = torch.nn.Module()
        m.__class__ = camera.B200CausalAttention
        m.head_dim = 128
        x = torch.zeros(1, 3, 8)
        assert torch.equal(m(x, kv_cache=None, global_idx=2), x + 1) and seen["global_idx"] == 2
        assert torch.equal(m(x, kv_cache={"_skip_append": False}, num_frame_per_block=3), x + 1)   # CPU tensor
    finally:
        camera._reference_causal_attention = orig


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lingbot_map")), reason="reference checkout not present")
def test_install_and_uninstall_restore_reference_names():
    sys.path.insert(0, REF)
    import lingbot_map.aggregator.stream as stream_mod
    import lingbot_map.layers.flashinfer_cache as cache_mod
    before = (stream_mod.FlashInferBlock, cache_mod.FlashInferKVCacheManager, stream_mod.AggregatorStream.__init__)
    P.select.install(patch_embed_attention=True)
    try:
        assert stream_mod.FlashInferBlock is P.B200Block
        agg = stream_mod.AggregatorStream(img_size=56, patch_size=14, embed_dim=1024, depth=1, num_heads=16,
                                          patch_embed="conv", enable_3d_rope=True, max_frame_num=32)
        assert isinstance(agg.frame_blocks[0].attn, P.B200FrameAttention)
    finally:
        P.select.uninstall()
    assert (stream_mod.FlashInferBlock, cache_mod.FlashInferKVCacheManager,
            stream_mod.AggregatorStream.__init__) == before


def test_entry_scripts_compile_and_parse_their_arguments():
    """bench.py and __graft_entry__.py byte-compile, and bench.py builds its argument parser (no GPU needed)."""
    import py_compile
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for name in ("bench.py", "bench_model.py", "__graft_entry__.py"):
        py_compile.compile(os.path.join(root, name), doraise=True)
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "--exact-softmax" in r.stdout and "--scale-frames" in r.stdout, r.stderr[-500:]


def test_clock_sampler_reports_samples_of_the_timed_region_only():
    """bench.py's clock sampler against a stand-in for nvidia-smi: rows before mark_begin() are dropped, throttle
    reasons of the kept rows are reported, and a region shorter than the sampling period still gets the nearest row."""
    import importlib.util
    import time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    fake = ("import time,sys\n"
            "rows=['1000, 1965, 300, Not Active, Not Active, Not Active, Not Active']*3+"
            "['1900, 1965, 900, Not Active, Not Active, Not Active, Active']*50\n"
            "for r in rows:\n    print(r, flush=True); time.sleep(0.05)\n")
    s = bench.ClockSampler.__new__(bench.ClockSampler)
    s.rows, s.proc, s.thread = [], None, None
    s.cmd = [sys.executable, "-c", fake]
    s.start()
    time.sleep(0.4)                      # the three 1000 MHz rows fall before the timed region
    s.mark_begin()
    time.sleep(0.5)
    got = s.stop()
    assert got["sm_mhz"] == 1900.0 and got["sm_max_mhz"] == 1965.0 and got["reasons"] == ["sw_power_cap"], got
    assert got["samples"] >= 3
