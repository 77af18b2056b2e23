"""Camera-head attention on the append-only device cache against the reference.

1. gct_decode_attention (through DecodeCache) against the float64 oracle: head_dim 128 and 64, one and several new
   tokens per call, stored and non-stored calls, a cache long enough to be split over many CTAs, growth of the buffers.
2. The reference's own CameraCausalHead (from baseline/_ref) with its attention modules converted, streaming the
   seeded sequence of tests/golden/camera_head_fp32.npz (made by make_goldens.py from the reference on CPU, fp32).
   Everything is fp32, so the bound is tight: 2e-4 max-abs on pose encodings of magnitude O(1)."""
import os
import sys

import numpy as np
import pytest
import torch

import seeded
import lingbot_map_b200 as P
from oracle import gct_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
G = os.path.join(os.path.dirname(__file__), "golden")


def _oracle(q, k, v):
    """softmax(q k^T / sqrt(D)) v per head; q [n, H, D], k/v [T, H, D] float64."""
    D = q.shape[-1]
    s = np.einsum("nhd,thd->hnt", q, k) / np.sqrt(D)
    s -= s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("hnt,thd->nhd", p, v)


@pytest.mark.parametrize("H,D", [(16, 128), (2, 128), (3, 64)])
def test_decode_cache_matches_oracle(H, D):
    c = P.DecodeCache(H, D, DEV, capacity=16)
    ks, vs = [], []
    rs = np.random.RandomState(H * 1000 + D)
    t = lambda a: torch.from_numpy(a.astype(np.float32)).to(DEV)
    calls = [(8, True), (1, True), (1, False), (3, True), (1, True)] + [(1, True)] * 30 + [(8, True)] * 150 + [(1, False), (1, True)]
    worst = 0.0
    for n, store in calls:
        q, k, v = (rs.standard_normal((n, H, D)) * s for s in (1.5, 1.5, 1.0))
        got = c.attend(t(q), t(k), t(v), store).double().cpu().numpy()
        kk = np.concatenate(ks + [k]) if ks else k
        vv = np.concatenate(vs + [v]) if vs else v
        f32 = lambda a: a.astype(np.float32).astype(np.float64)
        want = _oracle(f32(q), f32(kk), f32(vv))
        worst = max(worst, float(np.abs(got - want).max()))
        if store:
            ks.append(k)
            vs.append(v)
    assert c.count == sum(n for n, s in calls if s) and c.capacity >= c.count
    assert worst <= 2e-5, f"max abs {worst:.3e}"
    # the stored rows are the inputs, bit for bit
    assert np.array_equal(c.k[:c.count].cpu().numpy(), np.concatenate(ks).astype(np.float32))


def test_more_than_eight_new_tokens_in_one_call():
    H, D = 2, 128
    c = P.DecodeCache(H, D, DEV, capacity=8)
    rs = np.random.RandomState(5)
    t = lambda a: torch.from_numpy(a.astype(np.float32)).to(DEV)
    k0, v0 = rs.standard_normal((4, H, D)), rs.standard_normal((4, H, D))
    c.attend(t(k0), t(k0), t(v0), True)
    q, k, v = rs.standard_normal((19, H, D)), rs.standard_normal((19, H, D)), rs.standard_normal((19, H, D))
    got = c.attend(t(q), t(k), t(v), True).double().cpu().numpy()
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    want = _oracle(f32(q), f32(np.concatenate([k0, k])), f32(np.concatenate([v0, v])))
    assert c.count == 23 and np.abs(got - want).max() <= 2e-5


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lingbot_map")), reason="reference package not installed under baseline/_ref")
def test_camera_head_stream_matches_reference():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from lingbot_map.heads.camera_head import CameraCausalHead
    from lingbot_map_b200.camera import convert_camera_head, DecodeCache
    z = np.load(os.path.join(G, "camera_head_fp32.npz"))
    head = CameraCausalHead(dim_in=256, num_heads=2, trunk_depth=4, num_iterations=4, enable_3d_rope=True,
                            max_frame_num=64).eval()
    seeded.fill_model_(head, 13)
    head = head.to(DEV)
    assert convert_camera_head(head) == 4
    tol = 2e-4
    with torch.no_grad():
        x = torch.from_numpy(seeded.randn(700, 1, 3, 1, 256)).to(DEV)
        y = head([x], causal_inference=True, num_frame_per_block=3, num_frame_for_scale=3)
        assert np.abs(y[-1].cpu().numpy() - z["scale"]).max() <= tol
        for i in range(7):
            skip = i in (2, 5)
            for d in head.kv_cache:
                d["_skip_append"] = skip
            x = torch.from_numpy(seeded.randn(701 + i, 1, 1, 1, 256)).to(DEV)
            y = head([x], causal_inference=True, num_frame_per_block=1, num_frame_for_scale=3)
            d = float(np.abs(y[-1].cpu().numpy() - z[f"frame{i}"]).max())
            assert d <= tol, f"frame {i} ({'non-' if skip else ''}keyframe): {d:.3e}"
    caches = [v for d in head.kv_cache for k, v in d.items() if isinstance(v, DecodeCache)]
    assert len(caches) == 16 and all(c.count == int(z["cached_frames"][0]) for c in caches)
    head.clean_kv_cache()
    assert head.kv_cache is None
