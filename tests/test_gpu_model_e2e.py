"""End-to-end drop-in check on the GPU: the reference's own GCTStream model (aggregator, camera head, depth head),
built from an installed copy of the reference package with the B200 backend selected, against camera encodings and
depth recorded from the reference on CPU in fp32 (tests/golden/model_e2e_fp32.npz, made by make_goldens.py).

The reference package is looked for in baseline/_ref (python -m pip install --no-deps --target baseline/_ref
<reference checkout>); without it the test is skipped.  Weights and images are regenerated from seeds.

Tolerances (the model runs its Linear layers in fp32; q, k, v and the softmax weights are rounded to bf16 inside the
attention kernels of 48 blocks): camera encoding max-abs 5e-2 (values are O(1..5)), depth max-abs 5e-2 on values
O(1), both far below the differences between frames (O(0.5)) and between keyframe schedules (0.28).  Measured on
a B200: camera encoding 1.4e-2 to 1.7e-2, depth 4.7e-3 to 5.6e-3."""
import os
import sys

import numpy as np
import pytest
import torch

import seeded
import lingbot_map_b200 as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
G = os.path.join(os.path.dirname(__file__), "golden")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "lingbot_map")),
                                 reason="reference package not installed under baseline/_ref")]

CFG = dict(height=126, width=182, frames=8, scale_frames=2, window=3, weight_seed=7, image_seed=5, depth_stride=7)


@pytest.fixture(scope="module")
def model():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from lingbot_map.models.gct_stream import GCTStream
    P.select.install()
    try:
        m = GCTStream(img_size=518, patch_size=14, enable_3d_rope=True, max_frame_num=64,
                      kv_cache_sliding_window=CFG["window"], kv_cache_scale_frames=CFG["scale_frames"],
                      camera_num_iterations=4, use_sdpa=False).eval()
        seeded.fill_model_(m, CFG["weight_seed"])
        m = m.to("cuda:0")
        assert all(isinstance(b, P.B200Block) for b in m.aggregator.global_blocks)
        assert all(isinstance(b.attn, P.B200FrameAttention) for b in m.aggregator.frame_blocks)
        yield m
    finally:
        P.select.uninstall()


def images():
    c = CFG
    x = np.random.RandomState(c["image_seed"]).rand(c["frames"], 3, c["height"], c["width"]).astype(np.float32)
    return torch.from_numpy(x).to("cuda:0")


@pytest.mark.parametrize("tag,kf", [("paged_kf1", 1), ("paged_kf2", 2)])
def test_streaming_poses_and_depth_match_reference(model, tag, kf):
    z = np.load(os.path.join(G, "model_e2e_fp32.npz"))
    model.clean_kv_cache()
    with torch.no_grad():
        pred = model.inference_streaming(images(), num_scale_frames=CFG["scale_frames"], keyframe_interval=kf)
    mgr = model.aggregator.kv_cache_manager
    assert isinstance(mgr, P.B200KVCacheManager)
    st = CFG["depth_stride"]
    pose = pred["pose_enc"][0].float().cpu().numpy()
    depth = pred["depth"][0, :, ::st, ::st, 0].float().cpu().numpy()
    dp = float(np.abs(pose - z[f"{tag}_pose_enc"]).max())
    dd = float(np.abs(depth - z[f"{tag}_depth"]).max())
    print(f"{tag}: pose max-abs {dp:.3e}, depth max-abs {dd:.3e}")
    assert np.isfinite(pose).all() and np.isfinite(depth).all()
    assert dp <= 5e-2, f"camera encoding differs by {dp}"
    assert dd <= 5e-2, f"depth differs by {dd}"
    assert mgr.device_status() == 0


def test_patch_embed_attention_converted(model):
    """The 24 DINOv2 patch-embed attention layers (vision_transformer.py:144-171) through the dense kernel as well:
    same tolerances.  Runs last: the conversion is in place."""
    z = np.load(os.path.join(G, "model_e2e_fp32.npz"))
    n = P.select.convert_frame_attention(model.aggregator, patch_embed=True)
    assert n == len(model.aggregator.patch_embed.blocks) == 24
    model.clean_kv_cache()
    with torch.no_grad():
        pred = model.inference_streaming(images(), num_scale_frames=CFG["scale_frames"], keyframe_interval=1)
    st = CFG["depth_stride"]
    dp = float(np.abs(pred["pose_enc"][0].float().cpu().numpy() - z["paged_kf1_pose_enc"]).max())
    dd = float(np.abs(pred["depth"][0, :, ::st, ::st, 0].float().cpu().numpy() - z["paged_kf1_depth"]).max())
    print(f"patch embed converted: pose max-abs {dp:.3e}, depth max-abs {dd:.3e}")
    assert dp <= 5e-2 and dd <= 5e-2


CFG518 = dict(height=378, width=518, frames=8, num_scale_frames=2, weight_seed=7, image_seed=0, depth_stride=7)


def test_production_frame_size_378x518():
    """The reference's CPU-runnable configuration at the production frame size: 378x518 (1005 tokens per frame, pages
    of 999 tokens whose last 128-token block holds 103), default cache geometry (8 anchor frames, window 64), 8 frames
    U[0,1), 2 scale frames in phase 1 and 6 streaming frames, keyframe interval 1.  Golden: the reference's fp32 CPU
    run of the same seeded model (tests/golden/model_e2e_518_fp32.npz).  Same bound as above: 5e-2 max-abs on the
    camera encodings and on the depth samples."""
    z = np.load(os.path.join(G, "model_e2e_518_fp32.npz"))
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from lingbot_map.models.gct_stream import GCTStream
    c = CFG518
    P.select.install()
    try:
        m = GCTStream(img_size=518, patch_size=14, enable_3d_rope=True, max_frame_num=64, camera_num_iterations=4,
                      use_sdpa=False).eval()
        seeded.fill_model_(m, c["weight_seed"])
        m = m.to("cuda:0")
        x = np.random.RandomState(c["image_seed"]).rand(c["frames"], 3, c["height"], c["width"]).astype(np.float32)
        with torch.no_grad():
            pred = m.inference_streaming(torch.from_numpy(x).to("cuda:0"), num_scale_frames=c["num_scale_frames"],
                                         keyframe_interval=1)
        mgr = m.aggregator.kv_cache_manager
        assert isinstance(mgr, P.B200KVCacheManager) and mgr.tokens_per_frame == 1005 and mgr.page_size == 999
        assert mgr.build_visible_page_table(0) == list(z["visible_end"])
        st = c["depth_stride"]
        pose = pred["pose_enc"][0].float().cpu().numpy()
        depth = pred["depth"][0, :, ::st, ::st, 0].float().cpu().numpy()
        dp = float(np.abs(pose - z["pose_enc"]).max())
        dd = float(np.abs(depth - z["depth"]).max())
        print(f"378x518: pose max-abs {dp:.3e}, depth max-abs {dd:.3e}")
        assert np.isfinite(pose).all() and np.isfinite(depth).all()
        assert dp <= 5e-2, f"camera encoding differs by {dp}"
        assert dd <= 5e-2, f"depth differs by {dd}"
        assert mgr.device_status() == 0
    finally:
        P.select.uninstall()
