"""Generate the golden fixtures in this folder from the reference implementation.

Run in a container where the reference checkout is importable:

    python tests/golden/make_goldens.py --reference /path/to/lingbot-map

It imports the reference's own Python code on CPU (the FlashInfer wrapper class is replaced by a
no-op stub because its constructor needs a GPU; all bookkeeping and the fp32 gather+SDPA path of the
cache manager are the reference's own), drives it with seeded inputs (tests/golden/seeded.py) and
stores only the outputs.  The tests regenerate the inputs from the same seeds.
"""
import argparse
import gzip
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import seeded  # noqa: E402


def _import_reference(path):
    sys.dont_write_bytecode = True
    sys.path.insert(0, path)
    import flashinfer

    class _Stub:
        def __init__(self, *a, **k):
            pass
    flashinfer.BatchPrefillWithPagedKVCacheWrapper = _Stub


def _snap(m, b=0):
    return {"visible": [int(x) for x in m.build_visible_page_table(b)],
            "last_page_len": int(m.compute_last_page_len(b)),
            "stats": m.get_cache_stats(b),
            "n_scale": len(m.scale_patch_pages[b]), "n_window": len(m.live_window_patch_pages[b]),
            "free_patch": [int(x) for x in m.free_patch_pages[b]],
            "free_special": [int(x) for x in m.free_special_pages[b]]}


def manager_traces():
    import torch
    from lingbot_map.layers.flashinfer_cache import FlashInferKVCacheManager

    def make(tpf, scale, window, max_total, heads=1, nb=1):
        return FlashInferKVCacheManager(
            num_blocks=nb, max_num_frames=scale + window + 16, tokens_per_frame=tpf, num_heads=heads,
            head_dim=8, dtype=torch.float32, device=torch.device("cpu"), num_special_tokens=6,
            scale_frames=scale, sliding_window=window, max_total_frames=max_total, force_fp32=True)

    cases = []

    def geometry(m, tpf, scale, window, max_total):
        return {"tokens_per_frame": tpf, "scale_frames": scale, "sliding_window": window,
                "max_total_frames": max_total, "page_size": m.page_size,
                "max_patch_pages": m.max_patch_pages, "max_num_pages": m.max_num_pages}

    def run(name, tpf, scale, window, max_total, ops, snap_at=None):
        m = make(tpf, scale, window, max_total)
        k = torch.zeros(tpf, 1, 8)
        snaps = []
        for i, op in enumerate(ops):
            if op == "append":
                m.append_frame(0, k, k)
            elif op == "evict":
                m.evict_frames(0, scale, window)
            elif op == "defer_on":
                m._defer_eviction = True
            elif op == "defer_off":
                m._defer_eviction = False
            elif op == "exec_deferred":
                m.execute_deferred_eviction(0, scale, window)
            elif op == "rollback":
                m.rollback_last_frame(0)
            elif op == "reset":
                m.reset()
            else:
                raise ValueError(op)
            if snap_at is None or i in snap_at:
                s = _snap(m)
                s["op_index"] = i
                snaps.append(s)
        cases.append({"name": name, "geometry": geometry(m, tpf, scale, window, max_total),
                      "ops": ops, "snapshots": snaps})

    # the reference's own _sanity_check geometry (flashinfer_cache.py:577-631): 100 frames
    run("sanity_262", 262, 8, 64, 200, ["append", "evict"] * 100)
    # small geometry with a non-keyframe emulation at the end (block.py:256-263)
    run("small_26", 26, 2, 3, 40,
        ["append", "evict"] * 9 + ["defer_on", "append", "evict", "rollback", "defer_off"]
        + ["append", "evict"] * 3 + ["reset"] + ["append", "evict"] * 4)
    # production geometry 378x518: 1005 tokens, page 999, 400 keyframes, sparse snapshots
    frames = [1, 8, 9, 72, 73, 74, 166, 167, 168, 333, 334, 400]
    run("full_1005", 1005, 8, 64, 1124, ["append", "evict"] * 400,
        snap_at={2 * f - 1 for f in frames})
    # keyframe interval 3 at the production geometry: non-keyframes temp-append and roll back
    ops = ["append", "evict"] * 8
    for i in range(8, 260):
        if (i - 8) % 3 == 0:
            ops += ["append", "evict"]
        else:
            ops += ["defer_on", "append", "evict", "rollback", "defer_off"]
    run("full_1005_kf3", 1005, 8, 64, 1124, ops, snap_at=set(range(len(ops) - 40, len(ops))) | set(range(0, 60)))
    # random op sequences, incl. flow-style deferred eviction (gct_stream_window.py:362-419)
    for seed in range(4):
        rs = np.random.RandomState(100 + seed)
        tpf = [26, 11, 38, 70][seed]
        scale, window = [(2, 3), (1, 2), (3, 5), (0, 4)][seed]
        ops, depth, deferred, pending = [], 0, False, False
        for _ in range(220):
            r = rs.rand()
            if deferred:
                if not pending:
                    ops += ["append", "evict"]
                    depth += 1
                    pending = True
                elif r < 0.5:
                    ops += ["rollback", "defer_off"]
                    depth -= 1
                    deferred = pending = False
                else:
                    ops += ["exec_deferred", "defer_off"]
                    deferred = pending = False
            elif r < 0.55:
                ops += ["append", "evict"]
                depth += 1
            elif r < 0.85:
                ops += ["defer_on"]
                deferred = True
            elif r < 0.97 and depth > 0 and depth <= scale:
                # rollback right after an append in the scale phase (no eviction happened yet)
                ops += ["append", "rollback"]
            elif r >= 0.97:
                ops += ["reset"]
                depth = 0
        if deferred:
            ops += ["defer_off"]
        run(f"random_{seed}", tpf, scale, window, 150, ops)
    with gzip.open(os.path.join(HERE, "manager_traces.json.gz"), "wt") as f:
        json.dump(cases, f, separators=(",", ":"))
    print("manager_traces.json.gz:", len(cases), "cases")


def paged_attention_values():
    """Reference manager, fp32 gather+SDPA path (flashinfer_cache.py:372-383), seeded K/V/Q."""
    import torch
    from lingbot_map.layers.flashinfer_cache import FlashInferKVCacheManager
    out = {}
    specs = {  # name: (tokens_per_frame, heads, scale, window, frames, max_total, value scale, frames stored)
        "p20": (26, 4, 2, 3, 9, 40, 1.0, None),
        "p150": (156, 1, 1, 2, 30, 60, 1.0, {0, 1, 5, 24, 25, 29}),
        "p300": (306, 1, 2, 2, 12, 40, 0.125, {0, 3, 11}),
    }
    meta = {}
    for name, (tpf, H, scale, window, frames, max_total, vs, keep) in specs.items():
        m = FlashInferKVCacheManager(
            num_blocks=1, max_num_frames=scale + window + 16, tokens_per_frame=tpf, num_heads=H, head_dim=64,
            dtype=torch.float32, device=torch.device("cpu"), scale_frames=scale, sliding_window=window,
            max_total_frames=max_total, force_fp32=True)
        for t in range(frames):
            k = torch.from_numpy(seeded.randn(1000 + t, tpf, H, 64, scale=vs))
            v = torch.from_numpy(seeded.randn(2000 + t, tpf, H, 64, scale=vs))
            q = torch.from_numpy(seeded.randn(3000 + t, tpf, H, 64, scale=vs))
            m.append_frame(0, k, v)
            m.evict_frames(0, scale, window)
            if keep is None or t in keep:
                out[f"{name}_out_{t}"] = m.compute_attention(0, q).numpy()
        # one non-keyframe: deferred eviction + temporary append + attention + rollback
        k = torch.from_numpy(seeded.randn(1000 + frames, tpf, H, 64, scale=vs))
        v = torch.from_numpy(seeded.randn(2000 + frames, tpf, H, 64, scale=vs))
        q = torch.from_numpy(seeded.randn(3000 + frames, tpf, H, 64, scale=vs))
        m._defer_eviction = True
        m.append_frame(0, k, v)
        out[f"{name}_out_nonkf"] = m.compute_attention(0, q).numpy()
        m.rollback_last_frame(0)
        m._defer_eviction = False
        out[f"{name}_visible_end"] = np.array(m.build_visible_page_table(0), np.int32)
        meta[name] = dict(tokens_per_frame=tpf, heads=H, scale=scale, window=window, frames=frames,
                          max_total=max_total, value_scale=vs)
    out["meta_json"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "paged_attention_fp32.npz"), **out)
    print("paged_attention_fp32.npz:", len(out), "arrays")


def prepare_qkv_values():
    """prepare_qkv (attention.py:402-426) with 3-D RoPE, and Attention.forward's q/k path with 2-D RoPE."""
    import torch
    from lingbot_map.layers.attention import FlashInferAttention, Attention
    from lingbot_map.layers.rope import WanRotaryPosEmbed, RotaryPositionEmbedding2D, PositionGetter
    torch.manual_seed(0)
    out = {}
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    N = ns + pph * ppw
    rope2d = RotaryPositionEmbedding2D(frequency=100)
    att = FlashInferAttention(dim, num_heads=H, qk_norm=True, rope=rope2d).eval()
    seeded.fill_module_(att, 7)
    rope3d = WanRotaryPosEmbed(attention_head_dim=64, patch_size=(1, 14, 14), max_seq_len=64)
    for f in (0, 5, 41):
        x = torch.from_numpy(seeded.randn(50 + f, 1, N, dim))
        pos3d = rope3d(ppf=1, pph=pph, ppw=ppw, patch_start_idx=ns, device=torch.device("cpu"), f_start=f, f_end=f + 1)
        with torch.no_grad():
            qkv = att.qkv(x)[0]                                  # [N, 3*dim]
            q, k, v = att.prepare_qkv(x, pos=pos3d, enable_3d_rope=True)
        out[f"rope3d_f{f}_qkv"] = qkv.numpy()
        out[f"rope3d_f{f}_q"], out[f"rope3d_f{f}_k"], out[f"rope3d_f{f}_v"] = q.numpy(), k.numpy(), v.numpy()
    # 2-D: positions as the aggregator builds them (base.py:416-442)
    pos = PositionGetter()(1, pph, ppw, device=torch.device("cpu")) + 1
    pos = torch.cat([torch.zeros(1, ns, 2, dtype=pos.dtype), pos], dim=1)
    x = torch.from_numpy(seeded.randn(99, 1, N, dim))
    with torch.no_grad():
        qkv = att.qkv(x)[0]
        q, k, v = att.prepare_qkv(x, pos=pos, enable_3d_rope=False)
    out["rope2d_qkv"], out["rope2d_q"], out["rope2d_k"], out["rope2d_v"] = qkv.numpy(), q.numpy(), k.numpy(), v.numpy()
    out["rope2d_pos"] = pos[0].numpy()
    # dense frame attention incl. proj (attention.py:65-87), two frames as the batch dimension
    fa = Attention(dim, num_heads=H, qk_norm=True, rope=rope2d).eval()
    seeded.fill_module_(fa, 11)
    x = torch.from_numpy(seeded.randn(123, 2, N, dim))
    with torch.no_grad():
        y = fa(x, pos=pos.expand(2, -1, -1))
    out["frame_attn_out"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "prepare_qkv_fp32.npz"), **out)
    print("prepare_qkv_fp32.npz:", len(out), "arrays")


def block_stream_values():
    """FlashInferBlock (block.py:151-310) driven like AggregatorStream does: phase 1 with 2 scale frames,
    then 8 streaming frames with keyframe interval 2; and SDPABlock with interval 1 for the dict-cache path."""
    import torch
    from lingbot_map.layers.block import FlashInferBlock, SDPABlock
    from lingbot_map.layers.flashinfer_cache import FlashInferKVCacheManager
    from lingbot_map.layers.rope import WanRotaryPosEmbed, RotaryPositionEmbedding2D
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    P = ns + pph * ppw
    scale, window = 2, 3
    rope3d = WanRotaryPosEmbed(attention_head_dim=64, patch_size=(1, 14, 14), max_seq_len=64)
    dev = torch.device("cpu")
    out = {}

    def drive(block, cache, kf_interval, tag, is_paged):
        tfp = 0
        x = torch.from_numpy(seeded.randn(500, 1, scale * P, dim))
        pos = rope3d(ppf=scale, pph=pph, ppw=ppw, patch_start_idx=ns, device=dev, f_start=0, f_end=scale)
        kw = dict(num_patches=P - ns, num_special=ns, enable_3d_rope=True, kv_cache=cache, global_idx=0,
                  num_frame_for_scale=scale, num_register_tokens=4)
        with torch.no_grad():
            y = block(x, pos=pos, num_frames=scale, num_frame_per_block=scale, **kw)
        out[f"{tag}_phase1"] = y.numpy()
        tfp += scale
        for i in range(scale, scale + 8):
            is_kf = kf_interval <= 1 or (i - scale) % kf_interval == 0
            if is_paged:
                cache._skip_append = not is_kf
            x = torch.from_numpy(seeded.randn(500 + i, 1, P, dim))
            pos = rope3d(ppf=1, pph=pph, ppw=ppw, patch_start_idx=ns, device=dev, f_start=tfp, f_end=tfp + 1)
            with torch.no_grad():
                y = block(x, pos=pos, num_frames=1, num_frame_per_block=1, **kw)
            out[f"{tag}_frame{i}"] = y.numpy()
            if is_kf:
                tfp += 1
        if is_paged:
            cache._skip_append = False
            out[f"{tag}_visible_end"] = np.array(cache.build_visible_page_table(0), np.int32)
            out[f"{tag}_last_len_end"] = np.array([cache.compute_last_page_len(0)], np.int32)

    common = dict(dim=dim, num_heads=H, init_values=0.01, qk_norm=True,
                  rope=RotaryPositionEmbedding2D(frequency=100),
                  kv_cache_sliding_window=window, kv_cache_scale_frames=scale)
    blk = FlashInferBlock(**common).eval()
    seeded.fill_module_(blk, 21)
    mgr = FlashInferKVCacheManager(num_blocks=1, max_num_frames=scale + window + 16, tokens_per_frame=P, num_heads=H,
                                   head_dim=64, dtype=torch.float32, device=dev, scale_frames=scale,
                                   sliding_window=window, max_total_frames=40, force_fp32=True)
    drive(blk, mgr, 2, "paged_kf2", True)
    mgr.reset()
    drive(blk, mgr, 1, "paged_kf1", True)
    sblk = SDPABlock(**common).eval()
    seeded.fill_module_(sblk, 21)
    cache = {"k_0": None, "v_0": None, "k_0_special": None, "v_0_special": None}
    drive(sblk, cache, 1, "sdpa_kf1", False)
    out["param_names_json"] = np.frombuffer(json.dumps([n for n, _ in blk.named_parameters()]).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "block_stream_fp32.npz"), **out)
    print("block_stream_fp32.npz:", len(out), "arrays;",
          "max |paged_kf1 - sdpa_kf1| =",
          max(float(np.abs(out[f'paged_kf1_frame{i}'] - out[f'sdpa_kf1_frame{i}']).max()) for i in range(2, 10)))


MODEL_E2E = dict(height=126, width=182, frames=8, scale_frames=2, window=3, weight_seed=7, image_seed=5,
                 depth_stride=7)


def model_e2e_images():
    c = MODEL_E2E
    return np.random.RandomState(c["image_seed"]).rand(c["frames"], 3, c["height"], c["width"]).astype(np.float32)


def model_e2e_values():
    """The whole GCTStream model (models/gct_stream.py:350-470) with seeded weights, fp32 on CPU, streaming 8
    frames (2 scale frames, then one by one): the SDPA backend with keyframe interval 1, and the paged manager's
    fp32 gather+SDPA path (kv_cache_force_fp32) with keyframe interval 2.  Stores camera encodings and a strided
    sample of the depth maps."""
    import torch
    from lingbot_map.models.gct_stream import GCTStream
    c = MODEL_E2E
    kw = dict(img_size=518, patch_size=14, enable_3d_rope=True, max_frame_num=64,
              kv_cache_sliding_window=c["window"], kv_cache_scale_frames=c["scale_frames"], camera_num_iterations=4)
    imgs = torch.from_numpy(model_e2e_images())
    out = {}
    for tag, use_sdpa, kf in (("sdpa_kf1", True, 1), ("paged_kf2", False, 2), ("paged_kf1", False, 1)):
        model = GCTStream(use_sdpa=use_sdpa, **kw).eval()
        seeded.fill_model_(model, c["weight_seed"])
        if not use_sdpa:
            model.aggregator.kv_cache_force_fp32 = True
        with torch.no_grad():
            pred = model.inference_streaming(imgs, num_scale_frames=c["scale_frames"], keyframe_interval=kf)
        st = c["depth_stride"]
        out[f"{tag}_pose_enc"] = pred["pose_enc"][0].numpy().astype(np.float32)
        out[f"{tag}_depth"] = pred["depth"][0, :, ::st, ::st, 0].numpy().astype(np.float32)
        out[f"{tag}_depth_mean"] = pred["depth"][0].mean(dim=(1, 2, 3)).numpy().astype(np.float32)
        del model
    np.savez_compressed(os.path.join(HERE, "model_e2e_fp32.npz"), **out)
    print("model_e2e_fp32.npz:", {k: v.shape for k, v in out.items()})
    print("  max |paged_kf1 - sdpa_kf1| pose:", float(np.abs(out["paged_kf1_pose_enc"] - out["sdpa_kf1_pose_enc"]).max()),
          "depth:", float(np.abs(out["paged_kf1_depth"] - out["sdpa_kf1_depth"]).max()))
    print("  max |paged_kf2 - sdpa_kf1| pose:", float(np.abs(out["paged_kf2_pose_enc"] - out["sdpa_kf1_pose_enc"]).max()))


def block_stream_bf16_values():
    """FlashInferBlock with bf16 weights under bf16 autocast, the way demo.py runs the aggregator (demo.py:458-460,545):
    the reference's own block code on CPU, `block.to(bfloat16)`, bf16 input, torch.autocast("cpu", bfloat16); the
    paged manager in its fp32 gather + SDPA mode.  Phase 1 with 2 scale frames, then 5 streaming keyframes."""
    import torch
    from lingbot_map.layers.block import FlashInferBlock
    from lingbot_map.layers.flashinfer_cache import FlashInferKVCacheManager
    from lingbot_map.layers.rope import WanRotaryPosEmbed, RotaryPositionEmbedding2D
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    P = ns + pph * ppw
    scale, window = 2, 3
    rope3d = WanRotaryPosEmbed(attention_head_dim=64, patch_size=(1, 14, 14), max_seq_len=64)
    dev = torch.device("cpu")
    blk = FlashInferBlock(dim=dim, num_heads=H, init_values=0.01, qk_norm=True,
                          rope=RotaryPositionEmbedding2D(frequency=100), kv_cache_sliding_window=window,
                          kv_cache_scale_frames=scale).eval()
    seeded.fill_module_(blk, 21)
    blk = blk.to(torch.bfloat16)
    mgr = FlashInferKVCacheManager(num_blocks=1, max_num_frames=scale + window + 16, tokens_per_frame=P, num_heads=H,
                                   head_dim=64, dtype=torch.float32, device=dev, scale_frames=scale,
                                   sliding_window=window, max_total_frames=40, force_fp32=True)
    kw = dict(num_patches=P - ns, num_special=ns, enable_3d_rope=True, kv_cache=mgr, global_idx=0,
              num_frame_for_scale=scale, num_register_tokens=4)
    out = {}
    with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16):
        x = torch.from_numpy(seeded.randn(900, 1, scale * P, dim)).to(torch.bfloat16)
        pos = rope3d(ppf=scale, pph=pph, ppw=ppw, patch_start_idx=ns, device=dev, f_start=0, f_end=scale)
        y = blk(x, pos=pos, num_frames=scale, num_frame_per_block=scale, **kw)
        out["phase1"] = y.float().numpy()
        for i in range(5):
            x = torch.from_numpy(seeded.randn(901 + i, 1, P, dim)).to(torch.bfloat16)
            pos = rope3d(ppf=1, pph=pph, ppw=ppw, patch_start_idx=ns, device=dev, f_start=scale + i, f_end=scale + i + 1)
            y = blk(x, pos=pos, num_frames=1, num_frame_per_block=1, **kw)
            out[f"frame{i}"] = y.float().numpy()
    out["visible_end"] = np.array(mgr.build_visible_page_table(0), np.int32)
    np.savez_compressed(os.path.join(HERE, "block_stream_bf16.npz"), **out)
    print("block_stream_bf16.npz:", {k: (v.shape, float(np.abs(v).max())) for k, v in out.items()})


MODEL_E2E_518 = dict(height=378, width=518, frames=8, num_scale_frames=2, weight_seed=7, image_seed=0, depth_stride=7)


def model_e2e_518_images():
    c = MODEL_E2E_518
    return np.random.RandomState(c["image_seed"]).rand(c["frames"], 3, c["height"], c["width"]).astype(np.float32)


def model_e2e_518_values():
    """The whole GCTStream model at the production frame size 378x518 (1005 tokens per frame, page of 999 tokens with
    its 103-token tail block), default cache geometry (8 anchor frames, window 64), 8 frames U[0,1): 2 scale frames
    in phase 1, then 6 streaming frames, keyframe interval 1; fp32 on CPU through the paged manager's fp32
    gather + SDPA path.  Stores camera encodings and a strided sample of the depth maps."""
    import torch
    from lingbot_map.models.gct_stream import GCTStream
    c = MODEL_E2E_518
    model = GCTStream(img_size=518, patch_size=14, enable_3d_rope=True, max_frame_num=64, camera_num_iterations=4,
                      use_sdpa=False).eval()
    seeded.fill_model_(model, c["weight_seed"])
    model.aggregator.kv_cache_force_fp32 = True
    imgs = torch.from_numpy(model_e2e_518_images())
    with torch.no_grad():
        pred = model.inference_streaming(imgs, num_scale_frames=c["num_scale_frames"], keyframe_interval=1)
    st = c["depth_stride"]
    out = {"pose_enc": pred["pose_enc"][0].numpy().astype(np.float32),
           "depth": pred["depth"][0, :, ::st, ::st, 0].numpy().astype(np.float32),
           "visible_end": np.array(model.aggregator.kv_cache_manager.build_visible_page_table(0), np.int32)}
    np.savez_compressed(os.path.join(HERE, "model_e2e_518_fp32.npz"), **out)
    print("model_e2e_518_fp32.npz:", {k: v.shape for k, v in out.items()})


def camera_head_values():
    """CameraCausalHead (heads/camera_head.py:157-358) in streaming mode on CPU, fp32: 2 heads of 128 (dim 256),
    4 refinement iterations x 4 blocks with 3-D RoPE; first call with 3 scale frames at once, then 7 single frames of
    which two are non-keyframes (_skip_append: attend, do not store).  Stores every call's final pose encoding."""
    import torch
    from lingbot_map.heads.camera_head import CameraCausalHead
    head = CameraCausalHead(dim_in=256, num_heads=2, trunk_depth=4, num_iterations=4, enable_3d_rope=True,
                            max_frame_num=64).eval()
    seeded.fill_model_(head, 13)
    out = {}
    with torch.no_grad():
        x = torch.from_numpy(seeded.randn(700, 1, 3, 1, 256))
        y = head([x], causal_inference=True, num_frame_per_block=3, num_frame_for_scale=3)
        out["scale"] = y[-1].numpy()
        for i in range(7):
            skip = i in (2, 5)
            for d in head.kv_cache:
                d["_skip_append"] = skip
            x = torch.from_numpy(seeded.randn(701 + i, 1, 1, 1, 256))
            y = head([x], causal_inference=True, num_frame_per_block=1, num_frame_for_scale=3)
            out[f"frame{i}"] = y[-1].numpy()
    out["cached_frames"] = np.array([head.kv_cache[0]["k_0"].shape[2]], np.int32)
    np.savez_compressed(os.path.join(HERE, "camera_head_fp32.npz"), **out)
    print("camera_head_fp32.npz:", {k: v.shape for k, v in out.items()}, "cached", out["cached_frames"])


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LINGBOT_MAP_REFERENCE"), required="LINGBOT_MAP_REFERENCE" not in os.environ,
                    help="checkout of the reference repository (or set LINGBOT_MAP_REFERENCE)")
    ap.add_argument("--only", default="", help="comma-separated fixture names (default: all)")
    args = ap.parse_args()
    _import_reference(args.reference)
    todo = {"manager_traces": manager_traces, "paged_attention": paged_attention_values,
            "prepare_qkv": prepare_qkv_values, "block_stream": block_stream_values, "model_e2e": model_e2e_values,
            "block_stream_bf16": block_stream_bf16_values, "model_e2e_518": model_e2e_518_values,
            "camera_head": camera_head_values}
    for name, fn in todo.items():
        if (not args.only and name != "model_e2e_518") or name in args.only.split(","):
            fn()
