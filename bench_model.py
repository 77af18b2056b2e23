"""Whole-model streaming frames/s of the reference's GCTStream at a pre-filled KV cache, with either backend.

    python bench_model.py --reference <dir holding the lingbot_map package and gct_profile.py> \
        --backend b200|flashinfer --cached-frames 10000 --frames 40 [--no-compile]

A measurement tool beside bench.py (which runs it for its `whole_model` record); not part of the importable package.

The model, its random-init weights, the synthetic images (randn, seed 42), bf16 autocast and the optional
torch.compile of the hot modules are the ones of the reference's gct_profile.py (load_model / compile_model are
imported from it, gct_profile.py:26-57); only the way the steady state is reached differs: instead of streaming
`cached-frames` real frames first, phase 1 and a few streaming frames run for real, then the cache manager of
every global block is filled with seeded random K/V through its own public append_frame / evict_frames calls and
the frame counter that drives the 3-D RoPE is advanced (aggregator/stream.py:468-469,526-527).  After that
`--frames` real model.forward calls are timed with CUDA events, one frame at a time, as gct_profile.py does
(gct_profile.py:115-160).  With `--backend flashinfer` nothing of this package touches the model: it is the
reference's own FlashInfer path."""
import argparse
import contextlib
import importlib.util
import json
import os
import sys
import time

import torch


def _load_profile_module(reference_dir):
    path = os.path.join(reference_dir, "gct_profile.py")
    if not os.path.exists(path):
        raise SystemExit(f"{path} not found: --reference must hold gct_profile.py and the lingbot_map package")
    sys.path.insert(0, reference_dir)
    spec = importlib.util.spec_from_file_location("_gct_profile", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def prefill(model, cached_frames, seed=0):
    """Append seeded random K/V frames to every global block's cache until `cached_frames` keyframes are cached."""
    agg = model.aggregator
    mgr = agg.kv_cache_manager
    have = int(mgr.num_frames)
    todo = cached_frames - have
    if todo <= 0:
        return have
    blk = agg.global_blocks[0].attn
    g = torch.Generator(device="cuda").manual_seed(seed)
    shape = (mgr.tokens_per_frame, blk.num_heads, blk.head_dim)
    k = torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)
    for f in range(todo):
        for b in range(mgr.num_blocks):
            mgr.append_frame(b, k, v)
            mgr.evict_frames(block_idx=b, scale_frames=blk.kv_cache_scale_frames,
                             sliding_window=blk.kv_cache_sliding_window,
                             cross_frame_special=blk.kv_cache_cross_frame_special,
                             include_scale_frames=blk.kv_cache_include_scale_frames,
                             camera_only=blk.kv_cache_camera_only, num_register_tokens=4)
    agg.total_frames_processed += todo
    return int(mgr.num_frames)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", required=True)
    ap.add_argument("--backend", choices=["b200", "flashinfer"], default="b200")
    ap.add_argument("--cached-frames", type=int, default=10000)
    ap.add_argument("--frames", type=int, default=40)
    ap.add_argument("--img-h", type=int, default=378)
    ap.add_argument("--img-w", type=int, default=518)
    ap.add_argument("--no-compile", action="store_true")
    ap.add_argument("--patch-embed", action="store_true", help="b200 backend: also convert the DINOv2 patch-embed attention")
    args = ap.parse_args(argv)

    gp = _load_profile_module(os.path.abspath(args.reference))
    if args.backend == "b200":
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from lingbot_map_b200 import select
        select.install(patch_embed_attention=args.patch_embed)
    torch.manual_seed(0)
    model = gp.load_model("flashinfer", img_size=518, sliding_window=64, max_frame_num=args.cached_frames + 400,
                          camera_num_iterations=4)
    torch.manual_seed(42)
    n_real = 8 + 12 + 12 + args.frames
    images = torch.randn(1, n_real, 3, args.img_h, args.img_w, device="cuda").to(torch.bfloat16)
    ctx = torch.amp.autocast("cuda", dtype=torch.bfloat16)

    def stream(lo, hi):
        for i in range(lo, hi):
            torch.compiler.cudagraph_mark_step_begin()
            with torch.no_grad(), ctx:
                model.forward(images[:, i:i + 1], num_frame_for_scale=8, num_frame_per_block=1, causal_inference=True)

    model.clean_kv_cache()
    torch.compiler.cudagraph_mark_step_begin()
    with torch.no_grad(), ctx:
        model.forward(images[:, :8], num_frame_for_scale=8, num_frame_per_block=8, causal_inference=True)
    stream(8, 14)
    if not args.no_compile:
        gp.compile_model(model)
        stream(14, 20)
    t0 = time.perf_counter()
    cached = prefill(model, args.cached_frames)
    torch.cuda.synchronize()
    fill_s = time.perf_counter() - t0
    stream(20, 32)                                   # warm-up at the final cache size
    torch.cuda.synchronize()
    stats = model.aggregator.kv_cache_manager.get_cache_stats(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_frame = []
    for i in range(32, 32 + args.frames):
        e0.record()
        stream(i, i + 1)
        e1.record()
        torch.cuda.synchronize()
        per_frame.append(e0.elapsed_time(e1))
    in_order = [round(x, 2) for x in per_frame]
    per_frame.sort()
    med = per_frame[len(per_frame) // 2]
    mean = sum(per_frame) / len(per_frame)
    print(json.dumps({"backend": args.backend, "compiled": not args.no_compile, "cached_frames": cached,
                      "cache_stats_block0": {k: (int(v) if isinstance(v, (int, bool)) else v) for k, v in stats.items()
                                             if isinstance(v, (int, float, bool))},
                      "frames_timed": args.frames, "ms_per_frame_median": round(med, 3),
                      "ms_per_frame_mean": round(mean, 3), "frames_per_s_median": round(1000.0 / med, 2),
                      "frames_per_s_mean": round(1000.0 / mean, 2), "ms_per_frame_max": round(per_frame[-1], 3), "ms_in_order": in_order,
                      "prefill_s": round(fill_s, 1),
                      "image": f"{args.img_h}x{args.img_w}", "dtype": "bf16 autocast"}))


if __name__ == "__main__":
    main()
