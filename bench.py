#!/usr/bin/env python
"""Benchmark of the GCT streaming attention hot path on B200.

One "step" = one streaming frame at 518x378 (1005 tokens, 16 heads x 64) through the hot path of all 24
aggregator layers, at the steady state of a 10,000-frame sequence (8 anchor + 64 window frames of full
tokens + 6 memory tokens of every past frame = 131,928 visible KV tokens):
    frame block  : q/k LayerNorm + 2-D RoPE + bf16 cast  ->  dense attention 1005 x 1005
    global block : fused q/k LayerNorm + 3-D RoPE + bf16 K/V page append -> eviction -> paged attention
                   over the visible page table (split-KV + log-sum-exp merge)
The qkv/proj Linear layers, MLPs, DINOv2 and the heads are outside the measured path (`whole_model` in the
output line times the complete model behind the reference's interface, with either backend).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--mode streams|kvsplit]
                    [--streams-per-gpu S]

Prints ONE JSON line.  N > 1 is launched with torch.distributed.run, one rank per GPU:
`streams` (default) runs independent streams, S per GPU (weak scaling, no data-path collective), and adds a
`kvsplit` sub-record: ONE stream whose visible pages are sharded over the GPUs (strong scaling), checked against
the single-pass result before it is timed.  `--mode kvsplit` makes that the headline of the line instead.
`--impl reference` times the reference's SDPA streaming path on the host cores.

At N = 1 the line also carries, measured after and outside the timed regions:
  cpu_baseline      the reference's CPU path on a bounded sample;
  flashinfer_layer  the reference's own FlashInferKVCacheManager.compute_attention (plan once, run() timed) on a
                    cache with the same page table and contents as this backend's, kv = 131,928, same GPU;
  parity_at_headline  this backend's output for that layer against a float64 softmax over all rows of two heads
                    and against FlashInfer's bf16 output on every element;
  whole_model       frames/s of the whole GCTStream model at the 10k-frame cache with this backend and with the
                    reference's FlashInfer backend (bench_model.py, one subprocess each).
"""
import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

TPF, HEADS, HEAD_DIM, DEPTH = 1005, 16, 64, 24
PPH, PPW, NSPECIAL = 27, 37, 6
SCALE_FRAMES, WINDOW = 8, 64
METRIC = "streaming frames/s @518x378 bf16 (steady state, 10k-frame KV); attn % of TC peak"
UNIT = "frames/s"
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def visible_kv(n_cached):
    return (TPF - NSPECIAL) * min(n_cached, SCALE_FRAMES + WINDOW) + NSPECIAL * n_cached


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"bf16_tflops": d["bf16_tflops_sustained"], "bf16_tflops_burst": d.get("bf16_tflops"),
                "hbm_gbs": d["hbm_gbs"], "which": "measured (sustained)"}
    return {"bf16_tflops": 1400.0, "bf16_tflops_burst": 1590.0, "hbm_gbs": 6650.0, "which": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.rows, self.proc, self.thread = [], None, None
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
            self.cmd = ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                        "-lms", "200"]
        except Exception:
            self.cmd = None

    def start(self):
        if self.cmd is None:
            return
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def mark_begin(self):
        """Start of the timed region: only samples from here on (to a little past its end) are reported."""
        self.t_begin = time.perf_counter()

    def mark_end(self):
        self.t_end = time.perf_counter()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        t_end = getattr(self, "t_end", time.perf_counter())
        time.sleep(0.25)
        for _ in range(30):                    # a slow nvidia-smi start-up: wait for its first row rather than report none
            if self.rows:
                break
            time.sleep(0.1)
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t_begin = getattr(self, "t_begin", 0.0)
        inside = [r for t, r in self.rows if t_begin <= t <= t_end + 0.25]
        if not inside and self.rows:          # region shorter than the sampling period: the sample nearest to it
            inside = [min(self.rows, key=lambda tr: abs(tr[0] - t_end))[1]]
        for r in inside:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v == "Active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- host placement
def bind_to_gpu_numa_node(device_index):
    """Pin this process (and so the pinned host buffers it touches first) to the CPUs of the GPU's NUMA node.
    Best effort: returns {"numa_node": n or None, "cpus": count} for the output line."""
    info = {"numa_node": None, "cpus": len(os.sched_getaffinity(0))}
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        with open(path) as f:
            node = int(f.read().strip())
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info = {"numa_node": node, "cpus": len(cpus)}
    except Exception:
        pass
    return info


# ----------------------------------------------------------------------------- workload (GPU arm)
class HotPath:
    """State of one stream on one GPU: cache manager at the n_cached-frame steady state + synthetic inputs."""

    def __init__(self, device, n_cached, extra_frames, seed, shard=None, keyframe_interval=1):
        import lingbot_map_b200 as P
        from lingbot_map_b200 import _lib
        self.P, self.lib, self.dev = P, _lib, device
        self.shard = shard                      # (rank, world) for kvsplit, else None
        self.kf_interval = max(int(keyframe_interval), 1)
        self.step_index = 0
        g = torch.Generator(device=device).manual_seed(seed)
        self.mgr = P.B200KVCacheManager(DEPTH, SCALE_FRAMES + WINDOW + 16, TPF, HEADS, HEAD_DIM, device=device,
                                        scale_frames=SCALE_FRAMES, sliding_window=WINDOW,
                                        max_total_frames=n_cached + extra_frames + 100)
        for pool in self.mgr.kv_caches:         # cached K/V ~ N(0,1): logits q.k/8 have unit variance
            pool.normal_(generator=g)
        for b in range(DEPTH):                  # bookkeeping only: the pages already hold data
            for _ in range(n_cached):
                self.mgr.append_frame_bookkeeping(b)
                self.mgr.evict_frames(b, SCALE_FRAMES, WINDOW)
        self.mgr.rescan_key_norms()             # the pages were filled directly: recompute the key-norm maxima
        C = HEADS * HEAD_DIM
        rn = lambda *s: torch.randn(*s, device=device, generator=g)
        self.qkv_frame = [rn(TPF, 3 * C).to(torch.bfloat16) for _ in range(DEPTH)]
        self.qkv_global = [rn(TPF, 3 * C).to(torch.bfloat16) for _ in range(DEPTH)]
        self.norm = [[1 + 0.1 * rn(64), 0.1 * rn(64), 1 + 0.1 * rn(64), 0.1 * rn(64)] for _ in range(2 * DEPTH)]
        self.cs2d = P.ops.rope2d_table(PPH, PPW, NSPECIAL, device)
        self.cs3d = torch.empty(TPF, 32, 2, dtype=torch.float32, device=device)
        self.frame_index = n_cached
        self.outs = [None] * (2 * DEPTH)
        self.launches = 0
        self.keep_q = None                      # set to a list to keep the global layers' q of the last step

    def step(self, qkv_frame=None, qkv_global=None, before_layer=None, after_layer=None):
        P, lib, m = self.P, self.lib, self.mgr
        qkv_frame = qkv_frame or self.qkv_frame
        qkv_global = qkv_global or self.qkv_global
        # 3-D RoPE table of this frame; the reference keeps time indices below max_frame_num, so wrap
        P.ops.rope3d_table(self.frame_index % 1024, PPH, PPW, NSPECIAL, self.dev, out=self.cs3d)
        self.launches += 1
        # keyframe gate (gct_stream.py:450-464): every kf_interval-th frame stays in the cache; the others are
        # appended with eviction deferred, attended over and rolled back (block.py:256-263)
        keyframe = self.step_index % self.kf_interval == 0
        if not keyframe:
            m._defer_eviction = True
        for b in range(DEPTH):
            if before_layer is not None:
                before_layer(b)
            q, k, v = P.ops.prep_qkv(qkv_frame[b], HEADS, TPF, *self.norm[2 * b], self.cs2d, lib.ROPE_2D)
            self.outs[2 * b] = P.ops.dense_attention(q[None], k[None], v[None])
            qg = m.append_frame_fused(b, qkv_global[b], *self.norm[2 * b + 1], self.cs3d, lib.ROPE_3D)
            m.evict_frames(b, SCALE_FRAMES, WINDOW)      # no-op while deferred
            if self.keep_q is not None:
                self.keep_q.append(qg)
            if self.shard is None:
                self.outs[2 * b + 1] = m.compute_attention(b, qg)
                self.launches += 5          # prep, dense attention, fused append, paged attention, merge
            else:
                from lingbot_map_b200 import distributed as D
                self.outs[2 * b + 1] = D.sharded_attention(m, b, qg, *self.shard)
                self.launches += 5          # prep, dense attention, fused append, paged attention, exchange+merge
            if not keyframe:
                m.rollback_last_frame(b)
            if after_layer is not None:
                after_layer(b)
        if not keyframe:
            m._defer_eviction = False
        else:
            self.frame_index += 1               # a non-keyframe reuses the time index of the next keyframe
        self.step_index += 1


def _cos64(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-300))


def timed_steps(step_fn, n, barrier, dev, world):
    """n calls of step_fn between a barrier + synchronize on both sides; CUDA-event ms, max over ranks."""
    import torch.distributed as dist
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(n):
        step_fn()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    local_ms = float(ms.item())
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()), local_ms


def measure(hps, args, dev, rank, world, barrier, sampler, kvsplit):
    """The three timed regions for a list of streams on this GPU (one entry when kvsplit): device-resident inputs,
    a second pass over the same steps with the attention kernel bracketed by events, and the end-to-end pass."""
    import torch.distributed as dist
    m0 = hps[0].mgr

    def step_all():
        for hp in hps:
            hp.step()

    for _ in range(args.warmup):
        step_all()
    barrier()
    for hp in hps:
        assert hp.mgr.device_status() == 0
    # ---- timed region: device-resident inputs, no instrumentation ----
    if sampler is not None:
        sampler.mark_begin()
    launches0 = sum(hp.launches for hp in hps)
    t_wall = time.perf_counter()
    total_ms, _ = timed_steps(step_all, args.steps, barrier, dev, world)
    wall_s = time.perf_counter() - t_wall
    if sampler is not None:
        sampler.mark_end()
    gpu_launches = sum(hp.launches for hp in hps) - launches0
    # ---- second pass: the paged attention kernel alone, one CUDA-event pair per launch ----
    ksteps = max(1, min(args.steps, args.kernel_steps))
    m0.kernel_timing(ksteps * DEPTH)
    m0.kernel_time()
    for _ in range(ksteps):
        hps[0].step()
    attn_ms, attn_launches = m0.kernel_time()
    m0.kernel_timing(0)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for _ in range(ksteps):
        hps[0].step()
    t1.record()
    torch.cuda.synchronize()
    one_stream_step_ms = t0.elapsed_time(t1) / ksteps
    for hp in hps:
        assert hp.mgr.device_status() == 0 and hp.P.ops.device_status(dev) == 0

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region ----
    C3 = 3 * HEADS * HEAD_DIM
    # KV-sharded stream: the frame's inputs are the same on every rank, so each rank moves only its 1/W slice of the
    # rows over PCIe (host -> device, and of the results device -> host) and the ranks complete the inputs over NVLink:
    # one coalesced all-gather of the step's 48 slices at the start of the step, on the compute stream (the per-layer
    # exchange kernels wait on their peers and must not share the device with another kernel that does).  The slices
    # of step s+1 are uploaded while step s computes (two slice sets).  The bytes that cross PCIe per step are the
    # same in total as for one GPU.
    sliced = kvsplit and world > 1
    rows_pad = -(-TPF // world) * world if sliced else TPF
    sl = rows_pad // world if sliced else TPF
    r_lo = rank * sl if sliced else 0
    r_hi = min(r_lo + sl, TPF)

    def host_slice(t):
        full = torch.zeros(rows_pad, t.shape[1], dtype=t.dtype)
        full[:TPF].copy_(t.cpu())
        return full[r_lo:r_lo + sl].clone().pin_memory()

    e2e = []
    for hp in hps:
        st = {"hp": hp}
        st["h_in_f"] = [host_slice(t) for t in hp.qkv_frame]
        st["h_in_g"] = [host_slice(t) for t in hp.qkv_global]
        st["h_out"] = [torch.empty(max(r_hi - r_lo, 0), HEADS, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
                       for _ in range(2 * DEPTH)]
        st["d_buf_f"] = [torch.empty(rows_pad, C3, dtype=torch.bfloat16, device=dev) for _ in range(DEPTH)]
        st["d_buf_g"] = [torch.empty(rows_pad, C3, dtype=torch.bfloat16, device=dev) for _ in range(DEPTH)]
        st["d_in_f"] = [t[:TPF] for t in st["d_buf_f"]]
        st["d_in_g"] = [t[:TPF] for t in st["d_buf_g"]]
        if sliced:
            st["d_sl_f"] = [[torch.empty(sl, C3, dtype=torch.bfloat16, device=dev) for _ in range(DEPTH)] for _ in range(2)]
            st["d_sl_g"] = [[torch.empty(sl, C3, dtype=torch.bfloat16, device=dev) for _ in range(DEPTH)] for _ in range(2)]
        e2e.append(st)
    # Copies run on their own stream.  Streams of independent frames: the inputs of layer b are uploaded while layer
    # b-1 computes, and the outputs of layer b are downloaded while layer b+1 computes.  Events order every buffer
    # hand-over in both directions.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)

    def make_e2e_step(st):
        hp = st["hp"]
        ev_in = [torch.cuda.Event() for _ in range(DEPTH)]       # inputs of layer b are on the device
        ev_free = [torch.cuda.Event() for _ in range(DEPTH)]     # layer b no longer reads its input buffers
        ev_out = [torch.cuda.Event() for _ in range(DEPTH)]      # outputs of layer b are computed
        for e in ev_free:
            e.record(main_stream)

        def upload(b):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_free[b])
                st["d_in_f"][b].copy_(st["h_in_f"][b], non_blocking=True)
                st["d_in_g"][b].copy_(st["h_in_g"][b], non_blocking=True)
                ev_in[b].record(copy_stream)

        def before_layer(b):
            if b == 0:
                upload(0)
            if b + 1 < DEPTH:
                upload(b + 1)
            main_stream.wait_event(ev_in[b])

        def after_layer(b):
            ev_free[b].record(main_stream)
            ev_out[b].record(main_stream)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_out[b])
                for i in (2 * b, 2 * b + 1):
                    hp.outs[i].record_stream(copy_stream)
                    st["h_out"][i].copy_(hp.outs[i].view(TPF, HEADS, HEAD_DIM)[r_lo:r_hi], non_blocking=True)

        def e2e_step():
            hp.step(st["d_in_f"], st["d_in_g"], before_layer, after_layer)
            main_stream.wait_stream(copy_stream)                 # the step ends when its results are on the host

        if not sliced:
            return e2e_step

        ev_sl_in = [torch.cuda.Event() for _ in range(2)]        # slice set s of the next step is on the device
        ev_sl_free = [torch.cuda.Event() for _ in range(2)]      # the all-gather has read slice set s
        for e in ev_sl_free:
            e.record(main_stream)
        state = {"set": 0, "primed": False}

        def upload_slices(s):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_sl_free[s])
                for b in range(DEPTH):
                    st["d_sl_f"][s][b].copy_(st["h_in_f"][b], non_blocking=True)
                    st["d_sl_g"][s][b].copy_(st["h_in_g"][b], non_blocking=True)
                ev_sl_in[s].record(copy_stream)

        def after_layer_sliced(b):
            ev_out[b].record(main_stream)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_out[b])
                for i in (2 * b, 2 * b + 1):
                    hp.outs[i].record_stream(copy_stream)
                    st["h_out"][i].copy_(hp.outs[i].view(TPF, HEADS, HEAD_DIM)[r_lo:r_hi], non_blocking=True)

        def e2e_step_sliced():
            s = state["set"]
            if not state["primed"]:
                upload_slices(s)
                state["primed"] = True
            main_stream.wait_event(ev_sl_in[s])
            # one launch for the 48 gathers where the installed torch can coalesce them, else one launch each
            with getattr(dist, "_coalescing_manager", contextlib.nullcontext)():
                for b in range(DEPTH):
                    dist.all_gather_into_tensor(st["d_buf_f"][b], st["d_sl_f"][s][b])
                    dist.all_gather_into_tensor(st["d_buf_g"][b], st["d_sl_g"][s][b])
            ev_sl_free[s].record(main_stream)
            upload_slices(1 - s)                                 # the next step's slices cross PCIe under this step
            state["set"] = 1 - s
            hp.step(st["d_in_f"], st["d_in_g"], None, after_layer_sliced)
            main_stream.wait_stream(copy_stream)                 # the step ends when its result slices are on the host
        return e2e_step_sliced

    e2e_steps = [make_e2e_step(st) for st in e2e]

    def e2e_all():
        for f in e2e_steps:
            f()

    e2e_all()
    e2e_ms, e2e_local = timed_steps(e2e_all, args.e2e_steps, barrier, dev, world)
    per_rank = [e2e_local]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, e2e_local)
        per_rank = gathered
    streams = 1 if kvsplit else world * len(hps)
    return {
        "total_ms": total_ms, "wall_s": wall_s, "gpu_launches": gpu_launches, "attn_ms": attn_ms,
        "attn_launches": attn_launches, "one_stream_step_ms": one_stream_step_ms, "streams": streams,
        "value": streams * args.steps / (total_ms / 1e3),
        "e2e_value": streams * args.e2e_steps / (e2e_ms / 1e3),
        "e2e_per_rank_fps": [len(hps) * args.e2e_steps / (x / 1e3) for x in per_rank],
        # bytes that cross PCIe per step for one stream (a sharded stream moves them in W slices, one per rank)
        "h2d": 2 * DEPTH * TPF * C3 * 2, "d2h": 2 * DEPTH * TPF * HEADS * HEAD_DIM * 2,
    }


def kvsplit_parity(hp, rank, dev):
    """One frame of the KV-sharded stream; every global layer's merged output is compared on rank 0 with the
    single-pass attention of the same layer over the whole page list (every rank holds the whole replicated pool)."""
    m = hp.mgr
    hp.keep_q = []
    hp.step()
    qs, hp.keep_q = hp.keep_q, None
    torch.cuda.synchronize()
    worst_abs, worst_cos = 0.0, 1.0
    if rank == 0:
        for b in range(DEPTH):
            m.plan()                                            # the whole visible list
            full = m.compute_attention(b, qs[b])
            got = hp.outs[2 * b + 1].view(TPF, HEADS, HEAD_DIM)
            worst_abs = max(worst_abs, float((got.float() - full.float()).abs().max()))
            worst_cos = min(worst_cos, _cos64(got, full))
        m._shard_plan = None                                     # the next sharded call plans its slice again
    ok = worst_abs <= 1e-2 and worst_cos >= 0.99999
    return {"max_abs": worst_abs, "cosine": worst_cos, "layers": DEPTH, "ok": bool(ok),
            "bound": "max_abs <= 1e-2, cosine >= 0.99999 against the single-pass output on rank 0"}


def run_gpu(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    placement = bind_to_gpu_numa_node(local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    headline_kvsplit = args.mode == "kvsplit" and world > 1
    extra = 2 * args.steps + 2 * args.warmup + 3 * args.kernel_steps + 16 + 2 * args.e2e_steps
    # the sampler runs from before the set-up (nvidia-smi takes a while to start on a multi-GPU host); only its
    # samples from the timed region are reported
    sampler = ClockSampler(dev)
    sampler.start()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def build(kvsplit, n_streams):
        hps = []
        for s in range(n_streams):
            seed = 100 + (0 if kvsplit else rank * n_streams + s)
            hp = HotPath(dev, args.frames_cached, extra, seed=seed, shard=(rank, world) if kvsplit else None,
                         keyframe_interval=args.keyframe_interval)
            if args.exact_softmax:
                hp.mgr.set_bounded_mode(False)
            hps.append(hp)
        return hps

    hps = build(headline_kvsplit, 1 if headline_kvsplit else args.streams_per_gpu)
    parity = kvsplit_parity(hps[0], rank, dev) if headline_kvsplit else None
    res = measure(hps, args, dev, rank, world, barrier, sampler, headline_kvsplit)
    clocks = sampler.stop()
    n_cached_now = hps[0].mgr.num_frames
    kv_now = visible_kv(n_cached_now)

    sub = None
    line_holder = {}
    if world > 1 and not headline_kvsplit and not args.no_kvsplit:
        # strong-scaling sub-record: one stream, visible pages sharded over all ranks.  The headline numbers are
        # already measured; a watchdog makes sure they are printed even if the sub-record should get stuck.
        del hps
        torch.cuda.empty_cache()

        def give_up():
            if rank == 0 and "line" in line_holder:
                line_holder["line"]["kvsplit"] = {"unavailable": "the KV-sharded sub-record did not finish within %d s"
                                                                 % args.kvsplit_timeout}
                print(json.dumps(line_holder["line"]), flush=True)
            os._exit(0 if rank != 0 or "line" in line_holder else 1)

        watchdog = threading.Timer(args.kvsplit_timeout, give_up)
        watchdog.daemon = True
        line_holder["line"] = headline_line(args, res, clocks, placement, kv_now, n_cached_now, world, False, None, None) \
            if rank == 0 else None
        watchdog.start()
        sub_args = argparse.Namespace(**vars(args))
        sub_args.steps, sub_args.warmup, sub_args.e2e_steps = min(args.steps, 40), 3, min(args.e2e_steps, 5)
        try:
            khps = build(True, 1)
            kpar = kvsplit_parity(khps[0], rank, dev)
            kres = measure(khps, sub_args, dev, rank, world, barrier, None, True)
            sub = {"value": kres["value"], "unit": UNIT, "scaling": "strong", "steps": sub_args.steps,
                   "ms_per_step": kres["total_ms"] / sub_args.steps, "e2e": kres["e2e_value"], "parity": kpar,
                   "exchange": "peer memory" if getattr(khps[0].mgr, "_peer_exchange", None) is not None else "nccl all-gather",
                   "workload": "one stream, visible KV pages sharded over %d GPUs, exchange + LSE merge per layer" % world}
            del khps
        except Exception as e:                                          # noqa: BLE001
            sub = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}
        watchdog.cancel()

    if rank == 0:
        line = headline_line(args, res, clocks, placement, kv_now, n_cached_now, world, headline_kvsplit, parity, sub)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(max_seconds=25.0)
    if world == 1 and rank == 0:
        del hps
        torch.cuda.empty_cache()
        if not args.no_flashinfer:
            rec = headline_layer_record(dev)
            line["flashinfer_layer"] = rec["flashinfer_layer"]
            line["parity_at_headline"] = rec["parity_at_headline"]
        if not args.no_whole_model:
            line["whole_model"] = whole_model_record(args)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def headline_line(args, res, clocks, placement, kv_now, n_cached_now, world, headline_kvsplit, parity, sub):
    """The output line of the GPU arm from the measurements of run_gpu (rank 0)."""
    peaks = load_peaks()
    # algorithmic FLOPs of one launch of the paged attention kernel; a KV shard holds 1/world of the keys
    flops = 4.0 * TPF * kv_now * HEAD_DIM * HEADS / (world if headline_kvsplit else 1)
    kern_s = res["attn_ms"] / max(res["attn_launches"], 1) / 1e3
    achieved = flops / kern_s / 1e12 if res["attn_launches"] else None
    sm = clocks.get("sm_mhz")
    line = {
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["total_ms"] / args.steps,
        "higher_is_better": True, "scaling": "strong" if headline_kvsplit else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"GCT hot path, {DEPTH} layers x (frame attention 1005x1005 + fused K/V append + "
                               f"paged global attention), 518x378, {n_cached_now} cached frames, kv={kv_now} tokens, "
                               f"page 999, scale {SCALE_FRAMES} + window {WINDOW}, keyframe_interval {args.keyframe_interval}",
                   "parallelism": ("kv-pages sharded over %d GPUs, peer exchange + LSE merge" % world) if headline_kvsplit
                   else ("%d independent stream(s), %d per GPU" % (res["streams"], args.streams_per_gpu)),
                   "l2": (f"inputs larger than L2 (each layer streams {kv_now * 4096 / 1e6:.0f} MB of K/V)"
                          if kv_now * 4096 * DEPTH > 126e6 else
                          f"K/V of all layers ({kv_now * 4096 * DEPTH / 1e6:.0f} MB) fit in L2: not a metric configuration"),
                   "clock_samples": clocks.get("samples"), "timed_region_s": res["wall_s"],
                   "host_placement": placement},
        "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "e2e": {"value": res["e2e_value"], "unit": UNIT, "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "steps": args.e2e_steps, "per_rank": res["e2e_per_rank_fps"]},
        "gpu_launches": res["gpu_launches"],
        "roofline": {"bound": "tensor", "kernel": "gct_attn_kernel<2> (paged global attention, %s)" %
                               ("running row maximum" if args.exact_softmax else
                                "softmax reference folded into the S product"),
                     "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": (achieved / peaks["bf16_tflops"]) if achieved else None,
                     "frac_of_burst_peak": (achieved / peaks["bf16_tflops_burst"])
                     if achieved and peaks.get("bf16_tflops_burst") else None,
                     "peak_source": peaks["which"], "kernel_us": kern_s * 1e6,
                     "kernel_us_x_sm_mhz": (kern_s * 1e6 * sm) if sm else None,
                     "launches_timed": res["attn_launches"],
                     "timed_in": "a second pass over the same steps, one CUDA-event pair per launch",
                     "flops_per_launch": flops,
                     "attn_share_of_step": (res["attn_ms"] / max(res["attn_launches"], 1) * DEPTH) / res["one_stream_step_ms"],
                     "traffic": NCU_DRAM_BYTES_SMALL_CASE * kv_now / NCU_SMALL_CASE_KV / (world if headline_kvsplit else 1),
                     "traffic_source": "ncu small case scaled by KV tokens"},
    }
    if parity is not None:
        line["kvsplit_parity"] = parity
    if sub is not None:
        line["kvsplit"] = sub
    return line


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the paged attention kernel.  Captured with
# ncu on a small case (kv = 73,170 tokens: 348.5 MB, see profiles/gct_attn_kernel_paged_kv73k.md) and
# scaled to the benchmark's KV length by the number of key tokens, which the traffic is proportional to.
NCU_DRAM_BYTES_SMALL_CASE = 348.5e6
NCU_SMALL_CASE_KV = 73170


# ----------------------------------------------------------------------------- same-box FlashInfer layer + parity
def headline_layer_record(dev, n_cached=10000, repeats=30):
    """One global layer at the headline geometry, built twice with identical contents: this backend's manager and the
    reference's own FlashInferKVCacheManager (imported from baseline/_ref).  Times both (plan once, then run), and
    checks this backend's output against a float64 softmax (all 1005 rows of two heads) and against FlashInfer."""
    import lingbot_map_b200 as P
    out = {"flashinfer_layer": None, "parity_at_headline": None}
    g = torch.Generator(device=dev).manual_seed(7)
    kf = torch.randn(8, TPF, HEADS, HEAD_DIM, device=dev, generator=g).to(torch.bfloat16)     # 8 frames, cycled
    vf = torch.randn(8, TPF, HEADS, HEAD_DIM, device=dev, generator=g).to(torch.bfloat16)
    q = torch.randn(TPF, HEADS, HEAD_DIM, device=dev, generator=g).to(torch.bfloat16)
    m = P.B200KVCacheManager(1, SCALE_FRAMES + WINDOW + 16, TPF, HEADS, HEAD_DIM, device=dev,
                             scale_frames=SCALE_FRAMES, sliding_window=WINDOW, max_total_frames=n_cached + 100)
    for t in range(n_cached):
        m.append_frame(0, kf[t % 8], vf[t % 8])
        m.evict_frames(0, SCALE_FRAMES, WINDOW)
    kv = visible_kv(n_cached)

    def time_us(fn):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(repeats):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / repeats * 1e3

    m.plan()
    h = m._handle
    from lingbot_map_b200 import _lib
    ours = torch.empty(TPF, HEADS, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    run_ours = lambda: _lib.check(m._lib.gct_mgr_attention(h, 0, q.data_ptr(), _lib.BF16, TPF, ours.data_ptr(), None, s))
    b200_us = time_us(run_ours)
    assert m.device_status() == 0
    # float64 softmax on the same bf16 inputs, all rows of two heads (on the device, outside every timed region)
    kk, vv = m._gather_kv(0)
    assert kk.shape[0] == kv
    worst_abs, worst_cos = 0.0, 1.0
    for hd in (0, 11):
        sc = (q[:, hd].double() @ kk[:, hd].double().T) * 0.125
        want = torch.softmax(sc, dim=-1) @ vv[:, hd].double()
        del sc
        worst_abs = max(worst_abs, float((ours[:, hd].double() - want).abs().max()))
        worst_cos = min(worst_cos, _cos64(ours[:, hd], want))
    par = {"kv": kv, "vs_float64_softmax": {"rows": TPF, "heads": [0, 11], "max_abs": worst_abs, "cosine": worst_cos},
           "bound": "max_abs <= 2e-2, cosine >= 0.9999",
           "ok": bool(worst_abs <= 2e-2 and worst_cos >= 0.9999)}
    rec = {"kv": kv, "b200_layer_us": b200_us, "b200_tflops": 4.0 * TPF * kv * HEAD_DIM * HEADS / b200_us / 1e6}
    try:
        if not os.path.isdir(REF_DIR):
            raise RuntimeError("baseline/_ref is not installed")
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from lingbot_map.layers.flashinfer_cache import FlashInferKVCacheManager
        ref = FlashInferKVCacheManager(num_blocks=1, max_num_frames=SCALE_FRAMES + WINDOW + 16, tokens_per_frame=TPF,
                                       num_heads=HEADS, head_dim=HEAD_DIM, dtype=torch.bfloat16, device=dev,
                                       num_special_tokens=NSPECIAL, scale_frames=SCALE_FRAMES, sliding_window=WINDOW,
                                       max_total_frames=n_cached + 100)
        for t in range(n_cached):
            ref.append_frame(0, kf[t % 8], vf[t % 8])
            ref.evict_frames(0, SCALE_FRAMES, WINDOW)
        assert list(ref.build_visible_page_table(0)) == m.build_visible_page_table(0)
        fi = ref.compute_attention(0, q)                                   # plans (block 0) and runs
        run_fi = lambda: ref.prefill_wrapper.run(q=q, paged_kv_cache=ref.kv_caches[0])   # the run() half alone
        fi_us = time_us(run_fi)
        rec.update({"flashinfer_layer_us": fi_us, "ratio": fi_us / b200_us,
                    "flashinfer_tflops": 4.0 * TPF * kv * HEAD_DIM * HEADS / fi_us / 1e6,
                    "how": "reference FlashInferKVCacheManager from baseline/_ref, backend fa2: plan once, "
                           f"prefill_wrapper.run timed over {repeats} launches with CUDA events; same page table and K/V"})
        par["vs_flashinfer_bf16"] = {"elements": int(fi.numel()), "max_abs": float((ours.float() - fi.float()).abs().max()),
                                     "cosine": _cos64(ours, fi)}
        del ref
    except Exception as e:                                                   # noqa: BLE001
        rec["flashinfer"] = "unavailable: %s: %s" % (type(e).__name__, str(e)[:200])
    out["flashinfer_layer"], out["parity_at_headline"] = rec, par
    del m
    torch.cuda.empty_cache()
    return out


def whole_model_record(args):
    """Whole GCTStream model (reference code from baseline/_ref) at the 10k-frame cache: frames/s with this backend
    and with the reference's FlashInfer backend, each in its own process (bench_model.py)."""
    if not os.path.isdir(REF_DIR):
        return {"unavailable": "baseline/_ref is not installed"}
    rec = {"frames_timed": args.whole_model_frames, "cached_frames": args.frames_cached,
           "how": "bench_model.py: the reference's gct_profile.py model (random init, torch.compile as it does), "
                  "bf16 autocast, 378x518, cache pre-filled through the manager's own append_frame"}
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, REF_DIR, env.get("PYTHONPATH", "")])
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    for backend in ("b200", "flashinfer"):
        cmd = [sys.executable, os.path.join(ROOT, "bench_model.py"), "--reference", REF_DIR, "--backend", backend,
               "--cached-frames", str(args.frames_cached), "--frames", str(args.whole_model_frames)]
        try:
            r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.whole_model_timeout)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            if r.returncode != 0 or not lines:
                rec[backend] = {"unavailable": "exit %d: %s" % (r.returncode, (r.stderr or r.stdout)[-300:])}
                continue
            d = json.loads(lines[-1])
            rec[backend + "_fps"] = d["frames_per_s_median"]
            rec[backend + "_ms_per_frame"] = d["ms_per_frame_median"]
        except subprocess.TimeoutExpired:
            rec[backend] = {"unavailable": "timed out after %d s" % args.whole_model_timeout}
    if "b200_fps" in rec and "flashinfer_fps" in rec:
        rec["ratio"] = rec["b200_fps"] / rec["flashinfer_fps"]
    return rec


# ----------------------------------------------------------------------------- CPU arm
def _reference_layers():
    """The reference's own SDPAAttention / Attention modules (global and frame layer) from baseline/_ref, or None."""
    try:
        if not os.path.isdir(REF_DIR):
            return None
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from lingbot_map.layers.attention import Attention, SDPAAttention
        from lingbot_map.layers.rope import PositionGetter, RotaryPositionEmbedding2D, WanRotaryPosEmbed
        return Attention, SDPAAttention, PositionGetter, RotaryPositionEmbedding2D, WanRotaryPosEmbed
    except Exception:                                                        # noqa: BLE001
        return None


class CpuLayerPair:
    """One global layer + one frame layer of one streaming frame on the host cores, at the n_cached-frame steady
    state.  kind "reference": the reference's own SDPAAttention (dict KV cache: cat, evict, clone, SDPA; with its
    qkv/proj Linears, 1.5 % of the layer's flops) and Attention modules, imported from baseline/_ref.
    kind "port": oracle/sdpa_port.py, the CPU restatement, when the reference package is not installed."""

    def __init__(self, n_cached, threads):
        torch.set_num_threads(threads)
        self.n_cached, self.threads = n_cached, threads
        g = torch.Generator().manual_seed(1)
        self.rn = rn = lambda *s: torch.randn(*s, generator=g)
        C = HEADS * HEAD_DIM
        n_ev = max(n_cached - SCALE_FRAMES - WINDOW, 0)
        full = min(n_cached, SCALE_FRAMES + WINDOW)
        self.k = rn(1, HEADS, full, TPF, HEAD_DIM)
        self.v = rn(1, HEADS, full, TPF, HEAD_DIM)
        self.ks = rn(1, HEADS, n_ev, NSPECIAL, HEAD_DIM)
        self.vs = rn(1, HEADS, n_ev, NSPECIAL, HEAD_DIM)
        ref = _reference_layers()
        self.kind = "reference" if ref is not None else "port"
        if ref is not None:
            Attention, SDPAAttention, PositionGetter, Rope2D, Wan = ref
            torch.manual_seed(0)
            self.glob = SDPAAttention(dim=C, num_heads=HEADS, qk_norm=True, rope=object(),
                                      kv_cache_sliding_window=WINDOW, kv_cache_scale_frames=SCALE_FRAMES).eval()
            self.frame = Attention(dim=C, num_heads=HEADS, qk_norm=True, rope=Rope2D(frequency=100)).eval()
            self.pos3d = Wan(attention_head_dim=HEAD_DIM, patch_size=(1, 14, 14), max_seq_len=1024)(
                ppf=1, pph=PPH, ppw=PPW, patch_start_idx=NSPECIAL, device=torch.device("cpu"),
                f_start=n_cached % 1024, f_end=n_cached % 1024 + 1)
            pos = PositionGetter()(1, PPH, PPW, device=torch.device("cpu")) + 1
            self.pos2d = torch.cat([torch.zeros(1, NSPECIAL, 2, dtype=pos.dtype), pos], dim=1)
            self.x = rn(1, TPF, C)
        else:
            from oracle import sdpa_port as SP
            self.SP = SP
            self.params = {"qkv.weight": None, "qkv.bias": None, "proj.weight": None, "proj.bias": None,
                           "q_norm.weight": 1 + 0.1 * rn(64), "q_norm.bias": 0.1 * rn(64),
                           "k_norm.weight": 1 + 0.1 * rn(64), "k_norm.bias": 0.1 * rn(64)}
            self.qkv = rn(1, TPF, 3 * C)
            self.cos, self.sin = SP.rope3d_cos_sin(n_cached % 1024, 1, PPH, PPW, NSPECIAL)

    def sample(self):
        """Seconds for the pair; the cache state is rebuilt (views of the same storage) before every sample."""
        import torch.nn.functional as F
        if self.kind == "reference":
            cache = {"k_0": self.k, "v_0": self.v, "k_0_special": self.ks, "v_0_special": self.vs}
            t0 = time.perf_counter()
            with torch.no_grad():
                self.glob(self.x, pos=self.pos3d, enable_3d_rope=True, kv_cache=cache, global_idx=0,
                          num_frame_per_block=1, num_register_tokens=4)          # attention.py:595-670
                self.frame(self.x, pos=self.pos2d)                               # attention.py:65-87
            return time.perf_counter() - t0
        SP, params = self.SP, self.params
        port = SP.SdpaStreamPort(params, HEADS, SCALE_FRAMES, WINDOW, NSPECIAL)
        port.k, port.v, port.k_special, port.v_special = self.k, self.v, self.ks, self.vs

        def split(t):
            q, k, v = t.reshape(1, TPF, 3, HEADS, HEAD_DIM).permute(2, 0, 3, 1, 4).unbind(0)
            q = F.layer_norm(q, (HEAD_DIM,), params["q_norm.weight"], params["q_norm.bias"], 1e-5)
            k = F.layer_norm(k, (HEAD_DIM,), params["k_norm.weight"], params["k_norm.bias"], 1e-5)
            return q, k, v

        t0 = time.perf_counter()
        with torch.no_grad():
            q, k, v = split(self.qkv)                               # global layer (attention.py:601-670, minus Linears)
            q, k = SP.apply_rope3d(q, self.cos, self.sin), SP.apply_rope3d(k, self.cos, self.sin)
            port.attend(q, k, v, 1)
            q, k, v = split(self.qkv)                               # frame layer (attention.py:65-84, minus Linears)
            q, k = SP.apply_rope3d(q, self.cos, self.sin), SP.apply_rope3d(k, self.cos, self.sin)   # same cost as 2-D
            F.scaled_dot_product_attention(q, k, v)
        return time.perf_counter() - t0

    def describe(self):
        what = ("the reference's SDPAAttention.forward + Attention.forward from baseline/_ref (fp32, dict cache "
                "cat/evict/clone + SDPA, Linears included)") if self.kind == "reference" else \
               "oracle/sdpa_port.py (CPU restatement of the reference's SDPA path, Linears excluded)"
        return (f"1 of {DEPTH} layer pairs (global attention over kv={visible_kv(self.n_cached + 1)} + frame attention "
                f"1005x1005) x{DEPTH} per frame; {what}; torch CPU, {self.threads} threads")


def cpu_baseline(max_seconds=25.0, n_cached=10000):
    threads = os.cpu_count() or 1
    pair = CpuLayerPair(n_cached, threads)
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 and (not times or time.perf_counter() - t_start + times[-1] < max_seconds):
        times.append(pair.sample())
    best = min(times)
    return {"value": 1.0 / (DEPTH * best), "unit": UNIT, "cores": threads, "kind": pair.kind,
            "sample": pair.describe() + f", best of {len(times)}", "seconds_per_sample": best}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    pair = CpuLayerPair(args.frames_cached, threads)
    for _ in range(min(args.warmup, 1)):
        pair.sample()
    steps = min(args.steps, 8)            # each step is a bounded sample: 1 of 24 layer pairs
    t = [pair.sample() for _ in range(steps)]
    per_frame = DEPTH * (sum(t) / len(t))
    value = 1.0 / per_frame
    cb = {"value": value, "unit": UNIT, "cores": threads, "kind": pair.kind,
          "sample": pair.describe() + f"; {steps} steps timed (capped at 8 to stay within minutes)"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": per_frame * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "the reference's CPU (SDPA dict-cache) streaming path, same frame geometry and "
                               f"{args.frames_cached}-frame cache state as the GPU arm", "cores": threads},
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    global DEPTH, SCALE_FRAMES, WINDOW
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=160)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="streams", choices=["streams", "kvsplit"])
    ap.add_argument("--streams-per-gpu", type=int, default=1,
                    help="independent streams per GPU, interleaved step by step on one CUDA stream")
    ap.add_argument("--frames-cached", type=int, default=10000)
    ap.add_argument("--keyframe-interval", type=int, default=1,
                    help="every K-th streamed frame is a keyframe; the others are appended, attended over and rolled "
                         "back (the 10,000-frame / interval-5 configuration holds 2,007 keyframes: --frames-cached 2007)")
    ap.add_argument("--e2e-steps", type=int, default=0,
                    help="timed steps of the end-to-end pass (0: as many as --steps, so that both passes see the same "
                         "clocks under the power cap)")
    ap.add_argument("--kernel-steps", type=int, default=20,
                    help="steps of the second pass that brackets every attention launch with CUDA events")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-flashinfer", action="store_true", help="skip the same-box FlashInfer layer timing + parity record")
    ap.add_argument("--no-whole-model", action="store_true", help="skip the whole-model frames/s of both backends")
    ap.add_argument("--no-kvsplit", action="store_true", help="N > 1: skip the KV-sharded single-stream sub-record")
    ap.add_argument("--kvsplit-timeout", type=int, default=240,
                    help="N > 1: seconds after which the line is printed without the KV-sharded sub-record")
    ap.add_argument("--whole-model-frames", type=int, default=40)
    ap.add_argument("--whole-model-timeout", type=int, default=420)
    ap.add_argument("--exact-softmax", action="store_true",
                    help="force the attention instantiation that tracks the running row maximum (bounded mode off)")
    ap.add_argument("--scale-frames", type=int, default=SCALE_FRAMES,
                    help="anchor frames kept for ever (metric: 8; the single-layer microbenchmark uses 1)")
    ap.add_argument("--window", type=int, default=WINDOW,
                    help="sliding window of full frames (metric: 64; the single-layer microbenchmark uses 16)")
    ap.add_argument("--layers", type=int, default=24,
                    help="aggregator depth; the metric is defined at 24, smaller values are for profiler captures")
    args = ap.parse_args()
    if args.e2e_steps <= 0:
        args.e2e_steps = args.steps
    DEPTH = args.layers
    SCALE_FRAMES, WINDOW = args.scale_frames, args.window
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path for the product")
        run_gpu(args)


if __name__ == "__main__":
    main()
