"""KV-sharded single stream on real GPUs (needs at least two; skipped otherwise): one process per GPU over NCCL,
every rank holds the same replicated cache, attends over its slice of the visible pages and takes part in the peer
exchange kernel; the merged result on every rank is compared with the single-pass attention over the whole page list.

Ranks are child processes; NVLink multicast is switched off in every library used (NCCL_NVLS_ENABLE=0, the symmetric
memory allocator without multicast) and the exchange kernel uses plain peer loads and stores."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason="needs at least two GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1", LINGBOT_B200_KV_EXCHANGE=mode)
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import lingbot_map_b200 as P
        from lingbot_map_b200 import distributed as D
        tpf, H, blocks = 306, 4, 2
        m = P.B200KVCacheManager(blocks, 48, tpf, H, 64, device=dev, scale_frames=2, sliding_window=5, max_total_frames=200)
        g = torch.Generator(device=dev).manual_seed(77)              # same seed: replicated cache contents
        rn = lambda *s: torch.randn(*s, device=dev, generator=g).to(torch.bfloat16)
        worst_abs, worst_cos = 0.0, 1.0
        for frame in range(12):                                       # the visible list grows from 1 page: empty slices first
            outs, qs = [], []
            for b in range(blocks):
                k, v, q = rn(tpf, H, 64), rn(tpf, H, 64), rn(tpf, H, 64)
                m.append_frame(b, k, v)
                m.evict_frames(b, 2, 5)
                outs.append(D.sharded_attention(m, b, q, rank, world).clone())
                qs.append(q)
            for b in range(blocks):
                m.plan()
                full = m.compute_attention(b, qs[b]) if b == 0 else m.compute_attention(b, qs[b])
                a, c = outs[b].double().flatten(), full.double().flatten()
                worst_abs = max(worst_abs, float((a - c).abs().max()))
                worst_cos = min(worst_cos, float(a @ c / (a.norm() * c.norm())))
            m._shard_plan = None
        used_peer = getattr(m, "_peer_exchange", None) is not None
        ret[rank] = (worst_abs, worst_cos, m.device_status(), used_peer)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["peer", "allgather"])
def test_kv_sharded_attention_matches_single_pass(mode):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        worst_abs, worst_cos, status, used_peer = ret[r]
        assert status == 0
        assert worst_abs <= 1e-2 and worst_cos >= 0.99999, f"rank {r}: max_abs={worst_abs:.3e} cosine={worst_cos:.7f}"
        if mode == "peer":
            assert used_peer, "the peer exchange was not set up (symmetric memory unavailable?)"


def test_one_process_drives_two_gpus():
    """The shared-memory opt-in of the attention kernels and the SM count are per-device state: a process that has
    used GPU 0 must be able to launch the 2-tile kernel (176 KB of dynamic shared memory) on GPU 1 as well.  Small
    cases only: dense attention with one and two query tiles per CTA, and a paged call through a manager."""
    import numpy as np
    sys.path.insert(0, ROOT)
    import lingbot_map_b200 as P
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        g = torch.Generator().manual_seed(3)                          # host generator: identical inputs on both devices
        q = torch.randn(1, 300, 4, 64, generator=g).to(dev).to(torch.bfloat16)
        k = torch.randn(1, 700, 4, 64, generator=g).to(dev).to(torch.bfloat16)
        small = P.ops.dense_attention(q[:, :100], k, k)               # one tile per CTA
        big = P.ops.dense_attention(q, k, k)                          # two tiles per CTA
        ref = torch.nn.functional.scaled_dot_product_attention(q.float().permute(0, 2, 1, 3), k.float().permute(0, 2, 1, 3),
                                                               k.float().permute(0, 2, 1, 3)).permute(0, 2, 1, 3)
        assert float((big.float() - ref).abs().max()) < 2e-2 and float((small.float() - ref[:, :100]).abs().max()) < 2e-2
        m = P.B200KVCacheManager(1, 21, 262, 2, 64, device=dev, scale_frames=2, sliding_window=3, max_total_frames=40)
        kv = torch.randn(262, 2, 64, generator=g).to(dev)
        for _ in range(4):
            m.append_frame(0, kv, kv)
            m.evict_frames(0, 2, 3)
        out = m.compute_attention(0, kv.to(torch.bfloat16))
        assert torch.isfinite(out).all() and m.device_status() == 0 and P.ops.device_status(dev) == 0
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])                              # same seeds, same arithmetic on both devices
