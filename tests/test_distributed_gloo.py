"""The KV-sharded path on CPU ranks (gloo, world_size 2 and 3): page-range sharding, the packed
[O | lse] record exchange, and the merge math against single-pass attention from the oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_pages, page, last_len, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lingbot_map_b200 import distributed as D
        from oracle import gct_oracle as O
        import seeded
        n_q, H = 37, 3
        kv_len = (n_pages - 1) * page + last_len
        q, k, v = seeded.randn(1, n_q, H, 64), seeded.randn(2, kv_len, H, 64), seeded.randn(3, kv_len, H, 64)
        lo, hi = D.shard_page_range(n_pages, rank, world)
        local = torch.empty(D.record_floats(n_q, H), dtype=torch.float32)
        n = n_q * H * 64
        if hi > lo:
            t0, t1 = lo * page, min(hi * page, kv_len)
            o, lse = O.attention(q, k[t0:t1], v[t0:t1])
            local[:n] = torch.from_numpy(o.astype(np.float32).ravel())
            local[n:] = torch.from_numpy(lse.astype(np.float32).ravel())
        else:
            D.pack_empty_record(local, n_q, H)
        rec = D.gather_records(local, world)
        merged = D.merge_records_reference(rec, n_q, H).numpy()
        full, _ = O.attention(q, k, v)
        err = float(np.abs(merged - full).max())
        # the two-phase peer exchange (rows owned in slices: partials to the owner, merged slices to everybody)
        two_phase = D.exchange_host_model(local, n_q, H, rank, world).numpy()
        err = max(err, float(np.abs(two_phase - full).max()))
        # every rank must hold the same records
        chk = rec.double().sum().reshape(1)
        lst = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(lst, chk)
        same = all(float(x) == float(lst[0]) for x in lst)
        ret[rank] = (err, same, (lo, hi))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_pages,last_len", [(2, 9, 13), (2, 1, 20), (3, 7, 50), (3, 2, 50)])
def test_sharded_merge_on_gloo_ranks(world, n_pages, last_len):
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, n_pages, 50, last_len, ret), nprocs=world, join=True)
    assert len(ret) == world
    covered = []
    for r in range(world):
        err, same, (lo, hi) = ret[r]
        assert err < 1e-5 and same
        covered += list(range(lo, hi))
    assert covered == list(range(n_pages))        # every page owned exactly once, in order


def test_shard_page_range_properties():
    sys.path.insert(0, ROOT)
    from lingbot_map_b200 import distributed as D
    for n in (0, 1, 5, 72, 133, 1000):
        for w in (1, 2, 4, 8):
            spans = [D.shard_page_range(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        D.shard_page_range(4, 2, 2)
    # row slices of the peer exchange: contiguous, complete, balanced, and never larger than the receive slots
    for rows in (1, 7, 1005 * 16, 37 * 3):
        for w in (1, 2, 3, 8):
            spans = [D.row_slice(rows, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) <= (rows + w - 1) // w
