"""Pin the CPU oracle against fixtures produced by the reference implementation itself."""
import gzip
import json
import os

import numpy as np
import pytest

import seeded
from oracle import gct_oracle as O

G = os.path.join(os.path.dirname(__file__), "golden")


def _load_traces():
    with gzip.open(os.path.join(G, "manager_traces.json.gz"), "rt") as f:
        return json.load(f)


TRACES = _load_traces()


def apply_op(m, op, geo):
    if op == "append":
        m.append_frame(0)
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
    else:
        raise ValueError(op)


@pytest.mark.parametrize("case", TRACES, ids=[c["name"] for c in TRACES])
def test_manager_trace_bit_exact(case):
    geo = case["geometry"]
    m = O.PagedCacheOracle(1, geo["tokens_per_frame"], 1, 8, scale_frames=geo["scale_frames"],
                           sliding_window=geo["sliding_window"], max_total_frames=geo["max_total_frames"],
                           store=False)
    assert (m.page_size, m.max_patch_pages, m.max_num_pages) == (
        geo["page_size"], geo["max_patch_pages"], geo["max_num_pages"])
    snaps = {s["op_index"]: s for s in case["snapshots"]}
    for i, op in enumerate(case["ops"]):
        apply_op(m, op, geo)
        if i in snaps:
            got = m.snapshot(0)
            want = {k: v for k, v in snaps[i].items() if k != "op_index"}
            assert got == want, f"{case['name']} op {i} ({op})"


def test_sanity_check_known_answers():
    """The numbers the reference's _sanity_check asserts (flashinfer_cache.py:616-631)."""
    m = O.PagedCacheOracle(2, 262, 16, 64, scale_frames=8, sliding_window=64, max_total_frames=200, store=False)
    for b in range(2):
        for _ in range(100):
            m.append_frame(b)
            m.evict_frames(b, 8, 64)
        assert len(m.scale_pages[b]) == 8 and len(m.window_pages[b]) == 64
        assert len(m.special_pages[b]) == 3 and m.special_token_count[b] == 600
        assert m.compute_last_page_len(b) == 600 % 256
        vis = m.build_visible_page_table(b)
        assert all(p < m.max_patch_pages for p in vis[:72]) and all(p >= m.max_patch_pages for p in vis[72:])
    m.reset()
    assert m.frame_count[0] == 0


def test_paged_attention_values():
    z = np.load(os.path.join(G, "paged_attention_fp32.npz"))
    meta = json.loads(bytes(z["meta_json"]).decode())
    for name, g in meta.items():
        tpf, H = g["tokens_per_frame"], g["heads"]
        m = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=g["scale"], sliding_window=g["window"],
                               max_total_frames=g["max_total"])
        vs = g["value_scale"]
        for t in range(g["frames"] + 1):
            k = seeded.randn(1000 + t, tpf, H, 64, scale=vs)
            v = seeded.randn(2000 + t, tpf, H, 64, scale=vs)
            q = seeded.randn(3000 + t, tpf, H, 64, scale=vs)
            nonkf = t == g["frames"]
            if nonkf:
                m._defer_eviction = True
            m.append_frame(0, k, v)
            m.evict_frames(0, g["scale"], g["window"])
            key = f"{name}_out_nonkf" if nonkf else f"{name}_out_{t}"
            if key in z:
                got = m.compute_attention(0, q)
                assert np.abs(got - z[key]).max() < 5e-6, key
            if nonkf:
                m.rollback_last_frame(0)
                m._defer_eviction = False
        assert m.build_visible_page_table(0) == list(z[f"{name}_visible_end"])


def test_prepare_qkv_values():
    z = np.load(os.path.join(G, "prepare_qkv_fp32.npz"))
    H, pph, ppw, ns = 2, 3, 4, 6
    w = {n: seeded.param_value(7, n, (64,)) for n in ("q_norm.weight", "q_norm.bias", "k_norm.weight", "k_norm.bias")}
    for f in (0, 5, 41):
        q, k, v = O.prepare_qkv(z[f"rope3d_f{f}_qkv"], H, w["q_norm.weight"], w["q_norm.bias"], w["k_norm.weight"],
                                w["k_norm.bias"], rope="3d", f=f, pph=pph, ppw=ppw, num_special=ns)
        for got, key in ((q, "q"), (k, "k"), (v, "v")):
            assert np.abs(got - z[f"rope3d_f{f}_{key}"]).max() < 2e-5, (f, key)
    assert (O.positions_2d(pph, ppw, ns) == z["rope2d_pos"]).all()
    q, k, v = O.prepare_qkv(z["rope2d_qkv"], H, w["q_norm.weight"], w["q_norm.bias"], w["k_norm.weight"],
                            w["k_norm.bias"], rope="2d", pph=pph, ppw=ppw, num_special=ns)
    for got, key in ((q, "q"), (k, "k"), (v, "v")):
        assert np.abs(got - z[f"rope2d_{key}"]).max() < 2e-5, key


def test_frame_attention_values():
    """Attention.forward (attention.py:65-87) incl. qkv and proj Linear, restated with the oracle pieces."""
    z = np.load(os.path.join(G, "prepare_qkv_fp32.npz"))
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    N = ns + pph * ppw
    P = lambda n, s: seeded.param_value(11, n, s).astype(np.float64)
    x = seeded.randn(123, 2, N, dim).astype(np.float64)
    Wqkv, bqkv = P("qkv.weight", (3 * dim, dim)), P("qkv.bias", (3 * dim,))
    Wp, bp = P("proj.weight", (dim, dim)), P("proj.bias", (dim,))
    for b in range(2):
        qkv = x[b] @ Wqkv.T + bqkv
        q, k, v = O.prepare_qkv(qkv, H, P("q_norm.weight", (64,)), P("q_norm.bias", (64,)),
                                P("k_norm.weight", (64,)), P("k_norm.bias", (64,)),
                                rope="2d", pph=pph, ppw=ppw, num_special=ns)
        o, _ = O.attention(q, k, v)
        y = o.reshape(N, dim) @ Wp.T + bp
        assert np.abs(y - z["frame_attn_out"][b]).max() < 2e-5


def test_merge_partials_matches_single_pass():
    rs = np.random.RandomState(5)
    q, k, v = (rs.standard_normal((33, 3, 64)) for _ in range(3))
    k = rs.standard_normal((301, 3, 64))
    v = rs.standard_normal((301, 3, 64))
    full, lse = O.attention(q, k, v)
    cuts = [0, 17, 128, 129, 301]
    parts = [O.attention(q, k[a:b], v[a:b]) for a, b in zip(cuts[:-1], cuts[1:])]
    out, l2 = O.merge_partials([p[0] for p in parts], [p[1] for p in parts])
    assert np.abs(out - full).max() < 1e-12 and np.abs(l2 - lse).max() < 1e-12


def test_bf16_round():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 0.0, 65504.0], np.float32)
    r = O.bf16_round(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625)   # ties to even, then up
    assert (O.bf16_from_bits(O.bf16_bits(x)) == r).all()
    import torch
    t = torch.from_numpy(seeded.randn(3, 4096))
    assert (t.to(torch.bfloat16).float().numpy() == O.bf16_round(t.numpy())).all()
