"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the reference's golden outputs.

Tolerances (bf16 operands, fp32 accumulation): max-abs 2e-2 and cosine >= 0.9999 in float64 against the
float64 oracle evaluated on the same bf16-rounded inputs."""
import json
import os

import numpy as np
import pytest
import torch

import seeded
import lingbot_map_b200 as P
from lingbot_map_b200 import _lib
from oracle import gct_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def cosine64(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def assert_close(got, want, tag, max_abs=2e-2, cos=0.9999):
    got = got.float().cpu().numpy() if torch.is_tensor(got) else got
    d = float(np.abs(got.astype(np.float64) - want).max())
    c = cosine64(got, want)
    assert np.isfinite(got).all(), tag
    assert d <= max_abs and c >= cos, f"{tag}: max_abs={d:.3e} cosine={c:.7f}"


def bf(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(torch.bfloat16)


def r(x):
    return O.bf16_round(x).astype(np.float64)


# ---------------------------------------------------------------- paged attention vs reference goldens
@pytest.mark.parametrize("name", ["p20", "p150", "p300"])
@pytest.mark.parametrize("kdtype", ["bf16", "f32"])
def test_paged_attention_golden(name, kdtype):
    z = np.load(os.path.join(G, "paged_attention_fp32.npz"))
    g = json.loads(bytes(z["meta_json"]).decode())[name]
    tpf, H, vs = g["tokens_per_frame"], g["heads"], g["value_scale"]
    m = P.B200KVCacheManager(1, g["scale"] + g["window"] + 16, tpf, H, 64, device=DEV, scale_frames=g["scale"],
                             sliding_window=g["window"], max_total_frames=g["max_total"])
    orc = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=g["scale"], sliding_window=g["window"],
                             max_total_frames=g["max_total"])
    for t in range(g["frames"] + 1):
        k = seeded.randn(1000 + t, tpf, H, 64, scale=vs)
        v = seeded.randn(2000 + t, tpf, H, 64, scale=vs)
        q = seeded.randn(3000 + t, tpf, H, 64, scale=vs)
        nonkf = t == g["frames"]
        if nonkf:
            m._defer_eviction = True
            orc._defer_eviction = True
        if kdtype == "bf16":
            m.append_frame(0, bf(k), bf(v))
            qd = bf(q)
        else:   # fp32 K and q, bf16 V: what arrives under autocast
            m.append_frame(0, torch.from_numpy(k).to(DEV), bf(v))
            qd = torch.from_numpy(q).to(DEV)
        m.evict_frames(0, g["scale"], g["window"])
        orc.append_frame(0, r(k), r(v))
        orc.evict_frames(0, g["scale"], g["window"])
        assert m.build_visible_page_table(0) == orc.build_visible_page_table(0)
        assert m.compute_last_page_len(0) == orc.compute_last_page_len(0)
        out = m.compute_attention(0, qd)
        assert out.dtype == torch.bfloat16 and tuple(out.shape) == (tpf, H, 64)
        want = orc.compute_attention(0, r(q))
        assert_close(out, want, f"{name} frame {t} vs oracle", max_abs=2e-2 * max(vs, 0.05))
        key = f"{name}_out_nonkf" if nonkf else f"{name}_out_{t}"
        if key in z:
            # The reference's own fp32 result, computed on the UNROUNDED inputs.  This leg therefore also carries the
            # bf16 rounding of q, k and v themselves (relative 2^-9 each, independent per element), which the oracle
            # leg above removes by rounding its inputs the same way.  With outputs that are averages of about a hundred
            # v rows the rounding of v alone gives 1 - cosine ~ (2^-9)^2 / 3 = 1.3e-6 and the perturbed softmax weights
            # a few times that; 0.9999 holds with margin once the bf16 output rounding (another 1.3e-6) is added.
            assert_close(out, z[key].astype(np.float64), f"{name} frame {t} vs reference", cos=0.9999)
        if nonkf:
            m.rollback_last_frame(0)
            orc.rollback_last_frame(0)
            m._defer_eviction = False
    assert m.build_visible_page_table(0) == list(z[f"{name}_visible_end"])
    # page contents are bit-exact bf16 roundings of what was appended
    kk, vv = m._gather_kv(0)
    ok, ov = orc.gather_kv(0)
    assert (kk.float().cpu().numpy() == ok.astype(np.float32)).all()
    assert (vv.float().cpu().numpy() == ov.astype(np.float32)).all()
    assert m.device_status() == 0


def test_empty_cache_returns_zeros():
    m = P.B200KVCacheManager(1, 21, 26, 2, 64, device=DEV, scale_frames=2, sliding_window=3, max_total_frames=40)
    q = torch.randn(26, 2, 64, device=DEV)
    out = m.compute_attention(0, q)
    assert out.shape == q.shape and float(out.abs().max()) == 0.0       # flashinfer_cache.py:368-370


def test_plan_is_reused_across_blocks_and_lse():
    """plan at block 0, run on every block (flashinfer_cache.py:385-421); lse output; partial + merge."""
    tpf, H = 140, 3
    m = P.B200KVCacheManager(3, 21, tpf, H, 64, device=DEV, scale_frames=1, sliding_window=2, max_total_frames=60)
    orcs = O.PagedCacheOracle(3, tpf, H, 64, scale_frames=1, sliding_window=2, max_total_frames=60)
    for t in range(7):
        for b in range(3):
            k, v = seeded.randn(10 * t + b, tpf, H, 64), seeded.randn(500 + 10 * t + b, tpf, H, 64)
            m.append_frame(b, bf(k), bf(v))
            m.evict_frames(b, 1, 2)
            orcs.append_frame(b, r(k), r(v))
            orcs.evict_frames(b, 1, 2)
    for b in range(3):
        q = seeded.randn(900 + b, tpf, H, 64)
        out, lse = m.compute_attention(b, bf(q), return_lse=True)
        kk, vv = orcs.gather_kv(b)
        want, wl = O.attention(r(q), kk, vv)
        assert_close(out, want, f"block {b}")
        assert np.abs(lse.cpu().numpy() - wl).max() < 2e-3
    # KV-sharded: two page sub-ranges, partial results merged by log-sum-exp
    q = seeded.randn(77, tpf, H, 64)
    n = len(m.build_visible_page_table(0))
    parts, lses = [], []
    for lo, hi in ((0, 2), (2, n)):
        m.plan(lo, hi)
        o, l = m.compute_attention_partial(1, bf(q))
        parts.append(o)
        lses.append(l)
    merged = P.ops.lse_merge(torch.stack(parts), torch.stack(lses))
    kk, vv = orcs.gather_kv(1)
    assert_close(merged, O.attention(r(q), kk, vv)[0], "sharded merge")
    assert m.device_status() == 0


# ---------------------------------------------------------------- dense attention
@pytest.mark.parametrize("B,Nq,Nkv,H", [(1, 1, 1, 1), (1, 6, 130, 2), (2, 130, 257, 3), (1, 1005, 1005, 2),
                                         (3, 37, 128, 1), (1, 300, 2600, 2)])
def test_dense_attention_vs_oracle(B, Nq, Nkv, H):
    q, k, v = seeded.randn(1, B, Nq, H, 64), seeded.randn(2, B, Nkv, H, 64), seeded.randn(3, B, Nkv, H, 64)
    out = P.ops.dense_attention(bf(q), bf(k), bf(v))
    for b in range(B):
        assert_close(out[b], O.attention(r(q[b]), r(k[b]), r(v[b]))[0], f"dense b={b}")
    assert P.ops.device_status(DEV) == 0


def test_dense_attention_strided_views():
    """q/k/v as views into one qkv buffer [B, N, 3, H, 64] (the layout the qkv Linear produces)."""
    B, N, H = 2, 200, 4
    qkv = seeded.randn(9, B, N, 3, H, 64)
    t = bf(qkv)
    out = P.ops.dense_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2])
    for b in range(B):
        assert_close(out[b], O.attention(r(qkv[b, :, 0]), r(qkv[b, :, 1]), r(qkv[b, :, 2]))[0], f"strided b={b}")


def test_dense_attention_peaked_softmax():
    """Large logits (|s| up to ~60): running-max rescaling must hold."""
    Nq, Nkv, H = 140, 700, 2
    q, k, v = seeded.randn(4, 1, Nq, H, 64, scale=3.0), seeded.randn(5, 1, Nkv, H, 64, scale=3.0), seeded.randn(6, 1, Nkv, H, 64)
    out = P.ops.dense_attention(bf(q), bf(k), bf(v))
    # With logits of +-60 the softmax is nearly one-hot: an output row is (almost) a single v row, |v| up to ~4.
    # The result is stored as bf16, whose spacing at magnitude 2..4 is 2^-6 = 1.6e-2, so two results that differ by
    # one rounding step are already 1.6e-2 apart; and the weights P are rounded to bf16 before the PV product
    # (relative 2^-9 on the dominant weight, i.e. up to 4 * 2^-9 = 8e-3 on the output).  Bound: one output rounding
    # step + the weight rounding = 2.4e-2, stated as 2.5e-2; the cosine keeps the common 0.9999.
    assert_close(out[0], O.attention(r(q[0]), r(k[0]), r(v[0]))[0], "peaked", max_abs=2.5e-2, cos=0.9999)


# ---------------------------------------------------------------- fused prologue / append
def _norm_params(seed):
    names = ("q_norm.weight", "q_norm.bias", "k_norm.weight", "k_norm.bias")
    w = [seeded.param_value(seed, n, (64,)) for n in names]
    return w, [torch.from_numpy(x).to(DEV) for x in w]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_prep_qkv_golden(dtype):
    z = np.load(os.path.join(G, "prepare_qkv_fp32.npz"))
    H, pph, ppw, ns = 2, 3, 4, 6
    w, wd = _norm_params(7)
    tol = dict(max_abs=3e-2, cos=0.9999)
    for f in (0, 5, 41):
        qkv = z[f"rope3d_f{f}_qkv"]
        src = torch.from_numpy(qkv).to(DEV) if dtype == "f32" else bf(qkv)
        cs = P.ops.rope3d_table(f, pph, ppw, ns, DEV)
        ang = O.rope3d_angles(f, pph, ppw, ns)
        assert np.abs(cs[..., 0].cpu().numpy() - np.cos(ang)).max() < 1e-6
        assert np.abs(cs[..., 1].cpu().numpy() - np.sin(ang)).max() < 1e-6
        q, k, v = P.ops.prep_qkv(src, H, ns + pph * ppw, *wd, cs, _lib.ROPE_3D)
        if dtype == "f32":   # reference result on the same fp32 input, rounded once to bf16
            for got, key in ((q, "q"), (k, "k"), (v, "v")):
                assert_close(got, z[f"rope3d_f{f}_{key}"].astype(np.float64), f"3d f={f} {key}", **tol)
                ulp = np.abs(got.float().cpu().numpy() - O.bf16_round(z[f"rope3d_f{f}_{key}"]))
                assert (ulp <= np.abs(z[f"rope3d_f{f}_{key}"]) * 2 ** -7 + 1e-6).all()
        else:
            wq, wk, wv = O.prepare_qkv(r(qkv), H, *w, rope="3d", f=f, pph=pph, ppw=ppw, num_special=ns)
            for got, want, key in ((q, wq, "q"), (k, wk, "k"), (v, wv, "v")):
                assert_close(got, want, f"3d bf16 f={f} {key}", **tol)
    qkv = z["rope2d_qkv"]
    cs = P.ops.rope2d_table(pph, ppw, ns, DEV)
    q, k, v = P.ops.prep_qkv(torch.from_numpy(qkv).to(DEV), H, ns + pph * ppw, *wd, cs, _lib.ROPE_2D)
    for got, key in ((q, "q"), (k, "k"), (v, "v")):
        assert_close(got, z[f"rope2d_{key}"].astype(np.float64), f"2d {key}", **tol)


def test_append_fused_equals_prep_then_append():
    """Fused LayerNorm+RoPE+page write == prep_qkv followed by append_frame, bit for bit, incl. a special
    run that straddles two special pages."""
    H, pph, ppw, ns = 2, 3, 4, 6
    tpf = ns + pph * ppw                      # 18 tokens, page 12: specials straddle at frame 2 (12 = 2*6), 3...
    w, wd = _norm_params(3)
    kw = dict(device=DEV, scale_frames=1, sliding_window=2, max_total_frames=30)
    a = P.B200KVCacheManager(1, 19, tpf, H, 64, **kw)
    b = P.B200KVCacheManager(1, 19, tpf, H, 64, **kw)
    a2 = P.B200KVCacheManager(1, 19, 11, H, 64, num_special_tokens=4, **kw)   # page 7, 4 specials: 7 % 4 != 0
    b2 = P.B200KVCacheManager(1, 19, 11, H, 64, num_special_tokens=4, **kw)
    for t in range(9):
        qkv = torch.from_numpy(seeded.randn(40 + t, tpf, 3 * H * 64)).to(DEV)
        cs = P.ops.rope3d_table(t, pph, ppw, ns, DEV)
        q1 = a.append_frame_fused(0, qkv, *wd, cs, _lib.ROPE_3D)
        q2, k2, v2 = P.ops.prep_qkv(qkv, H, tpf, *wd, cs, _lib.ROPE_3D)
        b.append_frame(0, k2, v2)
        for m in (a, b):
            m.evict_frames(0, 1, 2)
        assert torch.equal(q1, q2)
        assert torch.equal(a.kv_caches[0], b.kv_caches[0])
        # geometry whose specials straddle pages (no rope: the table is sized for tpf tokens)
        qkv = torch.from_numpy(seeded.randn(80 + t, 11, 3 * H * 64)).to(DEV)
        q1 = a2.append_frame_fused(0, qkv, *wd, None, _lib.ROPE_NONE)
        q2, k2, v2 = P.ops.prep_qkv(qkv, H, 11, *wd, None, _lib.ROPE_NONE)
        b2.append_frame(0, k2, v2)
        for m in (a2, b2):
            m.evict_frames(0, 1, 2)
        assert torch.equal(q1, q2) and torch.equal(a2.kv_caches[0], b2.kv_caches[0])
    assert a.device_status() == 0 and a2.device_status() == 0
    # straddle really happened: 9 frames * 4 specials = 36 tokens over pages of 7
    assert len(a2.all_special_pages[0]) == 6 and a2.compute_last_page_len(0) == 1


# ---------------------------------------------------------------- production geometry
def test_full_geometry_properties():
    """378x518 geometry: 1005 tokens/frame, 16 heads, page 999, scale 8 + window 64, 80 keyframes.
    Checked through size-independent properties and the oracle on a sample of (head, query) pairs."""
    tpf, H = 1005, 16
    m = P.B200KVCacheManager(1, 88, tpf, H, 64, device=DEV, max_total_frames=400)
    gen = torch.Generator(device=DEV).manual_seed(2)
    for t in range(80):
        k = torch.randn(tpf, H, 64, device=DEV, generator=gen)
        v = torch.randn(tpf, H, 64, device=DEV, generator=gen)
        m.append_frame(0, k, v.to(torch.bfloat16))
        m.evict_frames(0, 8, 64)
    assert m.get_cache_stats(0) == {"frame_count": 80, "scale_pages": 8, "live_pages": 64, "free_pages": 16,
                                    "special_tokens": 480}
    q = torch.randn(tpf, H, 64, device=DEV, generator=gen).to(torch.bfloat16)
    out, lse = m.compute_attention(0, q, return_lse=True)
    kk, vv = m._gather_kv(0)
    assert kk.shape[0] == 999 * 72 + 480
    # oracle on a sample of heads and query rows
    rows = [0, 1, 127, 128, 500, 895, 896, 1004]
    for h in (0, 7, 15):
        want, wl = O.attention(q[rows][:, h:h + 1].float().cpu().numpy(), kk[:, h:h + 1].float().cpu().numpy(),
                               vv[:, h:h + 1].float().cpu().numpy())
        assert_close(out[rows][:, h:h + 1], want, f"full head {h}")
        assert np.abs(lse[rows][:, h].cpu().numpy() - wl[:, 0]).max() < 2e-3
    # property: V := 1 everywhere -> output == 1 (softmax weights sum to one)
    m.kv_caches[0][:, 1] = 1.0
    ones = m.compute_attention(0, q)
    assert float((ones.float() - 1.0).abs().max()) < 1e-2
    # property: the merge of two disjoint page ranges equals the single pass
    m.kv_caches[0][:, 1] = m.kv_caches[0][:, 0] * 0.5     # some non-trivial V again
    full = m.compute_attention(0, q)
    n = len(m.build_visible_page_table(0))
    parts, lses = [], []
    for lo, hi in ((0, 30), (30, n)):
        m.plan(lo, hi)
        o, l = m.compute_attention_partial(0, q)
        parts.append(o)
        lses.append(l)
    merged = P.ops.lse_merge(torch.stack(parts), torch.stack(lses))
    assert float((merged.float() - full.float()).abs().max()) < 1e-2
    assert cosine64(merged.float().cpu().numpy(), full.float().cpu().numpy()) > 0.99999
    assert m.device_status() == 0


def test_sharded_records_and_strided_merge():
    """The multi-GPU record format on one GPU: two page shards computed one after the other into packed
    [O | lse] records (what each rank all-gathers), merged by gct_lse_merge_strided; plus the world-size-1
    path of sharded_attention and the empty-shard record."""
    from lingbot_map_b200 import distributed as D
    tpf, H = 200, 2
    m = P.B200KVCacheManager(2, 21, tpf, H, 64, device=DEV, scale_frames=2, sliding_window=3, max_total_frames=60)
    orc = O.PagedCacheOracle(2, tpf, H, 64, scale_frames=2, sliding_window=3, max_total_frames=60)
    for t in range(9):
        for b in range(2):
            k, v = seeded.randn(20 * t + b, tpf, H, 64), seeded.randn(700 + 20 * t + b, tpf, H, 64)
            m.append_frame(b, bf(k), bf(v))
            m.evict_frames(b, 2, 3)
            orc.append_frame(b, r(k), r(v))
            orc.evict_frames(b, 2, 3)
    q = seeded.randn(4242, tpf, H, 64)
    kk, vv = orc.gather_kv(1)
    want = O.attention(r(q), kk, vv)[0]
    n_pages = len(m.build_visible_page_table(0))
    n = tpf * H * 64
    world = 3
    rec = torch.empty(world, D.record_floats(tpf, H), dtype=torch.float32, device=DEV)
    for rank in range(2):
        lo, hi = D.shard_page_range(n_pages, rank, 2)
        m.plan(lo, hi)
        m.compute_attention_partial(1, bf(q), out=rec[rank, :n].view(tpf, H, 64), lse=rec[rank, n:].view(tpf, H))
    D.pack_empty_record(rec[2], tpf, H)                       # a rank that owns no page
    out = torch.empty(tpf, H, 64, dtype=torch.bfloat16, device=DEV)
    _lib.check(_lib.load().gct_lse_merge_strided(rec.data_ptr(), rec.data_ptr() + 4 * n, world, tpf, H, rec.shape[1],
                                                 rec.shape[1], out.data_ptr(), None,
                                                 torch.cuda.current_stream().cuda_stream))
    assert_close(out, want, "strided merge of 2 shards + empty record")
    assert_close(D.merge_records_reference(rec, tpf, H).float(), want, "torch merge")
    # world size 1 through the public helper (plans at block 0, reuses the plan at block 1)
    m._shard_plan = None
    o0 = D.sharded_attention(m, 0, bf(q), 0, 1)
    o1 = D.sharded_attention(m, 1, bf(q), 0, 1)
    assert_close(o1, want, "sharded_attention world=1")
    assert o0.shape == o1.shape and m.device_status() == 0


@pytest.mark.parametrize("q_len", [1, 6, 130, 262])
@pytest.mark.parametrize("qdtype", ["bf16", "f32"])
def test_paged_attention_query_lengths(q_len, qdtype):
    """Query lengths below a full frame (the reference's wrapper takes any qo length), last special page
    partially filled, fp32 queries cast to bf16 like flashinfer_cache.py:419."""
    tpf, H = 262, 2                               # the reference's _sanity_check geometry: page of 256 tokens
    m = P.B200KVCacheManager(1, 30, tpf, H, 64, device=DEV, scale_frames=2, sliding_window=4, max_total_frames=100)
    orc = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=2, sliding_window=4, max_total_frames=100)
    for t in range(11):
        k, v = seeded.randn(300 + t, tpf, H, 64), seeded.randn(400 + t, tpf, H, 64)
        m.append_frame(0, bf(k), bf(v))
        m.evict_frames(0, 2, 4)
        orc.append_frame(0, r(k), r(v))
        orc.evict_frames(0, 2, 4)
    q = seeded.randn(555, q_len, H, 64)
    qd = bf(q) if qdtype == "bf16" else torch.from_numpy(q).to(DEV)
    m.plan()
    out = torch.empty(q_len, H, 64, dtype=torch.bfloat16, device=DEV)
    _lib.check(m._lib.gct_mgr_attention(m._handle, 0, qd.data_ptr(), _lib.BF16 if qdtype == "bf16" else _lib.F32, q_len,
                                        out.data_ptr(), None, torch.cuda.current_stream().cuda_stream))
    kk, vv = orc.gather_kv(0)
    assert kk.shape[0] == 256 * 6 + 66
    assert_close(out, O.attention(r(q), kk, vv)[0], f"q_len {q_len}")
    assert m.device_status() == 0


def test_argument_errors_are_reported_not_trapped():
    m = P.B200KVCacheManager(1, 21, 26, 2, 64, device=DEV, scale_frames=2, sliding_window=3, max_total_frames=40)
    k = torch.zeros(26, 2, 64, device=DEV)
    m.append_frame(0, k, k)
    lib = m._lib
    q = torch.zeros(26, 2, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    s = torch.cuda.current_stream().cuda_stream
    # no plan yet
    assert lib.gct_mgr_attention(m._handle, 0, q.data_ptr(), _lib.BF16, 26, out.data_ptr(), None, s) == _lib.ERR_INVALID
    assert b"plan" in lib.gct_last_error()
    m.plan()
    assert lib.gct_mgr_attention(m._handle, 3, q.data_ptr(), _lib.BF16, 26, out.data_ptr(), None, s) == _lib.ERR_INVALID
    assert lib.gct_mgr_attention(m._handle, 0, q.data_ptr(), _lib.BF16, 27, out.data_ptr(), None, s) == _lib.ERR_INVALID
    assert lib.gct_mgr_attention(m._handle, 0, q.data_ptr(), 7, 26, out.data_ptr(), None, s) == _lib.ERR_INVALID
    assert lib.gct_mgr_plan(m._handle, 2, 1, s) == _lib.ERR_INVALID
    with pytest.raises(TypeError):
        m.append_frame(0, k.half(), k.half())
    with pytest.raises(AssertionError, match="expected 20 patch tokens"):
        m.append_frame(0, torch.zeros(25, 2, 64, device=DEV), torch.zeros(25, 2, 64, device=DEV))
    assert m.device_status() == 0


def test_dense_attention_and_prologue_capture_into_a_cuda_graph():
    """The launches of gct_attn_dense and gct_prep_qkv are plain stream work: after one warm-up call (which sizes the
    per-device scratch) they capture into a CUDA graph and replay on new input values, as they do inside the
    reference's torch.compile(mode="reduce-overhead") wrappers."""
    import lingbot_map_b200 as P
    from lingbot_map_b200 import ops
    dev = "cuda:0"
    H, N = 4, 300
    g = torch.Generator(device=dev).manual_seed(3)
    qkv = torch.randn(N, 3 * H * 64, generator=g, device=dev)
    static_in = qkv.clone()

    def step(x):
        q, k, v = ops.prep_qkv(x, H, N, None, None, None, None, None, 0)
        return ops.dense_attention(q.view(1, N, H, 64), k.view(1, N, H, 64), v.view(1, N, H, 64))

    want0 = step(static_in).clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = step(static_in)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, want0)
    qkv2 = torch.randn(N, 3 * H * 64, generator=g, device=dev)
    static_in.copy_(qkv2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, step(qkv2))
    assert ops.device_status(dev) == 0


def _cache_with_frames(scale, n_frames, tpf=262, H=2, seed=11, kscale=1.0):
    import lingbot_map_b200 as P
    dev = "cuda:0"
    m = P.B200KVCacheManager(1, 2 + 4 + 16, tpf, H, 64, device=dev, scale_frames=2, sliding_window=4, max_total_frames=64)
    g = torch.Generator(device=dev).manual_seed(seed)
    for _ in range(n_frames):
        k = torch.randn(tpf, H, 64, generator=g, device=dev) * kscale
        v = torch.randn(tpf, H, 64, generator=g, device=dev)
        m.append_frame(0, k, v)
        m.evict_frames(0, 2, 4)
    q = (torch.randn(tpf, H, 64, generator=g, device=dev) * scale).to(torch.bfloat16)
    return m, q


@pytest.mark.parametrize("qscale,kscale,tag", [(1.0, 1.0, "bound small: fixed reference"),
                                               (12.0, 12.0, "bound too loose: exact kernel takes over")])
def test_bounded_and_exact_modes_agree_with_the_oracle(qscale, kscale, tag):
    """Bounded mode (|q| * max|k| as a fixed softmax reference, chosen on the device per call) and the exact mode
    compute the same softmax: both within the attention tolerance of the oracle, and of each other."""
    from oracle import gct_oracle as O
    m, q = _cache_with_frames(qscale, 9, kscale=kscale)
    kk, vv = m._gather_kv(0)
    out_b = m.compute_attention(0, q).float().cpu().numpy()
    m.set_bounded_mode(False)
    out_e = m.compute_attention(0, q).float().cpu().numpy()
    assert m.device_status() == 0
    ref, _ = O.attention(q.float().cpu().numpy().astype(np.float64), kk.float().cpu().numpy().astype(np.float64),
                         vv.float().cpu().numpy().astype(np.float64))
    for name, got in (("bounded", out_b), ("exact", out_e)):
        d = float(np.abs(got - ref).max())
        c = float((got.ravel() @ ref.ravel()) / (np.linalg.norm(got) * np.linalg.norm(ref)))
        assert d <= 2e-2 and c >= 0.9999, f"{tag}, {name}: max_abs={d:.3e} cosine={c:.6f}"
    assert float(np.abs(out_b - out_e).max()) <= 1e-2


def test_key_norm_tracking_survives_reset_and_direct_pool_writes():
    """The key-norm maximum restarts after reset(); bookkeeping-only appends switch bounded mode off until
    rescan_key_norms(), so pages written directly never meet a stale bound."""
    from oracle import gct_oracle as O
    m, q = _cache_with_frames(1.0, 7, kscale=30.0)          # huge keys first
    m.reset()
    g = torch.Generator(device="cuda:0").manual_seed(5)
    for _ in range(3):
        m.append_frame(0, torch.randn(262, 2, 64, generator=g, device="cuda:0"),
                       torch.randn(262, 2, 64, generator=g, device="cuda:0"))
        m.evict_frames(0, 2, 4)
    def check():
        kk, vv = m._gather_kv(0)
        got = m.compute_attention(0, q).float().cpu().numpy()
        ref, _ = O.attention(q.float().cpu().numpy().astype(np.float64), kk.float().cpu().numpy().astype(np.float64),
                             vv.float().cpu().numpy().astype(np.float64))
        assert float(np.abs(got - ref).max()) <= 2e-2
    check()
    m.append_frame_bookkeeping(0)                           # page content: whatever the pool holds
    m.evict_frames(0, 2, 4)
    m.kv_caches[0][:, 0] *= 50.0                            # direct write: keys far beyond the tracked maximum
    check()                                                 # exact kernel (bounded mode is off for the block)
    m.rescan_key_norms(0)
    check()                                                 # bound recomputed: too loose -> exact kernel again
    assert m.device_status() == 0


def test_key_norm_maxima_track_appends_and_rescan():
    """The tracked maximum bounds the true key norms from above within the 0.4 % rounding allowance, restarts after
    reset, and rescan_key_norms() reproduces the maximum over the whole pool."""
    m, _ = _cache_with_frames(1.0, 9, kscale=3.0)
    def pool_max():
        k = m.kv_caches[0][:, 0].float()                      # [pages, page_size, H, 64]
        return k.norm(dim=-1).amax(dim=(0, 1))
    true = pool_max()                                         # untouched pages are zero
    got = m.key_norm_max[0].clone()
    assert torch.all(got >= true * 0.999) and torch.all(got <= true * 1.01), (got, true)
    m.reset()
    g = torch.Generator(device="cuda:0").manual_seed(1)
    m.append_frame(0, torch.randn(262, 2, 64, generator=g, device="cuda:0") * 0.1,
                   torch.randn(262, 2, 64, generator=g, device="cuda:0"))
    assert torch.all(m.key_norm_max[0] < 2.0)                 # restarted: the old, larger keys no longer count
    m.rescan_key_norms(0)
    assert torch.allclose(m.key_norm_max[0], pool_max(), rtol=1e-3)   # whole pool, stale pages included


@pytest.mark.parametrize("n_past,kv_expected", [(1000, 23085), (10000, 77085)])
@pytest.mark.parametrize("dist", ["randn_over_8", "unit_variance"])
def test_single_layer_microbench_shapes(n_past, kv_expected, dist):
    """The single-layer configuration of the headline benchmark: one frame of 1005 query tokens x 16 heads x 64 over
    1 anchor frame + 16 window frames (full tokens) + 6 memory tokens for each of the past frames, built through the
    manager (scale 1, window 16) so that the page layout is the real one.  Values ~ N(0,1)/8 from seed 1 (logits are
    then almost uniform and the cosine is the binding check), and a unit-variance distribution with a peaked softmax."""
    tpf, H = 1005, 16
    m = P.B200KVCacheManager(1, 1 + 16 + 16, tpf, H, 64, device=DEV, scale_frames=1, sliding_window=16,
                             max_total_frames=n_past + 64)
    gen = torch.Generator(device=DEV).manual_seed(1)
    scale = 0.125 if dist == "randn_over_8" else 1.0
    kf = (torch.randn(8, tpf, H, 64, device=DEV, generator=gen) * scale).to(torch.bfloat16)   # 8 distinct frames, cycled
    vf = (torch.randn(8, tpf, H, 64, device=DEV, generator=gen) * scale).to(torch.bfloat16)
    for t in range(17 + n_past):
        m.append_frame(0, kf[t % 8], vf[t % 8])
        m.evict_frames(0, 1, 16)
    q = (torch.randn(tpf, H, 64, device=DEV, generator=gen) * scale).to(torch.bfloat16)
    out = m.compute_attention(0, q)
    kk, vv = m._gather_kv(0)
    assert kk.shape[0] == kv_expected
    rows = [0, 5, 6, 127, 128, 640, 1004]
    for h in (0, 9, 15):
        want, _ = O.attention(q[rows][:, h:h + 1].float().cpu().numpy(), kk[:, h:h + 1].float().cpu().numpy(),
                              vv[:, h:h + 1].float().cpu().numpy())
        assert_close(out[rows][:, h:h + 1], want, f"{dist} n_past={n_past} head {h}")
    assert m.device_status() == 0


# ---------------------------------------------------------------- headline geometry, every row
@pytest.fixture(scope="module")
def headline_cache():
    """The cache state the benchmark times: 10,000 keyframes at 378x518, i.e. 72 full pages + 61 special pages (the
    last one partly filled), kv = 131,928, built through append_frame from 8 cycled random frames."""
    tpf, H = 1005, 16
    m = P.B200KVCacheManager(1, 88, tpf, H, 64, device=DEV, max_total_frames=10100)
    gen = torch.Generator(device=DEV).manual_seed(3)
    kf = torch.randn(8, tpf, H, 64, device=DEV, generator=gen).to(torch.bfloat16)
    vf = torch.randn(8, tpf, H, 64, device=DEV, generator=gen).to(torch.bfloat16)
    for t in range(10000):
        m.append_frame(0, kf[t % 8], vf[t % 8])
        m.evict_frames(0, 8, 64)
    q = torch.randn(tpf, H, 64, device=DEV, generator=gen).to(torch.bfloat16)
    kk, vv = m._gather_kv(0)
    assert kk.shape[0] == 131928 and len(m.build_visible_page_table(0)) == 133
    assert len(m.all_special_pages[0]) == 61 and m.compute_last_page_len(0) == 60000 - 60 * 999
    heads = (0, 13)
    want = {h: O.attention(q[:, h:h + 1].float().cpu().numpy().astype(np.float64),
                           kk[:, h:h + 1].float().cpu().numpy().astype(np.float64),
                           vv[:, h:h + 1].float().cpu().numpy().astype(np.float64)) for h in heads}
    return m, q, want


@pytest.mark.parametrize("mode", ["bounded", "exact"])
def test_headline_kv_every_row_of_two_heads(headline_cache, mode):
    """kv = 131,928 (the only size the benchmark times): all 1005 query rows of two heads against the float64 oracle,
    with the softmax reference folded into the S product and with the running row maximum; log-sum-exps too."""
    m, q, want = headline_cache
    m.set_bounded_mode(mode == "bounded")
    try:
        out, lse = m.compute_attention(0, q, return_lse=True)
    finally:
        m.set_bounded_mode(True)
    # Log-sum-exp: with the running maximum the logits are exact products of the bf16 inputs (2e-3 leaves room for
    # the exponential approximations).  With the folded reference the Q tile is multiplied by scale * log2(e) BEFORE
    # it is rounded to bf16 for the tensor core (relative 2^-9 per element, the same perturbation for every key of a
    # row), which moves the logits of a row, and so its log-sum-exp, by up to |logit| * 2^-9 ~ 2e-3 at the logits of
    # this test (up to ~6 in natural units, measured 2.1e-3); the normalised output does not see a common shift.
    lse_tol = 2e-3 if mode == "exact" else 4e-3
    for h, (wo, wl) in want.items():
        assert_close(out[:, h:h + 1], wo, f"kv=131928 {mode} head {h}")
        assert np.abs(lse[:, h].cpu().numpy() - wl[:, 0]).max() < lse_tol
    assert m.device_status() == 0


@pytest.mark.parametrize("pages", [(0, 17), (33, 67), (116, 133)])
def test_page_slices_of_the_headline_cache(headline_cache, pages):
    """What one rank of a KV-sharded stream computes: attention over a slice of the visible page list (17 or 34 pages
    of the 133: 136 / 272 KV blocks, where the launch uses long KV ranges plus one short range per head and query
    group instead of equal ranges; the last slice ends with the partly filled special page).  All rows of one head,
    output and log-sum-exp, against the float64 oracle over the same tokens."""
    m, q, _ = headline_cache
    lo, hi = pages
    kk, vv = m._gather_kv(0)
    t0, t1 = lo * 999, min(hi * 999, kk.shape[0])
    h = 7
    wo, wl = O.attention(q[:, h:h + 1].float().cpu().numpy().astype(np.float64),
                         kk[t0:t1, h:h + 1].float().cpu().numpy().astype(np.float64),
                         vv[t0:t1, h:h + 1].float().cpu().numpy().astype(np.float64))
    try:
        m.plan(lo, hi)
        out, lse = m.compute_attention_partial(0, q)
    finally:
        m.plan()
    assert_close(out[:, h:h + 1], wo, f"pages [{lo}, {hi})")
    assert np.abs(lse[:, h].cpu().numpy() - wl[:, 0]).max() < 4e-3      # bounded mode: see the test above
    assert m.device_status() == 0


def test_bounded_mode_is_chosen_per_cta(headline_cache):
    """Two query rows (in different query tiles) get a norm that makes their Cauchy-Schwarz bound too loose: only the
    CTAs that hold them fall back to the running maximum, inside the same launch; every row still matches the oracle
    (the two rows themselves are compared in relative terms: their softmax is nearly one-hot)."""
    m, q, want = headline_cache
    qb = q.clone()
    qb[5] *= 20
    qb[700] *= 20
    out = m.compute_attention(0, qb)
    kk, vv = m._gather_kv(0)
    keep = [i for i in range(q.shape[0]) if i not in (5, 700)]
    for h, (wo, _) in want.items():
        assert_close(out[keep][:, h:h + 1], wo[keep], f"untouched rows, head {h}")
        wb, _ = O.attention(qb[[5, 700]][:, h:h + 1].float().cpu().numpy().astype(np.float64),
                            kk[:, h:h + 1].float().cpu().numpy().astype(np.float64),
                            vv[:, h:h + 1].float().cpu().numpy().astype(np.float64))
        got = out[[5, 700]][:, h:h + 1].float().cpu().numpy()
        assert np.abs(got - wb).max() <= 2 ** -6 * max(1.0, np.abs(wb).max()) and cosine64(got, wb) >= 0.9999
    assert m.device_status() == 0


def test_rows_past_the_valid_length_of_the_last_page_do_not_leak():
    """Rows of the last special page beyond last_page_len are read by the kernel (they are inside the tensor map) and
    masked.  Filled with large finite values (a pool that was not zeroed, or data left by a rolled-back frame) they
    must not change the result; the header asks for finite values there, since 0 * NaN would poison the PV product."""
    tpf, H = 262, 2
    m = P.B200KVCacheManager(1, 30, tpf, H, 64, device=DEV, scale_frames=2, sliding_window=4, max_total_frames=100)
    orc = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=2, sliding_window=4, max_total_frames=100)
    for t in range(11):
        k, v = seeded.randn(300 + t, tpf, H, 64), seeded.randn(400 + t, tpf, H, 64)
        m.append_frame(0, bf(k), bf(v))
        m.evict_frames(0, 2, 4)
        orc.append_frame(0, r(k), r(v))
        orc.evict_frames(0, 2, 4)
    last_page, last_len = m.build_visible_page_table(0)[-1], m.compute_last_page_len(0)
    assert last_len == 66
    m.kv_caches[0][last_page, 0, last_len:] = 3.0e3          # keys: inside the tracked norm bound would be too kind
    m.kv_caches[0][last_page, 1, last_len:] = -7.0e4         # values
    q = seeded.randn(556, tpf, H, 64)
    kk, vv = orc.gather_kv(0)
    want = O.attention(r(q), kk, vv)[0]
    for bounded in (True, False):
        m.set_bounded_mode(bounded)
        assert_close(m.compute_attention(0, bf(q)), want, f"garbage tail, bounded={bounded}")
    assert m.device_status() == 0


def test_exchange_kernel_with_one_rank_equals_single_pass():
    """gct_mgr_attention_exchange with world = 1: the rank's own buffers stand for the peer-mapped ones, so both
    phases of the exchange kernel (partials -> receive slots, merge of the row slice -> output) run on one GPU
    without any peer.  Twice on the same flag words (epochs 1, 2), with a split KV range and with a single pass."""
    import ctypes as C
    from lingbot_map_b200.cache import _stream_ptr
    lib = _lib.load()
    for tpf, H, frames in ((306, 2, 30), (134, 16, 3)):
        m = P.B200KVCacheManager(1, 48, tpf, H, 64, device=DEV, scale_frames=4, sliding_window=28, max_total_frames=200)
        orc = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=4, sliding_window=28, max_total_frames=200)
        for t in range(frames):
            k, v = seeded.randn(50 + t, tpf, H, 64), seeded.randn(150 + t, tpf, H, 64)
            m.append_frame(0, bf(k), bf(v))
            m.evict_frames(0, 4, 28)
            orc.append_frame(0, r(k), r(v))
            orc.evict_frames(0, 4, 28)
        rb, fb, sl = C.c_size_t(), C.c_size_t(), C.c_int()
        _lib.check(lib.gct_kv_exchange_sizes(tpf, H, 1, C.byref(rb), C.byref(fb), C.byref(sl)))
        assert sl.value == tpf * H
        recv = torch.zeros(rb.value // 4, dtype=torch.float32, device=DEV)
        flags = torch.zeros(64, dtype=torch.int32, device=DEV)
        out = torch.empty(tpf, H, 64, dtype=torch.bfloat16, device=DEV)
        one = lambda t: (C.c_void_p * 1)(t.data_ptr())
        m.plan()
        kk, vv = orc.gather_kv(0)
        for epoch in (1, 2):
            q = seeded.randn(600 + epoch, tpf, H, 64)
            qd = bf(q)
            out.zero_()
            _lib.check(lib.gct_mgr_attention_exchange(m._handle, 0, qd.data_ptr(), _lib.BF16, tpf, 0, 1, 1, one(recv),
                                                      one(out), one(flags), sl.value, epoch, _stream_ptr(m.device)))
            assert_close(out, O.attention(r(q), kk, vv)[0], f"exchange world=1 epoch {epoch} ({tpf}x{H})")
            assert flags[:2].tolist() == [epoch, epoch] and flags[2:4].tolist() == [0, 0]
        assert m.device_status() == 0


def test_exchange_wait_runs_out_when_a_peer_never_signals():
    """The exchange kernel's waits are bounded: with world = 2 and nobody playing rank 1 (its buffers are plain local
    tensors that nothing ever flags) the kernel gives up after about two seconds, records the time-out in the status
    word and returns; the host reads it as an error, and the device goes on working."""
    import ctypes as C
    import time
    from lingbot_map_b200.cache import _stream_ptr
    lib = _lib.load()
    tpf, H = 134, 2
    m = P.B200KVCacheManager(1, 24, tpf, H, 64, device=DEV, scale_frames=2, sliding_window=4, max_total_frames=64)
    for t in range(3):
        m.append_frame(0, bf(seeded.randn(900 + t, tpf, H, 64)), bf(seeded.randn(950 + t, tpf, H, 64)))
        m.evict_frames(0, 2, 4)
    rb, fb, sl = C.c_size_t(), C.c_size_t(), C.c_int()
    _lib.check(lib.gct_kv_exchange_sizes(tpf, H, 2, C.byref(rb), C.byref(fb), C.byref(sl)))
    recv = [torch.zeros(rb.value // 4, dtype=torch.float32, device=DEV) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(2)]
    out = [torch.zeros(tpf, H, 64, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    two = lambda ts: (C.c_void_p * 2)(*[t.data_ptr() for t in ts])
    m.plan()
    qd = bf(seeded.randn(990, tpf, H, 64))
    t0 = time.perf_counter()
    _lib.check(lib.gct_mgr_attention_exchange(m._handle, 0, qd.data_ptr(), _lib.BF16, tpf, 0, 2, 1, two(recv), two(out),
                                              two(flags), sl.value, 1, _stream_ptr(m.device)))
    with pytest.raises(Exception, match="device status"):
        m.device_status()
    waited = time.perf_counter() - t0
    assert 0.5 < waited < 20.0, waited
    assert flags[0][:2].tolist() == [1, 0] and flags[1][0].item() == 1     # rank 0 published, rank 1 never did
    assert float(out[0].float().abs().max()) == 0.0                          # nothing was merged or stored
    # the context is intact: a fresh manager (its own status word) computes as usual
    m2 = P.B200KVCacheManager(1, 24, tpf, H, 64, device=DEV, scale_frames=2, sliding_window=4, max_total_frames=64)
    orc = O.PagedCacheOracle(1, tpf, H, 64, scale_frames=2, sliding_window=4, max_total_frames=64)
    k, v = seeded.randn(901, tpf, H, 64), seeded.randn(951, tpf, H, 64)
    m2.append_frame(0, bf(k), bf(v))
    orc.append_frame(0, r(k), r(v))
    q = seeded.randn(991, tpf, H, 64)
    assert_close(m2.compute_attention(0, bf(q)), orc.compute_attention(0, r(q)), "after a timed-out exchange")
    assert m2.device_status() == 0
