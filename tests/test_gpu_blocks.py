"""Block-level parity on the GPU: B200Block / B200FrameAttention against outputs recorded from the reference's
FlashInferBlock (paged fp32 path), SDPABlock and Attention on CPU (tests/golden/*.npz).

Weights are fp32 and the Linear layers run in fp32; q/k/v are rounded to bf16 by the CUDA prologue, attention runs
on bf16 tensor cores.  Tolerance on block outputs: 2e-2 max-abs and cosine >= 0.9999 (float64)."""
import os

import numpy as np
import pytest
import torch

import seeded
import lingbot_map_b200 as P

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


class Rope2dStub:
    """Carries the base frequency the way RotaryPositionEmbedding2D does (rope.py:81-86)."""
    base_frequency = 100.0


def close(got, want, tag, max_abs=2e-2, cos=0.9999):
    g = got.double().cpu().numpy().ravel()
    w = np.asarray(want, np.float64).ravel()
    c = float(g @ w / (np.linalg.norm(g) * np.linalg.norm(w)))
    d = float(np.abs(g - w).max())
    assert np.isfinite(g).all() and d <= max_abs and c >= cos, f"{tag}: max_abs={d:.3e} cosine={c:.7f}"


def rope3d_pos(f_start, n_frames, pph, ppw, ns):
    """Complex frequency tensor [1,1,N,32] as WanRotaryPosEmbed.forward returns it (rope.py:336-425)."""
    from oracle import gct_oracle as O
    ang = np.concatenate([O.rope3d_angles(f, pph, ppw, ns) for f in range(f_start, f_start + n_frames)], axis=0)
    z = torch.polar(torch.ones(ang.shape, dtype=torch.float64), torch.from_numpy(ang))
    return z[None, None].to(DEV)


@pytest.mark.parametrize("kf", [2, 1])
def test_block_stream_matches_reference(kf):
    z = np.load(os.path.join(G, "block_stream_fp32.npz"))
    dim, H, pph, ppw, ns, scale, window = 128, 2, 3, 4, 6, 2, 3
    Ptok = ns + pph * ppw
    blk = P.B200Block(dim=dim, num_heads=H, init_values=0.01, qk_norm=True, rope=Rope2dStub(),
                      kv_cache_sliding_window=window, kv_cache_scale_frames=scale).eval().to(DEV)
    seeded.fill_module_(blk, 21)
    mgr = P.B200KVCacheManager(num_blocks=1, max_num_frames=scale + window + 16, tokens_per_frame=Ptok, num_heads=H,
                               head_dim=64, dtype=torch.float32, device=DEV, scale_frames=scale,
                               sliding_window=window, max_total_frames=40)
    tag = f"paged_kf{kf}"
    kw = dict(num_patches=Ptok - ns, num_special=ns, enable_3d_rope=True, kv_cache=mgr, global_idx=0,
              num_frame_for_scale=scale, num_register_tokens=4)
    tfp = 0
    with torch.no_grad():
        x = torch.from_numpy(seeded.randn(500, 1, scale * Ptok, dim)).to(DEV)
        y = blk(x, pos=rope3d_pos(0, scale, pph, ppw, ns), num_frames=scale, num_frame_per_block=scale, **kw)
        close(y, z[f"{tag}_phase1"], "phase 1")
        tfp += scale
        for i in range(scale, scale + 8):
            is_kf = kf <= 1 or (i - scale) % kf == 0
            mgr._skip_append = not is_kf
            x = torch.from_numpy(seeded.randn(500 + i, 1, Ptok, dim)).to(DEV)
            y = blk(x, pos=rope3d_pos(tfp, 1, pph, ppw, ns), num_frames=1, num_frame_per_block=1, **kw)
            close(y, z[f"{tag}_frame{i}"], f"frame {i} ({'KF' if is_kf else 'non-KF'})")
            if is_kf:
                tfp += 1
    mgr._skip_append = False
    # page table and eviction decisions bit-exact with the reference run
    assert mgr.build_visible_page_table(0) == list(z[f"{tag}_visible_end"])
    assert mgr.compute_last_page_len(0) == int(z[f"{tag}_last_len_end"][0])
    assert mgr.device_status() == 0


def test_block_attn_pre_contract():
    """attn_pre returns (q, k, v) [tokens, H, 64] like block.py:217-227 and equals what the fused append writes."""
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    Ptok = ns + pph * ppw
    blk = P.B200Block(dim=dim, num_heads=H, init_values=0.01, qk_norm=True, rope=Rope2dStub()).eval().to(DEV)
    seeded.fill_module_(blk, 5)
    mgr = P.B200KVCacheManager(1, 21, Ptok, H, 64, device=DEV, scale_frames=2, sliding_window=3, max_total_frames=40)
    x = torch.from_numpy(seeded.randn(1, 1, Ptok, dim)).to(DEV)
    pos = rope3d_pos(3, 1, pph, ppw, ns)
    with torch.no_grad():
        q, k, v = blk.attn_pre(x, pos=pos, enable_3d_rope=True)
        blk(x, pos=pos, num_frames=1, enable_3d_rope=True, kv_cache=mgr, global_idx=0)
    assert q.shape == (Ptok, H, 64) and q.dtype == torch.bfloat16
    kk, vv = mgr._gather_kv(0)
    # cache order: patch page first, then the special page (flashinfer_cache.py:446-450)
    assert torch.equal(kk, torch.cat([k[ns:], k[:ns]])) and torch.equal(vv, torch.cat([v[ns:], v[:ns]]))


def test_frame_attention_matches_reference():
    z = np.load(os.path.join(G, "prepare_qkv_fp32.npz"))
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    N = ns + pph * ppw
    fa = P.B200FrameAttention(dim, num_heads=H, qk_norm=True, rope=Rope2dStub()).eval().to(DEV)
    seeded.fill_module_(fa, 11)
    x = torch.from_numpy(seeded.randn(123, 2, N, dim)).to(DEV)
    pos = torch.from_numpy(z["rope2d_pos"]).to(DEV)[None].expand(2, -1, -1)
    with torch.no_grad():
        y = fa(x, pos=pos)
    close(y, z["frame_attn_out"], "frame attention")


def test_bf16_autocast_path():
    """demo.py casts the aggregator to bf16 and runs under autocast (demo.py:458-460,545): bf16 weights and
    activations, bf16 LayerNorm parameters.  Golden: the reference's own FlashInferBlock with `.to(bfloat16)` under
    bf16 autocast on CPU (tests/golden/block_stream_bf16.npz, make_goldens.py block_stream_bf16_values).

    Tolerance.  Both sides return bf16, whose spacing at the outputs' magnitude (up to 5.8 here) is 2^-5 = 3.1e-2
    for |y| in [4, 8) and 2^-6 for [2, 4); the two runs round every intermediate (LayerNorm output, qkv, attention
    output, proj, two MLP layers, two residual sums) to bf16 at slightly different values, so final results that
    differ by one or two output rounding steps are expected: max-abs bound = 2 steps at the largest magnitude
    = 6.3e-2.  The cosine over the whole output is insensitive to single steps and keeps 0.9999."""
    z = np.load(os.path.join(G, "block_stream_bf16.npz"))
    dim, H, pph, ppw, ns, scale, window = 128, 2, 3, 4, 6, 2, 3
    Ptok = ns + pph * ppw
    blk = P.B200Block(dim=dim, num_heads=H, init_values=0.01, qk_norm=True, rope=Rope2dStub(),
                      kv_cache_sliding_window=window, kv_cache_scale_frames=scale).eval().to(DEV)
    seeded.fill_module_(blk, 21)
    blk = blk.to(torch.bfloat16)
    mgr = P.B200KVCacheManager(1, scale + window + 16, Ptok, H, 64, device=DEV, scale_frames=scale,
                               sliding_window=window, max_total_frames=40)
    kw = dict(num_patches=Ptok - ns, num_special=ns, enable_3d_rope=True, kv_cache=mgr, global_idx=0,
              num_frame_for_scale=scale, num_register_tokens=4)
    tol = dict(max_abs=6.3e-2, cos=0.9999)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        x = torch.from_numpy(seeded.randn(900, 1, scale * Ptok, dim)).to(DEV).to(torch.bfloat16)
        y = blk(x, pos=rope3d_pos(0, scale, pph, ppw, ns), num_frames=scale, num_frame_per_block=scale, **kw)
        assert y.dtype == torch.bfloat16
        close(y, z["phase1"], "bf16 phase 1", **tol)
        for i in range(5):
            x = torch.from_numpy(seeded.randn(901 + i, 1, Ptok, dim)).to(DEV).to(torch.bfloat16)
            y = blk(x, pos=rope3d_pos(scale + i, 1, pph, ppw, ns), num_frames=1, num_frame_per_block=1, **kw)
            assert y.dtype == torch.bfloat16
            close(y, z[f"frame{i}"], f"bf16 frame {i}", **tol)
    assert mgr.build_visible_page_table(0) == list(z["visible_end"])
    assert mgr.device_status() == 0


def test_block_with_compiled_style_attn_pre_equals_fused_path():
    """With blk.attn_pre rebound on the instance (what compile_model does) the streaming forward goes through
    attn_pre + append_frame instead of the fused append; both write the same pages and give the same output."""
    dim, H, pph, ppw, ns = 128, 2, 3, 4, 6
    Ptok = ns + pph * ppw
    mk_blk = lambda: P.B200Block(dim=dim, num_heads=H, init_values=0.01, qk_norm=True, rope=Rope2dStub(),
                                 kv_cache_sliding_window=3, kv_cache_scale_frames=2).eval().to(DEV)
    a, b = mk_blk(), mk_blk()
    seeded.fill_module_(a, 9)
    seeded.fill_module_(b, 9)
    b.attn_pre = b.attn_pre                       # instance attribute, as after `b.attn_pre = torch.compile(b.attn_pre)`
    mk = lambda: P.B200KVCacheManager(1, 21, Ptok, H, 64, device=DEV, scale_frames=2, sliding_window=3, max_total_frames=40)
    ma, mb = mk(), mk()
    for i in range(7):
        skip = i in (3, 5)
        ma._skip_append = mb._skip_append = skip
        x = torch.from_numpy(seeded.randn(40 + i, 1, Ptok, dim)).to(DEV)
        pos = rope3d_pos(i, 1, pph, ppw, ns)
        with torch.no_grad():
            ya = a(x, pos=pos, num_frames=1, enable_3d_rope=True, kv_cache=ma, global_idx=0)
            yb = b(x, pos=pos, num_frames=1, enable_3d_rope=True, kv_cache=mb, global_idx=0)
        assert torch.equal(ya, yb)
        assert ma.build_visible_page_table(0) == mb.build_visible_page_table(0)
    assert torch.equal(ma._gather_kv(0)[0], mb._gather_kv(0)[0])


def test_plain_attention_without_norm_and_rope():
    """The DINOv2 patch-embed attention (vision_transformer.py:144-171 builds Block(attn_class=Attention) with
    qk_norm off and no RoPE; 1 class + 4 register + 999 patch tokens): B200FrameAttention against fp32 SDPA."""
    dim, H, N = 128, 2, 1004
    fa = P.B200FrameAttention(dim, num_heads=H, qk_norm=False, rope=None).eval().to(DEV)
    seeded.fill_module_(fa, 31)
    x = torch.from_numpy(seeded.randn(77, 2, N, dim)).to(DEV)
    with torch.no_grad():
        y = fa(x)
        qkv = fa.qkv(x).reshape(2, N, 3, H, 64).permute(2, 0, 3, 1, 4)
        ref = torch.nn.functional.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        ref = fa.proj(ref.transpose(1, 2).reshape(2, N, dim))
    close(y, ref.double().cpu().numpy(), "plain attention")
