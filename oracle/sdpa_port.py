"""CPU port of the reference's SDPA streaming path, in PyTorch on host cores.  TEST INFRASTRUCTURE ONLY.

This is the path the reference itself runs on a machine without FlashInfer (`--use_sdpa`): a dict KV cache
that grows by torch.cat, evicts by re-concatenating scale + window frames, keeps the 6 special tokens of
evicted frames, and calls F.scaled_dot_product_attention.  It is the timed CPU baseline of the benchmark
and an fp32 cross-check for the block-level parity tests.  Parity status: PINNED against outputs of the
reference's SDPABlock (tests/golden/block_stream_fp32.npz).

Restated from (paths relative to the reference repo):
  lingbot_map/layers/attention.py:595-718   SDPAAttention.forward, _apply_kv_cache_eviction
  lingbot_map/layers/block.py:510-532       SDPABlock.forward
  lingbot_map/layers/rope.py:435-461        apply_rotary_emb
"""
import torch
import torch.nn.functional as F


def rope3d_cos_sin(f_start, n_frames, pph, ppw, ns, fhw=(20, 22, 22), theta=10000.0):
    """cos/sin [n_frames*(ns+pph*ppw), 32] float64 of the 3-D RoPE (rope.py:293-433)."""
    def freqs(dim):
        return 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64)[: dim // 2] / dim))
    ft, fh, fw = (freqs(d) for d in fhw)
    rows = []
    for f in range(f_start, f_start + n_frames):
        sp = torch.arange(ns, dtype=torch.float64)
        rows.append(torch.cat([(f * ft).expand(ns, -1), sp[:, None] * fh, sp[:, None] * fw], dim=1))
        hh = (ns + torch.arange(pph, dtype=torch.float64)).repeat_interleave(ppw)
        ww = (ns + torch.arange(ppw, dtype=torch.float64)).repeat(pph)
        rows.append(torch.cat([(f * ft).expand(pph * ppw, -1), hh[:, None] * fh, ww[:, None] * fw], dim=1))
    ang = torch.cat(rows, dim=0)
    return ang.cos(), ang.sin()


def apply_rope3d(x, cos, sin):
    """x [B,H,N,D]; cos/sin [N, D/2] cast to x.dtype first (rope.py:450-461)."""
    c, s = cos.to(x.dtype)[None, None], sin.to(x.dtype)[None, None]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).reshape(x.shape)


class SdpaStreamPort:
    """One global attention layer with the reference's dict KV cache (attention.py:595-718).

    params: dict with qkv.weight/bias, q_norm.weight/bias, k_norm.weight/bias, proj.weight/bias tensors.
    """

    def __init__(self, params, num_heads, scale_frames=8, sliding_window=64, num_special=6):
        self.p = params
        self.H = num_heads
        self.scale_frames, self.sliding_window, self.ns = scale_frames, sliding_window, num_special
        self.reset()

    def reset(self):
        self.k = self.v = self.k_special = self.v_special = None

    def qkv(self, x):
        B, N, C = x.shape
        D = C // self.H
        t = F.linear(x, self.p["qkv.weight"], self.p["qkv.bias"]).reshape(B, N, 3, self.H, D).permute(2, 0, 3, 1, 4)
        q, k, v = t.unbind(0)
        q = F.layer_norm(q, (D,), self.p["q_norm.weight"], self.p["q_norm.bias"], 1e-5)
        k = F.layer_norm(k, (D,), self.p["k_norm.weight"], self.p["k_norm.bias"], 1e-5)
        return q, k, v

    def attend(self, q, k, v, frames_in_call):
        """q,k,v [B,H,N,D] already normalised and rotated.  Appends to the cache, evicts, attends."""
        B, H, N, D = k.shape
        kf = k.view(B, H, frames_in_call, N // frames_in_call, D)
        vf = v.view(B, H, frames_in_call, N // frames_in_call, D)
        if self.k is None:                                                   # :632-636
            self.k, self.v = kf, vf
        else:                                                                # :637-646
            self.k = torch.cat((self.k, kf), dim=2)
            self.v = torch.cat((self.v, vf), dim=2)
        self._evict()                                                        # :648-650
        kc, vc = self.k.clone(), self.v.clone()                              # :652-653
        a, b, c, d, e = kc.shape
        k_full, v_full = kc.reshape(a, b, c * d, e), vc.reshape(a, b, c * d, e)
        if self.k_special is not None:                                       # :658-663
            sa, sb, sc, sd, se = self.k_special.shape
            k_full = torch.cat([self.k_special.reshape(sa, sb, sc * sd, se), k_full], dim=2)
            v_full = torch.cat([self.v_special.reshape(sa, sb, sc * sd, se), v_full], dim=2)
        return F.scaled_dot_product_attention(q, k_full, v_full)             # :666-669

    def _evict(self):                                                        # :676-718
        sw, sf = self.sliding_window, self.scale_frames
        if self.k.shape[3] <= 1:
            return
        n = self.k.shape[2]
        if n <= sw + sf or n - sw <= sf:
            return
        ek, ev = self.k[:, :, sf:n - sw], self.v[:, :, sf:n - sw]
        nk, nv = ek[:, :, :, :self.ns].clone(), ev[:, :, :, :self.ns].clone()
        if self.k_special is None:
            self.k_special, self.v_special = nk, nv
        else:
            self.k_special = torch.cat([self.k_special, nk], dim=2)
            self.v_special = torch.cat([self.v_special, nv], dim=2)
        self.k = torch.cat([self.k[:, :, :sf], self.k[:, :, -sw:]], dim=2)
        self.v = torch.cat([self.v[:, :, :sf], self.v[:, :, -sw:]], dim=2)

    def forward(self, x, cos, sin, frames_in_call=1):
        """x [B, N, C] (after norm1) -> attention branch output incl. proj (attention.py:595-674)."""
        q, k, v = self.qkv(x)
        q, k = apply_rope3d(q, cos, sin), apply_rope3d(k, cos, sin)
        o = self.attend(q, k, v, frames_in_call)
        B, H, N, D = o.shape
        o = o.transpose(1, 2).reshape(B, N, H * D)
        return F.linear(o, self.p["proj.weight"], self.p["proj.bias"])


def block_forward(params, attn_port, x, cos, sin, frames_in_call=1):
    """SDPABlock.forward (block.py:510-532): x + ls1(attn(norm1 x)); x + ls2(mlp(norm2 x))."""
    C = x.shape[-1]
    h = F.layer_norm(x, (C,), params["norm1.weight"], params["norm1.bias"], 1e-5)
    x = x + attn_port.forward(h, cos, sin, frames_in_call) * params["ls1.gamma"]
    h = F.layer_norm(x, (C,), params["norm2.weight"], params["norm2.bias"], 1e-5)
    h = F.linear(F.gelu(F.linear(h, params["mlp.fc1.weight"], params["mlp.fc1.bias"])),
                 params["mlp.fc2.weight"], params["mlp.fc2.bias"])
    return x + h * params["ls2.gamma"]
