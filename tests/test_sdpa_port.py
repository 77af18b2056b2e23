"""Pin the PyTorch-CPU port of the reference's SDPA streaming path (the timed CPU baseline) against
outputs recorded from the reference's own SDPABlock."""
import json
import os

import numpy as np
import torch

import seeded
from oracle import sdpa_port as SP

G = os.path.join(os.path.dirname(__file__), "golden")


def block_params(seed, names_shapes):
    return {n: torch.from_numpy(seeded.param_value(seed, n, s)) for n, s in names_shapes.items()}


def block_shapes(dim):
    return {"norm1.weight": (dim,), "norm1.bias": (dim,), "attn.qkv.weight": (3 * dim, dim), "attn.qkv.bias": (3 * dim,),
            "attn.q_norm.weight": (64,), "attn.q_norm.bias": (64,), "attn.k_norm.weight": (64,),
            "attn.k_norm.bias": (64,), "attn.proj.weight": (dim, dim), "attn.proj.bias": (dim,),
            "ls1.gamma": (dim,), "norm2.weight": (dim,), "norm2.bias": (dim,), "mlp.fc1.weight": (4 * dim, dim),
            "mlp.fc1.bias": (4 * dim,), "mlp.fc2.weight": (dim, 4 * dim), "mlp.fc2.bias": (dim,), "ls2.gamma": (dim,)}


def test_parameter_names_match_reference_block():
    z = np.load(os.path.join(G, "block_stream_fp32.npz"))
    names = json.loads(bytes(z["param_names_json"]).decode())
    assert sorted(names) == sorted(block_shapes(128))


def test_sdpa_port_matches_reference_block_stream():
    z = np.load(os.path.join(G, "block_stream_fp32.npz"))
    dim, H, pph, ppw, ns, scale, window = 128, 2, 3, 4, 6, 2, 3
    P = ns + pph * ppw
    p = block_params(21, block_shapes(dim))
    attn = SP.SdpaStreamPort({k[5:]: v for k, v in p.items() if k.startswith("attn.")}, H, scale, window, ns)
    x = torch.from_numpy(seeded.randn(500, 1, scale * P, dim))
    cos, sin = SP.rope3d_cos_sin(0, scale, pph, ppw, ns)
    y = SP.block_forward(p, attn, x, cos, sin, frames_in_call=scale)
    assert float((y - torch.from_numpy(z["sdpa_kf1_phase1"])).abs().max()) < 5e-6
    for i in range(scale, scale + 8):
        x = torch.from_numpy(seeded.randn(500 + i, 1, P, dim))
        cos, sin = SP.rope3d_cos_sin(i, 1, pph, ppw, ns)
        y = SP.block_forward(p, attn, x, cos, sin)
        assert float((y - torch.from_numpy(z[f"sdpa_kf1_frame{i}"])).abs().max()) < 5e-6, i
    # 10 frames, scale 2 + window 3: 5 evicted frames keep their 6 special tokens
    assert tuple(attn.k.shape) == (1, H, 5, P, 64) and tuple(attn.k_special.shape) == (1, H, 5, ns, 64)
