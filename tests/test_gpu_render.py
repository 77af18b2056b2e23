"""Frustum culling and Morton voxelisation on the GPU against the float32 CPU restatement: every mask bit, Morton
code and voxel centre equal (the kernels use single rounded float operations for that reason).  Covers empty input,
sizes that are not a multiple of the four points a thread takes, points behind the camera / outside the planes /
on image borders, negative coordinates, and a multi-million point cloud through properties."""
import numpy as np
import pytest
import torch

from lingbot_map_b200 import render_ops as RO
from oracle import render_oracle as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _camera(seed):
    rs = np.random.RandomState(seed)
    q, _ = np.linalg.qr(rs.standard_normal((3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q.astype(np.float32), (rs.standard_normal(3) * 0.5).astype(np.float32)


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 100003])
def test_frustum_cull_bit_exact(n):
    rs = np.random.RandomState(n)
    pts = (rs.standard_normal((n, 3)) * 3).astype(np.float32)
    Rm, t = _camera(n + 1)
    args = (300.0, 310.0, 259.0, 189.0, 518, 378, 0.1, 6.0)
    got = RO.frustum_cull(torch.from_numpy(pts).to(DEV), torch.from_numpy(Rm).to(DEV), torch.from_numpy(t).to(DEV), *args)
    want = R.frustum_cull(pts, Rm, t, *args)
    assert got.dtype == torch.bool and got.shape == (n,)
    assert np.array_equal(got.cpu().numpy(), want)
    if n > 1000:
        assert 0.02 < want.mean() < 0.9          # the case exercises both outcomes


@pytest.mark.parametrize("n,voxel", [(0, 0.05), (1, 0.05), (7, 0.5), (4097, 0.05), (250000, 0.02)])
def test_voxelize_frame_bit_exact(n, voxel):
    rs = np.random.RandomState(n + 7)
    xyz = (rs.standard_normal((n, 3)) * 2).astype(np.float32)
    rgb = rs.rand(n, 3).astype(np.float32)
    c, col, codes = RO.voxelize_frame(torch.from_numpy(xyz).to(DEV), torch.from_numpy(rgb).to(DEV), voxel)
    wc, wcol, wcodes = R.voxelize_frame(xyz, rgb, voxel)
    assert np.array_equal(codes.cpu().numpy(), wcodes)
    assert np.array_equal(c.cpu().numpy(), wc)
    assert np.array_equal(col.cpu().numpy(), wcol)
    if n:
        assert np.all(np.diff(wcodes) > 0)       # sorted and unique


def test_large_cloud_properties():
    """8 M points (96 MB of xyz: larger than L2's share): idempotence of voxelisation on its own output centres, and
    the culled set is exactly the set whose projection the oracle accepts on a sample."""
    n = 8_000_000
    g = torch.Generator(device=DEV).manual_seed(1)
    xyz = torch.randn(n, 3, device=DEV, generator=g) * 2
    rgb = torch.rand(n, 3, device=DEV, generator=g)
    c, col, codes = RO.voxelize_frame(xyz, rgb, 0.05)
    assert torch.all(codes[1:] > codes[:-1])
    c2, _, codes2 = RO.voxelize_frame(c, col, 0.05)
    assert torch.equal(codes2, codes) and torch.equal(c2, c)          # centres map to their own voxels
    Rm, t = _camera(3)
    args = (300.0, 310.0, 259.0, 189.0, 518, 378, 0.1, 6.0)
    vis = RO.frustum_cull(xyz, torch.from_numpy(Rm), torch.from_numpy(t), *args)
    idx = torch.arange(0, n, 9973, device=DEV)
    want = R.frustum_cull(xyz[idx].cpu().numpy(), Rm, t, *args)
    assert np.array_equal(vis[idx].cpu().numpy(), want)
