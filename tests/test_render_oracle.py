"""Known answers for the CPU restatement of the reference's point-cloud helpers (oracle/render_oracle.py), worked
out by hand from demo_render/render_cuda_ext/frustum_cull/frustum_cull.cu:5-33 and voxel_morton/voxel_morton.cu:5-62."""
import numpy as np

from oracle import render_oracle as R


def test_frustum_cull_known_answers():
    I, t = np.eye(3, dtype=np.float32), np.zeros(3, np.float32)
    pts = np.array([[0, 0, 1],          # centre of the image: u = 50, v = 40
                    [0, 0, 0.05],       # in front of the near plane (0.1)
                    [0, 0, 100],        # at the far plane: pz >= far is culled
                    [-0.51, 0, 1],      # u = int(-51 + 50) = int(-1.0) = -1: outside
                    [-0.505, 0, 1],     # u = int(-0.5) = 0 (truncation toward zero): inside, as in the reference
                    [0.499, 0, 1],      # u = int(99.9) = 99 < W
                    [0.5, 0, 1],        # u = 100 = W: outside
                    [0, 0.4, 1],        # v = 80 = H: outside
                    [0, 0, -1]], np.float32)   # behind the camera
    got = R.frustum_cull(pts, I, t, 100.0, 100.0, 50.0, 40.0, 100, 80, 0.1, 100.0)
    assert got.tolist() == [True, False, False, False, True, True, False, False, False]
    # a translation moves the frustum
    got = R.frustum_cull(pts[:1], I, np.array([0, 0, -0.95], np.float32), 100.0, 100.0, 50.0, 40.0, 100, 80, 0.1, 100.0)
    assert got.tolist() == [False]


def test_morton_known_answers():
    # indices (0,0,0) -> offset 2^20 on every axis: bit 20 of x, y, z -> bits 60, 61, 62
    code, centre = R.morton_codes(np.array([[0.01, 0.01, 0.01]], np.float32), 0.1)
    assert int(code[0]) == (1 << 60) | (1 << 61) | (1 << 62)
    assert np.allclose(centre, 0.05)
    # (1, 0, 0) sets bit 0; (0, 1, 0) bit 1; (0, 0, 1) bit 2; (2, 0, 0) bit 3
    base = (1 << 60) | (1 << 61) | (1 << 62)
    for p, bit in (((0.15, 0.0, 0.0), 0), ((0.0, 0.15, 0.0), 1), ((0.0, 0.0, 0.15), 2), ((0.25, 0.0, 0.0), 3)):
        code, _ = R.morton_codes(np.array([p], np.float32), 0.1)
        assert int(code[0]) == base | (1 << bit), (p, hex(int(code[0])))
    # negative coordinates: floor(-0.05 / 0.1) = -1 -> 2^20 - 1 = twenty one-bits on that axis
    code, centre = R.morton_codes(np.array([[-0.05, 0.0, 0.0]], np.float32), 0.1)
    x_bits = sum(1 << (3 * b) for b in range(20))
    assert int(code[0]) == x_bits | (1 << 61) | (1 << 62)
    assert np.isclose(centre[0, 0], -0.05)


def test_voxelize_frame_merges_points_of_a_voxel():
    xyz = np.array([[0.31, 0.0, 0.0], [0.01, 0.0, 0.0], [0.02, 0.05, 0.09], [0.39, 0.0, 0.0]], np.float32)
    rgb = np.arange(12, dtype=np.float32).reshape(4, 3)
    centres, colours, codes = R.voxelize_frame(xyz, rgb, 0.1)
    assert centres.shape == (2, 3) and np.all(np.diff(codes) > 0)
    assert np.allclose(centres[:, 0], [0.05, 0.35])
    assert colours.tolist() == [rgb[1].tolist(), rgb[0].tolist()]      # first point of each voxel in stable code order
    e = R.voxelize_frame(np.zeros((0, 3), np.float32), np.zeros((0, 3), np.float32), 0.1)
    assert e[0].shape == (0, 3) and e[2].shape == (0,)
