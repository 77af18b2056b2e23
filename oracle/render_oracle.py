"""CPU restatement of the reference's point-cloud helpers.  TEST INFRASTRUCTURE ONLY.

float32 numpy, one rounded operation at a time, following
  demo_render/render_cuda_ext/frustum_cull/frustum_cull.cu:5-33   (frustum_cull)
  demo_render/render_cuda_ext/voxel_morton/voxel_morton.cu:5-62   (morton3D, compute_morton_kernel, mark_unique_kernel)
  demo_render/render_cuda_ext/voxel_morton/voxel_morton.cu:64-117 (voxelize_frame_cuda: sort, gather, compaction).
Parity status: UNPINNED against the reference binary (it is a torch CUDA extension that cannot run in a container
without a GPU, and the reference has no test vectors for it); pinned here by hand-computed known answers
(tests/test_render_oracle.py).  The reference's build may fuse a*b+c and uses fast division for the voxel index;
results can differ from it only for points within one rounding step of an image border or a voxel face."""
import numpy as np

F = np.float32


def frustum_cull(pts, R, t, fx, fy, cx, cy, W, H, near_plane, far_plane):
    pts = np.asarray(pts, F)
    R = np.asarray(R, F).reshape(3, 3)
    t = np.asarray(t, F).reshape(3)
    x, y, z = pts[:, 0], pts[:, 1], pts[:, 2]
    cam = [((R[i, 0] * x + R[i, 1] * y).astype(F) + R[i, 2] * z).astype(F) + t[i] for i in range(3)]
    px, py, pz = (c.astype(F) for c in cam)
    inside = ~((pz <= F(near_plane)) | (pz >= F(far_plane)))
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        fu = ((px / pz).astype(F) * F(fx)).astype(F) + F(cx)
        fv = ((py / pz).astype(F) * F(fy)).astype(F) + F(cy)
    ok = np.isfinite(fu) & np.isfinite(fv) & (np.abs(fu) < 2 ** 31) & (np.abs(fv) < 2 ** 31)
    u = np.trunc(np.where(ok, fu, -1)).astype(np.int64)
    v = np.trunc(np.where(ok, fv, -1)).astype(np.int64)
    return inside & ok & (u >= 0) & (u < W) & (v >= 0) & (v < H)


def _expand_bits(v):
    v = v.astype(np.uint64)
    for shift, mask in ((32, 0x1f00000000ffff), (16, 0x1f0000ff0000ff), (8, 0x100f00f00f00f00f),
                        (4, 0x10c30c30c30c30c3), (2, 0x1249249249249249)):
        v = (v | (v << np.uint64(shift))) & np.uint64(mask)
    return v


def morton_codes(xyz, voxel_size):
    xyz = np.asarray(xyz, F)
    idx = np.floor((xyz / F(voxel_size)).astype(F)).astype(np.int64)
    off = (idx + (1 << 20)).astype(np.uint32)
    code = _expand_bits(off[:, 0]) | (_expand_bits(off[:, 1]) << np.uint64(1)) | (_expand_bits(off[:, 2]) << np.uint64(2))
    centers = ((idx.astype(F) + F(0.5)).astype(F) * F(voxel_size)).astype(F)
    return code.astype(np.int64), centers


def voxelize_frame(xyz, rgb, voxel_size):
    """(centres, colours, codes) of the occupied voxels in code order; colour of the first point in a stable sort."""
    xyz, rgb = np.asarray(xyz, F), np.asarray(rgb, F)
    if xyz.shape[0] == 0:
        return np.zeros((0, 3), F), np.zeros((0, 3), F), np.zeros((0,), np.int64)
    codes, centers = morton_codes(xyz, voxel_size)
    order = np.argsort(codes, kind="stable")
    sc = codes[order]
    keep = np.ones(sc.shape[0], bool)
    keep[1:] = sc[1:] != sc[:-1]
    return centers[order][keep], rgb[order][keep], sc[keep]
