"""Point-cloud helpers of the reference's offline renderer on this library's kernels.

Same call signatures as demo_render/render_cuda_ext/render_cuda_ext/_api.py (`frustum_cull`, `voxelize_frame`);
the sort, gather and compaction around the Morton kernel are the same tensor-library calls the reference makes
(voxel_morton.cu:98-114 uses at::sort / index_select / nonzero).  The renderer itself (Open3D / Filament) needs a
graphics API and is not part of this package."""
import ctypes as C

import torch

from . import _lib
from .cache import _stream_ptr


def frustum_cull(pts: torch.Tensor, R_cw: torch.Tensor, t_cw: torch.Tensor, fx: float, fy: float, cx: float, cy: float,
                 W: int, H: int, near_plane: float, far_plane: float) -> torch.Tensor:
    """Visible mask [N] bool of points [N, 3] fp32 for the camera (R_cw, t_cw), frustum_cull.cu:35-53."""
    if not pts.is_cuda:
        raise RuntimeError("pts must be a CUDA tensor: there is no CPU path")
    pts = pts.contiguous().float()
    n = pts.shape[0]
    vis = torch.zeros(n, dtype=torch.uint8, device=pts.device)
    if n:
        R = (C.c_float * 9)(*[float(x) for x in R_cw.detach().float().cpu().reshape(-1).tolist()])
        t = (C.c_float * 3)(*[float(x) for x in t_cw.detach().float().cpu().reshape(-1).tolist()])
        with torch.cuda.device(pts.device):
            _lib.check(_lib.load().gct_frustum_cull(pts.data_ptr(), n, R, t, fx, fy, cx, cy, W, H, near_plane, far_plane,
                                                    vis.data_ptr(), _stream_ptr(pts.device)))
    return vis.bool()


def voxelize_frame(pts_xyz: torch.Tensor, pts_rgb: torch.Tensor, voxel_size: float):
    """(voxel centres [M, 3], colours [M, 3], Morton codes [M]) of the occupied voxels, sorted by code, the colour of
    the first point of each voxel in sorted order - voxelize_frame_cuda, voxel_morton.cu:64-117."""
    if not pts_xyz.is_cuda:
        raise RuntimeError("pts_xyz must be a CUDA tensor: there is no CPU path")
    dev = pts_xyz.device
    n = pts_xyz.shape[0]
    if n == 0:
        return (torch.zeros(0, 3, device=dev), torch.zeros(0, 3, device=dev), torch.zeros(0, dtype=torch.int64, device=dev))
    xyz, rgb = pts_xyz.contiguous().float(), pts_rgb.contiguous().float()
    codes = torch.empty(n, dtype=torch.int64, device=dev)
    centers = torch.empty(n, 3, dtype=torch.float32, device=dev)
    colors = torch.empty(n, 3, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.gct_voxel_morton(xyz.data_ptr(), rgb.data_ptr(), float(voxel_size), n, codes.data_ptr(),
                                        centers.data_ptr(), colors.data_ptr(), _stream_ptr(dev)))
        sorted_codes, order = torch.sort(codes, stable=True)      # ties: first point wins, deterministically
        centers, colors = centers.index_select(0, order), colors.index_select(0, order)
        mask = torch.empty(n, dtype=torch.uint8, device=dev)
        _lib.check(lib.gct_mark_unique(sorted_codes.data_ptr(), n, mask.data_ptr(), _stream_ptr(dev)))
    keep = torch.nonzero(mask).squeeze(1)
    return centers.index_select(0, keep), colors.index_select(0, keep), sorted_codes.index_select(0, keep)
