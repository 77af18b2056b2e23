// Point-cloud helpers of the offline renderer as plain CUDA: frustum culling and Morton voxelisation.
//
// Restates demo_render/render_cuda_ext/frustum_cull/frustum_cull.cu:5-33 and
// demo_render/render_cuda_ext/voxel_morton/voxel_morton.cu:5-62 of the reference (compute only; the renderer that
// consumes them needs a graphics API and is not part of this library).  Both are streams over AoS xyz floats:
// HBM bound, 13 B per point (cull) and 24 B read + 44 B written per point (voxelise).  A thread takes four points
// = three 16-byte loads, so a warp reads 1536 contiguous bytes; the tail is done point by point.
// Arithmetic is written with explicitly rounded single operations (no fused multiply-add, IEEE division), so that
// a float32 CPU restatement reproduces every mask bit and every Morton code exactly.
#include "gct_common.h"

namespace gct {
namespace {

struct CullArgs {
  float R[9], t[3];
  float fx, fy, cx, cy, near_plane, far_plane;
  int W, H;
};

__device__ __forceinline__ bool cull_one(float x, float y, float z, const CullArgs& a) {
  const float px = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(a.R[0], x), __fmul_rn(a.R[1], y)), __fmul_rn(a.R[2], z)), a.t[0]);
  const float py = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(a.R[3], x), __fmul_rn(a.R[4], y)), __fmul_rn(a.R[5], z)), a.t[1]);
  const float pz = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(a.R[6], x), __fmul_rn(a.R[7], y)), __fmul_rn(a.R[8], z)), a.t[2]);
  if (pz <= a.near_plane || pz >= a.far_plane) return false;            // frustum_cull.cu:25-28 (NaN depth: kept there too)
  const float fu = __fadd_rn(__fmul_rn(__fdiv_rn(px, pz), a.fx), a.cx);
  const float fv = __fadd_rn(__fmul_rn(__fdiv_rn(py, pz), a.fy), a.cy);
  // (int) of a float outside the int range is undefined in C; such points are outside every image
  if (!(fu > -2147483648.f && fu < 2147483648.f && fv > -2147483648.f && fv < 2147483648.f)) return false;
  const int u = static_cast<int>(fu), v = static_cast<int>(fv);       // truncation toward zero, as the reference
  return u >= 0 && u < a.W && v >= 0 && v < a.H;
}

__global__ void __launch_bounds__(256) gct_frustum_cull_kernel(const float* __restrict__ pts, CullArgs a, uint8_t* __restrict__ visible,
                                                               int64_t n) {
  const int64_t quads = n / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t qd = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; qd < quads; qd += stride) {
    const float4* p = reinterpret_cast<const float4*>(pts) + 3 * qd;
    const float4 a0 = p[0], a1 = p[1], a2 = p[2];                      // x0 y0 z0 x1 | y1 z1 x2 y2 | z2 x3 y3 z3
    uchar4 m;
    m.x = cull_one(a0.x, a0.y, a0.z, a);
    m.y = cull_one(a0.w, a1.x, a1.y, a);
    m.z = cull_one(a1.z, a1.w, a2.x, a);
    m.w = cull_one(a2.y, a2.z, a2.w, a);
    reinterpret_cast<uchar4*>(visible)[qd] = m;
  }
  if (blockIdx.x == 0 && threadIdx.x < n - 4 * quads) {
    const int64_t i = 4 * quads + threadIdx.x;
    visible[i] = cull_one(pts[3 * i], pts[3 * i + 1], pts[3 * i + 2], a);
  }
}

// Interleave the low 21 bits of x, y, z (voxel_morton.cu:5-18).
__device__ __forceinline__ uint64_t expand_bits(uint64_t v) {
  v = (v | (v << 32)) & 0x1f00000000ffffULL;
  v = (v | (v << 16)) & 0x1f0000ff0000ffULL;
  v = (v | (v << 8)) & 0x100f00f00f00f00fULL;
  v = (v | (v << 4)) & 0x10c30c30c30c30c3ULL;
  v = (v | (v << 2)) & 0x1249249249249249ULL;
  return v;
}

__global__ void __launch_bounds__(256) gct_voxel_morton_kernel(const float* __restrict__ xyz, const float* __restrict__ rgb,
                                                               float voxel_size, int64_t n, int64_t* __restrict__ codes,
                                                               float* __restrict__ centers, float* __restrict__ colors) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = xyz[3 * i], y = xyz[3 * i + 1], z = xyz[3 * i + 2];
    const int ix = static_cast<int>(floorf(__fdiv_rn(x, voxel_size)));
    const int iy = static_cast<int>(floorf(__fdiv_rn(y, voxel_size)));
    const int iz = static_cast<int>(floorf(__fdiv_rn(z, voxel_size)));
    constexpr int kOffset = 1 << 20;                                   // voxel_morton.cu:36-38
    const uint64_t code = expand_bits(static_cast<uint64_t>(static_cast<uint32_t>(ix + kOffset))) |
                          (expand_bits(static_cast<uint64_t>(static_cast<uint32_t>(iy + kOffset))) << 1) |
                          (expand_bits(static_cast<uint64_t>(static_cast<uint32_t>(iz + kOffset))) << 2);
    codes[i] = static_cast<int64_t>(code);
    centers[3 * i] = __fmul_rn(__fadd_rn(static_cast<float>(ix), 0.5f), voxel_size);
    centers[3 * i + 1] = __fmul_rn(__fadd_rn(static_cast<float>(iy), 0.5f), voxel_size);
    centers[3 * i + 2] = __fmul_rn(__fadd_rn(static_cast<float>(iz), 0.5f), voxel_size);
    colors[3 * i] = rgb[3 * i];
    colors[3 * i + 1] = rgb[3 * i + 1];
    colors[3 * i + 2] = rgb[3 * i + 2];
  }
}

__global__ void __launch_bounds__(256) gct_mark_unique_kernel(const int64_t* __restrict__ sorted, int64_t n, uint8_t* __restrict__ mask) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    mask[i] = (i == 0) || (sorted[i] != sorted[i - 1]);                // voxel_morton.cu:49-62
}

int grid_for(int64_t items) {
  const int64_t blocks = (items + 255) / 256;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace
}  // namespace gct

extern "C" {

int gct_frustum_cull(const float* pts_dev, int64_t n, const float R_cw[9], const float t_cw[3], float fx, float fy, float cx,
                     float cy, int width, int height, float near_plane, float far_plane, uint8_t* visible_dev, void* stream) {
  using namespace gct;
  if (n < 0 || R_cw == nullptr || t_cw == nullptr) return fail(GCT_ERR_INVALID, "gct_frustum_cull: bad argument");
  if (n == 0) return GCT_OK;
  if (pts_dev == nullptr || visible_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_frustum_cull: null argument");
  if ((reinterpret_cast<uintptr_t>(pts_dev) & 15) || (reinterpret_cast<uintptr_t>(visible_dev) & 3))
    return fail(GCT_ERR_INVALID, "gct_frustum_cull: points must be 16-byte aligned, the mask 4-byte aligned");
  CullArgs a;
  for (int i = 0; i < 9; ++i) a.R[i] = R_cw[i];
  for (int i = 0; i < 3; ++i) a.t[i] = t_cw[i];
  a.fx = fx; a.fy = fy; a.cx = cx; a.cy = cy;
  a.near_plane = near_plane; a.far_plane = far_plane;
  a.W = width; a.H = height;
  gct_frustum_cull_kernel<<<grid_for(n / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(pts_dev, a, visible_dev, n);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int gct_voxel_morton(const float* xyz_dev, const float* rgb_dev, float voxel_size, int64_t n, int64_t* codes_dev,
                     float* centers_dev, float* colors_dev, void* stream) {
  using namespace gct;
  if (n < 0 || !(voxel_size > 0.f)) return fail(GCT_ERR_INVALID, "gct_voxel_morton: bad argument");
  if (n == 0) return GCT_OK;
  if (xyz_dev == nullptr || rgb_dev == nullptr || codes_dev == nullptr || centers_dev == nullptr || colors_dev == nullptr)
    return fail(GCT_ERR_INVALID, "gct_voxel_morton: null argument");
  gct_voxel_morton_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(xyz_dev, rgb_dev, voxel_size, n, codes_dev,
                                                                                     centers_dev, colors_dev);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int gct_mark_unique(const int64_t* sorted_dev, int64_t n, uint8_t* mask_dev, void* stream) {
  using namespace gct;
  if (n < 0) return fail(GCT_ERR_INVALID, "gct_mark_unique: bad argument");
  if (n == 0) return GCT_OK;
  if (sorted_dev == nullptr || mask_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mark_unique: null argument");
  gct_mark_unique_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(sorted_dev, n, mask_dev);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

}  // extern "C"
