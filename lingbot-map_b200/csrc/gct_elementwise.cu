// HBM-bound helpers around the attention kernel: fused q/k LayerNorm + RoPE + bf16 cast with the
// K/V rows written straight into their cache pages, fp32->bf16 cast, split-KV merge, RoPE tables.
#include <math.h>

#include "gct_common.h"

namespace gct {
namespace {

__device__ __forceinline__ float2 load2(const void* base, int dtype, size_t elem) {
  if (dtype == GCT_F32) {
    return *reinterpret_cast<const float2*>(static_cast<const float*>(base) + elem);
  }
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(base) + elem);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// One warp per (token, group of heads); lane m owns elements (2m, 2m+1) of each 64-wide row.
//   LayerNorm(64), eps 1e-5, affine            lingbot_map/layers/attention.py:58-59,415
//   3-D RoPE: pair (2m,2m+1) rotated by angle m lingbot_map/layers/rope.py:450-461
//   2-D RoPE: inside each 32-wide half pair (j, j+16) rotated by angle j; table entry 16*half + j
//                                              lingbot_map/layers/rope.py:134-157,191-198
//   page write of K/V rows                     lingbot_map/layers/flashinfer_cache.py:503-505,547-549
constexpr int kHeadsPerWarp = 4;

__device__ __forceinline__ float2 norm_rope(float2 x, const float* w, const float* bia, float2 cs_mine,
                                            float2 cs_2d, int rope_mode, int lane) {
  if (w != nullptr) {
    const float mean = warp_sum(x.x + x.y) * (1.f / 64.f);
    const float dx = x.x - mean, dy = x.y - mean;
    const float var = warp_sum(dx * dx + dy * dy) * (1.f / 64.f);
    const float rstd = rsqrtf(var + 1e-5f);
    const float2 ww = *reinterpret_cast<const float2*>(w + 2 * lane);
    const float2 bb = *reinterpret_cast<const float2*>(bia + 2 * lane);
    x.x = dx * rstd * ww.x + bb.x;
    x.y = dy * rstd * ww.y + bb.y;
  }
  if (rope_mode == GCT_ROPE_3D) {
    const float c = cs_mine.x, s = cs_mine.y;
    const float a = x.x * c - x.y * s;
    const float b = x.x * s + x.y * c;
    x.x = a;
    x.y = b;
  } else if (rope_mode == GCT_ROPE_2D) {
    // lane m holds elements e = 2m, 2m+1; inside the half (e % 32) the partner of e is e +/- 16,
    // i.e. lane m ^ 8.  First 16 of a half: out = x*cos - partner*sin; last 16: out = x*cos + partner*sin.
    const float px = __shfl_xor_sync(0xffffffffu, x.x, 8);
    const float py = __shfl_xor_sync(0xffffffffu, x.y, 8);
    const bool upper = (lane & 8) != 0;
    // angle index for element e: 16*half + (e % 16); elements 2m and 2m+1 use consecutive angles
    const float sgn = upper ? 1.f : -1.f;
    x.x = x.x * cs_mine.x + sgn * px * cs_mine.y;
    x.y = x.y * cs_2d.x + sgn * py * cs_2d.y;
  }
  return x;
}

__global__ void __launch_bounds__(256) gct_prep_kernel(const PrepLaunch p) {
  const int lane = threadIdx.x & 31;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int head_groups = (p.heads + kHeadsPerWarp - 1) / kHeadsPerWarp;
  const int token = wid / head_groups;
  if (token >= p.tokens) return;
  const int h0 = (wid - token * head_groups) * kHeadsPerWarp;
  const int tf = token % p.tokens_per_frame;

  // rotation coefficients of this lane
  float2 cs_mine = make_float2(1.f, 0.f), cs_2d = make_float2(1.f, 0.f);
  if (p.rope_mode == GCT_ROPE_3D) {
    cs_mine = *reinterpret_cast<const float2*>(p.rope_cs + (static_cast<size_t>(tf) * 32 + lane) * 2);
  } else if (p.rope_mode == GCT_ROPE_2D) {
    const int half = lane >> 4;                 // elements 2m,2m+1 < 32 -> vertical half, else horizontal
    const int j0 = (2 * lane) & 15;             // angle index inside the half for element 2m
    cs_mine = *reinterpret_cast<const float2*>(p.rope_cs + (static_cast<size_t>(tf) * 32 + half * 16 + j0) * 2);
    cs_2d = *reinterpret_cast<const float2*>(p.rope_cs + (static_cast<size_t>(tf) * 32 + half * 16 + j0 + 1) * 2);
  }

  // destination rows of K and V for this token
  __nv_bfloat16* k_row = nullptr;
  __nv_bfloat16* v_row = nullptr;
  if (p.k_out != nullptr) {
    k_row = p.k_out + static_cast<size_t>(token) * p.heads * kHeadDim;
    v_row = p.v_out + static_cast<size_t>(token) * p.heads * kHeadDim;
  } else if (p.pool != nullptr) {
    int page, slot;
    if (token >= p.num_special) {
      page = p.patch_page;
      slot = token - p.num_special;
    } else if (token < p.sp_n0) {
      page = p.sp_page0;
      slot = p.sp_off0 + token;
    } else {
      page = p.sp_page1;
      slot = token - p.sp_n0;
    }
    if (page < 0 || page >= p.num_pages || slot < 0 || slot >= p.page_size) {
      if (lane == 0) atomicCAS(p.status, 0, kStatusBadIndex);
      return;
    }
    const size_t page_elems = static_cast<size_t>(p.page_size) * p.heads * kHeadDim;
    k_row = p.pool + (static_cast<size_t>(page) * 2) * page_elems + static_cast<size_t>(slot) * p.heads * kHeadDim;
    v_row = k_row + page_elems;
  }

  for (int h = h0; h < min(h0 + kHeadsPerWarp, p.heads); ++h) {
    const size_t src = static_cast<size_t>(token) * p.src_token_stride + static_cast<size_t>(h) * p.src_head_stride +
                       2 * lane;
    const size_t dst = static_cast<size_t>(h) * kHeadDim + 2 * lane;
    if (p.q_src != nullptr && p.q_out != nullptr) {
      float2 x = norm_rope(load2(p.q_src, p.src_dtype_qk, src), p.qn_w, p.qn_b, cs_mine, cs_2d, p.rope_mode, lane);
      *reinterpret_cast<__nv_bfloat162*>(p.q_out + static_cast<size_t>(token) * p.heads * kHeadDim + dst) =
          __floats2bfloat162_rn(x.x, x.y);
    }
    if (k_row != nullptr) {
      float2 x = norm_rope(load2(p.k_src, p.src_dtype_qk, src), p.kn_w, p.kn_b, cs_mine, cs_2d, p.rope_mode, lane);
      *reinterpret_cast<__nv_bfloat162*>(k_row + dst) = __floats2bfloat162_rn(x.x, x.y);
      float2 y = load2(p.v_src, p.src_dtype_v, src);
      *reinterpret_cast<__nv_bfloat162*>(v_row + dst) = __floats2bfloat162_rn(y.x, y.y);
    }
  }
}

__global__ void gct_cast_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n4) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&a);
    w.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(dst)[i] = w;
  }
}

// One warp per (query, head) row; lane m owns output elements (2m, 2m+1).
//   out = sum_g w_g O_g / sum_g w_g,  w_g = exp(lse_g - max_g lse_g)
__global__ void __launch_bounds__(256)
gct_merge_kernel(const float* __restrict__ parts, const float* __restrict__ lse, int groups, int64_t rows,
                 int64_t parts_stride, int64_t lse_stride, __nv_bfloat16* __restrict__ out_bf16,
                 float* __restrict__ out_f32, float* __restrict__ lse_out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  float mx = -INFINITY;
  for (int g = 0; g < groups; ++g) mx = fmaxf(mx, lse[static_cast<int64_t>(g) * lse_stride + row]);
  float den = 0.f;
  float2 acc = make_float2(0.f, 0.f);
  for (int g = 0; g < groups; ++g) {
    const float w = __expf(lse[static_cast<int64_t>(g) * lse_stride + row] - mx);
    const float2 v = *reinterpret_cast<const float2*>(parts + static_cast<int64_t>(g) * parts_stride + row * kHeadDim + 2 * lane);
    acc.x = fmaf(w, v.x, acc.x);
    acc.y = fmaf(w, v.y, acc.y);
    den += w;
  }
  const float inv = 1.f / den;
  if (out_bf16 != nullptr)
    *reinterpret_cast<__nv_bfloat162*>(out_bf16 + row * kHeadDim + 2 * lane) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  if (out_f32 != nullptr)
    *reinterpret_cast<float2*>(out_f32 + row * kHeadDim + 2 * lane) = make_float2(acc.x * inv, acc.y * inv);
  if (lse_out != nullptr && lane == 0) lse_out[row] = mx + logf(den);
}

// cs[token][m] = (cos, sin) of the m-th complex frequency; fp64 angles as the reference's table
// (lingbot_map/layers/rope.py:326-334,399-413): m<10 time (dim 20), m<21 height (dim 22), else width (dim 22).
__global__ void gct_rope3d_table_kernel(int f, int pph, int ppw, int ns, float* cs) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int tokens = ns + pph * ppw;
  if (idx >= tokens * 32) return;
  const int token = idx >> 5, m = idx & 31;
  int ph, pw;
  if (token < ns) {
    ph = pw = token;
  } else {
    const int pidx = token - ns;
    ph = ns + pidx / ppw;
    pw = ns + pidx % ppw;
  }
  double pos, expo;
  if (m < 10) {
    pos = f;
    expo = (2.0 * m) / 20.0;
  } else if (m < 21) {
    pos = ph;
    expo = (2.0 * (m - 10)) / 22.0;
  } else {
    pos = pw;
    expo = (2.0 * (m - 21)) / 22.0;
  }
  const double ang = pos * (1.0 / pow(10000.0, expo));
  cs[2 * idx] = static_cast<float>(cos(ang));
  cs[2 * idx + 1] = static_cast<float>(sin(ang));
}

// 2-D table (lingbot_map/layers/rope.py:105-119; positions lingbot_map/aggregator/base.py:436-440):
// entry 16*axis + j holds the angle pos_axis * base^(-2j/32), computed in fp32 like the reference.
__global__ void gct_rope2d_table_kernel(int pph, int ppw, int ns, float base, float* cs) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int tokens = ns + pph * ppw;
  if (idx >= tokens * 32) return;
  const int token = idx >> 5, e = idx & 31;
  const int axis = e >> 4, j = e & 15;
  int pos = 0;
  if (token >= ns) {
    const int pidx = token - ns;
    pos = (axis == 0 ? pidx / ppw : pidx % ppw) + 1;
  }
  const float inv = 1.0f / powf(base, static_cast<float>(2 * j) / 32.0f);
  const float ang = static_cast<float>(pos) * inv;
  cs[2 * idx] = cosf(ang);
  cs[2 * idx + 1] = sinf(ang);
}

}  // namespace

int launch_prep(const PrepLaunch& p, cudaStream_t stream) {
  if (p.tokens <= 0 || p.heads <= 0 || p.tokens_per_frame <= 0) return fail(GCT_ERR_INVALID, "prep: bad shape");
  if (p.rope_mode != GCT_ROPE_NONE && p.rope_cs == nullptr) return fail(GCT_ERR_INVALID, "prep: rope table missing");
  if ((p.src_token_stride | p.src_head_stride) & 1) return fail(GCT_ERR_INVALID, "prep: odd source stride");
  const int head_groups = (p.heads + kHeadsPerWarp - 1) / kHeadsPerWarp;
  const long long warps = static_cast<long long>(p.tokens) * head_groups;
  const int blocks = static_cast<int>((warps * 32 + 255) / 256);
  gct_prep_kernel<<<blocks, 256, 0, stream>>>(p);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int launch_cast_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t stream) {
  if (n % 4 != 0) return fail(GCT_ERR_INVALID, "cast: element count must be a multiple of 4");
  const int64_t n4 = n / 4;
  const int blocks = static_cast<int>(n4 / 256 + 1 < 1184 ? n4 / 256 + 1 : 1184);
  gct_cast_kernel<<<blocks, 256, 0, stream>>>(src, dst, n4);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int launch_merge(const float* parts, const float* lse, int groups, int64_t rows, __nv_bfloat16* out_bf16,
                 float* out_f32, float* lse_out, cudaStream_t stream, int64_t parts_stride, int64_t lse_stride) {
  if (groups <= 0 || rows <= 0) return fail(GCT_ERR_INVALID, "merge: bad shape");
  if (parts_stride <= 0) parts_stride = rows * kHeadDim;
  if (lse_stride <= 0) lse_stride = rows;
  if (parts_stride % 2 != 0) return fail(GCT_ERR_INVALID, "merge: group stride of the partial outputs must be even");
  const int blocks = static_cast<int>((rows * 32 + 255) / 256);
  gct_merge_kernel<<<blocks, 256, 0, stream>>>(parts, lse, groups, rows, parts_stride, lse_stride, out_bf16, out_f32,
                                               lse_out);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int launch_rope3d_table(int f, int pph, int ppw, int ns, float* cs, cudaStream_t stream) {
  const int n = (ns + pph * ppw) * 32;
  gct_rope3d_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(f, pph, ppw, ns, cs);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int launch_rope2d_table(int pph, int ppw, int ns, float base, float* cs, cudaStream_t stream) {
  const int n = (ns + pph * ppw) * 32;
  gct_rope2d_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(pph, ppw, ns, base, cs);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

}  // namespace gct
