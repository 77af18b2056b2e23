// HBM-bound helpers around the attention kernel: fused q/k LayerNorm + RoPE + bf16 cast with the
// K/V rows written straight into their cache pages, fp32->bf16 cast, split-KV merge, RoPE tables.
#include <math.h>

#include "gct_common.h"

namespace gct {
namespace {

// One warp per (token, group of four heads): lanes 8h..8h+7 own head h of the group, lane part s = lane & 7
// owns the eight consecutive elements 8s..8s+7 of the 64-wide row (one 16-byte bf16 or two 16-byte fp32
// loads), so a warp moves 512 contiguous bytes per tensor and all of q, k, v are in flight at once.
//   LayerNorm(64), eps 1e-5, affine            lingbot_map/layers/attention.py:58-59,415
//   3-D RoPE: pair (2m,2m+1) rotated by angle m lingbot_map/layers/rope.py:450-461
//   2-D RoPE: inside each 32-wide half pair (j, j+16) rotated by angle j; table entry 16*half + j
//                                              lingbot_map/layers/rope.py:134-157,191-198
//   page write of K/V rows                     lingbot_map/layers/flashinfer_cache.py:503-505,547-549
constexpr int kHeadsPerWarp = 4;

struct Row8 {
  float v[8];
};

__device__ __forceinline__ Row8 load8(const void* base, int dtype, size_t elem) {
  Row8 r;
  if (dtype == GCT_F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem + 4);
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      r.v[2 * i] = f.x;
      r.v[2 * i + 1] = f.y;
    }
  }
  return r;
}

__device__ __forceinline__ void store8(__nv_bfloat16* dst, const Row8& r) {
  uint4 u;
  __nv_bfloat162 p0 = __floats2bfloat162_rn(r.v[0], r.v[1]), p1 = __floats2bfloat162_rn(r.v[2], r.v[3]);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(r.v[4], r.v[5]), p3 = __floats2bfloat162_rn(r.v[6], r.v[7]);
  u.x = *reinterpret_cast<uint32_t*>(&p0);
  u.y = *reinterpret_cast<uint32_t*>(&p1);
  u.z = *reinterpret_cast<uint32_t*>(&p2);
  u.w = *reinterpret_cast<uint32_t*>(&p3);
  *reinterpret_cast<uint4*>(dst) = u;
}

// sum over the eight lanes of a row
__device__ __forceinline__ float row_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

// cs: the eight (cos, sin) pairs this lane needs.  3-D: entries 4s..4s+3 (pairs of its 8 elements), only
// cs[0..3] used.  2-D: entries 16*half + 8*(s&1) + i for its elements i = 0..7.
__device__ __forceinline__ void norm_rope8(Row8& x, const float* w, const float* bia, const float2 (&cs)[8],
                                           int rope_mode, int part) {
  if (w != nullptr) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += x.v[i];
    const float mean = row_sum(sum) * (1.f / 64.f);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x.v[i] -= mean;
      sq += x.v[i] * x.v[i];
    }
    const float rstd = rsqrtf(row_sum(sq) * (1.f / 64.f) + 1e-5f);
    const float4 w0 = *reinterpret_cast<const float4*>(w + 8 * part), w1 = *reinterpret_cast<const float4*>(w + 8 * part + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(bia + 8 * part), b1 = *reinterpret_cast<const float4*>(bia + 8 * part + 4);
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) x.v[i] = x.v[i] * rstd * ww[i] + bb[i];
  }
  if (rope_mode == GCT_ROPE_3D) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = x.v[2 * i] * cs[i].x - x.v[2 * i + 1] * cs[i].y;
      const float b = x.v[2 * i] * cs[i].y + x.v[2 * i + 1] * cs[i].x;
      x.v[2 * i] = a;
      x.v[2 * i + 1] = b;
    }
  } else if (rope_mode == GCT_ROPE_2D) {
    // element e' = 8*(part & 3) + i inside its 32-wide half; its partner e' +/- 16 lives two lanes away.
    // First 16 of a half: out = x*cos - partner*sin; last 16: out = x*cos + partner*sin.
    const float sgn = (part & 2) ? 1.f : -1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, x.v[i], 2);
      x.v[i] = x.v[i] * cs[i].x + sgn * partner * cs[i].y;
    }
  }
}

__global__ void __launch_bounds__(256) gct_prep_kernel(const PrepLaunch p) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int part = lane & 7;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int head_groups = (p.heads + kHeadsPerWarp - 1) / kHeadsPerWarp;
  const int token = wid / head_groups;
  if (token >= p.tokens) return;
  const int h = (wid - token * head_groups) * kHeadsPerWarp + (lane >> 3);
  const bool active = h < p.heads;          // inactive lanes still take part in the shuffles
  const int hh = active ? h : p.heads - 1;
  const int tf = token % p.tokens_per_frame;

  // rotation coefficients of this lane
  float2 cs[8];
  if (p.rope_mode == GCT_ROPE_3D) {
    const float4* t = reinterpret_cast<const float4*>(p.rope_cs + (static_cast<size_t>(tf) * 32 + 4 * part) * 2);
    const float4 a = t[0], b = t[1];
    cs[0] = make_float2(a.x, a.y);
    cs[1] = make_float2(a.z, a.w);
    cs[2] = make_float2(b.x, b.y);
    cs[3] = make_float2(b.z, b.w);
  } else if (p.rope_mode == GCT_ROPE_2D) {
    const int entry = (part >> 2) * 16 + (part & 1) * 8;      // 16*half + (e' % 16) for this lane's first element
    const float4* t = reinterpret_cast<const float4*>(p.rope_cs + (static_cast<size_t>(tf) * 32 + entry) * 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 a = t[i];
      cs[2 * i] = make_float2(a.x, a.y);
      cs[2 * i + 1] = make_float2(a.z, a.w);
    }
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

  const size_t src = static_cast<size_t>(token) * p.src_token_stride + static_cast<size_t>(hh) * p.src_head_stride +
                     8 * part;
  const size_t dst = static_cast<size_t>(hh) * kHeadDim + 8 * part;
  const bool do_q = p.q_src != nullptr && p.q_out != nullptr;
  const bool do_kv = k_row != nullptr;
  Row8 q, k, v;
  if (do_q) q = load8(p.q_src, p.src_dtype_qk, src);
  if (do_kv) {
    k = load8(p.k_src, p.src_dtype_qk, src);
    v = load8(p.v_src, p.src_dtype_v, src);
  }
  if (do_q) {
    norm_rope8(q, p.qn_w, p.qn_b, cs, p.rope_mode, part);
    if (active) store8(p.q_out + static_cast<size_t>(token) * p.heads * kHeadDim + dst, q);
  }
  if (do_kv) {
    norm_rope8(k, p.kn_w, p.kn_b, cs, p.rope_mode, part);
    if (active) {
      store8(k_row + dst, k);
      store8(v_row + dst, v);
    }
    if (p.key_norm_max != nullptr) {
      // running maximum of |k| per head (an upper bound: fp32 values, inflated for the bf16 rounding).  Positive
      // floats order like their bit patterns; the plain read first keeps atomics rare once the maximum settles.
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sq += k.v[i] * k.v[i];
      const float nrm = sqrtf(row_sum(sq)) * 1.004f;
      if (active && part == 0) {
        unsigned int* slot = reinterpret_cast<unsigned int*>(p.key_norm_max + hh);
        if (!(nrm <= __uint_as_float(*reinterpret_cast<volatile unsigned int*>(slot))))   // also taken for NaN
          atomicMax(slot, nrm == nrm ? __float_as_uint(nrm) : 0x7f800000u);
      }
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
  pdl_wait();
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

// Eight lanes per K row of the pool (16 bytes each), four rows per warp and load, four loads in flight per lane.
__global__ void __launch_bounds__(256)
gct_scan_keys_kernel(const __nv_bfloat16* __restrict__ pool, int64_t total_rows, int page_size, int heads,
                     float* key_norm_max) {
  const int lane = threadIdx.x & 31, part = lane & 7, sub = lane >> 3;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t rows_per_page = static_cast<int64_t>(page_size) * heads;
  constexpr int kUnroll = 4;
  for (int64_t base = ((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * (4 * kUnroll);
       base < total_rows; base += warps * (4 * kUnroll)) {
    uint4 v[kUnroll];
    int head[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t r = base + 4 * u + sub;
      const int64_t rr = r < total_rows ? r : total_rows - 1;          // tail: repeat the last row
      const int64_t page = rr / rows_per_page, in_page = rr - page * rows_per_page;
      head[u] = static_cast<int>(in_page % heads);
      v[u] = *reinterpret_cast<const uint4*>(pool + (page * 2 * rows_per_page + in_page) * kHeadDim + 8 * part);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        sq += f.x * f.x + f.y * f.y;
      }
      sq = row_sum(sq);
      if (part == 0) {
        const float nrm = sqrtf(sq);
        unsigned int* slot = reinterpret_cast<unsigned int*>(key_norm_max + head[u]);
        if (!(nrm <= __uint_as_float(*reinterpret_cast<volatile unsigned int*>(slot))))
          atomicMax(slot, nrm == nrm ? __float_as_uint(nrm) : 0x7f800000u);
      }
    }
  }
}

// cs[token][m] = (cos, sin) of the m-th complex frequency; fp64 angles as the reference's table
// (lingbot_map/layers/rope.py:326-334,399-413): m<10 time (dim 20), m<21 height (dim 22), else width (dim 22).
__global__ void gct_rope3d_table_kernel(int f, int pph, int ppw, int ns, float* cs) {
  pdl_wait();
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
  if ((p.src_token_stride | p.src_head_stride) & 7)
    return fail(GCT_ERR_INVALID, "prep: source strides must be multiples of 8 elements (16-byte vector loads)");
  auto misaligned = [](const void* q) { return q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
  if (misaligned(p.q_src) || misaligned(p.k_src) || misaligned(p.v_src) || misaligned(p.q_out) || misaligned(p.k_out) ||
      misaligned(p.v_out) || misaligned(p.pool) || misaligned(p.qn_w) || misaligned(p.qn_b) || misaligned(p.kn_w) ||
      misaligned(p.kn_b) || misaligned(p.rope_cs))
    return fail(GCT_ERR_INVALID, "prep: tensors must be 16-byte aligned");
  const int head_groups = (p.heads + kHeadsPerWarp - 1) / kHeadsPerWarp;
  const long long warps = static_cast<long long>(p.tokens) * head_groups;
  const int blocks = static_cast<int>((warps * 32 + 255) / 256);
  GCT_CUDA_CHECK(launch_pdl(gct_prep_kernel, dim3(blocks), dim3(256), 0, stream, p));
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
  GCT_CUDA_CHECK(launch_pdl(gct_merge_kernel, dim3(blocks), dim3(256), 0, stream, parts, lse, groups, rows, parts_stride,
                            lse_stride, out_bf16, out_f32, lse_out));
  return GCT_OK;
}

int launch_scan_keys(const __nv_bfloat16* pool, int num_pages, int page_size, int heads, float* key_norm_max,
                     cudaStream_t stream) {
  if (pool == nullptr || key_norm_max == nullptr || num_pages <= 0 || page_size <= 0 || heads <= 0)
    return fail(GCT_ERR_INVALID, "scan_keys: bad argument");
  GCT_CUDA_CHECK(cudaMemsetAsync(key_norm_max, 0, static_cast<size_t>(heads) * sizeof(float), stream));
  const int64_t total_rows = static_cast<int64_t>(num_pages) * page_size * heads;
  gct_scan_keys_kernel<<<148 * 8, 256, 0, stream>>>(pool, total_rows, page_size, heads, key_norm_max);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

int launch_rope3d_table(int f, int pph, int ppw, int ns, float* cs, cudaStream_t stream) {
  const int n = (ns + pph * ppw) * 32;
  GCT_CUDA_CHECK(launch_pdl(gct_rope3d_table_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, f, pph, ppw, ns, cs));
  return GCT_OK;
}

int launch_rope2d_table(int pph, int ppw, int ns, float base, float* cs, cudaStream_t stream) {
  const int n = (ns + pph * ppw) * 32;
  gct_rope2d_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(pph, ppw, ns, base, cs);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

}  // namespace gct
