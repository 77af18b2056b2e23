// Append-only one-token-per-frame KV cache attention ("decode" shape) for the camera head.
//
// The reference's CausalAttention (lingbot_map/layers/attention.py:90-349), as used by the camera head
// (lingbot_map/heads/camera_head.py:284-358), keeps one K and one V token per frame in a dict cache that grows by
// torch.cat every frame, is cloned, and is never evicted (the `shape[3] > 1` guard at attention.py:307); every new
// token attends to all cached tokens and to the tokens of its own call (all-true mask, attention.py:276-283).
// Here the cache is a preallocated [capacity, H, D] fp32 buffer per K and V; one kernel appends the new rows and
// computes softmax(q k^T / sqrt(D)) v for the n_q new query tokens over `cached` old + n_q new keys, fp32 throughout
// (the reference runs its heads in fp32 with autocast off).
//
// q_len is 1 (streaming) or the number of scale frames (first call), so the work is a stream over K and V:
// HBM bound, algorithmic bytes = 2 * (cached + n_q) * H * D * 4 per call.  Grid (H, splits): a CTA owns one head
// and a contiguous range of keys; a warp takes every fourth key of the range, each lane D/32 consecutive elements;
// running maximum / sum / weighted V per (warp, query); warps are combined through shared memory, splits through
// the workspace by the last CTA of each head to arrive (counter per head).
#include <algorithm>

#include "gct_common.h"

namespace gct {
namespace {

constexpr int kDecodeMaxQ = 8;
constexpr int kDecodeWarps = 4;

template <int D>
struct LaneVec;
template <>
struct LaneVec<128> {
  using T = float4;
  static __device__ __forceinline__ float dot(const T& a, const T& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
  static __device__ __forceinline__ void axpy(T& acc, float alpha, float w, const T& v) {
    acc.x = acc.x * alpha + w * v.x; acc.y = acc.y * alpha + w * v.y; acc.z = acc.z * alpha + w * v.z; acc.w = acc.w * alpha + w * v.w;
  }
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
};
template <>
struct LaneVec<64> {
  using T = float2;
  static __device__ __forceinline__ float dot(const T& a, const T& b) { return a.x * b.x + a.y * b.y; }
  static __device__ __forceinline__ void axpy(T& acc, float alpha, float w, const T& v) {
    acc.x = acc.x * alpha + w * v.x; acc.y = acc.y * alpha + w * v.y;
  }
  static __device__ __forceinline__ T zero() { return make_float2(0.f, 0.f); }
};

struct DecodeArgs {
  const float* q;        // [n_q, H, D]
  const float* k_new;    // [n_q, H, D]
  const float* v_new;
  float* cache_k;        // [capacity, H, D]
  float* cache_v;
  int cached, n_q, heads, store, splits;
  float scale;
  float* out;            // [n_q, H, D]
  float* part;           // [H][splits][n_q][D + 2]  (acc, m, l)
  int* counters;         // [H]
};

template <int D>
__global__ void __launch_bounds__(kDecodeWarps * 32) gct_decode_attn_kernel(const DecodeArgs a) {
  using V = typename LaneVec<D>::T;
  constexpr int kPer = D / 32;
  const int h = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = a.cached + a.n_q;
  const int j0 = static_cast<int>(static_cast<long long>(split) * total / a.splits);
  const int j1 = static_cast<int>(static_cast<long long>(split + 1) * total / a.splits);
  const size_t row_stride = static_cast<size_t>(a.heads) * D;
  const size_t head_off = static_cast<size_t>(h) * D + lane * kPer;

  V q[kDecodeMaxQ], acc[kDecodeMaxQ];
  float m[kDecodeMaxQ], l[kDecodeMaxQ];
#pragma unroll
  for (int i = 0; i < kDecodeMaxQ; ++i) {
    q[i] = i < a.n_q ? *reinterpret_cast<const V*>(a.q + i * row_stride + head_off) : LaneVec<D>::zero();
    acc[i] = LaneVec<D>::zero();
    m[i] = -INFINITY;
    l[i] = 0.f;
  }
  // the append: the first split of each head stores the new rows (every CTA reads them from k_new / v_new)
  if (a.store && split == 0 && warp == 0) {
    for (int i = 0; i < a.n_q; ++i) {
      *reinterpret_cast<V*>(a.cache_k + (a.cached + i) * row_stride + head_off) = *reinterpret_cast<const V*>(a.k_new + i * row_stride + head_off);
      *reinterpret_cast<V*>(a.cache_v + (a.cached + i) * row_stride + head_off) = *reinterpret_cast<const V*>(a.v_new + i * row_stride + head_off);
    }
  }
  for (int j = j0 + warp; j < j1; j += kDecodeWarps) {
    const float* kp = j < a.cached ? a.cache_k + j * row_stride : a.k_new + (j - a.cached) * row_stride;
    const float* vp = j < a.cached ? a.cache_v + j * row_stride : a.v_new + (j - a.cached) * row_stride;
    const V kv = *reinterpret_cast<const V*>(kp + head_off);
    const V vv = *reinterpret_cast<const V*>(vp + head_off);
#pragma unroll
    for (int i = 0; i < kDecodeMaxQ; ++i) {
      if (i < a.n_q) {
        float s = LaneVec<D>::dot(q[i], kv);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= a.scale;
        const float mn = fmaxf(m[i], s);
        const float alpha = __expf(m[i] - mn), w = __expf(s - mn);      // exp(-inf) = 0 on the first key
        LaneVec<D>::axpy(acc[i], alpha, w, vv);
        l[i] = l[i] * alpha + w;
        m[i] = mn;
      }
    }
  }
  // ---- combine the warps of the CTA ----
  __shared__ float s_acc[kDecodeWarps][kDecodeMaxQ][D];
  __shared__ float s_ml[kDecodeWarps][kDecodeMaxQ][2];
  __shared__ int s_last;
  for (int i = 0; i < a.n_q; ++i) {
    *reinterpret_cast<V*>(&s_acc[warp][i][lane * kPer]) = acc[i];
    if (lane == 0) {
      s_ml[warp][i][0] = m[i];
      s_ml[warp][i][1] = l[i];
    }
  }
  __syncthreads();
  const size_t rec = D + 2;
  for (int idx = threadIdx.x; idx < a.n_q * D; idx += blockDim.x) {
    const int i = idx / D, d = idx - i * D;
    float mx = -INFINITY;
    for (int w = 0; w < kDecodeWarps; ++w) mx = fmaxf(mx, s_ml[w][i][0]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float f = s_ml[w][i][0] == -INFINITY ? 0.f : __expf(s_ml[w][i][0] - mx);
      num += f * s_acc[w][i][d];
      den += f * s_ml[w][i][1];
    }
    float* p = a.part + ((static_cast<size_t>(h) * a.splits + split) * a.n_q + i) * rec;
    p[d] = num;
    if (d == 0) {
      p[D] = mx;
      p[D + 1] = den;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.counters + h, 1);
    s_last = prev == a.splits - 1;
    if (s_last) a.counters[h] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- last CTA of this head: merge the splits ----
  for (int idx = threadIdx.x; idx < a.n_q * D; idx += blockDim.x) {
    const int i = idx / D, d = idx - i * D;
    float mx = -INFINITY;
    for (int s = 0; s < a.splits; ++s)
      mx = fmaxf(mx, __ldcg(a.part + ((static_cast<size_t>(h) * a.splits + s) * a.n_q + i) * rec + D));
    float num = 0.f, den = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const float* p = a.part + ((static_cast<size_t>(h) * a.splits + s) * a.n_q + i) * rec;
      const float ms = __ldcg(p + D);
      const float f = ms == -INFINITY ? 0.f : __expf(ms - mx);
      num += f * __ldcg(p + d);
      den += f * __ldcg(p + D + 1);
    }
    a.out[i * row_stride + static_cast<size_t>(h) * D + d] = num / den;
  }
}

}  // namespace

size_t decode_counter_bytes(int heads) { return (static_cast<size_t>(heads) * sizeof(int) + 255) & ~size_t(255); }
size_t decode_workspace_bytes(int heads, int head_dim, int splits) {
  return decode_counter_bytes(heads) + static_cast<size_t>(heads) * splits * kDecodeMaxQ * (head_dim + 2) * sizeof(float);
}

int launch_decode_attention(const float* q, const float* k_new, const float* v_new, int n_q, float* cache_k, float* cache_v,
                            int cached, int capacity, int store, int heads, int head_dim, float* out, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream) {
  if (q == nullptr || k_new == nullptr || v_new == nullptr || cache_k == nullptr || cache_v == nullptr || out == nullptr ||
      workspace == nullptr)
    return fail(GCT_ERR_INVALID, "decode attention: null argument");
  if (head_dim != 64 && head_dim != 128) return fail(GCT_ERR_INVALID, "decode attention: head_dim must be 64 or 128");
  if (n_q < 1 || n_q > kDecodeMaxQ) return fail(GCT_ERR_INVALID, "decode attention: 1..8 new tokens per call");
  if (heads < 1 || cached < 0 || capacity < cached + (store ? n_q : 0))
    return fail(GCT_ERR_CAPACITY, "decode attention: cache capacity of " + std::to_string(capacity) + " rows exceeded");
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(q) || misaligned(k_new) || misaligned(v_new) || misaligned(cache_k) || misaligned(cache_v) || misaligned(out) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(GCT_ERR_INVALID, "decode attention: tensors must be 16-byte aligned, the workspace 256-byte aligned");
  int dev = 0, sms = 148;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  GCT_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int total = cached + n_q;
  // enough CTAs for two per SM, at least 64 keys each
  int splits = std::max(1, std::min((2 * sms + heads - 1) / heads, (total + 63) / 64));
  while (splits > 1 && decode_workspace_bytes(heads, head_dim, splits) > workspace_bytes) --splits;
  if (decode_workspace_bytes(heads, head_dim, splits) > workspace_bytes)
    return fail(GCT_ERR_CAPACITY, "decode attention: workspace too small");
  DecodeArgs a;
  a.q = q;
  a.k_new = k_new;
  a.v_new = v_new;
  a.cache_k = cache_k;
  a.cache_v = cache_v;
  a.cached = cached;
  a.n_q = n_q;
  a.heads = heads;
  a.store = store;
  a.splits = splits;
  a.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  a.out = out;
  a.counters = static_cast<int*>(workspace);                       // zeroed by the caller once; the kernel rezeroes
  a.part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + decode_counter_bytes(heads));
  const dim3 grid(heads, splits);
  if (head_dim == 128)
    gct_decode_attn_kernel<128><<<grid, kDecodeWarps * 32, 0, stream>>>(a);
  else
    gct_decode_attn_kernel<64><<<grid, kDecodeWarps * 32, 0, stream>>>(a);
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

}  // namespace gct

extern "C" {

int gct_decode_workspace_bytes(int heads, int head_dim, size_t* bytes_out) {
  if (heads < 1 || (head_dim != 64 && head_dim != 128) || bytes_out == nullptr)
    return gct::fail(GCT_ERR_INVALID, "gct_decode_workspace_bytes: bad argument");
  *bytes_out = gct::decode_workspace_bytes(heads, head_dim, 32);
  return GCT_OK;
}

int gct_decode_attention(const float* q_dev, const float* k_new_dev, const float* v_new_dev, int n_new, float* cache_k_dev,
                         float* cache_v_dev, int cached, int capacity, int store, int heads, int head_dim, float* out_dev,
                         void* workspace_dev, size_t workspace_bytes, void* stream) {
  return gct::launch_decode_attention(q_dev, k_new_dev, v_new_dev, n_new, cache_k_dev, cache_v_dev, cached, capacity, store,
                                      heads, head_dim, out_dev, workspace_dev, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
