// KV-sharded single stream: exchange and merge of the per-rank partial attention results over peer memory.
//
// Every rank attends over its slice of the visible page list and is left with S split-KV partials
// (normalised outputs + natural log-sum-exps) for all R = n_q * H rows.  The reference is single-GPU, so there is
// no counterpart; the semantics to reproduce are those of one attention pass over the union of the slices
// (lingbot_map/layers/flashinfer_cache.py:385-421).
//
// One kernel per layer and rank, two phases, plain loads and stores on peer-mapped addresses over NVLink:
//   phase 1  for every peer p: merge my S local partials of the rows in p's row slice and store the record
//            [O(64) | lse] into slot `rank` of p's receive buffer; the last CTA to finish raises flag1[rank] on every
//            peer.
//   phase 2  wait until flag1[r] of every rank r has reached this call's epoch; merge the W records of MY row slice
//            (log-sum-exp weights), round to bf16 and store the rows into every rank's output buffer; the last CTA to
//            finish raises flag2[rank] on every peer and CTA 0 waits for all flag2, so that the kernel's end on a
//            stream means the whole output has landed locally.
// Ordering: data stores -> CTA barrier -> one thread's system-scope fence -> CTA counter -> (last CTA) fence ->
// relaxed system-scope flag stores; on the other side relaxed polls of all flags, then one fence, then the CTA
// barrier.  One fence per batch of flags instead of a release / acquire per flag.
// Row slices are contiguous: rank r owns rows [r*R/W, (r+1)*R/W).  Each rank sends (W-1)/W of one record and one
// bf16 slice per peer instead of a whole record to everybody.
// Flags are epoch counters (monotonic per exchange object), never reset.  Every wait is bounded: on a timeout the
// kernel writes kStatusWaitTimeout to the status word and returns.  The grid is limited to what is co-resident on
// the device, since CTAs of different ranks wait on each other.
#include <algorithm>
#include <mutex>

#include "gct_common.h"

namespace gct {
namespace {

constexpr int kMaxWorld = 16;
constexpr long long kXchgWaitCycles = 4000000000LL;   // ~2 s

struct ExchangeArgs {
  const float* parts;     // [S][R][64] normalised partial outputs of this rank (null: this rank has no pages)
  const float* lses;      // [S][R]
  int splits;
  int rows;               // R
  int rank, world;
  int epoch;
  float* recv[kMaxWorld];           // rank r's receive buffer: [W][slice_max][64] floats, then [W][slice_max] lse
  __nv_bfloat16* out[kMaxWorld];    // rank r's output [R][64] bf16
  int* flags[kMaxWorld];            // rank r's flag words: flag1[W], flag2[W], then two CTA counters
  int slice_max;
  int* status;
};

// Flag traffic is relaxed at system scope; ordering comes from one system-scope fence before a batch of flag stores
// and one after a batch of flag polls (a release store or an acquire load per flag would pay a fence each, `world`
// times in a row).
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until all `world` flags at `f` have reached `epoch`, then fence (acquire side).  One thread polls, all flags
// per round (independent loads, one round trip); returns false on a timeout.
__device__ bool wait_flags(const int* f, int world, int epoch, int* status) {
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    int behind = 0;
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < world) behind |= (ld_relaxed_sys(f + r) - epoch) >> 31;   // epochs only grow; the difference handles wrap-around
    if (behind == 0) break;
    if ((it & 255u) == 0u) {
      if (clock64() - t0 > kXchgWaitCycles || *reinterpret_cast<volatile int*>(status) != 0) {
        atomicCAS(status, 0, kStatusWaitTimeout);
        return false;
      }
      __nanosleep(100);
    }
  }
  __threadfence_system();
  return true;
}

// Called by one thread of every CTA after the CTA's barrier: counts the CTA in; the last one to arrive publishes
// `epoch` in slot `rank` of every peer's flag row.  The fence before the count makes this CTA's stores (its other
// threads' stores reached this thread through the barrier) visible at system scope before the count can be seen,
// the fences around the publication chain that to the flag stores.
__device__ void count_in_and_publish(int* counter, int* const* flags, int slot, int world, int epoch) {
  __threadfence_system();
  const int prev = atomicAdd(counter, 1);
  if (prev == static_cast<int>(gridDim.x) - 1) {
    *counter = 0;
    __threadfence_system();
    for (int p = 0; p < world; ++p) st_relaxed_sys(flags[p] + slot, epoch);
  }
}

// A half-warp per row: 16 lanes x float4 = the 64 output elements; two rows per warp are in flight at once.
__global__ void __launch_bounds__(256, 4) gct_kv_exchange_kernel(const ExchangeArgs a) {
  __shared__ int s_flag;
  const int lane = threadIdx.x & 15;
  const int halves_per_cta = blockDim.x >> 4;
  const int ghalf = blockIdx.x * halves_per_cta + (threadIdx.x >> 4);
  const int nhalves = gridDim.x * halves_per_cta;
  const int R = a.rows, W = a.world;
  int* my_flags = a.flags[a.rank];
  int* counters = my_flags + 2 * W;
  pdl_wait();      // the attention kernel's partials (and everything earlier in the stream) are complete from here on

  // ---- phase 1: my partial of every row goes to the rank that owns the row ----
  for (int row = ghalf; row < R; row += nhalves) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float lse = -INFINITY;
    if (a.parts != nullptr) {
      float mx = -INFINITY;
      for (int s = 0; s < a.splits; ++s) mx = fmaxf(mx, a.lses[static_cast<size_t>(s) * R + row]);
      float den = 0.f;
      for (int s = 0; s < a.splits; ++s) {
        const float w = __expf(a.lses[static_cast<size_t>(s) * R + row] - mx);
        const float4 v = *reinterpret_cast<const float4*>(a.parts + (static_cast<size_t>(s) * R + row) * kHeadDim + 4 * lane);
        acc.x = fmaf(w, v.x, acc.x);
        acc.y = fmaf(w, v.y, acc.y);
        acc.z = fmaf(w, v.z, acc.z);
        acc.w = fmaf(w, v.w, acc.w);
        den += w;
      }
      const float inv = 1.f / den;
      acc.x *= inv;
      acc.y *= inv;
      acc.z *= inv;
      acc.w *= inv;
      lse = mx + __logf(den);
    }
    // owner of the row: the p with p*R/W <= row < (p+1)*R/W
    int p = static_cast<int>((static_cast<long long>(row) * W + W - 1) / R);
    if (p > W - 1) p = W - 1;
    while (p > 0 && static_cast<long long>(p) * R / W > row) --p;
    while (p + 1 < W && static_cast<long long>(p + 1) * R / W <= row) ++p;
    const int r0 = static_cast<int>(static_cast<long long>(p) * R / W);
    float* rbuf = a.recv[p];
    const size_t slot = static_cast<size_t>(a.rank) * a.slice_max + (row - r0);
    *reinterpret_cast<float4*>(rbuf + slot * kHeadDim + 4 * lane) = acc;
    if (lane == 0) rbuf[static_cast<size_t>(W) * a.slice_max * kHeadDim + slot] = lse;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA to get here publishes: everything this rank sent is visible before the flag
    count_in_and_publish(counters + 0, a.flags, a.rank, W, a.epoch);
    s_flag = wait_flags(my_flags, W, a.epoch, a.status) ? 1 : 0;
  }
  __syncthreads();
  if (s_flag == 0) return;

  // ---- phase 2: merge the W records of my row slice, bf16, to every rank's output ----
  const int r0 = static_cast<int>(static_cast<long long>(a.rank) * R / W);
  const int r1 = static_cast<int>(static_cast<long long>(a.rank + 1) * R / W);
  const float* rbuf = a.recv[a.rank];
  const float* rlse = rbuf + static_cast<size_t>(W) * a.slice_max * kHeadDim;
  for (int i = ghalf; i < r1 - r0; i += nhalves) {
    // independent loads first (one round trip per batch), then the arithmetic
    float ls[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) ls[r] = (r < W) ? __ldcg(rlse + static_cast<size_t>(r) * a.slice_max + i) : -INFINITY;
    float mx = -INFINITY;
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) mx = fmaxf(mx, ls[r]);
    float den = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int base = 0; base < kMaxWorld; base += 8) {
      if (base >= W) break;
      float4 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        v[r] = (base + r < W) ? __ldcg(reinterpret_cast<const float4*>(rbuf + (static_cast<size_t>(base + r) * a.slice_max + i) * kHeadDim + 4 * lane))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float w = (base + r < W) ? __expf(ls[base + r] - mx) : 0.f;   // exp(-inf) = 0: empty shard
        acc.x = fmaf(w, v[r].x, acc.x);
        acc.y = fmaf(w, v[r].y, acc.y);
        acc.z = fmaf(w, v[r].z, acc.z);
        acc.w = fmaf(w, v[r].w, acc.w);
        den += w;
      }
    }
    const float inv = 1.f / den;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    for (int p = 0; p < W; ++p)
      *reinterpret_cast<uint2*>(a.out[p] + static_cast<size_t>(r0 + i) * kHeadDim + 4 * lane) = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    count_in_and_publish(counters + 1, a.flags, W + a.rank, W, a.epoch);
    // the kernel ends on this rank only when every rank's slice has landed here (one CTA waits; a grid ends when
    // all of its CTAs have)
    if (blockIdx.x == 0) wait_flags(my_flags + W, W, a.epoch, a.status);
  }
}

}  // namespace

int launch_kv_exchange(const float* parts, const float* lses, int splits, int rows, int rank, int world, int epoch,
                       void* const* recv_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int slice_max, int* status,
                       cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return fail(GCT_ERR_INVALID, "exchange: bad rank / world");
  if (rows <= 0 || slice_max < (rows + world - 1) / world) return fail(GCT_ERR_INVALID, "exchange: receive slots too small");
  if ((parts == nullptr) != (lses == nullptr) || (parts != nullptr && splits < 1))
    return fail(GCT_ERR_INVALID, "exchange: partials and log-sum-exps must come together");
  if (status == nullptr || recv_ptrs == nullptr || out_ptrs == nullptr || flag_ptrs == nullptr)
    return fail(GCT_ERR_INVALID, "exchange: null argument");
  ExchangeArgs a;
  a.parts = parts;
  a.lses = lses;
  a.splits = splits;
  a.rows = rows;
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.slice_max = slice_max;
  a.status = status;
  for (int r = 0; r < world; ++r) {
    if (recv_ptrs[r] == nullptr || out_ptrs[r] == nullptr || flag_ptrs[r] == nullptr)
      return fail(GCT_ERR_INVALID, "exchange: null peer pointer");
    a.recv[r] = static_cast<float*>(recv_ptrs[r]);
    a.out[r] = static_cast<__nv_bfloat16*>(out_ptrs[r]);
    a.flags[r] = static_cast<int*>(flag_ptrs[r]);
  }
  // CTAs of different ranks wait on each other: launch no more than fit on the device at once
  int dev = 0, sms = 0, per_sm = 0;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  GCT_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  GCT_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gct_kv_exchange_kernel, 256, 0));
  if (per_sm < 1) return fail(GCT_ERR_CUDA, "exchange: kernel does not fit on an SM");
  const int grid = std::min(sms * std::min(per_sm, 4), (rows + 15) / 16);
  GCT_CUDA_CHECK(launch_pdl(gct_kv_exchange_kernel, dim3(grid), dim3(256), 0, stream, a));
  return GCT_OK;
}

}  // namespace gct
