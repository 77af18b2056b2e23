// Paged attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a serving process that hands the whole
// HBM to its own pool at start-up and forbids any later allocation, or a latency-critical loop in
// which cudaMalloc's device-wide synchronisation is not acceptable.  The regular paged-attention path
// needs scratch memory beyond its inputs and outputs (the device copy of the page table, the split-KV
// partial outputs with their log-sum-exps, a status word) and expects the caller to provide it as a
// workspace.  gct_attn_paged_static is the same computation with that scratch placed in a fixed
// array that is part of the loaded library image, so the call allocates nothing, anywhere.
//
// Cost and limits: every GPU that loads the library holds kScratchBytes (about 17 MB) until the process
// exits.  The array bounds the problem size: n_q * heads <= 16384 rows, at most 4 KV splits, at most
// 4096 visible pages.  All calls on one GPU share the array and it keeps the previous call's contents;
// the status word is cleared at the start of every call, the other regions are fully rewritten before
// they are read.  Two calls whose GPU work overlaps in time (different streams, or several host
// threads) race on it: serialise them.
#include <mutex>

#include "gct_common.h"

namespace {

constexpr int kStaticMaxRows = 16384;    // n_q * heads
constexpr int kStaticMaxSplits = 4;
constexpr int kStaticMaxPages = 4096;
constexpr size_t kStatusBytes = 256;
constexpr size_t kTableBytes = static_cast<size_t>(kStaticMaxPages) * sizeof(int32_t);
constexpr size_t kPartOBytes = static_cast<size_t>(kStaticMaxSplits) * kStaticMaxRows * gct::kHeadDim * sizeof(float);
constexpr size_t kPartLseBytes = static_cast<size_t>(kStaticMaxSplits) * kStaticMaxRows * sizeof(float);
constexpr size_t kScratchBytes = kStatusBytes + kTableBytes + kPartOBytes + kPartLseBytes;

// In host code this name is only a handle for the runtime, not a device address: the address each
// device gave the array comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

// Once per device, with that device current: ask the runtime where the array lives there.
int scratch_of_current_device(unsigned char** out) {
  int dev = -1;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return gct::fail(GCT_ERR_INVALID, "gct_attn_paged_static: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess)
      return gct::fail(GCT_ERR_CUDA, std::string("cudaGetSymbolAddress(g_static_scratch): ") + cudaGetErrorString(e));
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0)
      return gct::fail(GCT_ERR_CUDA, "gct_attn_paged_static: scratch array has no usable device address");
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return GCT_OK;
}

}  // namespace

extern "C" int gct_attn_paged_static(const void* pool_dev, int max_num_pages, int page_size, int heads,
                                     const int32_t* visible_pages_host, int n_pages, int last_page_len,
                                     const void* q_dev, int n_q, void* out_dev, void* stream,
                                     int* device_status_out) {
  using namespace gct;
  if (pool_dev == nullptr || visible_pages_host == nullptr || q_dev == nullptr || out_dev == nullptr)
    return fail(GCT_ERR_INVALID, "gct_attn_paged_static: null argument");
  if (max_num_pages <= 0 || page_size <= 0 || heads <= 0 || n_q <= 0 || n_pages <= 0 || last_page_len <= 0 ||
      last_page_len > page_size)
    return fail(GCT_ERR_INVALID, "gct_attn_paged_static: bad shape");
  if (static_cast<long long>(n_q) * heads > kStaticMaxRows)
    return fail(GCT_ERR_CAPACITY, "gct_attn_paged_static: n_q * heads = " + std::to_string(static_cast<long long>(n_q) * heads) +
                                      " exceeds the static scratch limit of " + std::to_string(kStaticMaxRows) +
                                      " rows; use gct_mgr_attention with a caller-provided workspace");
  if (n_pages > kStaticMaxPages)
    return fail(GCT_ERR_CAPACITY, "gct_attn_paged_static: " + std::to_string(n_pages) + " visible pages exceed the static limit of " +
                                      std::to_string(kStaticMaxPages));
  for (int i = 0; i < n_pages; ++i)
    if (visible_pages_host[i] < 0 || visible_pages_host[i] >= max_num_pages)
      return fail(GCT_ERR_INVALID, "gct_attn_paged_static: page id out of range at position " + std::to_string(i));

  unsigned char* scratch = nullptr;
  int rc = scratch_of_current_device(&scratch);
  if (rc != GCT_OK) return rc;
  int* status = reinterpret_cast<int*>(scratch);
  int32_t* table = reinterpret_cast<int32_t*>(scratch + kStatusBytes);
  float* part_o = reinterpret_cast<float*>(scratch + kStatusBytes + kTableBytes);
  float* part_lse = reinterpret_cast<float*>(scratch + kStatusBytes + kTableBytes + kPartOBytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // the status word is the only region that must start at zero; the page table and the partials of the
  // splits in use are rewritten below before anything reads them
  GCT_CUDA_CHECK(cudaMemsetAsync(status, 0, kStatusBytes, s));
  GCT_CUDA_CHECK(cudaMemcpyAsync(table, visible_pages_host, static_cast<size_t>(n_pages) * sizeof(int32_t),
                                 cudaMemcpyHostToDevice, s));

  AttnLaunch a;
  const __nv_bfloat16* pool = static_cast<const __nv_bfloat16*>(pool_dev);
  const int64_t page_elems = static_cast<int64_t>(page_size) * heads * kHeadDim;
  rc = make_tensor_map(&a.tm_k, pool, heads, page_size, max_num_pages, kHeadDim, static_cast<int64_t>(heads) * kHeadDim,
                       2 * page_elems);
  if (rc != GCT_OK) return rc;
  rc = make_tensor_map(&a.tm_v, pool + page_elems, heads, page_size, max_num_pages, kHeadDim,
                       static_cast<int64_t>(heads) * kHeadDim, 2 * page_elems);
  if (rc != GCT_OK) return rc;
  rc = make_tensor_map(&a.tm_q, q_dev, heads, n_q, 1, kHeadDim, static_cast<int64_t>(heads) * kHeadDim,
                       static_cast<int64_t>(n_q) * heads * kHeadDim);
  if (rc != GCT_OK) return rc;
  a.page_table = table;
  a.n_pages = n_pages;
  a.page_len = page_size;
  a.last_page_len = last_page_len;
  a.n_q = n_q;
  a.heads = heads;
  a.batch = 1;
  a.status = status;
  const int bpp = (page_size + kBlockN - 1) / kBlockN;
  const int total_blocks = (n_pages - 1) * bpp + (last_page_len + kBlockN - 1) / kBlockN;
  int dev = 0, sms = 148;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  GCT_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  choose_attention_config((n_q + kTileM - 1) / kTileM, heads, total_blocks, sms, kStaticMaxSplits, &a.q_tiles_per_cta,
                          &a.splits);
  if (a.splits == 1) {
    a.final_bf16 = true;
    a.out = static_cast<__nv_bfloat16*>(out_dev);
    rc = launch_attention(a, s);
  } else {
    a.final_bf16 = false;
    a.part_o = part_o;
    a.part_lse = part_lse;
    rc = launch_attention(a, s);
    if (rc == GCT_OK)
      rc = launch_merge(part_o, part_lse, a.splits, static_cast<int64_t>(n_q) * heads, static_cast<__nv_bfloat16*>(out_dev),
                        nullptr, nullptr, s);
  }
  if (rc != GCT_OK) return rc;
  if (device_status_out != nullptr) {
    int host = 0;
    GCT_CUDA_CHECK(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, s));
    GCT_CUDA_CHECK(cudaStreamSynchronize(s));
    *device_status_out = host;
    if (host != 0) return fail(GCT_ERR_DEVICE_STATUS, "gct_attn_paged_static: kernel reported device status " + std::to_string(host));
  }
  return GCT_OK;
}
