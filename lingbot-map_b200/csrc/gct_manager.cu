// C-ABI layer: the two-stream paged KV cache manager (host bookkeeping restating
// lingbot_map/layers/flashinfer_cache.py of the reference) and the entry points that launch the kernels.
#include <algorithm>
#include <deque>
#include <mutex>
#include <vector>

#include "gct_common.h"

namespace gct {

static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

// ---- driver entry point for tensor-map encoding (no link-time dependency on libcuda) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, int heads, int64_t tokens, int64_t pages, int64_t head_stride,
                    int64_t token_stride, int64_t page_stride) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(GCT_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(GCT_ERR_INVALID, "tensor base must be 16-byte aligned");
  if ((head_stride % 8) || (token_stride % 8) || (page_stride % 8))
    return fail(GCT_ERR_INVALID, "tensor strides must be multiples of 8 elements (16 bytes)");
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(pages)};
  // a stride of 0 is not encodable; dimensions of extent 1 get a dummy stride
  auto st = [](int64_t s) { return static_cast<cuuint64_t>((s > 0 ? s : kHeadDim) * 2); };
  cuuint64_t strides[3] = {st(head_stride), st(token_stride), st(page_stride)};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(kHeadDim), 1u, static_cast<cuuint32_t>(kBlockN), 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GCT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return GCT_OK;
}

// SM count of the current device, cached per device ordinal.
static int device_sm_count(int* out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int cached[kMaxDevices] = {0};
  int dev = 0;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(GCT_ERR_INVALID, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) GCT_CUDA_CHECK(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
  *out = cached[dev];
  return GCT_OK;
}

}  // namespace gct

using namespace gct;

// Per-block bookkeeping: the reference's deques and LIFO free lists (flashinfer_cache.py:150-170).
struct BlockState {
  std::deque<int32_t> scale_pages, window_pages;
  std::vector<int32_t> free_patch, special_pages, free_special;
  int64_t special_token_count = 0;
  int64_t frame_count = 0;
};

struct gct_mgr {
  gct_mgr_config_t cfg{};
  gct_mgr_geometry_t geo{};
  int patches = 0;
  bool defer_eviction = false;
  std::vector<BlockState> blocks;
  // device side (after bind)
  bool bound = false;
  std::vector<__nv_bfloat16*> pools;
  std::vector<CUtensorMap> tm_k, tm_v;
  uint8_t* ws = nullptr;
  size_t ws_bytes = 0;
  int* status_dev = nullptr;
  int32_t* table_dev = nullptr;
  __nv_bfloat16* q_stage = nullptr;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  int max_splits = 0;
  // bounded softmax reference: running max of |k| per (block, head) on the device, kept by every K write that goes
  // through the manager
  float* key_norm_max = nullptr;     // [num_blocks, H] inside the workspace header (null: does not fit)
  bool bounded_enabled = true;
  std::vector<char> key_norm_valid, key_norm_clear;
  // plan: the page table is staged through a small ring of pinned host slots so that its upload is a true
  // asynchronous copy (a pageable source would be staged by the runtime at call time)
  bool planned = false;
  int plan_pages = 0, plan_last_len = 0;
  static constexpr int kPlanSlots = 8;
  int32_t* plan_ring = nullptr;                  // [kPlanSlots][max_num_pages], cudaHostAlloc
  cudaEvent_t plan_done[kPlanSlots] = {};        // recorded after the copy out of each slot
  bool plan_used[kPlanSlots] = {};
  uint64_t plan_count = 0;
  // cached query tensor map
  const void* tmq_ptr = nullptr;
  int tmq_nq = 0;
  CUtensorMap tm_q{};
  int64_t launches = 0;
  // optional CUDA-event timing of the attention kernel alone (gct_mgr_kernel_timing)
  bool timing = false;
  std::vector<cudaEvent_t> ev_start, ev_stop;
  size_t ev_used = 0;
};

static constexpr size_t kWsHeader = 4096;      // status word
static constexpr int kMaxSplitsCap = 32;
// Largest |q| * max|k| * scale * log2(e) for which the bound may stand in for the row maximum: all exponents stay
// in [-2 * limit, 0], far inside the fp32 / bf16 exponent range.
static constexpr float kBoundedLimit = 40.0f;

static void reset_block(const gct_mgr* m, BlockState& b) {
  b.scale_pages.clear();
  b.window_pages.clear();
  b.special_pages.clear();
  b.free_patch.resize(m->geo.max_patch_pages);
  for (int i = 0; i < m->geo.max_patch_pages; ++i) b.free_patch[i] = i;
  const int nsp = m->geo.max_num_pages - m->geo.max_patch_pages;
  b.free_special.resize(nsp);
  for (int i = 0; i < nsp; ++i) b.free_special[i] = m->geo.max_patch_pages + i;
  b.special_token_count = 0;
  b.frame_count = 0;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WsLayout {
  size_t table_off, qstage_off, parto_off, partlse_off, total_min, per_split;
};
static constexpr size_t kWsKeyNormOff = 256;     // key_norm_max[num_blocks][H] up to the end of the header
static WsLayout ws_layout(const gct_mgr* m) {
  WsLayout w;
  const size_t rows = static_cast<size_t>(m->cfg.tokens_per_frame) * m->cfg.num_heads;
  w.table_off = kWsHeader;
  w.qstage_off = align_up(w.table_off + static_cast<size_t>(m->geo.max_num_pages) * 4, 256);
  w.parto_off = align_up(w.qstage_off + rows * kHeadDim * 2, 256);
  w.per_split = rows * kHeadDim * 4 + rows * 4;
  w.partlse_off = 0;
  w.total_min = w.parto_off + 2 * w.per_split + 256;
  return w;
}

static int check_bound_fwd(const gct_mgr* m);

extern "C" {

const char* gct_last_error(void) { return g_last_error.c_str(); }
int gct_version(void) { return 1; }

int gct_mgr_create(gct_mgr_t** out, const gct_mgr_config_t* cfg, gct_mgr_geometry_t* geo_out) {
  if (out == nullptr || cfg == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_create: null argument");
  if (cfg->head_dim != kHeadDim) return fail(GCT_ERR_INVALID, "gct_mgr_create: head_dim must be 64");
  if (cfg->num_blocks <= 0 || cfg->num_heads <= 0 || cfg->num_special_tokens < 0 || cfg->scale_frames < 0 ||
      cfg->sliding_window < 0 || cfg->max_total_frames <= 0)
    return fail(GCT_ERR_INVALID, "gct_mgr_create: bad configuration");
  if (cfg->tokens_per_frame <= cfg->num_special_tokens)
    return fail(GCT_ERR_INVALID, "tokens_per_frame=" + std::to_string(cfg->tokens_per_frame) +
                                     " <= num_special_tokens=" + std::to_string(cfg->num_special_tokens));
  gct_mgr* m = new gct_mgr();
  m->cfg = *cfg;
  m->patches = cfg->tokens_per_frame - cfg->num_special_tokens;
  m->geo.page_size = m->patches;                                              // flashinfer_cache.py:100-106
  m->geo.max_patch_pages = cfg->scale_frames + cfg->sliding_window + 16;      // :132
  const int64_t sp_tokens = static_cast<int64_t>(cfg->max_total_frames) * cfg->num_special_tokens;
  const int max_special = static_cast<int>((sp_tokens + m->geo.page_size - 1) / m->geo.page_size) + 16;   // :134-136
  m->geo.max_num_pages = m->geo.max_patch_pages + max_special;
  m->geo.pool_bytes = static_cast<int64_t>(m->geo.max_num_pages) * 2 * m->geo.page_size * cfg->num_heads * kHeadDim * 2;
  m->blocks.resize(cfg->num_blocks);
  for (auto& b : m->blocks) reset_block(m, b);
  if (geo_out != nullptr) *geo_out = m->geo;
  *out = m;
  return GCT_OK;
}

int gct_mgr_destroy(gct_mgr_t* m) {
  if (m != nullptr) {
    for (cudaEvent_t e : m->ev_start) cudaEventDestroy(e);
    for (cudaEvent_t e : m->ev_stop) cudaEventDestroy(e);
    if (m->plan_ring != nullptr) {
      for (int i = 0; i < gct_mgr::kPlanSlots; ++i)
        if (m->plan_done[i] != nullptr) cudaEventDestroy(m->plan_done[i]);
      cudaFreeHost(m->plan_ring);
    }
  }
  delete m;
  return GCT_OK;
}

int gct_mgr_kernel_timing(gct_mgr_t* m, int max_launches) {
  int rc = check_bound_fwd(m);
  if (rc != GCT_OK) return rc;
  for (cudaEvent_t e : m->ev_start) cudaEventDestroy(e);
  for (cudaEvent_t e : m->ev_stop) cudaEventDestroy(e);
  m->ev_start.clear();
  m->ev_stop.clear();
  m->ev_used = 0;
  m->timing = max_launches > 0;
  for (int i = 0; i < max_launches; ++i) {
    cudaEvent_t a, b;
    GCT_CUDA_CHECK(cudaEventCreate(&a));
    GCT_CUDA_CHECK(cudaEventCreate(&b));
    m->ev_start.push_back(a);
    m->ev_stop.push_back(b);
  }
  return GCT_OK;
}

int gct_mgr_kernel_time(gct_mgr_t* m, double* total_ms_out, int* launches_out) {
  int rc = check_bound_fwd(m);
  if (rc != GCT_OK) return rc;
  if (total_ms_out == nullptr || launches_out == nullptr) return fail(GCT_ERR_INVALID, "null argument");
  double total = 0.0;
  for (size_t i = 0; i < m->ev_used; ++i) {
    GCT_CUDA_CHECK(cudaEventSynchronize(m->ev_stop[i]));
    float ms = 0.f;
    GCT_CUDA_CHECK(cudaEventElapsedTime(&ms, m->ev_start[i], m->ev_stop[i]));
    total += ms;
  }
  *total_ms_out = total;
  *launches_out = static_cast<int>(m->ev_used);
  m->ev_used = 0;
  return GCT_OK;
}

int gct_mgr_workspace_bytes(const gct_mgr_t* m, size_t* bytes_out) {
  if (m == nullptr || bytes_out == nullptr) return fail(GCT_ERR_INVALID, "null argument");
  *bytes_out = ws_layout(m).total_min;
  return GCT_OK;
}

int gct_mgr_bind(gct_mgr_t* m, void* const* pools_dev, void* workspace_dev, size_t workspace_bytes) {
  if (m == nullptr || pools_dev == nullptr || workspace_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_bind: null argument");
  const WsLayout w = ws_layout(m);
  if (workspace_bytes < w.total_min)
    return fail(GCT_ERR_CAPACITY, "gct_mgr_bind: workspace of " + std::to_string(workspace_bytes) + " bytes, need " +
                                      std::to_string(w.total_min));
  if ((reinterpret_cast<uintptr_t>(workspace_dev) & 255) != 0) return fail(GCT_ERR_INVALID, "workspace must be 256-byte aligned");
  const int H = m->cfg.num_heads, P = m->geo.page_size;
  m->pools.assign(m->cfg.num_blocks, nullptr);
  m->tm_k.resize(m->cfg.num_blocks);
  m->tm_v.resize(m->cfg.num_blocks);
  const int64_t page_elems = static_cast<int64_t>(P) * H * kHeadDim;
  for (int b = 0; b < m->cfg.num_blocks; ++b) {
    if (pools_dev[b] == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_bind: null pool");
    m->pools[b] = static_cast<__nv_bfloat16*>(pools_dev[b]);
    int rc = make_tensor_map(&m->tm_k[b], m->pools[b], H, P, m->geo.max_num_pages, kHeadDim,
                             static_cast<int64_t>(H) * kHeadDim, 2 * page_elems);
    if (rc != GCT_OK) return rc;
    rc = make_tensor_map(&m->tm_v[b], m->pools[b] + page_elems, H, P, m->geo.max_num_pages, kHeadDim,
                         static_cast<int64_t>(H) * kHeadDim, 2 * page_elems);
    if (rc != GCT_OK) return rc;
  }
  m->ws = static_cast<uint8_t*>(workspace_dev);
  m->ws_bytes = workspace_bytes;
  m->status_dev = reinterpret_cast<int*>(m->ws);
  m->table_dev = reinterpret_cast<int32_t*>(m->ws + w.table_off);
  m->q_stage = reinterpret_cast<__nv_bfloat16*>(m->ws + w.qstage_off);
  const size_t avail = workspace_bytes - w.parto_off - 256;
  m->max_splits = static_cast<int>(std::min<size_t>(avail / w.per_split, kMaxSplitsCap));
  const size_t rows = static_cast<size_t>(m->cfg.tokens_per_frame) * H;
  m->part_o = reinterpret_cast<float*>(m->ws + w.parto_off);
  m->part_lse = reinterpret_cast<float*>(m->ws + w.parto_off + static_cast<size_t>(m->max_splits) * rows * kHeadDim * 4);
  GCT_CUDA_CHECK(cudaMemset(m->ws, 0, kWsHeader));
  const size_t kn_bytes = static_cast<size_t>(m->cfg.num_blocks) * H * sizeof(float);
  m->key_norm_max = kWsKeyNormOff + kn_bytes <= kWsHeader ? reinterpret_cast<float*>(m->ws + kWsKeyNormOff) : nullptr;
  // nothing is visible yet and the header was just zeroed: a maximum of 0 is exact
  m->key_norm_valid.assign(m->cfg.num_blocks, 1);
  m->key_norm_clear.assign(m->cfg.num_blocks, 0);
  if (m->plan_ring == nullptr) {
    GCT_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&m->plan_ring),
                                 static_cast<size_t>(gct_mgr::kPlanSlots) * m->geo.max_num_pages * sizeof(int32_t),
                                 cudaHostAllocDefault));
    for (int i = 0; i < gct_mgr::kPlanSlots; ++i)
      GCT_CUDA_CHECK(cudaEventCreateWithFlags(&m->plan_done[i], cudaEventDisableTiming));
  }
  m->bound = true;
  m->planned = false;
  m->tmq_ptr = nullptr;
  return GCT_OK;
}

// Where one frame's K/V rows go; the bookkeeping half of append_frame.
struct AppendPlan {
  int patch_page, sp_page0, sp_off0, sp_n0, sp_page1;
};

static int append_bookkeeping(gct_mgr* m, int block, AppendPlan* plan) {
  if (m == nullptr) return fail(GCT_ERR_INVALID, "null manager");
  if (block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "block index out of range");
  BlockState& b = m->blocks[block];
  const int P = m->geo.page_size, n = m->cfg.num_special_tokens;
  if (b.free_patch.empty())
    return fail(GCT_ERR_POOL_EXHAUSTED, "block " + std::to_string(block) + ": patch page pool exhausted - scale=" +
                                            std::to_string(b.scale_pages.size()) + ", window=" +
                                            std::to_string(b.window_pages.size()) + ", free=0");
  // check the special pool before mutating anything so a failed append leaves the state untouched
  {
    const int64_t off = b.special_token_count % P;
    const int64_t room = (off == 0) ? 0 : P - off;
    const int64_t need_pages = (n > room) ? (n - room + P - 1) / P : 0;
    if (static_cast<int64_t>(b.free_special.size()) < need_pages)
      return fail(GCT_ERR_POOL_EXHAUSTED, "block " + std::to_string(block) + ": special page pool exhausted at special_token_count=" +
                                              std::to_string(b.special_token_count) + ". Increase max_total_frames.");
  }
  AppendPlan pl{-1, -1, 0, 0, -1};
  pl.patch_page = b.free_patch.back();                       // LIFO pop (:496)
  b.free_patch.pop_back();
  if (static_cast<int>(b.scale_pages.size()) < m->cfg.scale_frames)   // :507-510
    b.scale_pages.push_back(pl.patch_page);
  else
    b.window_pages.push_back(pl.patch_page);
  int remaining = n, chunk = 0;
  while (remaining > 0) {                                     // :528-553
    const int off = static_cast<int>(b.special_token_count % P);
    if (off == 0) {
      b.special_pages.push_back(b.free_special.back());
      b.free_special.pop_back();
    }
    const int tail = b.special_pages.back();
    const int w = std::min(remaining, P - off);
    if (chunk == 0) {
      pl.sp_page0 = tail;
      pl.sp_off0 = off;
      pl.sp_n0 = w;
    } else if (chunk == 1) {
      pl.sp_page1 = tail;
    } else {
      return fail(GCT_ERR_INVALID, "special tokens of one frame span more than two pages");
    }
    b.special_token_count += w;
    remaining -= w;
    ++chunk;
  }
  b.frame_count += 1;
  if (plan != nullptr) *plan = pl;
  return GCT_OK;
}

int gct_mgr_append_bookkeeping(gct_mgr_t* m, int block) {
  const int rc = append_bookkeeping(m, block, nullptr);
  // the caller writes the pool itself: the key-norm maximum no longer covers what is visible (gct_mgr_scan_keys)
  if (rc == GCT_OK && m->bound && block >= 0 && block < static_cast<int>(m->key_norm_valid.size())) m->key_norm_valid[block] = 0;
  return rc;
}

static int check_bound(const gct_mgr* m) {
  if (m == nullptr) return fail(GCT_ERR_INVALID, "null manager");
  if (!m->bound) return fail(GCT_ERR_INVALID, "manager has no device memory bound (gct_mgr_bind)");
  return GCT_OK;
}
}  // extern "C"
static int check_bound_fwd(const gct_mgr* m) { return check_bound(m); }
extern "C" {

// Key-norm tracking of an append on `stream`: clear a maximum left over from before a reset, then let the kernel
// raise it.
static int track_key_norms(gct_mgr* m, int block, PrepLaunch* p, cudaStream_t stream) {
  if (m->key_norm_max == nullptr) return GCT_OK;
  float* slot = m->key_norm_max + static_cast<size_t>(block) * m->cfg.num_heads;
  if (m->key_norm_clear[block]) {
    GCT_CUDA_CHECK(cudaMemsetAsync(slot, 0, static_cast<size_t>(m->cfg.num_heads) * sizeof(float), stream));
    m->key_norm_clear[block] = 0;
  }
  p->key_norm_max = slot;
  return GCT_OK;
}

static void fill_paged_dst(const gct_mgr* m, int block, const AppendPlan& pl, PrepLaunch* p) {
  p->pool = m->pools[block];
  p->page_size = m->geo.page_size;
  p->num_pages = m->geo.max_num_pages;
  p->num_special = m->cfg.num_special_tokens;
  p->patch_page = pl.patch_page;
  p->sp_page0 = pl.sp_page0;
  p->sp_off0 = pl.sp_off0;
  p->sp_n0 = pl.sp_n0;
  p->sp_page1 = pl.sp_page1;
  p->status = m->status_dev;
  p->tokens = m->cfg.tokens_per_frame;
  p->tokens_per_frame = m->cfg.tokens_per_frame;
  p->heads = m->cfg.num_heads;
}

int gct_mgr_append(gct_mgr_t* m, int block, const void* k_dev, int k_dtype, const void* v_dev, int v_dtype, void* stream) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  if (k_dev == nullptr || v_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_append: null K/V");
  if ((k_dtype != GCT_F32 && k_dtype != GCT_BF16) || (v_dtype != GCT_F32 && v_dtype != GCT_BF16))
    return fail(GCT_ERR_INVALID, "gct_mgr_append: dtype must be GCT_F32 or GCT_BF16");
  AppendPlan pl;
  rc = append_bookkeeping(m, block, &pl);
  if (rc != GCT_OK) return rc;
  PrepLaunch p;
  fill_paged_dst(m, block, pl, &p);
  p.k_src = k_dev;
  p.v_src = v_dev;
  p.src_dtype_qk = k_dtype;
  p.src_dtype_v = v_dtype;
  p.src_token_stride = static_cast<int64_t>(m->cfg.num_heads) * kHeadDim;
  p.src_head_stride = kHeadDim;
  rc = track_key_norms(m, block, &p, static_cast<cudaStream_t>(stream));
  if (rc != GCT_OK) return rc;
  m->launches += 1;
  return launch_prep(p, static_cast<cudaStream_t>(stream));
}

int gct_mgr_append_fused(gct_mgr_t* m, int block, const void* qkv_dev, int qkv_dtype, int64_t qkv_row_stride,
                         const float* qn_w_dev, const float* qn_b_dev, const float* kn_w_dev, const float* kn_b_dev,
                         const float* rope_cs_dev, int rope_mode, void* q_out_dev, void* stream) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  if (qkv_dev == nullptr || q_out_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_append_fused: null argument");
  if (qkv_dtype != GCT_F32 && qkv_dtype != GCT_BF16) return fail(GCT_ERR_INVALID, "gct_mgr_append_fused: dtype");
  if ((qn_w_dev == nullptr) != (qn_b_dev == nullptr) || (kn_w_dev == nullptr) != (kn_b_dev == nullptr))
    return fail(GCT_ERR_INVALID, "gct_mgr_append_fused: norm weight and bias must come together");
  const int64_t C = static_cast<int64_t>(m->cfg.num_heads) * kHeadDim;
  if (qkv_row_stride < 3 * C) return fail(GCT_ERR_INVALID, "gct_mgr_append_fused: row stride smaller than 3*H*64");
  AppendPlan pl;
  rc = append_bookkeeping(m, block, &pl);
  if (rc != GCT_OK) return rc;
  PrepLaunch p;
  fill_paged_dst(m, block, pl, &p);
  const size_t esz = qkv_dtype == GCT_F32 ? 4 : 2;
  p.q_src = qkv_dev;
  p.k_src = static_cast<const uint8_t*>(qkv_dev) + C * esz;
  p.v_src = static_cast<const uint8_t*>(qkv_dev) + 2 * C * esz;
  p.src_dtype_qk = p.src_dtype_v = qkv_dtype;
  p.src_token_stride = qkv_row_stride;
  p.src_head_stride = kHeadDim;
  p.qn_w = qn_w_dev;
  p.qn_b = qn_b_dev;
  p.kn_w = kn_w_dev;
  p.kn_b = kn_b_dev;
  p.rope_cs = rope_cs_dev;
  p.rope_mode = rope_mode;
  p.q_out = static_cast<__nv_bfloat16*>(q_out_dev);
  rc = track_key_norms(m, block, &p, static_cast<cudaStream_t>(stream));
  if (rc != GCT_OK) return rc;
  m->launches += 1;
  return launch_prep(p, static_cast<cudaStream_t>(stream));
}

static void evict_now(gct_mgr* m, int block, int sliding_window) {
  BlockState& b = m->blocks[block];
  while (static_cast<int>(b.window_pages.size()) > sliding_window) {   // :252-254
    b.free_patch.push_back(b.window_pages.front());
    b.window_pages.pop_front();
  }
}

int gct_mgr_evict(gct_mgr_t* m, int block, int sliding_window) {
  if (m == nullptr || block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_evict: bad argument");
  if (m->defer_eviction) return GCT_OK;                                 // :250-251
  evict_now(m, block, sliding_window);
  return GCT_OK;
}

int gct_mgr_exec_deferred(gct_mgr_t* m, int block, int sliding_window) {
  if (m == nullptr || block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_exec_deferred: bad argument");
  evict_now(m, block, sliding_window);
  return GCT_OK;
}

int gct_mgr_set_defer(gct_mgr_t* m, int defer) {
  if (m == nullptr) return fail(GCT_ERR_INVALID, "null manager");
  m->defer_eviction = defer != 0;
  return GCT_OK;
}

int gct_mgr_get_defer(const gct_mgr_t* m, int* defer_out) {
  if (m == nullptr || defer_out == nullptr) return fail(GCT_ERR_INVALID, "null argument");
  *defer_out = m->defer_eviction ? 1 : 0;
  return GCT_OK;
}

int gct_mgr_rollback(gct_mgr_t* m, int block) {
  if (m == nullptr || block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_rollback: bad argument");
  BlockState& b = m->blocks[block];
  if (b.frame_count <= 0)
    return fail(GCT_ERR_UNDERFLOW, "block " + std::to_string(block) + ": cannot rollback, frame_count is 0");
  const int n = m->cfg.num_special_tokens, P = m->geo.page_size;
  const int64_t new_count = b.special_token_count - n;
  if (new_count < 0)
    return fail(GCT_ERR_UNDERFLOW, "block " + std::to_string(block) + ": special_token_count underflow");
  std::deque<int32_t>& src = (b.frame_count > m->cfg.scale_frames) ? b.window_pages : b.scale_pages;   // :281-284
  if (src.empty()) return fail(GCT_ERR_UNDERFLOW, "block " + std::to_string(block) + ": no page to roll back");
  b.free_patch.push_back(src.back());
  src.pop_back();
  const int64_t keep = new_count > 0 ? (new_count + P - 1) / P : 0;                                    // :294-297
  while (static_cast<int64_t>(b.special_pages.size()) > keep) {
    b.free_special.push_back(b.special_pages.back());
    b.special_pages.pop_back();
  }
  b.special_token_count = new_count;
  b.frame_count -= 1;
  return GCT_OK;
}

int gct_mgr_scan_keys(gct_mgr_t* m, int block, void* stream) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  if (block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_scan_keys: block index out of range");
  if (m->key_norm_max == nullptr) return GCT_OK;       // bounded mode unavailable for this geometry
  rc = launch_scan_keys(m->pools[block], m->geo.max_num_pages, m->geo.page_size, m->cfg.num_heads,
                        m->key_norm_max + static_cast<size_t>(block) * m->cfg.num_heads, static_cast<cudaStream_t>(stream));
  if (rc != GCT_OK) return rc;
  m->key_norm_valid[block] = 1;
  m->key_norm_clear[block] = 0;
  m->launches += 1;
  return GCT_OK;
}

int gct_mgr_set_bounded_mode(gct_mgr_t* m, int enable) {
  if (m == nullptr) return fail(GCT_ERR_INVALID, "null manager");
  m->bounded_enabled = enable != 0;
  return GCT_OK;
}

int gct_mgr_reset(gct_mgr_t* m) {
  if (m == nullptr) return fail(GCT_ERR_INVALID, "null manager");
  for (auto& b : m->blocks) reset_block(m, b);
  m->planned = false;
  // nothing is visible any more: the key-norm maxima restart from zero at the next append
  for (auto& f : m->key_norm_clear) f = 1;
  for (auto& f : m->key_norm_valid) f = 1;
  return GCT_OK;
}

static int last_page_len(const gct_mgr* m, const BlockState& b) {          // :452-470
  if (b.special_pages.empty()) return m->patches;
  const int tail = static_cast<int>(b.special_token_count % m->geo.page_size);
  return tail == 0 ? m->geo.page_size : tail;
}

int gct_mgr_visible_table(const gct_mgr_t* m, int block, int32_t* pages_out, int capacity, int* n_out, int* last_out) {
  if (m == nullptr || block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_visible_table: bad argument");
  const BlockState& b = m->blocks[block];
  const int n = static_cast<int>(b.scale_pages.size() + b.window_pages.size() + b.special_pages.size());
  if (n_out != nullptr) *n_out = n;
  if (last_out != nullptr) *last_out = last_page_len(m, b);
  if (pages_out != nullptr) {
    if (capacity < n) return fail(GCT_ERR_CAPACITY, "gct_mgr_visible_table: output buffer too small");
    int i = 0;
    for (int32_t p : b.scale_pages) pages_out[i++] = p;      // scale -> window -> special (:446-450)
    for (int32_t p : b.window_pages) pages_out[i++] = p;
    for (int32_t p : b.special_pages) pages_out[i++] = p;
  }
  return GCT_OK;
}

int gct_mgr_stats(const gct_mgr_t* m, int block, int64_t out[6]) {
  if (m == nullptr || out == nullptr || block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "gct_mgr_stats: bad argument");
  const BlockState& b = m->blocks[block];
  out[0] = b.frame_count;
  out[1] = static_cast<int64_t>(b.scale_pages.size());
  out[2] = static_cast<int64_t>(b.window_pages.size());
  out[3] = static_cast<int64_t>(b.free_patch.size());
  out[4] = b.special_token_count;
  out[5] = static_cast<int64_t>(b.special_pages.size());
  return GCT_OK;
}

int gct_mgr_free_list(const gct_mgr_t* m, int block, int which, int32_t* out, int capacity, int* n_out) {
  if (m == nullptr || block < 0 || block >= m->cfg.num_blocks || (which != 0 && which != 1))
    return fail(GCT_ERR_INVALID, "gct_mgr_free_list: bad argument");
  const std::vector<int32_t>& v = which == 0 ? m->blocks[block].free_patch : m->blocks[block].free_special;
  if (n_out != nullptr) *n_out = static_cast<int>(v.size());
  if (out != nullptr) {
    if (capacity < static_cast<int>(v.size())) return fail(GCT_ERR_CAPACITY, "gct_mgr_free_list: output buffer too small");
    std::copy(v.begin(), v.end(), out);
  }
  return GCT_OK;
}

int gct_mgr_plan(gct_mgr_t* m, int page_begin, int page_end, void* stream) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  const BlockState& b = m->blocks[0];
  std::vector<int32_t> vis;
  vis.reserve(b.scale_pages.size() + b.window_pages.size() + b.special_pages.size());
  for (int32_t p : b.scale_pages) vis.push_back(p);
  for (int32_t p : b.window_pages) vis.push_back(p);
  for (int32_t p : b.special_pages) vis.push_back(p);
  if (vis.empty()) return fail(GCT_ERR_INVALID, "visible page table is empty after append_frame");   // :393
  const int n = static_cast<int>(vis.size());
  if (page_end < 0) page_end = n;
  if (page_begin < 0 || page_begin >= page_end || page_end > n) return fail(GCT_ERR_INVALID, "gct_mgr_plan: bad page range");
  const int last = (page_end == n) ? last_page_len(m, b) : m->geo.page_size;
  if (last < 1 || last > m->geo.page_size)                                                          // :394-396
    return fail(GCT_ERR_INVALID, "block 0: last_page_len=" + std::to_string(last) + " out of range");
  // pinned staging slot: reused every kPlanSlots plans, after the copy out of it has completed
  const int slot = static_cast<int>(m->plan_count++ % gct_mgr::kPlanSlots);
  if (m->plan_used[slot]) GCT_CUDA_CHECK(cudaEventSynchronize(m->plan_done[slot]));
  int32_t* host = m->plan_ring + static_cast<size_t>(slot) * m->geo.max_num_pages;
  std::copy(vis.begin() + page_begin, vis.begin() + page_end, host);
  GCT_CUDA_CHECK(cudaMemcpyAsync(m->table_dev, host, static_cast<size_t>(page_end - page_begin) * 4,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  GCT_CUDA_CHECK(cudaEventRecord(m->plan_done[slot], static_cast<cudaStream_t>(stream)));
  m->plan_used[slot] = true;
  m->plan_pages = page_end - page_begin;
  m->plan_last_len = last;
  m->planned = true;
  return GCT_OK;
}

// Launch the attention kernel, bracketed by a CUDA-event pair when kernel timing is on.
static int timed_attention(gct_mgr* m, const AttnLaunch& a, cudaStream_t stream) {
  const bool t = m->timing && m->ev_used < m->ev_start.size();
  if (t) GCT_CUDA_CHECK(cudaEventRecord(m->ev_start[m->ev_used], stream));
  const int rc = launch_attention(a, stream);
  if (t) {
    GCT_CUDA_CHECK(cudaEventRecord(m->ev_stop[m->ev_used], stream));
    m->ev_used += 1;
  }
  return rc;
}

// splits_out != nullptr: stop after the attention kernel and leave its split partials (part_o, part_lse) in the
// workspace for the caller; *splits_out receives their count.
static int run_paged(gct_mgr* m, int block, const void* q_dev, int q_dtype, int n_q, __nv_bfloat16* out_bf16,
                     float* out_f32, float* lse_dev, cudaStream_t stream, int* splits_out = nullptr) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  if (block < 0 || block >= m->cfg.num_blocks) return fail(GCT_ERR_INVALID, "attention: block index out of range");
  if (!m->planned) return fail(GCT_ERR_INVALID, "attention: no plan (call gct_mgr_plan after the frame's append)");
  if (q_dev == nullptr || n_q <= 0 || n_q > m->cfg.tokens_per_frame)
    return fail(GCT_ERR_INVALID, "attention: n_q must be in [1, tokens_per_frame]");
  const int H = m->cfg.num_heads;
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(q_dev);
  if (q_dtype == GCT_F32) {          // the reference casts q to the storage dtype (:419)
    rc = launch_cast_bf16(static_cast<const float*>(q_dev), m->q_stage, static_cast<int64_t>(n_q) * H * kHeadDim, stream);
    if (rc != GCT_OK) return rc;
    m->launches += 1;
    q = m->q_stage;
  } else if (q_dtype != GCT_BF16) {
    return fail(GCT_ERR_INVALID, "attention: q dtype must be GCT_F32 or GCT_BF16");
  }
  if (m->tmq_ptr != q || m->tmq_nq != n_q) {
    rc = make_tensor_map(&m->tm_q, q, H, n_q, 1, kHeadDim, static_cast<int64_t>(H) * kHeadDim,
                         static_cast<int64_t>(n_q) * H * kHeadDim);
    if (rc != GCT_OK) return rc;
    m->tmq_ptr = q;
    m->tmq_nq = n_q;
  }
  AttnLaunch a;
  a.tm_q = m->tm_q;
  a.tm_k = m->tm_k[block];
  a.tm_v = m->tm_v[block];
  a.page_table = m->table_dev;
  a.n_pages = m->plan_pages;
  a.page_len = m->geo.page_size;
  a.last_page_len = m->plan_last_len;
  a.n_q = n_q;
  a.heads = H;
  a.batch = 1;
  a.status = m->status_dev;
  const int bpp = (m->geo.page_size + kBlockN - 1) / kBlockN;
  const int total_blocks = (a.n_pages - 1) * bpp + (a.last_page_len + kBlockN - 1) / kBlockN;
  int sms = 148;
  rc = device_sm_count(&sms);
  if (rc != GCT_OK) return rc;
  choose_attention_config((n_q + kTileM - 1) / kTileM, H, total_blocks, sms, m->max_splits, &a.q_tiles_per_cta, &a.splits,
                          &a.split_len);
  const int64_t rows = static_cast<int64_t>(n_q) * H;
  // Bounded mode: every key of this block's cache went through the manager, so |q_row| * max|k| bounds the row's
  // logits; while that bound stays small it replaces the running row maximum (decided per CTA inside the kernel).
  if (m->bounded_enabled && m->key_norm_max != nullptr && m->key_norm_valid[block] && a.q_tiles_per_cta == 2) {
    a.key_norm_max = m->key_norm_max + static_cast<size_t>(block) * H;
    a.bounded_limit = kBoundedLimit;
  }
  if (splits_out != nullptr) {
    a.final_bf16 = false;
    a.part_o = m->part_o;
    a.part_lse = m->part_lse;
    *splits_out = a.splits;
    m->launches += 1;
    return timed_attention(m, a, stream);
  }
  if (a.splits == 1 && out_bf16 != nullptr && lse_dev == nullptr) {
    a.final_bf16 = true;
    a.out = out_bf16;
    m->launches += 1;
    return timed_attention(m, a, stream);
  }
  a.final_bf16 = false;
  a.part_o = m->part_o;
  a.part_lse = m->part_lse;
  // partial rows are laid out with n_q rows per split
  rc = timed_attention(m, a, stream);
  if (rc != GCT_OK) return rc;
  m->launches += 2;
  return launch_merge(m->part_o, m->part_lse, a.splits, rows, out_bf16, out_f32, lse_dev, stream);
}

int gct_mgr_attention(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q, void* out_dev, float* lse_dev,
                      void* stream) {
  if (out_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_attention: null output");
  return run_paged(m, block, q_dev, q_dtype, n_q, static_cast<__nv_bfloat16*>(out_dev), nullptr, lse_dev,
                   static_cast<cudaStream_t>(stream));
}

int gct_mgr_attention_partial(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q, float* out_f32_dev,
                              float* lse_dev, void* stream) {
  if (out_f32_dev == nullptr || lse_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_mgr_attention_partial: null output");
  return run_paged(m, block, q_dev, q_dtype, n_q, nullptr, out_f32_dev, lse_dev, static_cast<cudaStream_t>(stream));
}

int gct_kv_exchange_sizes(int n_q, int heads, int world, size_t* recv_bytes_out, size_t* flag_bytes_out, int* slice_rows_out) {
  if (n_q <= 0 || heads <= 0 || world < 1 || world > 16) return fail(GCT_ERR_INVALID, "gct_kv_exchange_sizes: bad argument");
  const int64_t rows = static_cast<int64_t>(n_q) * heads;
  const int slice = static_cast<int>((rows + world - 1) / world);
  if (recv_bytes_out != nullptr) *recv_bytes_out = static_cast<size_t>(world) * slice * (kHeadDim + 1) * sizeof(float);
  if (flag_bytes_out != nullptr) *flag_bytes_out = static_cast<size_t>(2 * world + 2) * sizeof(int);
  if (slice_rows_out != nullptr) *slice_rows_out = slice;
  return GCT_OK;
}

int gct_mgr_attention_exchange(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q, int rank, int world,
                               int has_pages, void* const* recv_ptrs, void* const* out_ptrs, void* const* flag_ptrs,
                               int slice_rows, int epoch, void* stream) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows = static_cast<int64_t>(n_q) * m->cfg.num_heads;
  if (!has_pages) {
    m->launches += 1;
    return launch_kv_exchange(nullptr, nullptr, 0, static_cast<int>(rows), rank, world, epoch, recv_ptrs, out_ptrs, flag_ptrs,
                              slice_rows, m->status_dev, s);
  }
  int splits = 0;
  rc = run_paged(m, block, q_dev, q_dtype, n_q, nullptr, nullptr, nullptr, s, &splits);
  if (rc != GCT_OK) return rc;
  m->launches += 1;
  // partial rows are laid out with n_q rows per split, which is what the exchange kernel indexes
  return launch_kv_exchange(m->part_o, m->part_lse, splits, static_cast<int>(rows), rank, world, epoch, recv_ptrs, out_ptrs,
                            flag_ptrs, slice_rows, m->status_dev, s);
}

int gct_mgr_device_status(gct_mgr_t* m, void* stream, int* status_out) {
  int rc = check_bound(m);
  if (rc != GCT_OK) return rc;
  if (status_out == nullptr) return fail(GCT_ERR_INVALID, "null argument");
  int host = 0;
  GCT_CUDA_CHECK(cudaMemcpyAsync(&host, m->status_dev, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  GCT_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  *status_out = host;
  if (host != 0) return fail(GCT_ERR_DEVICE_STATUS, "a kernel reported device status " + std::to_string(host));
  return GCT_OK;
}

int gct_mgr_launch_count(const gct_mgr_t* m, int64_t* count_out) {
  if (m == nullptr || count_out == nullptr) return fail(GCT_ERR_INVALID, "null argument");
  *count_out = m->launches;
  return GCT_OK;
}

// ---- stand-alone operators ---------------------------------------------------------------

int gct_attn_launch_shape(int n_q, int heads, int kv_blocks, int num_sms, int max_splits, int* q_tiles_per_cta_out,
                          int* splits_out, int* split_len_out) {
  if (n_q <= 0 || heads <= 0 || kv_blocks <= 0 || num_sms <= 0 || max_splits <= 0 || q_tiles_per_cta_out == nullptr ||
      splits_out == nullptr || split_len_out == nullptr)
    return fail(GCT_ERR_INVALID, "gct_attn_launch_shape: bad argument");
  choose_attention_config((n_q + kTileM - 1) / kTileM, heads, kv_blocks, num_sms, max_splits, q_tiles_per_cta_out, splits_out,
                          split_len_out);
  return GCT_OK;
}

int gct_attn_dense(const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev, int batch, int n_q, int n_kv,
                   int heads, const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                   void* workspace_dev, size_t workspace_bytes, void* stream) {
  if (q_dev == nullptr || k_dev == nullptr || v_dev == nullptr || out_dev == nullptr || q_strides == nullptr ||
      k_strides == nullptr || v_strides == nullptr)
    return fail(GCT_ERR_INVALID, "gct_attn_dense: null argument");
  if (batch <= 0 || n_q <= 0 || n_kv <= 0 || heads <= 0) return fail(GCT_ERR_INVALID, "gct_attn_dense: bad shape");
  if (workspace_dev == nullptr || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace_dev) & 255))
    return fail(GCT_ERR_CAPACITY, "gct_attn_dense: needs a 256-byte aligned workspace of at least 256 bytes (status word)");
  AttnLaunch a;
  // strides are (batch, token, head) in elements
  int rc = make_tensor_map(&a.tm_q, q_dev, heads, n_q, batch, q_strides[2], q_strides[1], q_strides[0]);
  if (rc != GCT_OK) return rc;
  rc = make_tensor_map(&a.tm_k, k_dev, heads, n_kv, batch, k_strides[2], k_strides[1], k_strides[0]);
  if (rc != GCT_OK) return rc;
  rc = make_tensor_map(&a.tm_v, v_dev, heads, n_kv, batch, v_strides[2], v_strides[1], v_strides[0]);
  if (rc != GCT_OK) return rc;
  a.page_table = nullptr;
  a.n_pages = 1;
  a.page_len = n_kv;
  a.last_page_len = n_kv;
  a.n_q = n_q;
  a.heads = heads;
  a.batch = batch;
  a.status = static_cast<int*>(workspace_dev);
  const int total_blocks = (n_kv + kBlockN - 1) / kBlockN;
  const size_t rows = static_cast<size_t>(batch) * n_q * heads;
  const size_t per_split = rows * kHeadDim * 4 + rows * 4;
  const int max_splits = static_cast<int>(std::min<size_t>((workspace_bytes - 256) / per_split, kMaxSplitsCap));
  int sms = 148;
  rc = device_sm_count(&sms);
  if (rc != GCT_OK) return rc;
  choose_attention_config((n_q + kTileM - 1) / kTileM, heads * batch, total_blocks, sms, std::max(max_splits, 1),
                          &a.q_tiles_per_cta, &a.splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.splits == 1) {
    a.final_bf16 = true;
    a.out = static_cast<__nv_bfloat16*>(out_dev);
    return launch_attention(a, s);
  }
  a.final_bf16 = false;
  a.part_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace_dev) + 256);
  a.part_lse = a.part_o + static_cast<size_t>(a.splits) * rows * kHeadDim;
  rc = launch_attention(a, s);
  if (rc != GCT_OK) return rc;
  return launch_merge(a.part_o, a.part_lse, a.splits, static_cast<int64_t>(rows), static_cast<__nv_bfloat16*>(out_dev),
                      nullptr, nullptr, s);
}

int gct_prep_qkv(const void* qkv_dev, int qkv_dtype, int64_t qkv_row_stride, int tokens, int tokens_per_frame, int heads,
                 const float* qn_w_dev, const float* qn_b_dev, const float* kn_w_dev, const float* kn_b_dev,
                 const float* rope_cs_dev, int rope_mode, void* q_out_dev, void* k_out_dev, void* v_out_dev, void* stream) {
  if (qkv_dev == nullptr || q_out_dev == nullptr || k_out_dev == nullptr || v_out_dev == nullptr)
    return fail(GCT_ERR_INVALID, "gct_prep_qkv: null argument");
  if (qkv_dtype != GCT_F32 && qkv_dtype != GCT_BF16) return fail(GCT_ERR_INVALID, "gct_prep_qkv: dtype");
  if ((qn_w_dev == nullptr) != (qn_b_dev == nullptr) || (kn_w_dev == nullptr) != (kn_b_dev == nullptr))
    return fail(GCT_ERR_INVALID, "gct_prep_qkv: norm weight and bias must come together");
  const int64_t C = static_cast<int64_t>(heads) * kHeadDim;
  if (qkv_row_stride < 3 * C) return fail(GCT_ERR_INVALID, "gct_prep_qkv: row stride smaller than 3*H*64");
  PrepLaunch p;
  const size_t esz = qkv_dtype == GCT_F32 ? 4 : 2;
  p.q_src = qkv_dev;
  p.k_src = static_cast<const uint8_t*>(qkv_dev) + C * esz;
  p.v_src = static_cast<const uint8_t*>(qkv_dev) + 2 * C * esz;
  p.src_dtype_qk = p.src_dtype_v = qkv_dtype;
  p.src_token_stride = qkv_row_stride;
  p.src_head_stride = kHeadDim;
  p.tokens = tokens;
  p.tokens_per_frame = tokens_per_frame;
  p.heads = heads;
  p.qn_w = qn_w_dev;
  p.qn_b = qn_b_dev;
  p.kn_w = kn_w_dev;
  p.kn_b = kn_b_dev;
  p.rope_cs = rope_cs_dev;
  p.rope_mode = rope_mode;
  p.q_out = static_cast<__nv_bfloat16*>(q_out_dev);
  p.k_out = static_cast<__nv_bfloat16*>(k_out_dev);
  p.v_out = static_cast<__nv_bfloat16*>(v_out_dev);
  return launch_prep(p, static_cast<cudaStream_t>(stream));
}

int gct_rope3d_table(int frame_index, int pph, int ppw, int num_special, float* cs_out_dev, void* stream) {
  if (cs_out_dev == nullptr || pph <= 0 || ppw <= 0 || num_special < 0 || frame_index < 0)
    return fail(GCT_ERR_INVALID, "gct_rope3d_table: bad argument");
  return launch_rope3d_table(frame_index, pph, ppw, num_special, cs_out_dev, static_cast<cudaStream_t>(stream));
}

int gct_rope2d_table(int pph, int ppw, int num_special, float base, float* cs_out_dev, void* stream) {
  if (cs_out_dev == nullptr || pph <= 0 || ppw <= 0 || num_special < 0 || !(base > 0.f))
    return fail(GCT_ERR_INVALID, "gct_rope2d_table: bad argument");
  return launch_rope2d_table(pph, ppw, num_special, base, cs_out_dev, static_cast<cudaStream_t>(stream));
}

int gct_lse_merge(const float* parts_dev, const float* lse_dev, int groups, int n_q, int heads, void* out_dev,
                  float* lse_out_dev, void* stream) {
  if (parts_dev == nullptr || lse_dev == nullptr || out_dev == nullptr) return fail(GCT_ERR_INVALID, "gct_lse_merge: null argument");
  return launch_merge(parts_dev, lse_dev, groups, static_cast<int64_t>(n_q) * heads, static_cast<__nv_bfloat16*>(out_dev),
                      nullptr, lse_out_dev, static_cast<cudaStream_t>(stream));
}

int gct_lse_merge_strided(const float* parts_dev, const float* lse_dev, int groups, int n_q, int heads,
                          int64_t parts_group_stride, int64_t lse_group_stride, void* out_dev, float* lse_out_dev,
                          void* stream) {
  if (parts_dev == nullptr || lse_dev == nullptr || out_dev == nullptr)
    return fail(GCT_ERR_INVALID, "gct_lse_merge_strided: null argument");
  if (parts_group_stride <= 0 || lse_group_stride <= 0) return fail(GCT_ERR_INVALID, "gct_lse_merge_strided: bad stride");
  return launch_merge(parts_dev, lse_dev, groups, static_cast<int64_t>(n_q) * heads, static_cast<__nv_bfloat16*>(out_dev),
                      nullptr, lse_out_dev, static_cast<cudaStream_t>(stream), parts_group_stride, lse_group_stride);
}

}  // extern "C"
