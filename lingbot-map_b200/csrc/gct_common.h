// Shared declarations of the GCT B200 backend: error plumbing and the launch interfaces
// between the C-ABI layer (gct_manager.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>

#include "../../include/gct_b200.h"

namespace gct {

// Thread-local error text behind gct_last_error().
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define GCT_CUDA_CHECK(expr)                                                                  \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::gct::fail(GCT_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));   \
  } while (0)

// Programmatic dependent launch between this library's back-to-back kernels of one stream.  A kernel launched
// through launch_pdl may be scheduled while the last wave of its predecessor is still running; it does its private
// set-up (barriers, TMEM, descriptor prefetch) and then blocks in pdl_wait() until the predecessor has completed and
// its memory is visible, so stream order is preserved for every global access.  What is gained is the launch
// latency and the prologue of every kernel boundary of the five-launch layer loop.
#ifndef GCT_PDL
#define GCT_PDL 1
#endif
__device__ __forceinline__ void pdl_wait() {
#if GCT_PDL
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = GCT_PDL ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

constexpr int kHeadDim = 64;
constexpr int kBlockN = 128;   // KV tokens per attention block (one UMMA N tile)
constexpr int kTileM = 128;    // query rows per UMMA tile

// Codes written to the device status word by kernels (0 = ok).
constexpr int kStatusWaitTimeout = 1;   // a bounded mbarrier wait gave up
constexpr int kStatusBadIndex = 2;      // a page id / token offset failed its bounds check

// ---- attention -------------------------------------------------------------------------
// KV is a list of pages; every page but the last holds page_len tokens, the last one
// last_page_len.  A page is cut into blocks of kBlockN tokens (the tail block of a page is
// partial and masked).  With page_table == nullptr page i of batch item b is page id b
// (dense K/V: one page per batch item).
struct AttnLaunch {
  CUtensorMap tm_q, tm_k, tm_v;      // 4-D maps (d, head, token, page|batch), box {64,1,128,1}, 128B swizzle
  const int32_t* page_table = nullptr;
  int n_pages = 0;
  int page_len = 0;
  int last_page_len = 0;
  int n_q = 0, heads = 0, batch = 1;
  int q_tiles_per_cta = 2;           // 1 or 2
  int splits = 1;
  int split_len = 0;                 // 0: `splits` equal ranges of KV blocks; > 0: splits - 1 ranges of split_len blocks, the last
                                     // one takes the (shorter) rest and its CTAs are launched last
  bool final_bf16 = true;            // true: write bf16 out (requires splits == 1); false: partials
  __nv_bfloat16* out = nullptr;      // [batch, n_q, H, 64]
  float* part_o = nullptr;           // [splits, batch, n_q, H, 64] normalised partial outputs
  float* part_lse = nullptr;         // [splits, batch, n_q, H] natural log-sum-exp
  int* status = nullptr;             // device status word
  // bounded mode (two query tiles per CTA only): key_norm_max[h] bounds the 2-norm of every key of head h that the
  // page table reaches; a CTA uses |q_row| * key_norm_max[h] * scale * log2(e) as the fixed softmax reference of
  // its rows while that stays within bounded_limit, otherwise it tracks the running row maximum
  const float* key_norm_max = nullptr;   // [H]; null: no bounded mode
  float bounded_limit = 0.f;
};
int launch_attention(const AttnLaunch& a, cudaStream_t stream);
int attention_smem_bytes(int q_tiles_per_cta);

// Encode a 4-D bf16 tensor map {64, heads, tokens, pages} with the given element strides
// (head, token, page) and the box {64,1,128,1}.
int make_tensor_map(CUtensorMap* out, const void* base, int heads, int64_t tokens, int64_t pages,
                    int64_t head_stride, int64_t token_stride, int64_t page_stride);

// Pick (q_tiles_per_cta, splits) for a problem: n_q_tiles query tiles of 128 rows per (head,batch),
// total_blocks KV blocks, on num_sms SMs, with at most max_splits partial results.  With split_len != nullptr the
// plan may also be splits - 1 long ranges plus one short one (AttnLaunch::split_len), which fills the SMs that a whole
// number of equal ranges leaves idle; *split_len = 0 when equal ranges are at least as good.
void choose_attention_config(int n_q_tiles, int heads_x_batch, int total_blocks, int num_sms, int max_splits,
                             int* q_tiles_per_cta, int* splits, int* split_len = nullptr);

// ---- elementwise kernels ---------------------------------------------------------------
struct PrepLaunch {
  // sources: rows of 64 elements; element strides between tokens and heads
  const void* q_src = nullptr; const void* k_src = nullptr; const void* v_src = nullptr;
  int src_dtype_qk = GCT_BF16;       // dtype of q_src and k_src
  int src_dtype_v = GCT_BF16;
  int64_t src_token_stride = 0, src_head_stride = 64;
  int tokens = 0, heads = 0, tokens_per_frame = 0;
  const float* qn_w = nullptr; const float* qn_b = nullptr;   // null: no LayerNorm
  const float* kn_w = nullptr; const float* kn_b = nullptr;
  const float* rope_cs = nullptr;    // [tokens_per_frame, 32, 2] cos,sin; null or mode NONE: no rotation
  int rope_mode = GCT_ROPE_NONE;
  __nv_bfloat16* q_out = nullptr;    // [tokens, H, 64] or null
  // K/V destination, dense: [tokens, H, 64]
  __nv_bfloat16* k_out = nullptr; __nv_bfloat16* v_out = nullptr;
  // K/V destination, paged (k_out == null): pool [pages, 2, page_size, H, 64]
  __nv_bfloat16* pool = nullptr;
  int page_size = 0, num_pages = 0, num_special = 0;
  int patch_page = -1;               // tokens >= num_special go to row (token - num_special) of this page
  int sp_page0 = -1, sp_off0 = 0, sp_n0 = 0, sp_page1 = -1;   // specials: first sp_n0 at sp_off0 of page0, rest at row 0.. of page1
  int* status = nullptr;
  float* key_norm_max = nullptr;     // [H] running maximum of the 2-norms of the K rows written (paged destination)
};
int launch_prep(const PrepLaunch& p, cudaStream_t stream);

// key_norm_max[head] = max over all K rows of the pool [pages, 2, page_size, heads, 64] of their 2-norm
int launch_scan_keys(const __nv_bfloat16* pool, int num_pages, int page_size, int heads, float* key_norm_max,
                     cudaStream_t stream);
int launch_cast_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t stream);
// parts_stride / lse_stride: elements between consecutive groups (0 = densely packed).
int launch_merge(const float* parts, const float* lse, int groups, int64_t rows /* n_q*H */, __nv_bfloat16* out_bf16,
                 float* out_f32, float* lse_out, cudaStream_t stream, int64_t parts_stride = 0, int64_t lse_stride = 0);
// KV-sharded single stream: two-phase exchange + merge over peer-mapped buffers (gct_exchange.cu).
// parts/lses: this rank's split partials [S][rows][64], [S][rows] (null: the rank owns no page);
// recv/out/flag pointers: one per rank, addresses valid on this device.
int launch_kv_exchange(const float* parts, const float* lses, int splits, int rows, int rank, int world, int epoch,
                       void* const* recv_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int slice_max, int* status,
                       cudaStream_t stream);
int launch_rope3d_table(int f, int pph, int ppw, int ns, float* cs, cudaStream_t stream);
int launch_rope2d_table(int pph, int ppw, int ns, float base, float* cs, cudaStream_t stream);

}  // namespace gct
