/*
 * gct_b200.h - C ABI of the B200 (sm_100a) attention backend for the streaming
 * Geometric Context Transformer: paged two-stream KV cache manager, fused
 * q/k-norm + RoPE + bf16 page append, tcgen05 paged/dense attention, split-KV merge.
 *
 * Conventions
 *   - Every function returns an int status: 0 = ok, otherwise one of GCT_ERR_*.
 *     Nothing throws, nothing traps.  gct_last_error() returns a thread-local,
 *     human-readable description of the last failure on the calling thread.
 *   - Pointers named *_dev are device pointers on the current CUDA device; `stream` is a
 *     cudaStream_t passed as void*.  A manager belongs to the device that was current at
 *     gct_mgr_bind: make that device current for every later call on it.  The library never allocates or frees device memory:
 *     page pools, workspace and outputs belong to the caller.
 *   - Token-major "NHD" tensors: [tokens, heads, head_dim] with head_dim == 64.
 *   - dtype codes: GCT_F32 = 0, GCT_BF16 = 1.
 *
 * The comments cite the interface of the reference implementation (paths relative to the
 * Robbyant/lingbot-map repository) that each entry point stands in for.
 */
#ifndef GCT_B200_H
#define GCT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GCT_OK 0
#define GCT_ERR_INVALID 1        /* bad argument (shape, dtype, null pointer, unbound pools) */
#define GCT_ERR_POOL_EXHAUSTED 2 /* no free patch/special page: flashinfer_cache.py:489-494,533-537 */
#define GCT_ERR_UNDERFLOW 3      /* rollback with nothing to roll back: flashinfer_cache.py:276-293 */
#define GCT_ERR_CUDA 4           /* a CUDA runtime/driver call failed */
#define GCT_ERR_DEVICE_STATUS 5  /* a kernel reported a bounded-wait timeout or an index check */
#define GCT_ERR_CAPACITY 6       /* caller-provided buffer or workspace too small */

#define GCT_F32 0
#define GCT_BF16 1

#define GCT_ROPE_NONE 0
#define GCT_ROPE_2D 1 /* rotate-half inside each 32-wide half: lingbot_map/layers/rope.py:134-198 */
#define GCT_ROPE_3D 2 /* interleaved pairs (2m,2m+1): lingbot_map/layers/rope.py:435-461 */

typedef struct gct_mgr gct_mgr_t;

/* Geometry of one cache manager: arguments of FlashInferKVCacheManager.__init__
 * (lingbot_map/layers/flashinfer_cache.py:75-90). */
typedef struct gct_mgr_config {
  int32_t num_blocks;
  int32_t tokens_per_frame;   /* patches + specials, specials first */
  int32_t num_heads;
  int32_t head_dim;           /* must be 64 */
  int32_t num_special_tokens; /* 6 */
  int32_t scale_frames;       /* 8 */
  int32_t sliding_window;     /* 64 */
  int32_t max_total_frames;   /* sizes the special-page pool */
} gct_mgr_config_t;

/* Derived sizes (flashinfer_cache.py:100-138). */
typedef struct gct_mgr_geometry {
  int32_t page_size;       /* tokens per page = patches per frame */
  int32_t max_patch_pages; /* scale + window + 16 */
  int32_t max_num_pages;   /* patch pages + special pages */
  int64_t pool_bytes;      /* bytes of one block's pool [max_num_pages,2,page_size,H,64] bf16 */
} gct_mgr_geometry_t;

const char* gct_last_error(void);
int gct_version(void);

/* ---- cache manager: host bookkeeping (bit-exact with the reference) ------------------- */

/* FlashInferKVCacheManager.__init__ (flashinfer_cache.py:75-196), minus allocation. */
int gct_mgr_create(gct_mgr_t** out, const gct_mgr_config_t* cfg, gct_mgr_geometry_t* geo_out);
int gct_mgr_destroy(gct_mgr_t* m);

/* Hand the manager the caller-allocated device memory: one bf16 pool per block laid out
 * [max_num_pages, 2 (K,V), page_size, H, 64] (flashinfer_cache.py:141-148) and a workspace for
 * split-KV partial results, the device page table and the status word (the reference's
 * workspace_buffer, flashinfer_cache.py:184-186).  Needs a CUDA device.
 * Every row of a pool must hold finite values, also rows that no append has written yet: the attention kernel reads
 * whole 128-token blocks, masks the rows past the valid length of a page, and multiplies their (zero) weights with
 * whatever V holds there - zero-initialise the pools (0 * NaN would be NaN). */
int gct_mgr_bind(gct_mgr_t* m, void* const* pools_dev, void* workspace_dev, size_t workspace_bytes);
/* Smallest workspace gct_mgr_bind accepts for this geometry. */
int gct_mgr_workspace_bytes(const gct_mgr_t* m, size_t* bytes_out);

/* append_frame (flashinfer_cache.py:202-227, 474-553): allocate one patch page (LIFO), route it to
 * the scale or window list, append the specials to the special stream, and write K/V as bf16.
 * k_dev/v_dev: [tokens_per_frame, H, 64] contiguous, dtype GCT_F32 or GCT_BF16. */
int gct_mgr_append(gct_mgr_t* m, int block, const void* k_dev, int k_dtype, const void* v_dev, int v_dtype,
                   void* stream);
/* Same bookkeeping without touching device memory (tests, dry runs, replicas that do not own a page).  The
 * caller is then responsible for the page contents; bounded mode (below) is switched off for the block until
 * gct_mgr_scan_keys is called. */
int gct_mgr_append_bookkeeping(gct_mgr_t* m, int block);

/* Bounded mode of the paged attention (no counterpart in the reference): the manager keeps, per block and head,
 * the largest 2-norm of the K rows written through gct_mgr_append / gct_mgr_append_fused.  |q_row| times that
 * maximum bounds every logit of the row, and while the bound is small (checked on the device for every call) it
 * replaces the running row maximum of the online softmax, which removes the maximum and rescale work from the
 * kernel; otherwise the exact kernel runs.  Results are the same softmax either way.
 * The maxima are floats [num_blocks][H] at byte offset 256 of the bound workspace (the mode is unavailable when they
 * do not fit into its 4096-byte header, i.e. num_blocks * H > 960).
 * gct_mgr_scan_keys recomputes the maxima of a block from its whole pool (after writing pages directly);
 * gct_mgr_set_bounded_mode(m, 0) forces the exact kernel. */
int gct_mgr_scan_keys(gct_mgr_t* m, int block, void* stream);
int gct_mgr_set_bounded_mode(gct_mgr_t* m, int enable);

/* Fused tail of FlashInferAttention.prepare_qkv (lingbot_map/layers/attention.py:413-426) and
 * append_frame: from the qkv Linear output [tokens, 3*H*64] apply LayerNorm(64) to q and k
 * (attention.py:58-59,415), rotate them with the per-token cos/sin table `rope_cs_dev`
 * [tokens, 32, 2] fp32, write q as bf16 NHD to q_out_dev and K/V straight into their pages. */
int gct_mgr_append_fused(gct_mgr_t* m, int block, const void* qkv_dev, int qkv_dtype, int64_t qkv_row_stride,
                         const float* qn_w_dev, const float* qn_b_dev, const float* kn_w_dev, const float* kn_b_dev,
                         const float* rope_cs_dev, int rope_mode, void* q_out_dev, void* stream);

/* evict_frames (flashinfer_cache.py:229-254): no-op while eviction is deferred. */
int gct_mgr_evict(gct_mgr_t* m, int block, int sliding_window);
/* execute_deferred_eviction (flashinfer_cache.py:256-266). */
int gct_mgr_exec_deferred(gct_mgr_t* m, int block, int sliding_window);
/* the _defer_eviction attribute (flashinfer_cache.py:172-175; set by block.py:258-263). */
int gct_mgr_set_defer(gct_mgr_t* m, int defer);
int gct_mgr_get_defer(const gct_mgr_t* m, int* defer_out);
/* rollback_last_frame (flashinfer_cache.py:268-301). */
int gct_mgr_rollback(gct_mgr_t* m, int block);
/* reset (flashinfer_cache.py:423-432). */
int gct_mgr_reset(gct_mgr_t* m);

/* build_visible_page_table + compute_last_page_len (flashinfer_cache.py:438-470):
 * page ids in the order scale, window, special. */
int gct_mgr_visible_table(const gct_mgr_t* m, int block, int32_t* pages_out, int capacity, int* n_out,
                          int* last_page_len_out);
/* get_cache_stats (flashinfer_cache.py:303-322): frame_count, scale_pages, live_pages, free_pages,
 * special_tokens, special_pages. */
int gct_mgr_stats(const gct_mgr_t* m, int block, int64_t out[6]);
/* Free lists in stack order (bottom first): which = 0 patch, 1 special. */
int gct_mgr_free_list(const gct_mgr_t* m, int block, int which, int32_t* out, int capacity, int* n_out);

/* ---- cache manager: attention ------------------------------------------------------ */

/* The plan() half of compute_attention (flashinfer_cache.py:385-414): snapshot block 0's visible
 * table and upload it; valid for every block until the next plan.  page_begin/page_end select a
 * sub-range of the visible list (0, -1 = all) for KV-sharded execution. */
int gct_mgr_plan(gct_mgr_t* m, int page_begin, int page_end, void* stream);

/* The run() half (flashinfer_cache.py:416-421): softmax(q k^T / 8) v over the planned pages of `block`.
 * q_dev [n_q, H, 64] (GCT_F32 or GCT_BF16; cast to bf16 first as the reference does, :419),
 * out_dev [n_q, H, 64] bf16.  lse_dev (optional, may be NULL) receives the natural log-sum-exp
 * [n_q, H] fp32. */
int gct_mgr_attention(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q, void* out_dev,
                      float* lse_dev, void* stream);
/* Same, but leaves the result un-rounded: out_f32_dev [n_q, H, 64] fp32 plus lse_dev (required).
 * Used when partial results over a page sub-range are merged across GPUs. */
int gct_mgr_attention_partial(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q,
                              float* out_f32_dev, float* lse_dev, void* stream);

/* Reads the device status word (blocks on `stream`): 0 if no kernel reported a problem. */
int gct_mgr_device_status(gct_mgr_t* m, void* stream, int* status_out);
/* Measurement aid (no counterpart in the reference): bracket every launch of the attention kernel
 * with a CUDA-event pair on the launching stream, for up to max_launches launches (0 switches it
 * off); gct_mgr_kernel_time waits for them, returns the summed kernel time and rearms the events. */
int gct_mgr_kernel_timing(gct_mgr_t* m, int max_launches);
int gct_mgr_kernel_time(gct_mgr_t* m, double* total_ms_out, int* launches_out);
/* Number of kernels this manager has launched since creation. */
int gct_mgr_launch_count(const gct_mgr_t* m, int64_t* count_out);

/* How a paged attention call of the manager is cut into CTAs (host arithmetic only, no device needed; the reference
 * leaves this to FlashInfer's plan(), flashinfer_cache.py:398-410): n_q query rows, `heads` heads, kv_blocks KV
 * blocks of 128 tokens, on a device with num_sms SMs, at most max_splits partial results per row.  Outputs: query
 * tiles of 128 rows per CTA (1 or 2), the number of KV ranges per (head, query group), and split_len: 0 = equal
 * ranges, > 0 = splits - 1 ranges of split_len blocks followed by one shorter range whose CTAs are launched last. */
int gct_attn_launch_shape(int n_q, int heads, int kv_blocks, int num_sms, int max_splits, int* q_tiles_per_cta_out,
                          int* splits_out, int* split_len_out);

/* ---- stand-alone operators --------------------------------------------------------- */

/* Dense non-causal attention, the F.scaled_dot_product_attention call of Attention.forward
 * (lingbot_map/layers/attention.py:76) and of the phase-1 branch (attention.py:490).
 * q [batch, n_q, H, 64], k/v [batch, n_kv, H, 64], all bf16, arbitrary element strides
 * (multiples of 8 elements; head_dim contiguous); out [batch, n_q, H, 64] bf16 contiguous.
 * workspace is needed only when the call splits the KV range (n_kv large, few query tiles). */
int gct_attn_dense(const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev, int batch, int n_q,
                   int n_kv, int heads, const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], void* workspace_dev, size_t workspace_bytes, void* stream);

/* q/k LayerNorm + RoPE + bf16 cast for one batch of frames without a cache (frame blocks,
 * attention.py:67-73): qkv [tokens, 3*H*64] -> q,k,v bf16 [tokens, H, 64].  rope_cs_dev is indexed
 * by (token % tokens_per_frame). */
int gct_prep_qkv(const void* qkv_dev, int qkv_dtype, int64_t qkv_row_stride, int tokens, int tokens_per_frame,
                 int heads, const float* qn_w_dev, const float* qn_b_dev, const float* kn_w_dev,
                 const float* kn_b_dev, const float* rope_cs_dev, int rope_mode, void* q_out_dev, void* k_out_dev,
                 void* v_out_dev, void* stream);

/* cos/sin tables [tokens_per_frame, 32, 2] fp32.
 * 3-D (rope.py:293-433): time index f, specials at (f,i,i), patch (r,c) at (f,ns+r,ns+c), theta 1e4,
 * axis split 20/22/22, angles in fp64.  2-D (rope.py:88-122, base.py:416-442): specials at (0,0),
 * patches at (r+1,c+1), base 100, angles in fp32. */
int gct_rope3d_table(int frame_index, int pph, int ppw, int num_special, float* cs_out_dev, void* stream);
int gct_rope2d_table(int pph, int ppw, int num_special, float base, float* cs_out_dev, void* stream);

/* Merge G partial attention results: out = sum_g e^{lse_g-m} O_g / sum_g e^{lse_g-m}.
 * parts_dev [G, n_q, H, 64] fp32 (each already normalised), lse_dev [G, n_q, H] fp32,
 * out_dev [n_q, H, 64] bf16; lse_out_dev optional. */
int gct_lse_merge(const float* parts_dev, const float* lse_dev, int groups, int n_q, int heads, void* out_dev,
                  float* lse_out_dev, void* stream);
/* Same with explicit distances (in floats) between consecutive groups, for partials that arrive packed as
 * one [O | lse] record per rank from a single all-gather (no counterpart in the reference, which is
 * single-GPU). */
int gct_lse_merge_strided(const float* parts_dev, const float* lse_dev, int groups, int n_q, int heads,
                          int64_t parts_group_stride, int64_t lse_group_stride, void* out_dev, float* lse_out_dev,
                          void* stream);

/* KV-sharded single stream over several GPUs (no counterpart in the reference, which is single-GPU; the result
 * equals compute_attention, flashinfer_cache.py:385-421, over the union of the ranks' page slices).  Every rank has
 * planned its own slice of the visible page list (gct_mgr_plan with a sub-range; has_pages = 0 for a rank whose
 * slice is empty) and calls this once per layer, all ranks in the same order.  The call runs the paged attention
 * over the slice and then one kernel that (1) stores, for every peer, this rank's partial result of the rows the
 * peer owns into the peer's receive buffer and raises a flag there, (2) waits for every rank's flag, merges the
 * partials of its own row slice by their log-sum-exps, rounds to bf16 and stores the rows into every rank's output
 * buffer, (3) waits until every rank's rows have arrived.  Plain loads and stores on peer-mapped addresses.
 *   recv_ptrs[r], out_ptrs[r], flag_ptrs[r]: rank r's receive buffer (gct_kv_exchange_sizes bytes), output
 *   [n_q, H, 64] bf16 and flag words (zeroed once before the first call), as addresses valid on THIS device
 *   (symmetric / peer-mapped memory; entry `rank` is local memory).  epoch: 1, 2, 3, ... per call on the same flag
 *   words, identical on every rank.  All waits are bounded; a timeout sets the manager's device status word.
 *   The exchange kernel's CTAs wait on their peers and its grid is sized to be resident at once on an otherwise
 *   idle device: do not run another kernel that itself waits on a peer (a collective on a second stream, say)
 *   beside it - each could keep the other's CTAs from being scheduled until the bounded waits give up. */
int gct_kv_exchange_sizes(int n_q, int heads, int world, size_t* recv_bytes_out, size_t* flag_bytes_out,
                          int* slice_rows_out);
int gct_mgr_attention_exchange(gct_mgr_t* m, int block, const void* q_dev, int q_dtype, int n_q, int rank, int world,
                               int has_pages, void* const* recv_ptrs, void* const* out_ptrs, void* const* flag_ptrs,
                               int slice_rows, int epoch, void* stream);

/* Append-only cache of ONE token per frame with its attention, for the camera head: CausalAttention's streaming
 * branch (lingbot_map/layers/attention.py:222-283) as the camera head drives it (lingbot_map/heads/camera_head.py:
 * 284-358): the dict cache there grows by torch.cat every frame, is cloned and never evicted (attention.py:307).
 * cache_k_dev / cache_v_dev: [capacity, H, D] fp32 owned by the caller, `cached` rows valid.  The n_new (1..8) new
 * tokens q/k_new/v_new [n_new, H, D] fp32 attend to the cached rows and to each other (all-true mask,
 * attention.py:276-283); with store != 0 their K/V rows are appended at row `cached` (the caller then counts them),
 * with store == 0 they are used for this call only (a non-keyframe, attention.py:243-249).  head_dim 64 or 128,
 * fp32 arithmetic (the reference runs its heads in fp32).  The workspace (gct_decode_workspace_bytes) holds the
 * split partials and per-head counters; its first 4*H bytes must be zero before the first call. */
int gct_decode_workspace_bytes(int heads, int head_dim, size_t* bytes_out);
int gct_decode_attention(const float* q_dev, const float* k_new_dev, const float* v_new_dev, int n_new,
                         float* cache_k_dev, float* cache_v_dev, int cached, int capacity, int store, int heads,
                         int head_dim, float* out_dev, void* workspace_dev, size_t workspace_bytes, void* stream);

/* ---- point-cloud helpers of the offline renderer (compute only) ---------------------------- */

/* frustum_cull (demo_render/render_cuda_ext/frustum_cull/frustum_cull.cu:5-53): visible[i] = point i, moved to the
 * camera frame p = R_cw x + t_cw, lies strictly between the near and far plane and projects into the W x H image.
 * pts_dev [n, 3] fp32 (16-byte aligned), R_cw / t_cw on the HOST (row-major 3x3, 3), visible_dev [n] bytes (0/1).
 * Single rounded float operations, no fused multiply-add: a float32 CPU restatement gives the same bits; the
 * reference's build may contract a*b+c and can differ for points within one rounding step of an image border. */
int gct_frustum_cull(const float* pts_dev, int64_t n, const float R_cw[9], const float t_cw[3], float fx, float fy,
                     float cx, float cy, int width, int height, float near_plane, float far_plane, uint8_t* visible_dev,
                     void* stream);
/* compute_morton_kernel (demo_render/render_cuda_ext/voxel_morton/voxel_morton.cu:5-47): voxel index
 * floor(p / voxel_size) per axis, 63-bit Morton code of the indices offset by 2^20, voxel centre, colour copy. */
int gct_voxel_morton(const float* xyz_dev, const float* rgb_dev, float voxel_size, int64_t n, int64_t* codes_dev,
                     float* centers_dev, float* colors_dev, void* stream);
/* mark_unique_kernel (voxel_morton.cu:49-62): mask[i] = i == 0 or sorted[i] != sorted[i-1]. */
int gct_mark_unique(const int64_t* sorted_dev, int64_t n, uint8_t* mask_dev, void* stream);

/* Paged attention that allocates nothing (this entry point has no counterpart in the reference).
 * For hosts that cannot call cudaMalloc - e.g. a process that gave all device memory to its own pool
 * at start-up, or a loop that cannot afford cudaMalloc's device-wide synchronisation - and therefore
 * cannot provide the workspace gct_mgr_attention needs.  Same computation as gct_mgr_attention over the
 * pages `visible_pages_host[0..n_pages)` of one block's pool [max_num_pages, 2, page_size, heads, 64]
 * bf16; q_dev and out_dev are [n_q, heads, 64] bf16.  The scratch (device page table, split-KV
 * partials, status word) is a fixed array inside the library image, about 17 MB on every GPU that
 * loads the library, held until the process exits.
 * Limits: n_q * heads <= 16384, n_pages <= 4096 (GCT_ERR_CAPACITY beyond), at most 4 KV splits.
 * The first call on a device looks up the array's address on that device (cudaGetSymbolAddress); make
 * that first call before any stream capture begins.  All calls on a GPU share the array: calls whose
 * GPU work can overlap (several streams or host threads) race and must be serialised by the caller.
 * The pool belongs to the caller: every row of a visible page must hold finite values, also the rows of the last
 * page past last_page_len (they are read, masked, and their zero weights multiplied with what V holds there).
 * visible_pages_host is copied to the GPU by an asynchronous copy on `stream`: if it is pinned memory it must
 * stay alive and unchanged until `stream` has passed the call (pageable memory is staged before the call returns).
 * device_status_out may be NULL; otherwise the call synchronises `stream` and stores the kernels'
 * status word (0 = ok). */
int gct_attn_paged_static(const void* pool_dev, int max_num_pages, int page_size, int heads,
                          const int32_t* visible_pages_host, int n_pages, int last_page_len, const void* q_dev,
                          int n_q, void* out_dev, void* stream, int* device_status_out);

#ifdef __cplusplus
}
#endif
#endif /* GCT_B200_H */
