// Paged / dense non-causal attention for sm_100a: softmax(Q K^T / 8) V with head_dim 64, bf16 operands,
// fp32 accumulation.  Stands in for the reference's FlashInfer BatchPrefillWithPagedKVCacheWrapper.run
// (lingbot_map/layers/flashinfer_cache.py:416-421) and its F.scaled_dot_product_attention calls
// (lingbot_map/layers/attention.py:76,490).
//
// One CTA owns QT (1 or 2) query tiles of 128 rows of one head and one contiguous range of KV blocks
// (128 tokens each).  Warp roles:
//   warps [0, 4*QT)        softmax: one thread per query row; warp w owns TMEM lanes 32*(w%4)..+31
//   warp  4*QT             producer: TMA loads of Q once, then K and V blocks into two 4-stage rings
//   warps 4*QT+1 .. +QT    MMA issuers, one per query tile: tcgen05.mma
//                              S  = Q K^T   (M128 N128 K64,  A and B from shared memory)
//                              O += P V     (M128 N64  K128, A = P from TMEM, B = V from shared memory)
// TMEM columns (fp32): S_t at [128t, +128), O_t at [128QT + 64t, +64), P_t (bf16 pairs) at [192QT + 64t, +64).
// Per KV block j of tile t:
//   softmax   wait s_full; copy the S row into 128 registers; arrive s_empty  -> S_{j+1} may overwrite S
//             row max; the reference maximum only moves when the row max grows by more than 2^8
//             (then O is rescaled in TMEM, which is rare after the first blocks);
//             P = exp2(S*c - m*c) as bf16 pairs into TMEM; arrive p_full
//   MMA       wait s_empty, K_{j+1}: issue S_{j+1} (runs under the softmax of block j) -> s_full, k_empty
//             wait p_full,  V_j    : issue O += P_j V_j                                -> pv_full, v_empty
// Every mbarrier wait is bounded and reports through the status word instead of spinning forever.
//
// Bounded mode (gct_attn_kernel<2, true>, paged attention through the cache manager).  key_norm_max[h] bounds the
// 2-norm of every key of head h in the cache, so ref = |q_row| * key_norm_max[h] bounds every logit of the row
// (Cauchy-Schwarz) and can stand in for the running row maximum while it is small.  The softmax threads prepare
// this once per CTA from the Q tile in shared memory: they multiply their row by scale * log2(e) in place,
// derive ref from the scaled row, and write two small operand tiles, Qx (column 0 = -ref) and Kx (column 0 = 1).
// A fifth K16 step of the S product, S += Qx Kx^T, then subtracts ref inside the tensor core: S arrives in TMEM
// as the finished base-2 exponent, and the sweep is exp2, row sum and bf16 packing only - no row maximum, no
// multiply-add in front of the exponential, no rescale of O.  A CTA in which some row's ref exceeds the limit
// (or is not finite) takes a compact two-pass softmax with a running maximum instead; the choice is made per
// CTA inside the one launch.
#include <algorithm>
#include <mutex>
#include <vector>

#include "gct_common.h"

namespace gct {
namespace {

constexpr uint32_t kTileBytes = 128 * 64 * 2;      // one 128x64 bf16 tile, 128B-swizzled
constexpr long long kWaitLimitCycles = 4000000000LL;  // ~2 s at 2 GHz; only reached on a bug

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false when the CTA is aborting (this or another thread ran out of time, or
// another CTA flagged the status word); the caller then leaves its role loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*cta_abort) return false;
      if ((it & 1023u) == 0u && *reinterpret_cast<volatile int*>(status) != 0) {
        *cta_abort = 1;
        return false;
      }
      if (clock64() - t0 > kWaitLimitCycles) {
        *cta_abort = 1;
        atomicCAS(status, 0, kStatusWaitTimeout);
        return false;
      }
    }
  }
}

// ---- TMA ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// ---- tcgen05 ------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The MMA warps keep their control flow warp-uniform and predicate only the tcgen05 instructions on
// one elected lane (`lead` != 0 in that lane).  Descriptors and addresses computed by the whole warp
// can live in uniform registers; computed by a single lane inside a divergent branch they are moved
// there one by one before every instruction, which limits the issue rate to one MMA per ~60-90 clocks
// (measured), well below the 32-64 clocks an N=64/128, K=16 instruction occupies the tensor core.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t e;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
  return e;
}
__device__ __forceinline__ void tc_commit_elected(uint32_t lead, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "setp.ne.b32 e, %1, 0;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(lead)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 x bf16 -> fp32, issued by the elected lane.
__device__ __forceinline__ void umma_ss(uint32_t lead, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128B swizzle, descriptor version 1 (sm_100).
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1      bits [61,64) layout = 2 (SWIZZLE_128B)
// K-major tile (rows of 128 B, 8-row groups 1024 B apart): SBO = 1024, LBO unused (1).
// MN-major tile (k-rows of 128 B holding 64 contiguous MN elements): SBO = 1024 between 8-k-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor (kind::f16): c_format F32 (bit 4), a/b format BF16 (bits 7, 10),
// b_major at bit 16 (1 = MN-major), N>>3 at bits [17,23), M>>4 at bits [24,29).
constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV =
    (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

// D[tmem] (+)= A[tmem] * B[smem]: A is read from TMEM (lane = row, two bf16 per 32-bit column).
__device__ __forceinline__ void umma_ts(uint32_t lead, uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for two logits on the FMA pipe instead of the special-function unit: clamp to >= -125, split
// x = n + f with n = round(x) (adding 1.5 * 2^23 leaves n in the low mantissa bits), 2^f on [-0.5, 0.5] by a
// degree-3 polynomial (relative error 7.5e-5, far below bf16 resolution), then n is added to the exponent.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  constexpr float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = __fadd2_rn(x, make_float2(kMagic, kMagic));
  const float2 n = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
  const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
  p = __ffma2_rn(p, f, make_float2(0.6932609677f, 0.6932609677f));
  p = __ffma2_rn(p, f, make_float2(0.9999280572f, 0.9999280572f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}
// Same for exponents known to lie in [-126, 1]: no clamp.  kDeg 3: relative error 7.7e-5; kDeg 2: 1.8e-3.
// `shift` (a non-negative integer value) is subtracted from the exponent first, at no cost: it rides in the rounding
// constant.
template <int kDeg>
__device__ __forceinline__ float2 exp2_poly2_inrange(float2 x, float shift = 0.f) {
  constexpr float kMagic = 12582912.f;
  const float ms = kMagic - shift;                       // exact: both are integers below 2^24
  const float2 t = __fadd2_rn(x, make_float2(ms, ms));   // 1.5 * 2^23 + round(x - shift)
  const float2 n = __fadd2_rn(t, make_float2(-ms, -ms)); // round(x - shift) + shift
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 p;
  if constexpr (kDeg == 3) {
    p = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
    p = __ffma2_rn(p, f, make_float2(0.6932609677f, 0.6932609677f));
    p = __ffma2_rn(p, f, make_float2(0.9999280572f, 0.9999280572f));
  } else {
    p = __ffma2_rn(make_float2(0.23783042f, 0.23783042f), f, make_float2(0.70339652f, 0.70339652f));
    p = __ffma2_rn(p, f, make_float2(1.0005137f, 1.0005137f));
  }
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

struct KernelArgs {
  const int32_t* page_table;
  int n_pages, page_len, last_page_len, blocks_per_page, total_blocks;
  int n_q, heads, batch, q_groups, splits, split_len, final_bf16;
  float scale_log2;
  __nv_bfloat16* out;
  float* part_o;
  float* part_lse;
  int* status;
  // Bounded mode: key_norm_max[h] >= the 2-norm of every key of head h that the page table can reach;
  // bounded_limit is the largest row reference (in base-2 exponent units) a CTA accepts before it falls back
  // to the running-maximum softmax.  Null: the kernel instantiation without the bounded mode is launched.
  const float* key_norm_max;
  float bounded_limit;
};

constexpr int kKStages = 4;
constexpr int kVStages = 4;
#ifndef GCT_POLY_EVERY
#define GCT_POLY_EVERY 3
#endif
constexpr int kPolyEvery = GCT_POLY_EVERY;   // 0: all exponentials on the special-function unit
#ifndef GCT_FFMA_AHEAD
#define GCT_FFMA_AHEAD 4
#endif
#ifndef GCT_SUM_LAG
#define GCT_SUM_LAG 2
#endif
constexpr int kFfmaAhead = GCT_FFMA_AHEAD;   // software pipeline of the exponential sweep, in pairs of logits
constexpr int kSumLag = GCT_SUM_LAG;
#ifndef GCT_MAX_CHAINS
#define GCT_MAX_CHAINS 4
#endif
#ifndef GCT_PV_WAIT_AT
#define GCT_PV_WAIT_AT 31
#endif
constexpr int kPvWaitAt = GCT_PV_WAIT_AT;    // pair (31..61) after which the sweep waits for the previous PV and stores P[0,64)
constexpr int kMaxChains = GCT_MAX_CHAINS;
// Bounded mode: pair q of the sweep takes the polynomial when floor((q+1) * NUM / DEN) != floor(q * NUM / DEN),
// i.e. NUM of every DEN pairs, evenly spread; the rest go to the special-function unit.
#ifndef GCT_BOUNDED_POLY_NUM
#define GCT_BOUNDED_POLY_NUM 2
#endif
#ifndef GCT_BOUNDED_POLY_DEN
#define GCT_BOUNDED_POLY_DEN 5
#endif
#ifndef GCT_BOUNDED_POLY_DEG
#define GCT_BOUNDED_POLY_DEG 3
#endif
#ifndef GCT_BOUNDED_HALF_AT
#define GCT_BOUNDED_HALF_AT 30
#endif
constexpr int kBoundedPolyNum = GCT_BOUNDED_POLY_NUM, kBoundedPolyDen = GCT_BOUNDED_POLY_DEN;
constexpr int kBoundedPolyDeg = GCT_BOUNDED_POLY_DEG;
constexpr int kBoundedHalfAt = GCT_BOUNDED_HALF_AT;   // pair before which the second half of the S row must have landed
static_assert(kBoundedHalfAt >= 0 && kBoundedHalfAt <= 32, "the second half of the row is needed from pair 32 on");
// 1: P of a block is announced to the MMA warp as soon as its stores have completed, at the end of the block's
// iteration; 0: by the next iteration, after it has issued its first S loads (hides the store latency, but the
// PV product then starts later and its completion is waited for in the middle of the next sweep).
#ifndef GCT_EARLY_P_FULL
#define GCT_EARLY_P_FULL 1
#endif
// 1: the row reference is subtracted by a fifth K16 step of the S product (Qx Kx^T); 0: by the softmax threads
// (the reference is then rounded up to an integer, which the polynomial exponentials absorb into their rounding
// constant for free; only the pairs that go to the special-function unit pay a packed add).
#ifndef GCT_BOUNDED_FOLD
#define GCT_BOUNDED_FOLD 1
#endif
constexpr bool kBoundedFold = GCT_BOUNDED_FOLD != 0;
constexpr bool kEarlyPFull = GCT_EARLY_P_FULL != 0;
// 1: the waits inside the KV loop of the softmax warps end with a warp vote.  The outcome of a wait is the same in
// every lane without it: the lanes of a converged warp poll one mbarrier phase, one clock and one abort word with the
// same instructions, so they all see the same values; the vote costs 1.3 % of the kernel and is kept for the waits
// outside the loop only.
#ifndef GCT_VOTE_WAITS
#define GCT_VOTE_WAITS 0
#endif
// Register budget at two query tiles per CTA: 384 threads start with 168 registers each (64512 in total);
// the control warpgroup shrinks to kControlRegs and the two softmax warpgroups grow to kSoftmaxRegs:
// 128 * kControlRegs + 256 * kSoftmaxRegs <= 64512, both multiples of 8.
#ifndef GCT_CONTROL_REGS
#define GCT_CONTROL_REGS 64
#endif
#ifndef GCT_SOFTMAX_REGS
#define GCT_SOFTMAX_REGS 208
#endif
constexpr int kControlRegs = GCT_CONTROL_REGS;
constexpr int kSoftmaxRegs = GCT_SOFTMAX_REGS;
static_assert(128 * kControlRegs + 256 * kSoftmaxRegs <= 64512, "register pool of the CTA exceeded");   // power of two, independent dependency chains of the row maximum
constexpr float kRescaleThreshold = 8.0f;   // in log2 units of the scaled logits

template <int QT>
struct SmemLayout {
  static constexpr uint32_t q_off = 0;
  static constexpr uint32_t k_off = q_off + QT * kTileBytes;
  static constexpr uint32_t v_off = k_off + kKStages * kTileBytes;
  // bounded mode (QT == 2): one more 128B-swizzled 128 x 64 tile whose K16 column groups hold the extra operands
  // of the S product: bf16 columns [0,16) Qx of tile 0, [16,32) Qx of tile 1, [32,48) Kx
  static constexpr uint32_t x_off = v_off + kVStages * kTileBytes;
  static constexpr uint32_t bar_off = x_off + (QT == 2 ? kTileBytes : 0);
  // barriers: q_full, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], per tile s_full, s_empty, p_full, pv_full,
  // then q_ready (bounded mode: Q scaled, Qx and Kx written)
  static constexpr int n_bars = 1 + 2 * kKStages + 2 * kVStages + 4 * QT + 1;
  static constexpr uint32_t misc_off = bar_off + n_bars * 8;
  static constexpr uint32_t total = misc_off + 16;
};

// Threads per CTA: the softmax warpgroups plus one control warpgroup slot (producer + QT MMA warps; at
// QT == 2 a fourth, idle warp completes the warpgroup so that registers can be moved between
// warpgroups with setmaxnreg).
template <int QT>
constexpr int kThreads = (QT == 2) ? 384 : 192;

template <int QT, bool kBounded>
__global__ void __launch_bounds__(kThreads<QT>, 1)
gct_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  using L = SmemLayout<QT>;
  static_assert(!kBounded || QT == 2, "the bounded mode exists for two query tiles per CTA");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + L::bar_off;
  auto bar_q_full = [&]() { return bars; };
  auto bar_k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_k_empty = [&](int s) { return bars + 8u * (1 + kKStages + s); };
  auto bar_v_full = [&](int s) { return bars + 8u * (1 + 2 * kKStages + s); };
  auto bar_v_empty = [&](int s) { return bars + 8u * (1 + 2 * kKStages + kVStages + s); };
  constexpr int kTileBars = 1 + 2 * kKStages + 2 * kVStages;
  auto bar_s_full = [&](int t) { return bars + 8u * (kTileBars + 4 * t + 0); };
  auto bar_s_empty = [&](int t) { return bars + 8u * (kTileBars + 4 * t + 1); };
  auto bar_p_full = [&](int t) { return bars + 8u * (kTileBars + 4 * t + 2); };
  auto bar_pv_full = [&](int t) { return bars + 8u * (kTileBars + 4 * t + 3); };
  auto bar_q_ready = [&]() { return bars + 8u * (kTileBars + 4 * QT); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::misc_off);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + L::misc_off + 4);
  volatile int* cta_unsafe = reinterpret_cast<volatile int*>(smem + L::misc_off + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kProducerWarp = 4 * QT;
  constexpr int kFirstMmaWarp = 4 * QT + 1;
  constexpr uint32_t kTmemCols = (QT == 2) ? 512u : 256u;
  constexpr uint32_t kOCol = 128u * QT;
  constexpr uint32_t kPCol = 192u * QT;

  // ---- work coordinates ----
  // The query groups of one (head, KV range) are neighbours in launch order: they stream the same K/V through L2 at
  // the same time.  Equal ranges: the ranges of a head follow each other.  Long ranges + one short one: range-major,
  // so that the short CTAs are handed out last, to the SMs that run out of long ones first.
  int idx = blockIdx.x;
  const int qg = idx % a.q_groups;
  idx /= a.q_groups;
  int split, h, b, g0, g1;
  if (a.split_len == 0) {
    split = idx % a.splits;
    idx /= a.splits;
    h = idx % a.heads;
    b = idx / a.heads;
    g0 = static_cast<int>(static_cast<long long>(split) * a.total_blocks / a.splits);
    g1 = static_cast<int>(static_cast<long long>(split + 1) * a.total_blocks / a.splits);
  } else {
    h = idx % a.heads;
    idx /= a.heads;
    b = idx % a.batch;
    split = idx / a.batch;
    g0 = split * a.split_len;
    g1 = (split == a.splits - 1) ? a.total_blocks : g0 + a.split_len;
  }
  const int nblk = g1 - g0;

  // ---- set-up ----
  if (threadIdx.x == 0) {
    mbar_init(bar_q_full(), 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(bar_k_full(s), 1);
      mbar_init(bar_k_empty(s), QT);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(bar_v_full(s), 1);
      mbar_init(bar_v_empty(s), QT);
    }
    for (int t = 0; t < QT; ++t) {
      mbar_init(bar_s_full(t), 1);
      mbar_init(bar_s_empty(t), 4);
      mbar_init(bar_p_full(t), 4);
      mbar_init(bar_pv_full(t), 1);
    }
    mbar_init(bar_q_ready(), 4 * QT);            // one arrival per softmax warp
    *cta_abort = 0;
    *cta_unsafe = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kFirstMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();      // everything above is private to the CTA; from here on global memory of earlier kernels is read

  // QT == 2: 384 threads share 64K registers (168 each at launch); the control warpgroup gives most of its
  // share to the two softmax warpgroups, whose threads hold a whole 128-column S row.
  if (warp == kProducerWarp) {
    // =========================== producer ===========================
    if constexpr (QT == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q_full(), QT * kTileBytes);
      for (int t = 0; t < QT; ++t)
        tma_load_4d(sbase + L::q_off + t * kTileBytes, &tm_q, bar_q_full(), 0, h, (qg * QT + t) * kTileM, b);
      int page = b, cur_pi = -1;
      for (int j = 0; j < nblk; ++j) {
        const int g = g0 + j;
        const int pi = g / a.blocks_per_page;
        const int jb = g - pi * a.blocks_per_page;
        if (a.page_table != nullptr && pi != cur_pi) {
          page = __ldg(a.page_table + pi);
          cur_pi = pi;
        }
        const int ks = j % kKStages, vs = j % kVStages;
        if (!mbar_wait(bar_k_empty(ks), ((j / kKStages) & 1) ^ 1u, cta_abort, a.status)) break;
        mbar_arrive_expect_tx(bar_k_full(ks), kTileBytes);
        tma_load_4d(sbase + L::k_off + ks * kTileBytes, &tm_k, bar_k_full(ks), 0, h, jb * kBlockN, page);
        if (!mbar_wait(bar_v_empty(vs), ((j / kVStages) & 1) ^ 1u, cta_abort, a.status)) break;
        mbar_arrive_expect_tx(bar_v_full(vs), kTileBytes);
        tma_load_4d(sbase + L::v_off + vs * kTileBytes, &tm_v, bar_v_full(vs), 0, h, jb * kBlockN, page);
      }
    }
  } else if (warp >= kFirstMmaWarp) {
    // =========================== MMA issuer of tile t ===========================
    if constexpr (QT == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
    const int t = warp - kFirstMmaWarp;
    if (t < QT) {
      // all 32 lanes run the loop and the waits; `lead` marks the lane that issues
      const uint32_t lead = elect_one();
      auto issue_s = [&](int ks) {
        const uint64_t ad = smem_desc(sbase + L::q_off + t * kTileBytes, 16, 1024);
        const uint64_t bd = smem_desc(sbase + L::k_off + ks * kTileBytes, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // 64 = 4 x K16; +32 B per step inside the 128 B swizzle row
          umma_ss(lead, tmem_base + t * 128, ad + 2 * k, bd + 2 * k, kIdescS, k > 0);
        if constexpr (kBounded && kBoundedFold) {     // S += Qx_t Kx^T: subtracts the row reference (column groups t and 2 of the x tile)
          const uint64_t xd = smem_desc(sbase + L::x_off, 16, 1024);
          umma_ss(lead, tmem_base + t * 128, xd + 2 * t, xd + 4, kIdescS, 1u);
        }
      };
      auto issue_pv = [&](int vs, uint32_t accumulate) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // 128 tokens = 8 x K16: 8 TMEM columns of P and 16 V rows per step
          const uint64_t bd = smem_desc(sbase + L::v_off + vs * kTileBytes + k * 2048, 16, 1024);
          umma_ts(lead, tmem_base + kOCol + t * 64, tmem_base + kPCol + t * 64 + k * 8, bd, kIdescPV,
                  (k > 0) ? 1u : accumulate);
        }
      };
      auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, cta_abort, a.status));
      };
      bool ok = wait(kBounded ? bar_q_ready() : bar_q_full(), 0) && wait(bar_k_full(0), 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        tc_commit_elected(lead, bar_s_full(t));
        tc_commit_elected(lead, bar_k_empty(0));
      }
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) {
          const int ks = (j + 1) % kKStages;
          if (!(ok = wait(bar_s_empty(t), j & 1))) break;
          if (!(ok = wait(bar_k_full(ks), ((j + 1) / kKStages) & 1))) break;
          tc_fence_after();
          issue_s(ks);
          tc_commit_elected(lead, bar_s_full(t));
          tc_commit_elected(lead, bar_k_empty(ks));
        }
        const int vs = j % kVStages;
        if (!(ok = wait(bar_p_full(t), j & 1))) break;
        if (!(ok = wait(bar_v_full(vs), (j / kVStages) & 1))) break;
        tc_fence_after();
        issue_pv(vs, j > 0 ? 1u : 0u);
        tc_commit_elected(lead, bar_pv_full(t));
        tc_commit_elected(lead, bar_v_empty(vs));
      }
    }
  } else {
    // =========================== softmax ===========================
    if constexpr (QT == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int t = warp >> 2;                       // query tile of this warp
    const int row = ((warp & 3) << 5) | lane;      // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + t * 128;
    const uint32_t o_addr = tmem_base + lane_addr + kOCol + t * 64;
    const uint32_t p_addr = tmem_base + lane_addr + kPCol + t * 64;
    const float c = kBounded ? 1.f : a.scale_log2;  // bounded mode: the Q tile already carries scale * log2(e)
    float m = -INFINITY, l = 0.f;                   // m: reference maximum (raw logit units)
    float ref_fixed = 0.f;                          // bounded mode: upper bound of this row's exponents
    bool ok = true;
    bool running_max = false;                       // bounded kernel: this CTA fell back to the running maximum
    // waits whose outcome the whole warp shares (the tcgen05 loads and stores that follow are warp-wide): with a
    // vote outside the KV loop, by construction inside it (see GCT_VOTE_WAITS)
    auto wait_v = [&](uint32_t bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, cta_abort, a.status));
    };
    auto wait_u = [&](uint32_t bar, uint32_t parity) -> bool {
#if GCT_VOTE_WAITS
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, cta_abort, a.status));
#else
      return mbar_wait(bar, parity, cta_abort, a.status);
#endif
    };

    if constexpr (kBounded) {
      // ---- once per CTA: scale the Q row in place, derive its reference, write Qx and Kx ----
      ok = wait_v(bar_q_full(), 0);
      const uint32_t q_row = sbase + L::q_off + t * kTileBytes + row * 128;
      const uint32_t swz = static_cast<uint32_t>(row & 7);
      float sq = 0.f;
      if (ok) {
        const float cs = a.scale_log2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {              // 16-byte chunk j of the row sits at chunk j ^ (row & 7)
          const uint32_t addr = q_row + ((static_cast<uint32_t>(j) ^ swz) << 4);
          uint32_t w[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(w[i] << 16) * cs, hi = __uint_as_float(w[i] & 0xffff0000u) * cs;
            w[i] = pack_bf16x2(lo, hi);
            const float rlo = __uint_as_float(w[i] << 16), rhi = __uint_as_float(w[i] & 0xffff0000u);
            sq = fmaf(rlo, rlo, fmaf(rhi, rhi, sq));
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        }
        // rounded up to bf16 (the precision of the Qx operand) so that the value used is still an upper bound
        const float ref = sqrtf(sq) * __ldg(a.key_norm_max + h);
        if (!(ref <= a.bounded_limit)) *cta_unsafe = 1;            // too loose, infinite or NaN
        ref_fixed = kBoundedFold ? __uint_as_float((__float_as_uint(ref) + 0xffffu) & 0xffff0000u) : ceilf(ref);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(128 * QT) : "memory");   // all softmax threads, also after a failed wait
      running_max = *cta_unsafe != 0;
      if (running_max) ref_fixed = 0.f;
      if (ok && !kBoundedFold) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the scaled Q rows -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q_ready());
      }
      if (ok && kBoundedFold) {
        const uint32_t x_row = sbase + L::x_off + row * 128;
        const uint32_t negref = running_max ? 0u : ((__float_as_uint(ref_fixed) >> 16) | 0x8000u);
        auto st_chunk = [&](int j, uint32_t first) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %2, %2};" ::"r"(x_row + ((static_cast<uint32_t>(j) ^ swz) << 4)),
                       "r"(first), "r"(0u) : "memory");
        };
        st_chunk(2 * t, negref);                   // Qx_t: column 0 = -ref, columns 1..15 = 0
        st_chunk(2 * t + 1, 0u);
        if (t == 0) {                              // Kx: column 0 = 1
          st_chunk(4, 0x3f80u);
          st_chunk(5, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q_ready());
      }
    }
    uint32_t s[128];

    int pi = g0 / a.blocks_per_page;               // page and block-in-page of block j, advanced incrementally
    int jb = g0 - pi * a.blocks_per_page;
    if (kBounded && running_max) {
      // ---- fallback of the bounded kernel: two passes over the S row in TMEM, 32 columns at a time ----
      // pass 1 takes the masked row maximum, pass 2 exponentiates against the running maximum (moved only when the
      // row maximum outgrows it by 2^kRescaleThreshold) and stores P; compact rather than fast.
      for (int j = 0; ok && j < nblk; ++j) {
        if (!(ok = wait_v(bar_s_full(t), j & 1))) break;
        tc_fence_after();
        const int plen = (pi == a.n_pages - 1) ? a.last_page_len : a.page_len;
        const int valid = min(kBlockN, plen - jb * kBlockN);
        if (++jb == a.blocks_per_page) {
          jb = 0;
          ++pi;
        }
        uint32_t r[32];
        float mx = -INFINITY;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(s_addr + 32 * ch, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (32 * ch + i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
        float alpha = 1.f;
        if (mx - m > kRescaleThreshold) {            // always true on the first block (m = -inf)
          alpha = fast_exp2(m - mx);
          m = mx;
        }
        if (j > 0) {
          if (!(ok = wait_v(bar_pv_full(t), (j - 1) & 1))) break;
          tc_fence_after();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
              tmem_ld32(o_addr + hh * 32, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(o_addr + hh * 32, r);
            }
          }
        }
        float sum = 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(s_addr + 32 * ch, r);
          tmem_wait_ld();
          uint32_t pk16[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = 32 * ch + 2 * i;
            const float e0 = col < valid ? fast_exp2(__uint_as_float(r[2 * i]) - m) : 0.f;
            const float e1 = col + 1 < valid ? fast_exp2(__uint_as_float(r[2 * i + 1]) - m) : 0.f;
            sum += e0 + e1;
            pk16[i] = pack_bf16x2(e0, e1);
          }
          tmem_st16(p_addr + 16 * ch, pk16);
        }
        l = fmaf(l, alpha, sum);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar_s_empty(t));               // S was read twice: only now may the next block overwrite it
          mbar_arrive(bar_p_full(t));
        }
      }
    } else
    for (int j = 0; ok && j < nblk; ++j) {
      if (!(ok = wait_u(bar_s_full(t), j & 1))) break;
      tc_fence_after();
      // valid tokens of this block
      const int plen = (pi == a.n_pages - 1) ? a.last_page_len : a.page_len;
      const int valid = min(kBlockN, plen - jb * kBlockN);
      if (++jb == a.blocks_per_page) {
        jb = 0;
        ++pi;
      }
      // keys past the valid length: -inf (exp2 gives 0); bounded mode: an exponent the polynomial can take
      // (without the fold the reference is still to be subtracted from it)
      const uint32_t kMaskBits = !kBounded ? 0xff800000u : (kBoundedFold ? 0xc2fc0000u /* -126.f */ : __float_as_uint(ref_fixed - 126.f));
      // masked maximum of s[lo, lo+64): four independent chains of 3-input max
      auto half_max = [&](int lo) -> float {
        if (valid < lo + 64) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (lo + i >= valid) s[lo + i] = kMaskBits;
        }
        if constexpr (kBounded) {
          return 0.f;                             // the reference is fixed: only the masking above is needed
        } else {
        // kMaxChains independent chains of 3-input max, merged by a tree at the end
        float mxc[kMaxChains];
#pragma unroll
        for (int ch = 0; ch < kMaxChains; ++ch) mxc[ch] = __uint_as_float(s[lo + ch]);
        constexpr int kRounds = (64 - kMaxChains) / (2 * kMaxChains);   // full rounds of one max3 per chain
#pragma unroll
        for (int r = 0; r < kRounds; ++r)
#pragma unroll
          for (int ch = 0; ch < kMaxChains; ++ch) {
            const int i = kMaxChains + 2 * (r * kMaxChains + ch);
            mxc[ch] = max3(mxc[ch], __uint_as_float(s[lo + i]), __uint_as_float(s[lo + i + 1]));
          }
        {
          constexpr int kDone = kMaxChains + 2 * kRounds * kMaxChains;   // elements consumed so far
#pragma unroll
          for (int i = kDone; i < 64; i += 2) {
            const int ch = ((i - kDone) / 2) % kMaxChains;
            mxc[ch] = max3(mxc[ch], __uint_as_float(s[lo + i]), __uint_as_float(s[lo + i + 1]));
          }
        }
#pragma unroll
        for (int w = kMaxChains / 2; w >= 1; w /= 2)
#pragma unroll
          for (int ch = 0; ch < w; ++ch) mxc[ch] = fmaxf(mxc[ch], mxc[ch + w]);
        return mxc[0];
        }
      };
      // the second half of the row is still arriving from TMEM while the first half is reduced
      float mx;
      {
        uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
        uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
        uint32_t(&s2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[64]);
        uint32_t(&s3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[96]);
        tmem_ld32(s_addr, s0);
        tmem_ld32(s_addr + 32, s1);
        if (j > 0 && !(kBounded && kEarlyPFull)) {
          // P of the previous block: its stores completed while the loads above were issued
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p_full(t));
        }
        if constexpr (kBounded && kBoundedHalfAt == 0) {
          // the whole row at once (a row takes under a hundred clocks to arrive): S is released right away
          tmem_ld32(s_addr + 64, s2);
          tmem_ld32(s_addr + 96, s3);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_s_empty(t));
          if (valid < 128) {
#pragma unroll
            for (int i = 64; i < 128; ++i)
              if (i >= valid) s[i] = kMaskBits;
          }
        } else {
          tmem_wait_ld();
          tmem_ld32(s_addr + 64, s2);
          tmem_ld32(s_addr + 96, s3);
        }
        const float mlo = half_max(0);
        if constexpr (!kBounded) {
          tmem_wait_ld();
          // the S tile is in registers: the tensor core may overwrite it with the next block
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_s_empty(t));
          mx = fmaxf(mlo, half_max(64));
        } else {
          mx = mlo;                                // unused: the second half is masked after its load, inside the sweep
        }
      }
      // move the reference maximum only when the row maximum outgrew it by more than 2^kRescaleThreshold;
      // until then exponentials stay below 2^8 and every sum remains exact enough in fp32
      float alpha = 1.f;
      if constexpr (!kBounded) {
        if ((mx - m) * c > kRescaleThreshold) {      // always true on the first block (m = -inf)
          alpha = fast_exp2((m - mx) * c);           // exp2(-inf) = 0 on the first block
          m = mx;
        }
      }
      const float mc = m * c;                        // bounded mode: unused, the tensor core already subtracted ref

      // P (and O) of this tile are free once the PV product of the previous block has completed.  The wait
      // sits in the middle of the exponential sweep, right before the first store of P, so that the
      // round trip softmax -> MMA warp -> tensor core -> mbarrier hides under the first half of the sweep.
      auto wait_prev_pv_and_rescale = [&]() -> bool {
        if (j > 0) {
          if (!wait_u(bar_pv_full(t), (j - 1) & 1)) return false;
          tc_fence_after();
          if (!kBounded && __any_sync(0xffffffffu, alpha != 1.f)) {   // rare: rescale this warp's 32 rows of O in TMEM
            uint32_t ob[32];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              tmem_ld32(o_addr + hh * 32, ob);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ob[i] = __float_as_uint(__uint_as_float(ob[i]) * alpha);
              tmem_st32(o_addr + hh * 32, ob);
            }
          }
        }
        return true;
      };
      // P = exp2(S*c - m*c), software-pipelined over pairs of logits so that the exponentials (the scarce
      // pipe) are interleaved with independent work: pair p+4 gets its packed FFMA, pair p its two EX2,
      // pair p-2 its packed add into the row sum and its bf16 conversion (two K values per TMEM column).
      // Bounded mode: S already is the exponent, the packed FFMA is gone.
      const float2 c2 = make_float2(c, c), nmc2 = make_float2(-mc, -mc);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
      uint32_t pk[kPvWaitAt > 31 ? 64 : 32];
      auto pair_ffma = [&](int q) {
        if constexpr (!kBounded) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[2 * q]), __uint_as_float(s[2 * q + 1])), c2, nmc2);
          s[2 * q] = __float_as_uint(x.x);
          s[2 * q + 1] = __float_as_uint(x.y);
        }
      };
      auto pair_exp = [&](int q) {
        // some pairs are exponentiated on the FMA pipe: the special-function unit delivers only 16 results per
        // clock and SM, half of what the tensor core consumes at head_dim 64
        const bool poly = kBounded ? ((q + 1) * kBoundedPolyNum) / kBoundedPolyDen != (q * kBoundedPolyNum) / kBoundedPolyDen
                                   : (kPolyEvery > 0 && (q % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery - 1));
        if (poly) {
          const float2 x = make_float2(__uint_as_float(s[2 * q]), __uint_as_float(s[2 * q + 1]));
          float2 e;
          if constexpr (kBounded) e = exp2_poly2_inrange<kBoundedPolyDeg>(x, kBoundedFold ? 0.f : ref_fixed);   // exponents lie in [-126, 1]
          else e = exp2_poly2(x);
          s[2 * q] = __float_as_uint(e.x);
          s[2 * q + 1] = __float_as_uint(e.y);
        } else if constexpr (kBounded && !kBoundedFold) {
          const float2 y = __fadd2_rn(make_float2(__uint_as_float(s[2 * q]), __uint_as_float(s[2 * q + 1])),
                                      make_float2(-ref_fixed, -ref_fixed));
          s[2 * q] = __float_as_uint(fast_exp2(y.x));
          s[2 * q + 1] = __float_as_uint(fast_exp2(y.y));
        } else {
          s[2 * q] = __float_as_uint(fast_exp2(__uint_as_float(s[2 * q])));
          s[2 * q + 1] = __float_as_uint(fast_exp2(__uint_as_float(s[2 * q + 1])));
        }
      };
      auto pair_sum = [&](int q) {
        const float2 e = make_float2(__uint_as_float(s[2 * q]), __uint_as_float(s[2 * q + 1]));
        if (q & 1) acc1 = __fadd2_rn(acc1, e); else acc0 = __fadd2_rn(acc0, e);
        pk[kPvWaitAt > 31 ? q : (q & 31)] = pack_bf16x2(e.x, e.y);
      };
#pragma unroll
      for (int q = 0; q < kFfmaAhead; ++q) pair_ffma(q);
#pragma unroll
      for (int q = 0; q < 64; ++q) {
        if constexpr (kBounded) {
          // bounded mode needs no row maximum: the second half of the S row arrives under the first half of the sweep
          if (kBoundedHalfAt > 0 && q == kBoundedHalfAt) {
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_empty(t));
            if (valid < 128) {
#pragma unroll
              for (int i = 64; i < 128; ++i)
                if (i >= valid) s[i] = kMaskBits;
            }
          }
        }
        if (q + kFfmaAhead < 64) pair_ffma(q + kFfmaAhead);
        pair_exp(q);
        if (q >= kSumLag) {
          pair_sum(q - kSumLag);
          if (q - kSumLag == kPvWaitAt) {               // at least the first 64 keys are done
            ok = wait_prev_pv_and_rescale();
            if (ok) tmem_st32(p_addr, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
          }
        }
      }
#pragma unroll
      for (int q = 64 - kSumLag; q < 64; ++q) pair_sum(q);
      if (!ok) break;
      tmem_st32(p_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[kPvWaitAt > 31 ? 32 : 0]));
      const float rs0 = acc0.x, rs1 = acc0.y, rs2 = acc1.x, rs3 = acc1.y;
      l = fmaf(l, alpha, (rs0 + rs1) + (rs2 + rs3));
      if (j + 1 == nblk || (kBounded && kEarlyPFull)) {   // otherwise the next iteration announces P after its first loads
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full(t));
      }
    }

    // ---- epilogue: O / l ----
    if (ok && nblk > 0) ok = wait_v(bar_pv_full(t), (nblk - 1) & 1);
    const int qrow = (qg * QT + t) * kTileM + row;
    if (ok && nblk > 0) {
      tc_fence_after();
      const float inv = 1.f / l;
      const size_t rowidx = (static_cast<size_t>(b) * a.n_q + (qrow < a.n_q ? qrow : 0)) * a.heads + h;
      const size_t prow = static_cast<size_t>(split) * a.batch * a.n_q * a.heads + rowidx;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t ob[32];
        tmem_ld32(o_addr + hh * 32, ob);      // warp-wide: every lane takes part, also rows past n_q
        tmem_wait_ld();
        if (qrow < a.n_q) {
          if (a.final_bf16) {
            uint4* dst = reinterpret_cast<uint4*>(a.out + rowidx * kHeadDim + hh * 32);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(ob[q4 * 8 + 0]) * inv, __uint_as_float(ob[q4 * 8 + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(ob[q4 * 8 + 2]) * inv, __uint_as_float(ob[q4 * 8 + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(ob[q4 * 8 + 4]) * inv, __uint_as_float(ob[q4 * 8 + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(ob[q4 * 8 + 6]) * inv, __uint_as_float(ob[q4 * 8 + 7]) * inv);
              dst[q4] = w;
            }
          } else {
            float4* dst = reinterpret_cast<float4*>(a.part_o + prow * kHeadDim + hh * 32);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              dst[q4] = make_float4(__uint_as_float(ob[q4 * 4 + 0]) * inv, __uint_as_float(ob[q4 * 4 + 1]) * inv,
                                    __uint_as_float(ob[q4 * 4 + 2]) * inv, __uint_as_float(ob[q4 * 4 + 3]) * inv);
          }
        }
      }
      if (qrow < a.n_q && !a.final_bf16)
        a.part_lse[prow] = (((kBounded && !running_max) ? ref_fixed : m * c) + log2f(l)) * 0.6931471805599453f;
    }
  }

  // ---- teardown: every thread arrives here, also after an abort ----
  if (*cta_abort) {
    // give copies and MMAs that may still be in flight time to land before TMEM and smem are released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kFirstMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

int attention_smem_bytes(int qt) {
  return static_cast<int>((qt == 2 ? SmemLayout<2>::total : SmemLayout<1>::total) + 1024);
}

// The kernels need more dynamic shared memory than the default limit; the opt-in is a per-device attribute of each
// kernel, so it is recorded per device ordinal.
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_attr_mutex;
bool g_attr_set[kMaxDevices] = {false};

int opt_in_shared_memory() {
  int dev = -1;
  GCT_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(GCT_ERR_INVALID, "attention: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  if (!g_attr_set[dev]) {
    const int s2 = attention_smem_bytes(2), s1 = attention_smem_bytes(1);
    GCT_CUDA_CHECK(cudaFuncSetAttribute(gct_attn_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, s2));
    GCT_CUDA_CHECK(cudaFuncSetAttribute(gct_attn_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, s2));
    GCT_CUDA_CHECK(cudaFuncSetAttribute(gct_attn_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, s1));
    g_attr_set[dev] = true;
  }
  return GCT_OK;
}
}  // namespace

int launch_attention(const AttnLaunch& a, cudaStream_t stream) {
  if (a.n_q <= 0 || a.heads <= 0 || a.batch <= 0 || a.n_pages <= 0 || a.page_len <= 0 || a.last_page_len <= 0 ||
      a.last_page_len > a.page_len)
    return fail(GCT_ERR_INVALID, "attention: bad shape");
  if (a.q_tiles_per_cta != 1 && a.q_tiles_per_cta != 2) return fail(GCT_ERR_INVALID, "attention: q_tiles_per_cta");
  if (a.status == nullptr) return fail(GCT_ERR_INVALID, "attention: status word missing");
  KernelArgs k;
  k.page_table = a.page_table;
  k.n_pages = a.n_pages;
  k.page_len = a.page_len;
  k.last_page_len = a.last_page_len;
  k.blocks_per_page = (a.page_len + kBlockN - 1) / kBlockN;
  k.total_blocks = (a.n_pages - 1) * k.blocks_per_page + (a.last_page_len + kBlockN - 1) / kBlockN;
  k.n_q = a.n_q;
  k.heads = a.heads;
  k.batch = a.batch;
  const int rows_per_cta = kTileM * a.q_tiles_per_cta;
  k.q_groups = (a.n_q + rows_per_cta - 1) / rows_per_cta;
  k.splits = a.splits;
  k.split_len = a.split_len;
  k.final_bf16 = a.final_bf16 ? 1 : 0;
  k.scale_log2 = 0.125f * 1.4426950408889634f;   // 1/sqrt(64) * log2(e)
  k.out = a.out;
  k.part_o = a.part_o;
  k.part_lse = a.part_lse;
  k.status = a.status;
  k.key_norm_max = a.key_norm_max;
  k.bounded_limit = a.bounded_limit;
  const bool bounded = a.key_norm_max != nullptr;
  if (bounded && (a.q_tiles_per_cta != 2 || !(a.bounded_limit > 0.f)))
    return fail(GCT_ERR_INVALID, "attention: bounded mode needs two query tiles per CTA and a positive limit");
  if (a.splits < 1 || a.splits > k.total_blocks) return fail(GCT_ERR_INVALID, "attention: splits out of range");
  if (a.split_len != 0) {     // splits - 1 full ranges and a non-empty, not longer rest
    const long long rest = static_cast<long long>(k.total_blocks) - static_cast<long long>(a.splits - 1) * a.split_len;
    if (a.split_len < 0 || a.splits < 2 || rest < 1 || rest > a.split_len)
      return fail(GCT_ERR_INVALID, "attention: split_len does not cover the KV blocks");
  }
  if (a.final_bf16 && (a.splits != 1 || a.out == nullptr)) return fail(GCT_ERR_INVALID, "attention: final output needs splits == 1");
  if (!a.final_bf16 && (a.part_o == nullptr || a.part_lse == nullptr))
    return fail(GCT_ERR_INVALID, "attention: partial buffers missing");
  const long long grid = static_cast<long long>(k.q_groups) * a.splits * a.heads * a.batch;
  if (grid <= 0 || grid > 0x7fffffffLL) return fail(GCT_ERR_INVALID, "attention: grid too large");
  const int smem = attention_smem_bytes(a.q_tiles_per_cta);
  int rc = opt_in_shared_memory();
  if (rc != GCT_OK) return rc;
  const dim3 g(static_cast<unsigned>(grid));
  if (a.q_tiles_per_cta == 2) {
    if (bounded)
      GCT_CUDA_CHECK(launch_pdl(gct_attn_kernel<2, true>, g, dim3(kThreads<2>), smem, stream, a.tm_q, a.tm_k, a.tm_v, k));
    else
      GCT_CUDA_CHECK(launch_pdl(gct_attn_kernel<2, false>, g, dim3(kThreads<2>), smem, stream, a.tm_q, a.tm_k, a.tm_v, k));
  } else {
    GCT_CUDA_CHECK(launch_pdl(gct_attn_kernel<1, false>, g, dim3(kThreads<1>), smem, stream, a.tm_q, a.tm_k, a.tm_v, k));
  }
  GCT_CUDA_CHECK(cudaGetLastError());
  return GCT_OK;
}

namespace {

// Finish time, in KV blocks of one two-tile CTA, of `n_long` CTAs of `len_long` blocks followed by `n_short` CTAs of
// `len_short` blocks handed out in that order to `sms` SMs, each to the SM that is free first; every CTA pays
// `fixed` blocks of prologue and epilogue.
double list_schedule(int n_long, double len_long, int n_short, double len_short, int sms, double fixed) {
  // the long CTAs are equal: after them n_long % sms SMs have run one more than the others
  const int full = n_long / sms, extra = n_long % sms;
  std::vector<double> heap(static_cast<size_t>(sms));           // min-heap of the SMs' finish times
  for (int i = 0; i < sms; ++i) heap[i] = (full + (i < extra ? 1 : 0)) * (len_long + fixed);
  auto cmp = [](double x, double y) { return x > y; };
  std::make_heap(heap.begin(), heap.end(), cmp);
  for (int i = 0; i < n_short; ++i) {
    std::pop_heap(heap.begin(), heap.end(), cmp);
    heap.back() += len_short + fixed;
    std::push_heap(heap.begin(), heap.end(), cmp);
  }
  return *std::max_element(heap.begin(), heap.end());
}

struct SplitPlanKey {
  int n_q_tiles, heads_x_batch, total_blocks, num_sms, max_splits;
  bool operator==(const SplitPlanKey& o) const {
    return n_q_tiles == o.n_q_tiles && heads_x_batch == o.heads_x_batch && total_blocks == o.total_blocks &&
           num_sms == o.num_sms && max_splits == o.max_splits;
  }
};
struct SplitPlan {
  int qt, splits, split_len;
};

}  // namespace

void choose_attention_config(int n_q_tiles, int heads_x_batch, int total_blocks, int num_sms, int max_splits,
                             int* q_tiles_per_cta, int* splits, int* split_len) {
  // Cost model in units of "one KV block for one CTA": a CTA with two query tiles takes about as long
  // per block as one with a single tile takes for 0.6 blocks-worth of its pair; every CTA pays a fixed
  // prologue/epilogue of about two blocks, and a split result needs the merge kernel afterwards (a launch
  // of its own, about five blocks).  Pick the cheapest (tiles per CTA, splits).
#ifndef GCT_MERGE_COST
#define GCT_MERGE_COST 5.0
#endif
  constexpr double kMergeCost = GCT_MERGE_COST;
  constexpr double kFixed = 2.0;
  // the plan of the previous call with the same arguments (a frame asks 24 times for the same one)
  static thread_local SplitPlanKey last_key = {-1, -1, -1, -1, -1};
  static thread_local SplitPlan last_plan = {1, 1, 0};
  const SplitPlanKey key = {n_q_tiles, heads_x_batch, total_blocks, num_sms, max_splits};
  if (split_len != nullptr && key == last_key) {
    *q_tiles_per_cta = last_plan.qt;
    *splits = last_plan.splits;
    *split_len = last_plan.split_len;
    return;
  }
  double best = 1e300;
  int best_qt = 1, best_s = 1, best_len = 0;
  for (int qt = 2; qt >= 1; --qt) {
    const long long items = static_cast<long long>((n_q_tiles + qt - 1) / qt) * heads_x_batch;
    const double per_block = (qt == 2) ? 1.0 : 0.6;
    const int smax = total_blocks < max_splits ? total_blocks : max_splits;
    for (int s = 1; s <= smax; ++s) {
      const long long ctas = items * s;
      const long long waves = (ctas + num_sms - 1) / num_sms;
      const int blocks = (total_blocks + s - 1) / s;
      const double cost = static_cast<double>(waves) * (blocks * per_block + kFixed) + (s > 1 ? kMergeCost : 0.0);
      if (cost < best - 1e-9) {
        best = cost;
        best_qt = qt;
        best_s = s;
        best_len = 0;
      }
    }
    // s - 1 long ranges and a short one, the short CTAs last: try a few lengths of the short range per s
    if (split_len == nullptr || items * 2 > 4096) continue;
    for (int s = 2; s <= smax; ++s) {
      const int even = (total_blocks + s - 1) / s;
      for (int step = 1; step <= 12; ++step) {
        const int rest = even * step / 13;                       // short range: 1/13 ... 12/13 of an even share
        if (rest < 1) continue;
        const int len = (total_blocks - rest + s - 2) / (s - 1);   // long ranges, rounded up
        const int real_rest = total_blocks - (s - 1) * len;
        if (len < 1 || real_rest < 1 || real_rest > len) continue;
        const double cost = list_schedule(static_cast<int>(items * (s - 1)), len * per_block, static_cast<int>(items),
                                          real_rest * per_block, num_sms, kFixed) + kMergeCost;
        // only for a clear gain over the best plan so far: a long back-to-back run at the board's power limit gains
        // nothing from filling idle SMs (measured 0.6 % slower at 1057 blocks, where the model promises 2.5 %)
        if (cost < best * 0.96) {
          best = cost;
          best_qt = qt;
          best_s = s;
          best_len = len;
        }
      }
    }
  }
  *q_tiles_per_cta = best_qt;
  *splits = best_s;
  if (split_len != nullptr) {
    *split_len = best_len;
    last_key = key;
    last_plan = {best_qt, best_s, best_len};
  }
}

}  // namespace gct
