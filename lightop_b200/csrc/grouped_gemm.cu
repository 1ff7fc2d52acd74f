// Grouped block-INT8 GEMM for sm_100a: TMA-fed tcgen05 kind::i8 MMAs with int32
// partial sums in tensor memory, promoted to fp32 register sums once per 128-wide K block.
//
// Orientation ("swap-AB").  The 128 rows of a weight tile are the M side of the
// MMA and the tokens of one expert are its N side (N = tokens rounded up to 16,
// at most 160 in the block-scaled modes, 256 per channel).  A chunk of 1..160
// tokens therefore costs one pass over the weight tile with no padding to 128
// rows, which is what a weight-streaming (HBM-bound) MoE needs, and the same
// kernel serves prefill and decode sizes.  In tensor memory a lane is an output
// column n and a column is a token.
//
// Work item = (chunk of expert-sorted rows, 128-row output tile; for gate_up the gate tile and
// the up tile of the same 128 output columns, run as two passes over K).  Items are ordered
// chunk-major so that CTAs running side by side share the chunk's activation rows, and the
// chunks of one expert (adjacent in the table) read the same weight tiles at about the same
// time: weight tiles are loaded with an evict-first L2 policy unless the chunk table says that
// another chunk of the expert follows.  Persistent CTAs take items round-robin.
//
// Warp roles in a CTA of 20 or 24 warps:
//   warp 0      : two TMA producers on two lanes with their own control flow: lane 0 streams
//                 the weight tiles (HBM) into ring w[], lane 16 the chunk's token rows (L2) into
//                 ring a[].  Token rows are read from an expert-sorted copy of the activations,
//                 so a chunk is a run of consecutive rows and one tiled TMA load fetches it.
//   warps 1, 3  : MMA issuers, alternating K-block steps (warp 1 alone in the per-channel
//                 mode).  Three lanes of an issuer each follow one barrier ring (weights,
//                 activations, free partial buffer), poll in the same instruction and agree by
//                 a vote; lane 0 then issues the four MMAs of the step and one commit to done[].
//                 Warp 1 owns the tensor-memory allocation.
//   warp 2      : scale producer: the token scales of the K block (fetched two steps ahead)
//                 times the weight-block scale -> per-step table in shared memory
//   warps 4..   : promotion / epilogue, four warps (one per lane quarter of tensor memory) per
//                 column group; the chunk's tokens are dealt to the groups in pieces of 16.  A
//                 thread keeps the fp32 running sums of its output column for its pieces in
//                 registers: per K block it loads 16 int32 partials, converts and does one
//                 fused multiply-add per value with the scale product.
// Pipelines: the two shared-memory rings (full_w / full_a, refilled when done[] says the MMAs
// that read a slot have completed) and NBUF tensor-memory partial buffers (done[] as "full",
// tmem_empty as "free") between the issuers and the promotion warps.
//
// Epilogues run out of the register sums through a staging tile in shared memory, so that the
// global stores are whole rows: gate_up keeps bf16(gate) there during the up pass, then forms
// SiLU(gate)*up, the 128-wide group maximum and the int8 row; down stages bf16 rows and applies
// the routed weight on the way out.
//
// Per-channel mode (one scale per token and one per output channel instead of 128x128 blocks) uses
// the same pipeline without the promotion: a tensor-memory buffer is the int32 accumulator of a whole
// item, summed over every K block by the tensor core, and the promotion warps only run an epilogue
// (int32 -> fp32, times token scale, times channel scale) while the MMAs of the next items fill the
// other buffers.  The scale-producer warp idles in that mode.
//
// Every wait is bounded: after about a second a waiter records a timeout in the
// status word, raises a CTA-wide abort flag, and all roles fall through to the
// common exit where tensor memory is released.
#include "common.h"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <map>
#include <tuple>

namespace lo {
namespace {

// Build parameters (the defaults are the measured best; the others exist so that a variant can be built and compared).
// Column groups of the instantiations for chunks above 64 rows: five keep a group at two pieces of 16 tokens.
#ifndef LO_NCG_WIDE
#define LO_NCG_WIDE 5
#endif
// Interval between two polls of a barrier, in nanoseconds, by role.  A polling warp competes for issue slots with the
// promotion warps that share its scheduler; longer intervals for the waiters with slack measured no different.
#ifndef LO_SLEEP_PRODUCER
#define LO_SLEEP_PRODUCER 128u
#endif
#ifndef LO_SLEEP_SCALE
#define LO_SLEEP_SCALE 128u
#endif
#ifndef LO_SLEEP_MMA
#define LO_SLEEP_MMA 20u
#endif
#ifndef LO_SLEEP_PROMO
#define LO_SLEEP_PROMO 32u
#endif
#ifndef LO_SLEEP_PROMO_SLACK
#define LO_SLEEP_PROMO_SLACK 32u
#endif

constexpr int TILE_N = 128;      // weight rows per accumulator (MMA M)
constexpr int TILE_K = 128;      // int8 elements (= bytes) per K block
constexpr int T_MAX = 128;       // default bound of the rows of a chunk
constexpr int T_WIDE = 160;      // widest block-scaled chunk: three partial buffers of 160 columns fill tensor memory
constexpr int FIRST_EPI_WARP = 4;
constexpr int MAX_NCG = 5;
constexpr int W_TILE_BYTES = TILE_N * TILE_K;   // 16 KiB
constexpr int OUT_ROW_BYTES = TILE_N * 2;       // one token's 128 outputs as bf16 in the staging tile
constexpr uint32_t TMEM_COLS = 512;
constexpr int ND = 16;                          // completion ring, see Smem::done
constexpr int SMEM_LIMIT = 227 * 1024;          // dynamic shared memory a CTA can be given on this part

// A_ROWS is the largest chunk (token count) the instantiation accepts: with few tokens per call no
// expert can receive more than that many rows, the activation tiles shrink and more weight tiles fit
// into shared memory (more weight bytes in flight per SM).
template <int MODE, int A_ROWS> struct Cfg {
  // gate_up: an item is two passes over K on the same chunk, first the gate tile, then the up tile
  static constexpr int PHASES = MODE == GEMM_GATE_UP ? 2 : 1;
  // Column groups: the chunk's tokens are dealt, in pieces of 16, to this many sets of four promotion warps (one
  // warp per lane quarter of tensor memory).  Five groups keep a group at two pieces for chunks of up to 160
  // tokens (the group with the most pieces paces the K loop); the CTA then has 24 warps and 80 registers per
  // thread.  Narrow chunks use four groups: more warps would only add idle ones that have to keep step.
  static constexpr int NCG = A_ROWS > 64 ? LO_NCG_WIDE : 4;
  static constexpr int EPI_WARPS = 4 * NCG;
  static constexpr int NUM_THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int A_TILE_BYTES = A_ROWS * TILE_K;
  // Two rings.  Activation tiles come from L2 (the chunk's rows are read by every output tile of the expert): a
  // slot is refilled only after the MMAs that read it have completed, so the ring has to cover the load latency
  // plus the MMA queue, four K blocks at least.  Weight tiles come from HBM and get the shared memory that is left.
  static constexpr int NA_FIT = (64 * 1024) / A_TILE_BYTES;
  static constexpr int NA = NA_FIT < 4 ? 4 : (NA_FIT > 10 ? 10 : NA_FIT);
  // staging tile of the epilogue: [A_ROWS][128] bf16 (gate_up keeps the gate values there during the up pass)
  static constexpr int STAGING_BYTES = MODE == GEMM_CHANNEL ? 0 : A_ROWS * OUT_ROW_BYTES;
  static constexpr int FIXED_BYTES = 14 * 1024;   // scale tables, maxima, barriers, alignment slack (checked below)
  static constexpr int NW_FIT = (SMEM_LIMIT - FIXED_BYTES - STAGING_BYTES - NA * A_TILE_BYTES) / W_TILE_BYTES;
  static constexpr int NW = NW_FIT > 12 ? 12 : NW_FIT;
  // tensor memory is cut into partial buffers of A_ROWS columns, one int32 accumulator each (at most 8 are used):
  // the partial of one 128-wide K block in the block-scaled modes (the fp32 running sums live in the registers of
  // the promotion warps), the accumulator of a whole item in the per-channel mode
  static constexpr int NBUF = (int)TMEM_COLS / A_ROWS > 8 ? 8 : (int)TMEM_COLS / A_ROWS;
  // Ring of scale-product tables.  A slot written for K-block step i was last read at step
  // i - SC_SLOTS; the producer of step i has seen the MMAs of step i - NW complete, which were
  // issued after the promotion of step i - NW - NBUF finished, so NW + NBUF slots suffice.
  static constexpr int SC_SLOTS = MODE == GEMM_CHANNEL ? 1 : NW + NBUF;
};

template <int MODE, int A_ROWS> struct Smem {
  using C = Cfg<MODE, A_ROWS>;
  // operand tiles first: each is a multiple of 1024 bytes, base is 1024-aligned
  uint8_t w[C::NW][W_TILE_BYTES];
  uint8_t a[C::NA][C::A_TILE_BYTES];
  // epilogue staging, row = token (column of the chunk), 256 bytes per row
  uint8_t staging[C::STAGING_BYTES > 0 ? C::STAGING_BYTES : 16];
  float sc[C::SC_SLOTS][A_ROWS];           // token scale x weight-block scale, ring indexed by the K-block counter
  // gate_up epilogue: |act| maxima per (item parity, lane quarter, token); a stub in the other modes
  uint32_t amax[MODE == GEMM_GATE_UP ? 2 : 1][4][MODE == GEMM_GATE_UP ? A_ROWS : 1];
  uint64_t full_w[C::NW];
  uint64_t full_a[C::NA];
  // done[u % ND]: the MMAs of K-block step u have completed.  One tcgen05.commit per step serves everybody who
  // waits for that event: the producers (a weight slot is free NW steps later, an activation slot NA steps later),
  // the scale warp, and in the block-scaled modes the promotion warps (the partial of step u is in its buffer).
  // ND exceeds every ring depth, so a waiter cannot be overtaken by the barrier's next phase.
  uint64_t done[ND];
  uint64_t tmem_full[C::NBUF];             // per-channel mode: the accumulator of an item is complete
  uint64_t tmem_empty[C::NBUF];
  uint64_t esync[MAX_NCG];                 // rendezvous of the 128 epilogue threads of a column group
  uint64_t isync;                          // rendezvous of all promotion warps, once per item
  uint32_t tmem_base;
  volatile int abort_flag;
};

// ------------------------------ PTX wrappers --------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread until the phase completes (or the
// hint runs out) instead of returning at once: waiting warps then stop competing for issue slots
// with the warps that have work (without it, polling made up most of the executed instructions).
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(200000u)
      : "memory");
  return ok != 0;
}
// Upper bound of one wait, in SM clock cycles (about 1.5 s at 1.9 GHz).
constexpr long long WAIT_LIMIT_CYCLES = 3000000000ll;

// Bounded wait.  Returns false when the CTA is aborting (this waiter timed out or another one
// did); `code` identifies the waiter in the status word.  The clock is only consulted every
// 256 failed polls, so a wait that completes quickly costs nothing but the polls.  A waiter sleeps
// `sleep_ns` between two polls: a polling warp is always eligible, and the scheduler it shares with
// four others was observed to give it most of the issue slots (a promotion warp's dozen loop
// instructions between two K blocks took several hundred cycles).  Waiters far off the critical path
// (producers that run stages ahead, promotion warps without columns in a narrow chunk) sleep longer.
template <class S>
__device__ __forceinline__ bool mbar_wait(S &sm, uint64_t *bar, uint32_t parity, int32_t *status, int code, uint32_t sleep_ns = LO_SLEEP_PROMO) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  while (true) {
    // the polls between two looks at the clock carry no bookkeeping but their count
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      __nanosleep(sleep_ns);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (sm.abort_flag) return false;
    const long long now = clock64();
    if (t0 == 0) t0 = now;
    if (now - t0 > WAIT_LIMIT_CYCLES) {
      sm.abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}

// The same wait and arrive for a barrier given by its shared-memory address.
__device__ __forceinline__ bool mbar_try_wait_addr(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(200000u)
      : "memory");
  return ok != 0;
}
template <class S>
__device__ __forceinline__ bool mbar_wait_addr(S &sm, uint32_t bar, uint32_t parity, int32_t *status, int code, uint32_t sleep_ns = LO_SLEEP_PROMO) {
  if (mbar_try_wait_addr(bar, parity)) return true;
  long long t0 = 0;
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      __nanosleep(sleep_ns);
      if (mbar_try_wait_addr(bar, parity)) return true;
    }
    if (sm.abort_flag) return false;
    const long long now = clock64();
    if (t0 == 0) t0 = now;
    if (now - t0 > WAIT_LIMIT_CYCLES) {
      sm.abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}
// One non-blocking look at a barrier: has the phase of this parity completed?
__device__ __forceinline__ bool mbar_test_addr(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive_addr(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// 2-D tiled TMA load global -> shared (this CTA), completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int32_t x, int32_t y, uint64_t *bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte
// swizzle, 8-row groups 1024 bytes apart (tile base 1024-aligned).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                     // leading byte offset (unused with swizzle), 16-byte units
  d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                     // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                     // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: int8 x int8 -> int32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
  uint32_t d = 0;
  d |= 2u << 4;            // accumulator format: S32
  d |= 1u << 7;            // A format: signed 8-bit
  d |= 1u << 10;           // B format: signed 8-bit
  d |= (n >> 3) << 17;     // N / 8
  d |= (128u >> 4) << 24;  // M / 16
  return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive tensor-memory columns of this thread's lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One promotion step on N (8 or 16) tokens of this thread's output channel: acc = fma(float(raw), scale product, acc).
// The 128-long int8 dot is below 2^21 in magnitude, so the conversion is exact; one rounding per K block.
// `sc_addr` is the shared-memory address of the N scale products.
// Plain fp32 multiply-adds: the packed f32x2 form needs its operands in aligned register pairs, and assembling the
// pairs from the converted values cost more than the packed instruction saved (measured: -6 % on the gate_up launch).
template <int N>
__device__ __forceinline__ void promote(const uint32_t *raw, float *acc, uint32_t sc_addr) {
#pragma unroll
  for (int j4 = 0; j4 < N / 4; ++j4) {
    float s0, s1, s2, s3;               // scale products of four tokens
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(s0), "=f"(s1), "=f"(s2), "=f"(s3) : "r"(sc_addr + 16u * j4));
    acc[j4 * 4 + 0] = __fmaf_rn(__int2float_rn((int32_t)raw[j4 * 4 + 0]), s0, acc[j4 * 4 + 0]);
    acc[j4 * 4 + 1] = __fmaf_rn(__int2float_rn((int32_t)raw[j4 * 4 + 1]), s1, acc[j4 * 4 + 1]);
    acc[j4 * 4 + 2] = __fmaf_rn(__int2float_rn((int32_t)raw[j4 * 4 + 2]), s2, acc[j4 * 4 + 2]);
    acc[j4 * 4 + 3] = __fmaf_rn(__int2float_rn((int32_t)raw[j4 * 4 + 3]), s3, acc[j4 * 4 + 3]);
  }
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// Reciprocal refined by one Newton step, and the quotient a / b from it with the remainder folded back in
// (q = a*y, then q + (a - b*q)*y): the IEEE round-to-nearest quotient for operands whose quotient and reciprocal
// are normal numbers, which holds for every division of the epilogues (denominators in [1, 1e38] or a group
// scale of at least 1e-10 / 127).  Inline, so the sixteen divisions of a piece overlap; the library division is
// a subroutine call each, and two of them per output made the epilogue a fifth of the kernel's time.
__device__ __forceinline__ float rcp_refined(float b) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(b));
  return __fmaf_rn(__fmaf_rn(-b, y, 1.0f), y, y);
}
__device__ __forceinline__ float div_by(float a, float b, float y) {
  const float q = __fmul_rn(a, y);
  return __fmaf_rn(__fmaf_rn(-b, q, a), y, q);
}

struct KParams {
  const float *a_scale;     // [positions, KB]
  const float *b_scale;
  int64_t n_rows_per_expert;
  int64_t n_store;          // output columns that exist (< n_tiles*128 only for a dense E = 1 call)
  int KB;
  int n_tiles;
  const int32_t *sorted_ids;
  int64_t numel_valid;
  const Chunk *chunks;
  const int32_t *num_chunks;
  int8_t *act_q;
  float *act_s;
  __nv_bfloat16 *C;
  const float *topk_weights;
  int weight_mode;
  float act_eps;
  int32_t *status;
  int out_by_position;      // bf16 output row = sorted position instead of the sorted id
  const int64_t *row_dst;   // single mode: address of the output row of every sorted id (null: C + id * n_store)
};

// Four tensor maps of the sorted activation matrix, box heights 16 / 32 / 64 / 128 rows.  A chunk of
// more than 128 rows (per-channel mode only) is fetched as a 128-row box plus a second box for the rest.
struct AMaps {
  CUtensorMap m[4];
};

__device__ __forceinline__ int a_map_index(int T) { return T <= 16 ? 0 : (T <= 32 ? 1 : (T <= 64 ? 2 : 3)); }

template <int MODE, int A_ROWS>
__global__ void __launch_bounds__((Cfg<MODE, A_ROWS>::NUM_THREADS), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ AMaps a_maps, const KParams p) {
  using SM = Smem<MODE, A_ROWS>;
  using CF = Cfg<MODE, A_ROWS>;
  constexpr int SC_SLOTS = CF::SC_SLOTS;
  constexpr int NW = CF::NW;
  constexpr int NA = CF::NA;
  constexpr int NBUF = CF::NBUF;
  constexpr int PHASES = CF::PHASES;
  constexpr int NCG = CF::NCG;
  constexpr int EPI_WARPS = CF::EPI_WARPS;
  extern __shared__ uint8_t smem_raw[];
  SM &sm = *reinterpret_cast<SM *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  // broadcast from lane 0 so that the compiler knows the warp index (and everything derived from it:
  // roles, tensor-memory addresses, barrier addresses) is uniform across the warp
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;

  // ------------------------------ set-up -----------------------------------
  if (tid == 0) {
    for (int s = 0; s < NW; ++s) {
      // weight producer (arrive.expect_tx) + the scale warp (per-channel mode has no scale tables)
      mbar_init(&sm.full_w[s], MODE == GEMM_CHANNEL ? 1 : 2);
    }
    for (int s = 0; s < NA; ++s) mbar_init(&sm.full_a[s], 1);
    for (int s = 0; s < ND; ++s) mbar_init(&sm.done[s], 1);   // tcgen05.commit of the MMA thread
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&sm.tmem_full[b], 1);
      mbar_init(&sm.tmem_empty[b], EPI_WARPS);
    }
    for (int b = 0; b < NCG; ++b) mbar_init(&sm.esync[b], 128);
    mbar_init(&sm.isync, EPI_WARPS);
    sm.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 32) {
    // descriptors into the descriptor cache while the set-up runs
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a_maps.m[i])) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  // Everything above touches this CTA's shared and tensor memory only and may run while the kernel before this
  // one in the stream is still at work (dependent launch); its outputs (chunk table, activations, scales) are
  // read from here on.
  dependency_wait();
  dependency_release();

  const int num_chunks = *p.num_chunks;
  const int64_t num_items = (int64_t)num_chunks * p.n_tiles;
  const int KB = p.KB;

  if (warp < FIRST_EPI_WARP) {
    if (warp == 0) {
      // ============ weight producer: one 128 x 128 tile per K block (gate_up: gate pass, then up pass) ============
      if (lane == 0) {
        const uint64_t pol_stream = policy_evict_first();
        const uint64_t pol_keep = policy_evict_normal();
        uint32_t it = 0;
        int s = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
          const Chunk ch = p.chunks[item / p.n_tiles];
          const int nt = (int)(item % p.n_tiles);
          if (ch.expert < 0) continue;
          // weight tiles are streamed (evict-first) unless another chunk of the same expert is about to read
          // them again: those stay in L2 under the normal policy
          const uint64_t pol_w = ch.pad ? pol_keep : pol_stream;
          for (int ph = 0; ph < PHASES && ok; ++ph) {
            const int32_t row_g = (int32_t)(ch.expert * p.n_rows_per_expert + (int64_t)(ph * p.n_tiles + nt) * TILE_N);
            for (int kb = 0; kb < KB; ++kb, ++it) {
              // slot s was read by step it - NW
              if (it >= (uint32_t)NW && !mbar_wait(sm, &sm.done[(it - NW) % ND], ((it - NW) / ND) & 1u, p.status, 1, LO_SLEEP_PRODUCER)) { ok = false; break; }
              mbar_arrive_expect_tx(&sm.full_w[s], W_TILE_BYTES);
              tma_load_2d(sm.w[s], &w_map, kb * TILE_K, row_g, &sm.full_w[s], pol_w);
              s = s + 1 == NW ? 0 : s + 1;
            }
          }
        }
      } else if (lane == 16) {
      // ============ activation producer (a second lane of the same warp, on its own path): the chunk's token
      // rows of every K block.  Token rows are read from an expert-sorted copy of the activations, so a chunk is
      // a run of consecutive rows and one tiled load fetches it (a second one for the rows beyond 128).
        const uint64_t pol_a = policy_evict_last();
        uint32_t it = 0;
        int s = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
          const Chunk ch = p.chunks[item / p.n_tiles];
          if (ch.expert < 0) continue;
          const int T = (ch.rows + 15) & ~15;
          const int T0 = T > 128 ? 128 : T;                  // first box; the rest (if any) goes into a second one
          const int mi = a_map_index(T0);
          const int mi2 = T > 128 ? a_map_index(T - 128) : -1;
          const uint32_t a_bytes = (16u << mi) * TILE_K + (mi2 >= 0 ? (16u << mi2) * TILE_K : 0u);
          for (int ph = 0; ph < PHASES && ok; ++ph) {
            for (int kb = 0; kb < KB; ++kb, ++it) {
              if (it >= (uint32_t)NA && !mbar_wait(sm, &sm.done[(it - NA) % ND], ((it - NA) / ND) & 1u, p.status, 6, LO_SLEEP_PRODUCER)) { ok = false; break; }
              mbar_arrive_expect_tx(&sm.full_a[s], a_bytes);
              tma_load_2d(sm.a[s], &a_maps.m[mi], kb * TILE_K, ch.row0, &sm.full_a[s], pol_a);
              if constexpr (A_ROWS > 128) {
                if (mi2 >= 0)
                  tma_load_2d(sm.a[s] + 128 * TILE_K, &a_maps.m[mi2], kb * TILE_K, ch.row0 + 128, &sm.full_a[s], pol_a);
              }
              s = s + 1 == NA ? 0 : s + 1;
            }
          }
        }
      }
    } else if (warp == 1 || warp == 3) {
      // ============================ MMA issuers ===============================
      // A step of this role is a chain of dependent scalar instructions and barrier round trips (a barrier poll
      // takes more than a hundred cycles even when the phase has long completed), which costs more time than the
      // 16 KB of weights of a step take to arrive however little the tensor core has to do.  So: lane 0 issues,
      // lanes 0, 1 and 2 each own one of the step's three barriers (weights landed, activations landed, partial
      // buffer free) with its ring position and poll it in the same instruction; one commit per step; and in the
      // block-scaled modes two warps share the steps (even ones here, odd ones there: the partials of different
      // steps are independent, a commit tracks the MMAs of its own thread, and the ring positions of a warp simply
      // advance by two).  Per-channel mode accumulates an item's steps into one buffer, in order: warp 1 issues
      // them all and the buffer ring advances once per item.
      constexpr uint32_t NISS = MODE == GEMM_CHANNEL ? 1u : 2u;
      const uint32_t which = warp == 1 ? 0u : 1u;
      if (which < NISS) {
        const uint32_t my_n = lane == 0 ? (uint32_t)NW : (lane == 1 ? (uint32_t)NA : (uint32_t)NBUF);
        const uint32_t my_base = lane == 0 ? smem_u32(&sm.full_w[0]) : (lane == 1 ? smem_u32(&sm.full_a[0]) : smem_u32(&sm.tmem_empty[0]));
        // ring position and phase parity of this lane's barrier at this warp's next step (global step index `it`);
        // a fresh "buffer free" barrier is waited for with the opposite parity
        uint32_t my_slot = which % my_n;
        uint32_t my_par = ((which / my_n) & 1u) ^ (lane == 2 ? 1u : 0u);
        uint32_t it = which, it_base = 0;
        const uint64_t desc_w0 = make_smem_desc(smem_u32(sm.w[0])), desc_a0 = make_smem_desc(smem_u32(sm.a[0]));
        bool ok = true;
        for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
          const Chunk ch = p.chunks[item / p.n_tiles];
          if (ch.expert < 0) continue;
          const uint32_t idesc = make_idesc((uint32_t)((ch.rows + 15) & ~15));
          const uint32_t steps = (uint32_t)(PHASES * KB);
          for (uint32_t u = it - it_base; u < steps; u += NISS, it += NISS) {
            // per-channel mode: the accumulator buffer is waited for at the item's first step only
            const bool poll = lane < 2 || (lane == 2 && (MODE != GEMM_CHANNEL || u == 0));
            const bool mine = poll ? mbar_wait_addr(sm, my_base + 8u * my_slot, my_par, p.status, 3 + lane, LO_SLEEP_MMA) : true;
            if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
            const uint32_t sw = __shfl_sync(0xffffffffu, my_slot, 0);
            const uint32_t sa = __shfl_sync(0xffffffffu, my_slot, 1);
            const uint32_t b = __shfl_sync(0xffffffffu, my_slot, 2);
            if (lane == 0) {
              tc_fence_after();
              // descriptor start addresses are in 16-byte units
              const uint64_t adesc = desc_w0 + (uint64_t)(sw * (W_TILE_BYTES >> 4));
              const uint64_t bdesc = desc_a0 + (uint64_t)(sa * (uint32_t)(CF::A_TILE_BYTES >> 4));
              const uint32_t d = tmem_base + b * (uint32_t)A_ROWS;
#pragma unroll
              for (int k4 = 0; k4 < TILE_K / 32; ++k4)
                umma_i8(d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc,
                        (MODE == GEMM_CHANNEL ? (u | (uint32_t)k4) : (uint32_t)k4) != 0u ? 1u : 0u);
              umma_commit(&sm.done[it & (uint32_t)(ND - 1)]);
              if (MODE == GEMM_CHANNEL && u == steps - 1) umma_commit(&sm.tmem_full[b]);
            }
            __syncwarp();
            // per-channel mode: the buffer ring (lane 2) advances once per item
            if (MODE != GEMM_CHANNEL || lane != 2 || u == steps - 1) {
              my_slot += (MODE == GEMM_CHANNEL && lane == 2) ? 1u : NISS;
              if (my_slot >= my_n) { my_slot -= my_n; my_par ^= 1u; }
            }
          }
          it_base += steps;
        }
      }
    } else if (MODE != GEMM_CHANNEL) {
      // ========================= scale producer (warp 2) ====================
      // Thread g owns tokens g, g + 32, ... of the chunk.  The scales of a K block are fetched two steps before
      // they are used (they come from L2: the chunk's scale rows are read by every output tile of the expert), one
      // value per token and step, which keeps this role to a few registers per token.
      const int g = lane;
      constexpr int NU = (A_ROWS + 31) / 32;
      uint32_t it = 0;
      int s = 0, slot = 0;
      bool ok = true;
      const int64_t nblk = (p.n_rows_per_expert + TILE_N - 1) / TILE_N;
      for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const Chunk ch = p.chunks[item / p.n_tiles];
        const int nt = (int)(item % p.n_tiles);
        if (ch.expert < 0) continue;
        const int T = (ch.rows + 15) & ~15;
        const float *as_base = p.a_scale + (int64_t)ch.row0 * KB;
        uint32_t as_off[NU];          // offset of the token's scale row; a token beyond the chunk reads row 0
#pragma unroll
        for (int u = 0; u < NU; ++u) as_off[u] = (uint32_t)((g + u * 32 < ch.rows ? g + u * 32 : 0) * KB);
        for (int ph = 0; ph < PHASES && ok; ++ph) {
          const float *bs_ptr = p.b_scale + ((int64_t)ch.expert * nblk + nt + (int64_t)ph * p.n_tiles) * KB;
          float a0[NU], a1[NU], b0, b1;     // scales of this step and of the next one
#pragma unroll
          for (int u = 0; u < NU; ++u) {
            a0[u] = __ldg(as_base + as_off[u]);
            a1[u] = KB > 1 ? __ldg(as_base + as_off[u] + 1) : 0.f;
          }
          b0 = __ldg(bs_ptr);
          b1 = KB > 1 ? __ldg(bs_ptr + 1) : 0.f;
          for (int kb = 0; kb < KB; ++kb, ++it) {
            float as_now[NU];
            const float bs_now = b0;
            b0 = b1;
            if (kb + 2 < KB) b1 = __ldg(bs_ptr + kb + 2);
#pragma unroll
            for (int u = 0; u < NU; ++u) {
              as_now[u] = a0[u];
              a0[u] = a1[u];
              if (kb + 2 < KB) a1[u] = __ldg(as_base + as_off[u] + kb + 2);
            }
            // the slot of this step is free once the weight stage is (see SC_SLOTS)
            if (it >= (uint32_t)NW &&
                !__all_sync(0xffffffffu, mbar_wait(sm, &sm.done[(it - NW) % ND], ((it - NW) / ND) & 1u, p.status, 4, LO_SLEEP_SCALE))) { ok = false; break; }
#pragma unroll
            for (int u = 0; u < NU; ++u) {
              const int t = g + u * 32;
              if (t < T) sm.sc[slot][t] = t < ch.rows ? __fmul_rn(as_now[u], bs_now) : 0.f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.full_w[s]);
            s = s + 1 == NW ? 0 : s + 1;
            slot = slot + 1 == SC_SLOTS ? 0 : slot + 1;
          }
        }
      }
    }
  } else {
    // ====================== promotion + epilogue (16 warps) ====================
    const int pw = warp - FIRST_EPI_WARP;   // 0..15
    const int q = warp & 3;              // lane quarter of tensor memory this warp may access
    const int cg = pw >> 2;              // column group: which share of the chunk's tokens
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int n_local = q * 32 + lane;
    uint32_t ab = 0, eph = 0, iph = 0, item_par = 0;
    uint32_t sc_slot = 0, buf = 0, step = 0;     // block-scaled modes: ring positions of the K loop, K-block step count
    bool ready = false;                          // the coming step's barrier was already seen complete
    bool ok = true;
    for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const Chunk ch = p.chunks[item / p.n_tiles];
      const int nt = (int)(item % p.n_tiles);
      if (ch.expert < 0) {
        // block of a non-local expert: its output rows are zero
        if (MODE != GEMM_GATE_UP && p.C != nullptr) {
          for (int t = cg; t < ch.rows; t += NCG) {
            const int32_t sid = p.sorted_ids ? p.sorted_ids[ch.row0 + t] : ch.row0 + t;
            if (sid >= 0 && sid < p.numel_valid && (int64_t)nt * TILE_N + n_local < p.n_store)
              p.C[(int64_t)(p.out_by_position ? ch.row0 + t : sid) * p.n_store + (int64_t)nt * TILE_N + n_local] =
                  __float2bfloat16_rn(0.f);
          }
        }
        continue;
      }
      // The chunk's T columns (a multiple of 16) are dealt to the column groups in pieces of 16, as evenly as
      // that allows; a group owns at most two pieces (32 tokens) of a chunk of up to 160 tokens, four of a chunk
      // of up to 256.
      const int T = (ch.rows + 15) & ~15;
      const int n_pieces = T >> 4;
      const int my_p = n_pieces / NCG + (cg < n_pieces % NCG ? 1 : 0);
      const int col_begin = (cg * (n_pieces / NCG) + min(cg, n_pieces % NCG)) * 16;

      // Row id and routed weight of token col_begin + 32 * u + lane, fetched now so that the latency is
      // hidden behind the K loop; broadcast by shuffle in the epilogue: piece pc of the group is in
      // register set pc / 2, lanes 16 * (pc & 1) .. + 15.
      constexpr int NPF = ((A_ROWS / 16 + NCG - 1) / NCG + 1) / 2;   // sets of 32 tokens that cover a group's pieces
      int32_t sid_r[NPF];
      float wgt_r[NPF];
      // single mode: address of the row's first output column (0 = no row), so that the epilogue's row stores
      // serve a table of row addresses (rows in a peer's memory) and the plain matrix alike
      unsigned long long rowp_r[MODE == GEMM_SINGLE ? NPF : 1];
      rowp_r[0] = 0ull;
#pragma unroll
      for (int u = 0; u < NPF; ++u) {
        sid_r[u] = -1;
        wgt_r[u] = 0.f;
        if (MODE == GEMM_SINGLE) rowp_r[MODE == GEMM_SINGLE ? u : 0] = 0ull;
        if (MODE != GEMM_GATE_UP || p.weight_mode != LO_WEIGHT_NONE) {
          const int t = col_begin + u * 32 + lane;
          if (u * 32 + lane < my_p * 16 && t < ch.rows) {
            // without a sorted-id table the id of a row is its position
            int32_t sid = p.sorted_ids ? p.sorted_ids[ch.row0 + t] : ch.row0 + t;
            if (sid < 0 || sid >= p.numel_valid) sid = -1;
            if (sid >= 0 && p.weight_mode != LO_WEIGHT_NONE) wgt_r[u] = p.topk_weights[sid];
            if (MODE == GEMM_SINGLE && sid >= 0 && p.row_dst != nullptr)
              rowp_r[MODE == GEMM_SINGLE ? u : 0] = (unsigned long long)p.row_dst[sid];
            if (sid >= 0 && p.out_by_position) sid = ch.row0 + t;
            if (MODE == GEMM_SINGLE && sid >= 0 && p.row_dst == nullptr)
              rowp_r[MODE == GEMM_SINGLE ? u : 0] = (unsigned long long)(p.C + (int64_t)sid * p.n_store);
            sid_r[u] = sid;
          }
        }
      }

      if constexpr (MODE == GEMM_CHANNEL) {
        // ---------------- per-channel mode: one pass over the finished int32 accumulator ----------------
        // token scale of column col_begin + lane (broadcast by shuffle) and the scale of this thread's channel
        float as_r[NPF];
#pragma unroll
        for (int u = 0; u < NPF; ++u) {
          const int t = col_begin + u * 32 + lane;
          as_r[u] = (u * 32 + lane < my_p * 16 && t < ch.rows) ? __ldg(p.a_scale + ch.row0 + t) : 0.f;
        }
        const int64_t n_glob = (int64_t)nt * TILE_N + n_local;
        const bool n_ok = n_glob < p.n_store;
        const float bs = n_glob < p.n_rows_per_expert ? __ldg(p.b_scale + (int64_t)ch.expert * p.n_rows_per_expert + n_glob) : 0.f;
        const uint32_t b = ab % NBUF;
        const uint32_t aph = (ab / NBUF) & 1u;
        ++ab;
        if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.tmem_full[b], aph, p.status, 5))) { ok = false; break; }
        tc_fence_after();
        const uint32_t part = tmem_base + lane_off + b * (uint32_t)A_ROWS + (uint32_t)col_begin;
#pragma unroll 1
        for (int pc = 0; pc < my_p; ++pc) {
          uint32_t raw[16];
          tmem_ld16(part + pc * 16, raw);
          tmem_ld_wait();
          if (pc == my_p - 1) {
            // every value this warp needs is in registers: hand the buffer back before the stores
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.tmem_empty[b]);
          }
          // piece pc holds tokens 16 * pc .. 16 * pc + 15 of this group: register set pc / 2, lanes 16 * (pc & 1) ..
          const int u = NPF > 1 ? (pc >> 1) : 0;
          const int32_t sid_u = NPF > 1 && u ? sid_r[NPF - 1] : sid_r[0];
          const float wgt_u = NPF > 1 && u ? wgt_r[NPF - 1] : wgt_r[0];
          const float as_u = NPF > 1 && u ? as_r[NPF - 1] : as_r[0];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int src = (pc & 1) * 16 + j;
            const int32_t sid = __shfl_sync(0xffffffffu, sid_u, src);
            const float wgt = __shfl_sync(0xffffffffu, wgt_u, src);
            const float as = __shfl_sync(0xffffffffu, as_u, src);
            if (sid >= 0 && n_ok) {
              float v = __int2float_rn((int32_t)raw[j]);
              if (p.weight_mode == LO_WEIGHT_FP32) v = __fmul_rn(v, wgt);
              v = __fmul_rn(__fmul_rn(v, as), bs);
              if (p.weight_mode == LO_WEIGHT_BF16_PRODUCT) v = bf16_round(v) * bf16_round(wgt);
              p.C[(int64_t)sid * p.n_store + n_glob] = __float2bfloat16_rn(v);
            }
          }
        }
        if (my_p == 0) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.tmem_empty[b]);
        }
      } else {
        // ---------------- block-scaled modes: promotion once per K block, sums in registers ----------------
        // This warp owns the columns [col_begin, col_begin + 16 * my_p) of its 32 lanes.  Their fp32 running sums
        // stay in registers over the whole K loop (NP pieces of 16 columns at most; the piece loop is unrolled and
        // a piece beyond the chunk's width is skipped), so tensor memory holds nothing but partial buffers and a
        // K block costs one tensor-memory load per piece.
        constexpr int NP = (A_ROWS / 16 + NCG - 1) / NCG;
        float acc[NP][16];
        // Addresses of this item, formed once: the loops below only add constants to them.  Ring positions
        // (scale slot, partial buffer and its phase) are carried as counters instead of being divided out of
        // the step numbers.
        const uint32_t part0 = tmem_base + lane_off + (uint32_t)col_begin;
        const uint32_t sc0 = smem_u32(&sm.sc[0][0]) + (uint32_t)col_begin * 4u;
        const uint32_t done0 = smem_u32(&sm.done[0]), empty0 = smem_u32(&sm.tmem_empty[0]);
        // a warp with fewer pieces than the busiest group of the item has that much slack per step and polls at a
        // longer interval; a warp without columns only has to keep step
        const int max_p = (n_pieces + NCG - 1) / NCG;
        const uint32_t wait_ns = my_p == 0 ? 256u : (my_p < max_p ? LO_SLEEP_PROMO_SLACK : LO_SLEEP_PROMO);
        // this thread's column of the staging tile: row = token, 2 bytes per output channel.  Plain loads and
        // stores (no volatile asm), so that the compiler can overlap the sixteen tokens of a piece; the barrier
        // operations between the phases are compiler barriers as well.
        __nv_bfloat16 *const stg_mine = reinterpret_cast<__nv_bfloat16 *>(&sm.staging[0]) + col_begin * TILE_N + n_local;
#pragma unroll 1
        for (int ph = 0; ph < PHASES; ++ph) {
#pragma unroll
          for (int pc = 0; pc < NP; ++pc)
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[pc][j] = 0.f;
#pragma unroll 1
          for (int kb = 0; kb < KB; ++kb) {
            const uint32_t sc_step = sc0 + sc_slot * (uint32_t)(A_ROWS * 4);
            sc_slot = sc_slot + 1 == (uint32_t)SC_SLOTS ? 0u : sc_slot + 1;
            const uint32_t b = buf;
            buf = buf + 1 == (uint32_t)NBUF ? 0u : buf + 1;
            const uint32_t dn = step & (uint32_t)(ND - 1), dph = (step >> 4) & 1u;
            ++step;
            // The scale products of this step were written to shared memory before the weight stage's full
            // barrier completed, which the MMA thread observed before it issued the MMAs whose
            // completion this wait observes.  Warp-uniform outcome: the accesses below are warp-collective.
            if (!ready && !__all_sync(0xffffffffu, mbar_wait_addr(sm, done0 + 8u * dn, dph, p.status, 5, wait_ns))) { ok = false; break; }
            tc_fence_after();
            // an early look at the next step's barrier: the answer arrives while this step's columns are promoted
            // (a barrier round trip takes more than a hundred cycles even when the phase has long completed)
            const bool next_done = mbar_test_addr(done0 + 8u * (step & (uint32_t)(ND - 1)), (step >> 4) & 1u);
            const uint32_t part = part0 + b * (uint32_t)A_ROWS;
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
              if (pc < my_p) {
                uint32_t r16[16];
                tmem_ld16(part + pc * 16, r16);
                tmem_ld_wait();
                promote<16>(r16, &acc[pc][0], sc_step + (uint32_t)(pc * 64));
              }
            }
            ready = __all_sync(0xffffffffu, next_done);
            // every load of the partial has completed: hand the buffer back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_addr(empty0 + 8u * b);
          }
          if (!ok) break;
          if (MODE == GEMM_GATE_UP && ph == 0) {
            // End of the gate pass: bf16(gate) goes to this thread's column of the staging tile and is read back by
            // the same thread after the up pass.  The rows may still be in use by the row stores of the previous
            // item's epilogue, by any warp (the split of the rows over the column groups follows the chunk's
            // width): all promotion warps meet first.
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.isync);
            if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.isync, iph, p.status, 8))) { ok = false; break; }
            iph ^= 1u;
#pragma unroll
            for (int pc = 0; pc < NP; ++pc) {
              if (pc < my_p) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  float gte = acc[pc][j];
                  if (p.weight_mode == LO_WEIGHT_FP32)
                    gte *= __shfl_sync(0xffffffffu, NPF > 1 && (pc >> 1) ? wgt_r[NPF - 1] : wgt_r[0], (pc & 1) * 16 + j);
                  stg_mine[(pc * 16 + j) * TILE_N] = __float2bfloat16_rn(gte);
                }
              }
            }
          }
        }
        if (!ok) break;

        // ------------------------------ epilogue -------------------------------
        // One rolled loop over the warp's pieces: the body always works on piece 0 of the register sums and the
        // remaining pieces move down one place afterwards (registers cannot be indexed by a loop counter, and an
        // epilogue unrolled over the pieces would be fetched cold once per item).  Outputs go through the staging
        // tile so that global memory sees whole rows: a thread holds one output channel of 16 tokens, a row of the
        // output is 128 channels of one token.
        if constexpr (MODE == GEMM_GATE_UP) {
          const int64_t I = (int64_t)p.n_tiles * TILE_N;
          uint32_t(*amax_tab)[A_ROWS] = sm.amax[item_par];
#pragma unroll 1
          for (int pc = 0; pc < my_p; ++pc) {
            float *av = &acc[0][0];
            const __nv_bfloat16 *gs = stg_mine + pc * 16 * TILE_N;
            // Pass A: act = bf16(bf16(silu(bf16(gate))) * bf16(up)) in place of the up sums; maximum of |act|
            // over this warp's 32 output columns, lane j keeps the one of token j.
            float gte[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) gte[j] = __bfloat162float(gs[j * TILE_N]);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float up = av[j];
              if (p.weight_mode == LO_WEIGHT_FP32)
                up *= __shfl_sync(0xffffffffu, NPF > 1 && (pc >> 1) ? wgt_r[NPF - 1] : wgt_r[0], (pc & 1) * 16 + j);
              up = bf16_round(up);
              // 1 + exp(-gate) capped below the fp32 maximum: the quotient is then zero instead of an invalid
              // operation in the refinement (the exact quotient would be -0 or a number below 1e-36)
              const float den = fminf(1.0f + expf(-gte[j]), 1e38f);
              const float sl = bf16_round(div_by(gte[j], den, rcp_refined(den)));
              av[j] = bf16_round(sl * up);
            }
            uint32_t own = 0u;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(av[j]) & 0x7fffffffu);
              if (j == lane) own = m;
            }
            if (lane < 16) amax_tab[q][col_begin + pc * 16 + lane] = own;
            // the four warps of this column group exchange their maxima (the table alternates between two
            // copies from item to item; the pieces of one item use different entries); every gate value of the
            // piece has been read when they have met
            mbar_arrive(&sm.esync[cg]);
            if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.esync[cg], eph, p.status, 9))) { ok = false; break; }
            eph ^= 1u;
            // Pass B: lane j (< 16) forms the group scale of token j of the piece, amax / 127; every thread then
            // quantises its column of the 16 tokens, q = trunc(clamp(act / scale)), into byte n of the token's
            // staging row.
            float scale_r = 1.f, rcp_r = 1.f;
            const int t_own = col_begin + pc * 16 + (lane & 15);
            {
              const uint32_t m = max(max(amax_tab[0][t_own], amax_tab[1][t_own]), max(amax_tab[2][t_own], amax_tab[3][t_own]));
              scale_r = __fdiv_rn(fmaxf(__uint_as_float(m), p.act_eps), 127.0f);
              rcp_r = rcp_refined(scale_r);
              if (q == 0 && lane < 16 && t_own < ch.rows) p.act_s[((int64_t)ch.row0 + t_own) * p.n_tiles + nt] = scale_r;
            }
            int8_t *qs = reinterpret_cast<int8_t *>(&sm.staging[0]) + (col_begin + pc * 16) * OUT_ROW_BYTES + n_local;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float scale = __shfl_sync(0xffffffffu, scale_r, j);
              float r = div_by(av[j], scale, __shfl_sync(0xffffffffu, rcp_r, j));
              r = fminf(fmaxf(r, -128.0f), 127.0f);
              qs[j * OUT_ROW_BYTES] = (int8_t)__float2int_rz(r);
            }
            mbar_arrive(&sm.esync[cg]);
            if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.esync[cg], eph, p.status, 10))) { ok = false; break; }
            eph ^= 1u;
            // rows out: this warp takes tokens 4q .. 4q+3 of the piece, eight lanes x 16 bytes per row
            {
              const int t = col_begin + pc * 16 + 4 * q + (lane >> 3);
              if (t < ch.rows) {
                const uint4 v = *reinterpret_cast<const uint4 *>(&sm.staging[t * OUT_ROW_BYTES + (lane & 7) * 16]);
                *reinterpret_cast<uint4 *>(p.act_q + ((int64_t)ch.row0 + t) * I + (int64_t)nt * TILE_N + (lane & 7) * 16) = v;
              }
            }
#pragma unroll
            for (int pp = 0; pp + 1 < NP; ++pp)
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[pp][j] = acc[pp + 1][j];
          }
          if (!ok) break;
          item_par ^= 1u;
        } else {
          // the staging rows may still be read by the row stores of the previous item, by any warp (the split of
          // the rows over the column groups follows the chunk's width): all promotion warps meet first
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.isync);
          if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.isync, iph, p.status, 8))) { ok = false; break; }
          iph ^= 1u;
          const bool vec_ok = (p.n_store & 7) == 0;
#pragma unroll 1
          for (int pc = 0; pc < my_p; ++pc) {
            const float *av = &acc[0][0];
            __nv_bfloat16 *os = stg_mine + pc * 16 * TILE_N;
            const unsigned long long rowp_u = NPF > 1 && (pc >> 1) ? rowp_r[NPF - 1] : rowp_r[0];
            const float wgt_u = NPF > 1 && (pc >> 1) ? wgt_r[NPF - 1] : wgt_r[0];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = av[j];
              if (p.weight_mode == LO_WEIGHT_FP32) v *= __shfl_sync(0xffffffffu, wgt_u, (pc & 1) * 16 + j);
              os[j * TILE_N] = __float2bfloat16_rn(v);
            }
            mbar_arrive(&sm.esync[cg]);
            if (!__all_sync(0xffffffffu, mbar_wait(sm, &sm.esync[cg], eph, p.status, 9))) { ok = false; break; }
            eph ^= 1u;
            // rows out: this warp takes tokens 4q .. 4q+3 of the piece, two rows per step, sixteen lanes x 16 bytes per row
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int tp = 4 * q + 2 * i + (lane >> 4);                       // token of the piece
              const unsigned long long rowp = __shfl_sync(0xffffffffu, rowp_u, (pc & 1) * 16 + tp);
              // bf16-product order: bf16(sum) * bf16(w), rounded once more: one packed multiply per two outputs
              const __nv_bfloat162 w2 = __float2bfloat162_rn(__shfl_sync(0xffffffffu, wgt_u, (pc & 1) * 16 + tp));
              const int64_t n0 = (int64_t)nt * TILE_N + (lane & 15) * 8;
              if (rowp != 0ull && n0 < p.n_store) {
                const uint8_t *src = &sm.staging[(col_begin + pc * 16 + tp) * OUT_ROW_BYTES + (lane & 15) * 16];
                __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(rowp) + n0;
                uint4 v = *reinterpret_cast<const uint4 *>(src);
                if (p.weight_mode == LO_WEIGHT_BF16_PRODUCT) {
                  __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
                  for (int e = 0; e < 4; ++e) h[e] = __hmul2(h[e], w2);
                }
                if (vec_ok) {
                  *reinterpret_cast<uint4 *>(dst) = v;
                } else {
                  for (int e = 0; e < 8 && n0 + e < p.n_store; ++e) dst[e] = reinterpret_cast<const __nv_bfloat16 *>(&v)[e];
                }
              }
            }
#pragma unroll
            for (int pp = 0; pp + 1 < NP; ++pp)
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[pp][j] = acc[pp + 1][j];
          }
          if (!ok) break;
        }
      }
    }
  }

  // ------------------------------ teardown -----------------------------------
  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag) {
    // give copies that may still be in flight time to land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) {
    }
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------ host side ----------------------------------

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// Tensor map of a [rows, K] int8 matrix, box `box_rows` x 128 bytes, 128-byte swizzle.
// Encoded maps are cached by (base, rows, K, box_rows).
int make_tile_map(CUtensorMap *map, const int8_t *base, int64_t rows, int64_t K, int box_rows) {
  static std::mutex mu;
  static std::map<std::tuple<const void *, int64_t, int64_t, int>, CUtensorMap> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple((const void *)base, rows, K, box_rows);
  auto itc = cache.find(key);
  if (itc != cache.end()) {
    *map = itc->second;
    return LO_OK;
  }
  auto encode = get_encode_fn();
  if (!encode) return fail(LO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LO_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (cache.size() > 1024) cache.clear();
  cache[key] = *map;
  return LO_OK;
}

template <int MODE, int A_ROWS>
int launch_mode(const GemmArgs &a, cudaStream_t stream) {
  using SM = Smem<MODE, A_ROWS>;
  static_assert(sizeof(SM) + 1024 <= SMEM_LIMIT, "shared-memory layout exceeds what a CTA can be given");
  static_assert(ND == 16, "the promotion warps take the completion-ring phase from bit 4 of the step count");
  static_assert(Cfg<MODE, A_ROWS>::NW >= 4, "too few weight stages");
  static_assert(Cfg<MODE, A_ROWS>::NW < ND && Cfg<MODE, A_ROWS>::NA < ND && Cfg<MODE, A_ROWS>::NBUF < ND, "completion ring too short");
  const size_t smem_bytes = sizeof(SM) + 1024;
  // the attribute belongs to the (kernel, device) pair: set it once per device this thread launches on
  static thread_local uint64_t configured_devices = 0;
  int dev = 0;
  LO_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !((configured_devices >> dev) & 1u)) {
    LO_CUDA_OK(cudaFuncSetAttribute(grouped_gemm_kernel<MODE, A_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    if (dev >= 0 && dev < 64) configured_devices |= (uint64_t)1 << dev;
  }
  CUtensorMap wmap;
  int rc = make_tile_map(&wmap, a.B, (int64_t)a.E * a.n_rows_per_expert, a.K, TILE_N);
  if (rc != LO_OK) return rc;
  AMaps amaps;
  for (int i = 0; i < 4; ++i) {
    rc = make_tile_map(&amaps.m[i], a.A, a.rows_a, a.K, 16 << i);
    if (rc != LO_OK) return rc;
  }
  KParams p;
  p.a_scale = a.a_scale; p.b_scale = a.b_scale;
  p.n_rows_per_expert = a.n_rows_per_expert; p.n_store = a.n_store > 0 ? a.n_store : a.n_rows_per_expert; p.KB = (int)(a.K / TILE_K); p.n_tiles = a.n_tiles;
  p.sorted_ids = a.sorted_ids; p.numel_valid = a.numel_valid;
  p.chunks = a.chunks; p.num_chunks = a.num_chunks; p.act_q = a.act_q; p.act_s = a.act_s; p.C = a.C; p.row_dst = a.row_dst;
  p.topk_weights = a.topk_weights; p.weight_mode = a.weight_mode; p.act_eps = a.act_eps; p.status = a.status;
  p.out_by_position = a.out_by_position;
  const int grid = sm_count();
  if (grid <= 0) return fail(LO_ERR_CUDA, "no CUDA device");
  LO_CUDA_OK(launch_dependent(grouped_gemm_kernel<MODE, A_ROWS>, dim3(grid), dim3(Cfg<MODE, A_ROWS>::NUM_THREADS), smem_bytes, stream, wmap,
                              amaps, p));
  return LO_OK;
}

}  // namespace

int launch_grouped_gemm(GemmMode mode, const GemmArgs &a, cudaStream_t stream) {
  LO_REQUIRE(a.K % TILE_K == 0 && a.K >= TILE_K, "grouped gemm: K=%lld must be a positive multiple of 128", (long long)a.K);
  LO_REQUIRE(a.n_rows_per_expert % TILE_N == 0 || (a.E == 1 && mode != GEMM_GATE_UP),
             "grouped gemm: N=%lld must be a multiple of 128", (long long)a.n_rows_per_expert);
  LO_REQUIRE((int64_t)a.E * a.n_rows_per_expert < (1LL << 31), "grouped gemm: E*N exceeds the tensor-map row range");
  LO_REQUIRE(a.rows_a >= 1 && a.rows_a < (1LL << 31), "grouped gemm: activation row count out of range");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(a.B) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.A) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a.a_scale) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.b_scale) & 15) == 0,
             "grouped gemm: operands and scales must be 16-byte aligned");
  LO_REQUIRE(a.weight_mode == LO_WEIGHT_NONE || a.topk_weights != nullptr, "grouped gemm: weight mode %d needs topk_weights", a.weight_mode);
  LO_REQUIRE(a.row_dst == nullptr || (mode == GEMM_SINGLE && a.n_rows_per_expert % 8 == 0 && a.out_by_position == 0),
             "grouped gemm: a table of row addresses serves the single block-scaled mode with N a multiple of 8");
  LO_REQUIRE(mode == GEMM_GATE_UP || a.C != nullptr || a.row_dst != nullptr, "grouped gemm: no output");
  // no chunk can hold more rows than max_chunk_rows (a bound the caller derives from the token count)
  const int cap = a.max_chunk_rows <= 0 ? T_MAX : a.max_chunk_rows;
  if (mode == GEMM_GATE_UP) {
    LO_REQUIRE(a.n_rows_per_expert == 2 * (int64_t)a.n_tiles * TILE_N, "grouped gemm: gate_up needs N = 2*I");
    LO_REQUIRE(cap <= T_WIDE, "grouped gemm: block-scaled chunks hold at most 160 rows");
    if (cap <= 32) return launch_mode<GEMM_GATE_UP, 32>(a, stream);
    if (cap <= 64) return launch_mode<GEMM_GATE_UP, 64>(a, stream);
    if (cap <= 128) return launch_mode<GEMM_GATE_UP, 128>(a, stream);
    return launch_mode<GEMM_GATE_UP, T_WIDE>(a, stream);
  }
  LO_REQUIRE((int64_t)a.n_tiles * TILE_N >= a.n_rows_per_expert && (int64_t)(a.n_tiles - 1) * TILE_N < a.n_rows_per_expert,
             "grouped gemm: tile count mismatch");
  if (mode == GEMM_CHANNEL) {
    LO_REQUIRE(cap <= 256, "grouped gemm: per-channel chunks hold at most 256 rows");
    if (cap <= 32) return launch_mode<GEMM_CHANNEL, 32>(a, stream);
    if (cap <= 64) return launch_mode<GEMM_CHANNEL, 64>(a, stream);
    if (cap <= 128) return launch_mode<GEMM_CHANNEL, 128>(a, stream);
    return launch_mode<GEMM_CHANNEL, 256>(a, stream);
  }
  LO_REQUIRE(cap <= T_WIDE, "grouped gemm: block-scaled chunks hold at most 160 rows");
  if (cap <= 32) return launch_mode<GEMM_SINGLE, 32>(a, stream);
  if (cap <= 64) return launch_mode<GEMM_SINGLE, 64>(a, stream);
  if (cap <= 128) return launch_mode<GEMM_SINGLE, 128>(a, stream);
  return launch_mode<GEMM_SINGLE, T_WIDE>(a, stream);
}

}  // namespace lo
