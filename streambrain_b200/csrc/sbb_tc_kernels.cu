// tcgen05 / TMEM / TMA contraction kernels for sm_100a.
//
// One persistent, warp-specialised kernel template serves both contractions of
// the layer step:
//
//   trace update   D[i, j] = sum_b x[b, i] * y[b, j]   A = x  (MN-major), B = y (MN-major), K = batch
//   forward        D[b, j] = sum_k x[b, k] * w[k, j]   A = x  (K-major),  B = w (MN-major), K = in_features
//
// float32 accuracy on TF32 tensor cores: every operand value v is used as
// hi = v truncated to TF32 (what the tensor core reads of the raw float32) and
// lo = tf32(v - hi), and each k-step issues three MMAs  hi*hi + hi*lo + lo*hi
// into one float32 accumulator in tensor memory (the dropped lo*lo term is
// below 2^-20 relative).  A's hi and lo parts are staged in tensor memory, B's
// lo parts beside the raw tile in shared memory: the tensor core fetches only B
// from shared memory.
//
// Roles inside a CTA (512 threads, one CTA per SM, tiles walked persistently):
//   warps 0-3   A converters: wait for a TMA stage, write A's hi / lo parts to tensor
//               memory (one tile row per thread)
//               and (multi-chain trace update, raw products) B's lo parts to shared memory
//   warps 14-15 B converters (forward product, single-chain trace update): B's lo parts to shared memory
//   warps 4-11  epilogue: tcgen05.ld the accumulator (16x256b shape, so that four
//               lanes cover 32 contiguous bytes of a row) and either store it or run
//               the trace / weight arithmetic against 32 x 32 blocks of Cij that TMA
//               stages in shared memory two blocks ahead
//   warp 12     TMA producer (one lane): cp.async.bulk.tensor loads, no multicast
//   warp 13     MMA issuer (one lane) and owner of the TMEM allocation
// CTA pairs (PAIR; the forward product and the fused trace update): the kernel is launched in clusters of
// two CTAs that work on two vertically adjacent row tiles with one 256-row tcgen05.mma.cta_group::2 per k-step,
// issued by the leader CTA.  Each CTA stages and converts its own 128 rows of A into its own tensor memory and
// half of the tile's columns of B into its own shared memory; the converters and the epilogue warps of both
// CTAs report to the leader's mbarriers (mapa + remote arrive), tcgen05.commit with a cluster multicast reports
// back to both.  No TMA load uses multicast: every CTA loads into its own shared memory only.
// Hand-offs use mbarriers; every wait is bounded by a count of SM clock cycles:
// a wait that gives up records a code in a global status word, raises the CTA's
// abort flag, and every role falls through to the common tear-down (drain the
// tensor pipe, free TMEM) instead of spinning.
#include "sbb_tc.cuh"

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "sbb_math.cuh"

namespace sbb {
namespace {

constexpr int kConvWarps = 4;
constexpr int kEpiWarps = 8;
constexpr int kTmaWarp = kConvWarps + kEpiWarps;
constexpr int kMmaWarp = kTmaWarp + 1;
constexpr int kBConvWarps = 2;                 // warps kMmaWarp + 1 ..: the low parts of B
constexpr int kThreads = (kMmaWarp + 1 + kBConvWarps) * 32;  // 512: with 128 registers each, the whole register file
constexpr long long kWaitLimitCycles = 4000000000ll;  // default limit of one wait: about 2 s of SM clock

enum WaitCode { kWaitEmpty = 1, kWaitFull = 2, kWaitConv = 3, kWaitAccEmpty = 4, kWaitAccFull = 5, kWaitDrain = 6, kWaitSlab = 7 };

struct TcWork {
  int m_tiles, n_tiles, splits;
  int k_total;      // extent of the reduction dimension
  int k_per_split;  // multiple of the stage depth
  int m_fastest;    // tile order: row tiles fastest (1) or column tiles fastest (0)
  int a_row0;       // offset added to the A row coordinate (first output row of this launch)
  int a_box3;       // A stage fetched by one 3-D box (MN-major A whose row length is a multiple of 32)
  int b_box3_tiles; // column tiles [0, b_box3_tiles) fetch their B stage by one 3-D box
  int b_prefetch;   // B k-blocks requested into L2 ahead of the load into shared memory (0 = none)
  long long wait_limit;  // SM clock cycles after which a wait on an mbarrier gives up
  int lose_arrive;  // test hook: converter thread 0 of CTA 0 skips its arrival for the first stage
  int chain_kb;     // kernels without register-resident sums (CHAIN == 0): k-blocks per tensor-memory
                    // accumulation chain (0 = the whole k-range); later chains are added to the result of
                    // the earlier ones by the epilogue, through the output itself
};

struct TcEpilogue {
  // raw store: out[(split*rows + m)*ld + n]
  float *out;
  long rows, cols, ld;
  // fused trace step (rows = row_end - row_begin, global row = row0 + m)
  const float *rci;    // per global row: 1 / Ci, or 0 when Ci < cthr
  const float *rcj;    // per column: 1 / Cj, or 0 when Cj < cthr
  float *Cij;
  float *W;
  const uint8_t *wmask;
  const int *col_hc;
  uint32_t hc_magic;   // ceil(2^32 / Mc) when floor(n * magic / 2^32) == n / Mc for every column, else 0
  long H, Mc, row0;
  int fast_ok;         // select-word epilogue usable: Mc >= 32 (or no mask) and cthr^4 a normal float
  TraceParams<float> p;
  float ema_scale;  // taupdt / batch: weight of the batch sum in the moving average
  // raw store of an MN-major product: the tile leaves through shared memory and TMA stores of 32 x 32 blocks
  // (tmC = the output, row 0 = first row of this launch) instead of register stores: whole 128-byte rows per
  // request, which is what a destination in another GPU's memory needs to be written at link speed
  int tma_store;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr float kLn2 = 0.693147180559945309f;
// log2 by the special-function unit alone (subnormal arguments read as zero).
__device__ __forceinline__ float lg2_ftz(float v) {
  float r;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting or the time limit passed
// (in which case it raises the abort flag and records `code`).  The limit is
// counted on the SM's own cycle counter: %globaltimer is read through the memory
// system and costs microseconds per read on a busy GPU, which a wait taken
// thousands of times per launch cannot afford.
// The limit (cycles) sits in shared memory right behind the abort flag (written once at start-up).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                            int code, bool heed_abort = true) {
  const long long t0 = clock64();
  const long long limit = *reinterpret_cast<volatile long long *>(abort_flag + 1);
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 1023u) == 0) {
      if (heed_abort && *abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// One box over the 3-D view [chunk][row][32] of an MN-major matrix: a whole stage of an operand
// (every 32-element group along MN, all k-rows) in a single instruction.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// The same boxes requested into L2 only: takes DRAM latency out of the shared-memory pipeline.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// One box from shared memory to global memory (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most one store group of this thread may still be reading its shared-memory source
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// ---- CTA pairs (cluster of two CTAs driving one 256-row tcgen05.mma.cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster (own rank: local).
__device__ __forceinline__ void mbar_arrive_rank(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(bar), "r"(rank)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[256 x N] (+)= A[256 x 8] * B[8 x N] over the pair: each CTA holds its 128 rows of A and D in its own tensor
// memory and N / 2 columns of B in its own shared memory, all at the same addresses; issued by the leader alone.
__device__ __forceinline__ void mma_tf32_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Completion of the pair's MMAs issued so far, signalled on the mbarrier at this offset in both CTAs.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// D[128 x N] (+)= A[128 x 8] * B[8 x N]: A read from tensor memory (128 lanes x 8 columns of 32-bit
// values at a_tmem), B through a shared-memory descriptor, TF32 inputs, float32 accumulation.
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with A through a shared-memory descriptor as well.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Each lane writes NCOL (16 or 32) consecutive 32-bit columns of its own tensor-memory lane.
template <int NCOL>
__device__ __forceinline__ void tmem_st_32x32b(uint32_t taddr, const uint32_t (&r)[NCOL]) {
  static_assert(NCOL == 16 || NCOL == 32, "column count");
  if constexpr (NCOL == 32) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
  }
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 TMEM lanes x 32 columns: thread t gets, for rep = 0..3, registers
//   r[4*rep+0..1] = lane t/4,     columns 8*rep + 2*(t%4) + {0,1}
//   r[4*rep+2..3] = lane t/4 + 8, same columns.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, float (&r)[16]) {
  uint32_t u[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int k = 0; k < 16; ++k) r[k] = __uint_as_float(u[k]);
}

// Shared-memory matrix descriptor (sm_100 version field set).
//   K-major operand:  rows of 128 bytes along k, 128-byte swizzle with 16-byte base (layout type 2);
//                     SBO = 1024 (eight rows), LBO unused.
//   MN-major 32-bit operand: the only layout the tensor core accepts is the 128-byte swizzle with
//                     32-byte base (layout type 1): atoms of 4 k-rows x 128 bytes (32 elements along
//                     MN); SBO = distance between consecutive 4-row atoms along k, LBO = distance
//                     between 32-element groups along MN.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version
  d |= (uint64_t)layout_type << 61;
  return d;
}
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t saddr, uint32_t lbo_bytes) {
  return smem_desc(saddr, lbo_bytes, 512u, 1u);       // MN-major, SWIZZLE_128B_BASE32B
}

// Optional timeline (compile with -DSBB_TC_TRACE): CTA 0 stamps clock64() at the hand-offs of its first
// 64 tiles -- event numbers: 0 / 8 first / last TMA issue, 5 / 9 first / last conversion, 7 accumulator
// free, 1 first MMA, 2 accumulator committed, 3 epilogue start, 10 epilogue data ready, 13-15 column
// groups done, 4 epilogue end -- and sbb_tc_trace_read copies the 64 x 16 stamps out.  Compiled out otherwise.
#ifdef SBB_TC_TRACE
__device__ unsigned long long g_tc_trace[64 * 16];
#define TC_TRACE(tile, ev) do { if (blockIdx.x == 0 && (tile) < 64) g_tc_trace[(tile) * 16 + (ev)] = (unsigned long long)clock64(); } while (0)
#else
#define TC_TRACE(tile, ev)
#endif

// ------------------------------------------------------------------ the kernel
constexpr int kSlabBytes = 32 * 32 * 4;  // one epilogue warp's 32-row x 32-column block of the trace matrix

// The A operand's hi / lo parts live in tensor memory (written by the converters), so only B
// has a "lo" copy in shared memory and the tensor core fetches only B from there.
// PRESPLIT: the low parts of both operands come from memory (written by the column-sum kernels that run just
// before), so a stage is four TMA landing zones [A | B | B lo | A lo], nothing is converted inside the kernel
// and the tensor core takes both operands from shared memory.
// PAIR: two CTAs share one 256-row MMA; each stages its own 128 rows of A and BN / 2 columns of B.
template <int BN, int BK, int STAGES, bool SLABS, bool PRESPLIT = false, bool PAIR = false>
struct TcSmem {
  static constexpr int A_BYTES = 128 * BK * 4;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 4;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;  // TMA landing zone: the raw values serve as "hi"
  static constexpr int STAGE_BYTES = PRESPLIT ? 2 * RAW_BYTES : RAW_BYTES + B_BYTES;   // + B's lo parts (+ A's)
  static constexpr int TX_BYTES = PRESPLIT ? 2 * RAW_BYTES : RAW_BYTES;                // bytes TMA lands per stage
  // tensor memory: two accumulators, then (not PRESPLIT) per stage BK columns of A hi and BK of A lo
  static constexpr int TMEM_A_COL = 2 * BN;
  static constexpr int TMEM_COLS = 512;
  static_assert(2 * BN + (PRESPLIT ? 0 : STAGES * 2 * BK) <= TMEM_COLS, "tensor memory budget");
  static_assert(STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte swizzle alignment");
  static constexpr int SLAB_OFFSET = STAGES * STAGE_BYTES;
  // two 32 x 32 block buffers per epilogue warp: landing zones for blocks of the trace matrix (fused
  // epilogue) or staging for the TMA stores of the raw product
  static constexpr int SLAB_TOTAL = SLABS ? kEpiWarps * 2 * kSlabBytes : 0;
  static constexpr int BAR_OFFSET = SLAB_OFFSET + SLAB_TOTAL;
  // full, conv, empty per stage; acc_full[2], acc_empty[2], drain; slab[warp][2]
  static constexpr int NUM_BARS = 3 * STAGES + 5 + 2 * kEpiWarps;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // + tmem ptr, abort flag, alignment slack
  static_assert(TOTAL <= 232448, "shared memory budget");
};

// Two 16-lane halves of a warp's TMEM lane quarter, 32 columns each, one wait.
__device__ __forceinline__ void tmem_ld_pair(uint32_t taddr_lo, uint32_t taddr_hi, float (&a)[16], float (&b)[16]) {
  uint32_t u[16], v[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr_lo)
      : "memory");
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr_hi)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    a[k] = __uint_as_float(u[k]);
    b[k] = __uint_as_float(v[k]);
  }
}

// CHAIN = number of k-blocks accumulated in tensor memory before the running sum
// is taken over by float32 registers (0 = the whole k-range in tensor memory).
// The tensor core adds each MMA into its accumulator with less than IEEE
// rounding, so the error of a chain grows with its length; long reductions
// (the forward pass sums over in_features) are cut into short chains whose
// results the epilogue warps add in full float32.
// MULTI (kernels without register-resident sums, CHAIN == 0): the k-range of a tile is cut into chains of
// wk.chain_kb k-blocks and the epilogue carries the running sum through its output in memory; without it a
// tile is one chain and the epilogue is the plain one.
template <bool A_KMAJOR, int BN, int BK, int STAGES, bool FUSED, int CHAIN, bool MULTI = false, bool PRESPLIT = false,
          bool PAIR = false>
// 14 warps are allocated registers as 16: 128 registers per thread is the most that fits one CTA per SM.
__global__ void __launch_bounds__(kThreads, 1)
    tc_contraction_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmA3, const __grid_constant__ CUtensorMap tmB3,
                          const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAlo,
                          const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmA3lo,
                          const __grid_constant__ CUtensorMap tmB3lo, TcWork wk, TcEpilogue ep, int *status) {
  using SM = TcSmem<BN, BK, STAGES, FUSED || !A_KMAJOR, PRESPLIT, PAIR>;
  static_assert(!(PRESPLIT && A_KMAJOR), "pre-split operands are the two MN-major ones of the batch contractions");
  static_assert(!PAIR || (!PRESPLIT && BN % 64 == 0), "CTA pairs convert their operands themselves");
  // In a pair, CTA `rank` of the cluster works on row tile 2 * (pair's tile) + rank; the leader (rank 0) issues the MMAs.
  // B's low parts by the two extra warps (see their role below): forward product and single-chain trace update
  constexpr bool BWARPS = !PRESPLIT && !MULTI && (A_KMAJOR || FUSED);
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  constexpr int BNH = PAIR ? BN / 2 : BN;   // columns of B this CTA stages
  static_assert(!A_KMAJOR || BK == 32, "a K-major operand is loaded as one 128-byte-wide box");
  static_assert(BN % 64 == 0 && BN <= 256 && BK % 8 == 0 && BK <= 32, "tile shape");
  static_assert(!(FUSED && CHAIN > 0), "the fused epilogue consumes a whole-range accumulator");
  static_assert(CHAIN == 0 || BN <= 128, "register-resident running sums are sized for 128 columns");
  static_assert(!(MULTI && CHAIN > 0), "chains are carried either in registers or through memory");
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t dyn_base = smem_u32(smem_dyn);
  const uint32_t base = (dyn_base + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t *smem = smem_dyn + (base - dyn_base);
  const uint32_t bars = base + SM::BAR_OFFSET;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_conv = [&](int s) { return bars + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (3 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
  const uint32_t bar_drain = bars + 8u * (3 * STAGES + 4);
  auto bar_slab = [&](int e, int b) { return bars + 8u * (3 * STAGES + 5 + 2 * e + b); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + SM::BAR_OFFSET + SM::NUM_BARS * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_conv(s), (PAIR ? 2 : 1) * (kConvWarps + (BWARPS ? kBConvWarps : 0)) * 32);   // the leader's counts both CTAs' converters
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), (PAIR ? 2 : 1) * kEpiWarps * 32);
    }
    mbar_init(bar_drain, 1);
    for (int e = 0; e < kEpiWarps; ++e) {
      mbar_init(bar_slab(e, 0), 1);
      mbar_init(bar_slab(e, 1), 1);
    }
    *abort_flag = 0;
    *reinterpret_cast<volatile long long *>(abort_flag + 1) = wk.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), SM::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), SM::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // PAIR: the work items are pairs of row tiles, and the two CTAs of a cluster walk them together
  const int m_units = PAIR ? (wk.m_tiles + 1) / 2 : wk.m_tiles;
  const long total = (long)m_units * wk.n_tiles * wk.splits;
  const long w_first = PAIR ? (long)(blockIdx.x >> 1) : (long)blockIdx.x;
  const long w_step = PAIR ? (long)(gridDim.x >> 1) : (long)gridDim.x;
  // Decode a work index into (m_tile, n_tile, split) and its k-block range.
  auto decode = [&](long w, int &mt, int &nt, int &sp, int &kbeg, int &nkb) {
    if (wk.m_fastest) {
      mt = (int)(w % m_units);
      const long r = w / m_units;
      nt = (int)(r % wk.n_tiles);
      sp = (int)(r / wk.n_tiles);
    } else {
      nt = (int)(w % wk.n_tiles);
      const long r = w / wk.n_tiles;
      mt = (int)(r % m_units);
      sp = (int)(r / m_units);
    }
    if (PAIR) mt = 2 * mt + (int)rank;   // may be one past the last row tile: such a CTA stages zeros and stores nothing
    kbeg = sp * wk.k_per_split;
    const int kend = min(wk.k_total, kbeg + wk.k_per_split);
    nkb = (kend - kbeg + BK - 1) / BK;
  };

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long w = w_first; w < total && ok; w += w_step) {
        int mt, nt, sp, kbeg, nkb;
        decode(w, mt, nt, sp, kbeg, nkb);
        auto prefetch_b = [&](int kb) {   // k-block kb of this unit's B operand -> L2
          const int k0 = kbeg + kb * BK;
          if (nt < wk.b_box3_tiles) {
            tma_prefetch_3d(&tmB3, 0, k0, nt * (BN / 32));
          } else {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tma_prefetch_2d(&tmB, nt * BN + 32 * c, k0);
          }
        };
        for (int kb = 0; kb < wk.b_prefetch && kb < nkb; ++kb) prefetch_b(kb);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (wk.b_prefetch > 0 && kb + wk.b_prefetch < nkb) prefetch_b(kb + wk.b_prefetch);
          if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, status, kWaitEmpty)) { ok = false; break; }
          if (kb == 0) TC_TRACE((w - w_first) / w_step, 0);
          if (kb == nkb - 1) TC_TRACE((w - w_first) / w_step, 8);
          mbar_arrive_expect_tx(bar_full(s), SM::TX_BYTES);
          const uint32_t a_dst = base + s * SM::STAGE_BYTES;
          const uint32_t b_dst = a_dst + SM::A_BYTES;
          const int k0 = kbeg + kb * BK;
          if constexpr (PRESPLIT) {   // the low parts, same boxes from the low-part planes
            const uint32_t blo_dst = a_dst + SM::RAW_BYTES, alo_dst = blo_dst + SM::B_BYTES;
            if (wk.a_box3) {
              tma_load_3d(alo_dst, &tmA3lo, 0, k0, (wk.a_row0 + mt * 128) / 32, bar_full(s));
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                tma_load_2d(alo_dst + c * (BK * 128), &tmAlo, wk.a_row0 + mt * 128 + 32 * c, k0, bar_full(s));
            }
            if (nt < wk.b_box3_tiles) {
              tma_load_3d(blo_dst, &tmB3lo, 0, k0, nt * (BN / 32), bar_full(s));
            } else {
#pragma unroll
              for (int c = 0; c < BN / 32; ++c)
                tma_load_2d(blo_dst + c * (BK * 128), &tmBlo, nt * BN + 32 * c, k0, bar_full(s));
            }
          }
          if (A_KMAJOR) {
            tma_load_2d(a_dst, &tmA, k0, wk.a_row0 + mt * 128, bar_full(s));
          } else if (wk.a_box3) {
            tma_load_3d(a_dst, &tmA3, 0, k0, (wk.a_row0 + mt * 128) / 32, bar_full(s));
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_load_2d(a_dst + c * (BK * 128), &tmA, wk.a_row0 + mt * 128 + 32 * c, k0, bar_full(s));
          }
          // (PAIR: this CTA's half of the tile's columns; the 3-D map's box is BNH / 32 chunks deep)
          if (nt < wk.b_box3_tiles) {
            tma_load_3d(b_dst, &tmB3, 0, k0, nt * (BN / 32) + (int)rank * (BNH / 32), bar_full(s));
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 32; ++c)
              tma_load_2d(b_dst + c * (BK * 128), &tmB, nt * BN + (int)rank * BNH + 32 * c, k0, bar_full(s));
          }
        }
      }
      if (!ok) {
        // Loads already issued still land in this CTA's shared memory: give them
        // a bounded moment before the CTA retires.
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) {
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      // D float32, A and B TF32; A (tensor memory) K-major, B (shared memory) MN-major
      // (PRESPLIT: A from shared memory too, MN-major like B; PAIR: 256 rows over the two CTAs)
      constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((PRESPLIT ? 1u : 0u) << 15) | (1u << 16) |
                                 ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((PAIR ? 256 : 128) >> 4) << 24);
      uint32_t it = 0, chain = 0;
      bool ok = true;
      for (long w = w_first; w < total && ok; w += w_step) {
        int mt, nt, sp, kbeg, nkb;
        decode(w, mt, nt, sp, kbeg, nkb);
        int kb = 0;
        while (kb < nkb && ok) {
          const uint32_t buf = chain & 1u, aph = (chain >> 1) & 1u;
          if (!mbar_wait(bar_acc_empty(buf), aph ^ 1u, abort_flag, status, kWaitAccEmpty)) { ok = false; break; }
          TC_TRACE(chain, 7);
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb_end = CHAIN > 0 ? min(nkb, kb + CHAIN) : (MULTI ? min(nkb, kb + wk.chain_kb) : nkb);
          for (bool first = true; kb < kb_end; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1u;
            // the stage is ready when the converters have split it, or (PRESPLIT) as soon as TMA has landed it
            if (!mbar_wait(PRESPLIT ? bar_full(s) : bar_conv(s), ph, abort_flag, status, kWaitConv)) { ok = false; break; }
            if (first) TC_TRACE(chain, 1);
            tc_fence_after();
            const uint32_t b_hi = base + s * SM::STAGE_BYTES + SM::A_BYTES;
            const uint32_t b_lo = base + s * SM::STAGE_BYTES + SM::RAW_BYTES;
            const uint32_t ta_hi = tmem_base + SM::TMEM_A_COL + s * (2 * BK);
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
              // One MMA consumes 8 k-values: 8 columns of A in tensor memory, eight 128-byte rows
              // (two 4-row swizzle atoms) of the MN-major B in shared memory.
              const uint64_t db_hi = smem_desc_mn(b_hi + kk * 1024, BK * 128);
              const uint64_t db_lo = smem_desc_mn(b_lo + kk * 1024, BK * 128);
              if constexpr (PRESPLIT) {
                const uint32_t a_hi = base + s * SM::STAGE_BYTES, a_lo = b_lo + SM::B_BYTES;
                const uint64_t da_hi = smem_desc_mn(a_hi + kk * 1024, BK * 128);
                const uint64_t da_lo = smem_desc_mn(a_lo + kk * 1024, BK * 128);
                mma_tf32_ss(d_tmem, da_lo, db_hi, idesc, (first && kk == 0) ? 0u : 1u);
                mma_tf32_ss(d_tmem, da_hi, db_lo, idesc, 1u);
                mma_tf32_ss(d_tmem, da_hi, db_hi, idesc, 1u);
              } else if constexpr (PAIR) {
                mma_tf32_ts_pair(d_tmem, ta_hi + BK + kk * 8, db_hi, idesc, (first && kk == 0) ? 0u : 1u);
                mma_tf32_ts_pair(d_tmem, ta_hi + kk * 8, db_lo, idesc, 1u);
                mma_tf32_ts_pair(d_tmem, ta_hi + kk * 8, db_hi, idesc, 1u);
              } else {
                mma_tf32_ts(d_tmem, ta_hi + BK + kk * 8, db_hi, idesc, (first && kk == 0) ? 0u : 1u);
                mma_tf32_ts(d_tmem, ta_hi + kk * 8, db_lo, idesc, 1u);
                mma_tf32_ts(d_tmem, ta_hi + kk * 8, db_hi, idesc, 1u);
              }
            }
            first = false;
            // the stage may be refilled once these MMAs have read it (PAIR: in both CTAs)
            if constexpr (PAIR) mma_commit_pair(bar_empty(s));
            else mma_commit(bar_empty(s));
          }
          if (ok) {
            TC_TRACE(chain, 2);
            if constexpr (PAIR) mma_commit_pair(bar_acc_full(buf));
            else mma_commit(bar_acc_full(buf));
            ++chain;
          }
        }
      }
      // Drain: nothing of this CTA may still be running in the tensor pipe when TMEM is freed.
      // (bounded by time alone: also a CTA that is giving up lets its MMAs in flight finish before TMEM goes)
      if constexpr (PAIR) mma_commit_pair(bar_drain);   // (the peer's copy of this barrier is not waited on)
      else mma_commit(bar_drain);
      if (!mbar_try_wait(bar_drain, 0)) mbar_wait_slow(bar_drain, 0, abort_flag, status, kWaitDrain, false);
    }
  } else if (warp < kConvWarps) {
    // ------------------------------------------------------------ hi / lo converters (idle when PRESPLIT)
    uint32_t it = 0;
    bool ok = true;
    for (long w = w_first; !PRESPLIT && w < total && ok; w += w_step) {
      int mt, nt, sp, kbeg, nkb;
      decode(w, mt, nt, sp, kbeg, nkb);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait(bar_full(s), ph, abort_flag, status, kWaitFull)) { ok = false; break; }
        if (threadIdx.x == 0 && kb == 0) TC_TRACE((w - w_first) / w_step, 5);
        if (threadIdx.x == 0 && kb == nkb - 1) TC_TRACE((w - w_first) / w_step, 9);
        static_assert(kConvWarps == 4, "one A row (tensor-memory lane) per converter thread");
        // A: this thread's row of the tile goes to its lane of tensor memory, hi (the raw bits) in BK
        // columns and lo in the next BK.
        uint32_t r[BK];
        if constexpr (A_KMAJOR) {
          // K-major tile, 128-byte rows: 16-byte chunk c of row m sits at chunk c ^ (m % 8)
          static_assert(BK == 32, "a K-major row is one 128-byte swizzle span");
          const uint8_t *arow = smem + s * SM::STAGE_BYTES + threadIdx.x * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 q4 = *reinterpret_cast<const uint4 *>(arow + ((c ^ (threadIdx.x & 7)) << 4));
            r[4 * c + 0] = q4.x; r[4 * c + 1] = q4.y; r[4 * c + 2] = q4.z; r[4 * c + 3] = q4.w;
          }
        } else {
          // MN-major tile [32-row chunk][k][32 rows]: element (k, m) of chunk m / 32 sits in the
          // 128-byte line k at 32-byte piece ((m % 32) / 8) ^ (k % 4); a warp reads one line per k.
          const uint8_t *acol = smem + s * SM::STAGE_BYTES + warp * (BK * 128) + ((lane & 7) << 2);
#pragma unroll
          for (int k = 0; k < BK; ++k)
            r[k] = *reinterpret_cast<const uint32_t *>(acol + k * 128 + ((((lane >> 3) ^ (k & 3))) << 5));
        }
        const uint32_t ta = tmem_base + SM::TMEM_A_COL + s * (2 * BK) + ((uint32_t)(warp * 32) << 16);
        tmem_st_32x32b<BK>(ta, r);
#pragma unroll
        for (int k = 0; k < BK; ++k) r[k] = __float_as_uint(tf32_lo(__uint_as_float(r[k])));
        tmem_st_32x32b<BK>(ta + BK, r);
        if constexpr (!BWARPS) {
          // B: lo parts beside the raw tile in shared memory.  Every load is issued before the first
          // store: the hand-off to the MMA warp costs one shared-memory round trip, not one per piece.
          constexpr int kConvThreads = kConvWarps * 32;
          const float4 *rawb = reinterpret_cast<const float4 *>(smem + s * SM::STAGE_BYTES + SM::A_BYTES);
          float4 *lob = reinterpret_cast<float4 *>(smem + s * SM::STAGE_BYTES + SM::RAW_BYTES);
          constexpr int kPieces = SM::B_BYTES / 16 / kConvThreads;
          static_assert(SM::B_BYTES % (16 * kConvThreads) == 0, "a whole number of 16-byte pieces per thread");
          float4 v[kPieces];
#pragma unroll
          for (int i = 0; i < kPieces; ++i) v[i] = rawb[threadIdx.x + i * kConvThreads];
#pragma unroll
          for (int i = 0; i < kPieces; ++i)
            lob[threadIdx.x + i * kConvThreads] =
                make_float4(tf32_lo(v[i].x), tf32_lo(v[i].y), tf32_lo(v[i].z), tf32_lo(v[i].w));
          fence_async_smem();  // make the generic-proxy writes visible to the tensor pipe
        }
        tmem_wait_st();
        tc_fence_before();
        // (test hook: one lost arrival leaves the MMA warp waiting until its time limit, see tc_debug_lose_arrive)
        if (!(wk.lose_arrive && it == 0 && threadIdx.x == 0 && blockIdx.x == 0)) {
          if constexpr (PAIR) mbar_arrive_rank(bar_conv(s), 0);   // the leader's MMA warp waits for both CTAs
          else mbar_arrive(bar_conv(s));
        }
      }
    }
  } else if (warp > kMmaWarp) {
    // ------------------------------------------------------------ B's lo parts (BWARPS kernels)
    // Two warps of their own: on the A converters' path this work lengthens the chain (wait for the stage, load,
    // split, store, fence, arrive) that every k-block of the MMA stream waits for.  Measured: forward product
    // 0.437 -> 0.396 ms, single-chain trace update 0.561 -> 0.557 ms; the multi-chain trace update, whose eight
    // epilogue warps keep the SM's issue slots and shared memory busier, lost 5 %, so there the A converters
    // keep this work and these two warps go straight to the tear-down.
    uint32_t it = 0;
    bool ok = true;
    const int t = threadIdx.x - (kMmaWarp + 1) * 32;   // 0 .. 63
    for (long w = w_first; BWARPS && w < total && ok; w += w_step) {
      int mt, nt, sp, kbeg, nkb;
      decode(w, mt, nt, sp, kbeg, nkb);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait(bar_full(s), ph, abort_flag, status, kWaitFull)) { ok = false; break; }
        // lo parts beside the raw tile in shared memory; every load is issued before the first store
        constexpr int kBThreads = kBConvWarps * 32;
        const float4 *rawb = reinterpret_cast<const float4 *>(smem + s * SM::STAGE_BYTES + SM::A_BYTES);
        float4 *lob = reinterpret_cast<float4 *>(smem + s * SM::STAGE_BYTES + SM::RAW_BYTES);
        constexpr int kPieces = SM::B_BYTES / 16 / kBThreads;
        static_assert(SM::B_BYTES % (16 * kBThreads) == 0, "a whole number of 16-byte pieces per thread");
        float4 v[kPieces];
#pragma unroll
        for (int i = 0; i < kPieces; ++i) v[i] = rawb[t + i * kBThreads];
#pragma unroll
        for (int i = 0; i < kPieces; ++i)
          lob[t + i * kBThreads] = make_float4(tf32_lo(v[i].x), tf32_lo(v[i].y), tf32_lo(v[i].z), tf32_lo(v[i].w));
        fence_async_smem();  // make the generic-proxy writes visible to the tensor pipe
        if constexpr (PAIR) mbar_arrive_rank(bar_conv(s), 0);
        else mbar_arrive(bar_conv(s));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Thread (lane) owns four tile rows (16*hh + lane/4 + 8*rr) of its warp's TMEM lane
    // quarter and, per 32-column group, the column pairs 8*rep + 2*(lane%4) + {0,1}:
    // four lanes cover 32 contiguous bytes of a row, so global accesses fill whole sectors.
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int ch = (warp - kConvWarps) >> 2;     // which half of the tile's columns
    const int lr = lane >> 2, lc = (lane & 3) * 2;
    constexpr int NG = BN / 64;                  // 32-column groups per warp
    uint32_t chain = 0;
    bool ok = true;
    const int ew = warp - kConvWarps;            // epilogue warp index
    uint32_t swz[4];                             // byte offset of column pair `rep` inside a swizzled 128-byte row
#pragma unroll
    for (int rep = 0; rep < 4; ++rep) swz[rep] = ((uint32_t)((2 * rep + (lc >> 2)) ^ lr) << 4) + (uint32_t)(lc & 3) * 4u;
    uint32_t slab = 0;                           // blocks of the trace matrix consumed so far (fused epilogue)
    // Hypercolumn of a column: exact multiply-shift division when the host verified it, else the table.
    auto hc_of = [&](long n) -> int {
      return ep.hc_magic ? (int)__umulhi((uint32_t)n, ep.hc_magic) : __ldg(ep.col_hc + n);
    };
    // Block number s of this warp (buffer s % 2): column group g of tile (mt, nt).
    auto issue_slab_at = [&](uint32_t s, int mt, int nt, int g) {
      const uint32_t b = s & 1u;
      mbar_arrive_expect_tx(bar_slab(ew, b), kSlabBytes);
      tma_load_2d(base + SM::SLAB_OFFSET + (ew * 2 + b) * kSlabBytes, &tmC, nt * BN + ch * (BN / 2) + g * 32,
                  (int)ep.row0 + mt * 128 + 32 * q, bar_slab(ew, b));
    };
    if (FUSED && lane == 0 && w_first < total) {
      int mt, nt, sp, kbeg, nkb;
      decode(w_first, mt, nt, sp, kbeg, nkb);
      issue_slab_at(0, mt, nt, 0);
      issue_slab_at(1, mt, nt, 1);
    }
    // Raw product leaving by TMA: this warp's 32 x 32 block of column group g (lo: tile rows lr, lr + 8; hi:
    // 16 + lr, 24 + lr; four column pairs each) goes to a staging buffer in the swizzled layout of the
    // tensor map and one lane sends it.  Blocks past the edge of the output are clipped by the TMA unit.
    uint32_t stores = 0;
    auto store_block = [&](const float (&lo)[16], const float (&hi)[16], int mt, int nt, int g) {
      const uint32_t sb = stores & 1u;
      if (lane == 0) bulk_wait_read_1();   // the store that used this buffer two blocks ago has read it
      __syncwarp();
      uint8_t *sl = smem + SM::SLAB_OFFSET + (ew * 2 + sb) * kSlabBytes + lr * 128;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int rep = 0; rep < 4; ++rep) {
          *reinterpret_cast<float2 *>(sl + (8 * rr) * 128 + swz[rep]) = make_float2(lo[rep * 4 + rr * 2], lo[rep * 4 + rr * 2 + 1]);
          *reinterpret_cast<float2 *>(sl + (16 + 8 * rr) * 128 + swz[rep]) =
              make_float2(hi[rep * 4 + rr * 2], hi[rep * 4 + rr * 2 + 1]);
        }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmC, base + SM::SLAB_OFFSET + (ew * 2 + sb) * kSlabBytes, nt * BN + ch * (BN / 2) + g * 32,
                     mt * 128 + 32 * q);
        bulk_commit();
      }
      ++stores;
    };
    for (long w = w_first; w < total && ok; w += w_step) {
      int mt, nt, sp, kbeg, nkb;
      decode(w, mt, nt, sp, kbeg, nkb);
      int mt_next = 0, nt_next = 0;
      if (FUSED && w + w_step < total) {
        int sp2, kb2, nk2;
        decode(w + w_step, mt_next, nt_next, sp2, kb2, nk2);
      }
      const long m_base = (long)mt * 128 + 32 * q;   // first tile row of this warp's lane quarter
      const long n_base = (long)nt * BN + ch * (BN / 2);
      bool rv[4];
      long grow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long m = m_base + 16 * (j >> 1) + lr + 8 * (j & 1);
        rv[j] = m < ep.rows;
        grow[j] = m;
      }
      if constexpr (CHAIN > 0) {
        // ---- running sums in registers, one TMEM chain at a time (forward product)
        float sum[NG][2][16];
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
#pragma unroll
            for (int k = 0; k < 16; ++k) sum[g][hh][k] = 0.f;
        const int nchains = (nkb + CHAIN - 1) / CHAIN;
        for (int c = 0; c < nchains && ok; ++c, ++chain) {
          const uint32_t buf = chain & 1u, aph = (chain >> 1) & 1u;
          if (!mbar_wait(bar_acc_full(buf), aph, abort_flag, status, kWaitAccFull)) { ok = false; break; }
          __syncwarp();
          tc_fence_after();
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            float a0[16], a1[16];
            const uint32_t t0 = tmem_base + buf * BN + ch * (BN / 2) + g * 32 + ((uint32_t)(32 * q) << 16);
            tmem_ld_pair(t0, t0 + (16u << 16), a0, a1);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              sum[g][0][k] += a0[k];
              sum[g][1][k] += a1[k];
            }
          }
          tc_fence_before();
          if constexpr (PAIR) mbar_arrive_rank(bar_acc_empty(buf), 0);
          else mbar_arrive(bar_acc_empty(buf));
        }
        if (ok && !A_KMAJOR && ep.tma_store) {
#pragma unroll
          for (int g = 0; g < NG; ++g) store_block(sum[g][0], sum[g][1], mt, nt, g);
        } else if (ok) {
#pragma unroll
          for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (!rv[j]) continue;
              float *orow = ep.out + ((long)sp * ep.rows + grow[j]) * ep.ld;
#pragma unroll
              for (int rep = 0; rep < 4; ++rep) {
                const long n = n_base + g * 32 + rep * 8 + lc;
                if (n < ep.cols)
                  __stcs(reinterpret_cast<float2 *>(orow + n),
                         make_float2(sum[g][j >> 1][rep * 4 + (j & 1) * 2], sum[g][j >> 1][rep * 4 + (j & 1) * 2 + 1]));
              }
            }
        }
      } else {
        // The k-range of a tile may be cut into several tensor-memory accumulation chains (the tensor core
        // truncates every accumulate, so the error of a chain grows with its length): chain 0 forms the
        // result as if it were the whole sum, every later chain adds its part to what the earlier ones
        // stored (read back through L2), and only the last chain clamps the trace and writes the weight.
        const int nchains = MULTI ? (nkb + wk.chain_kb - 1) / wk.chain_kb : 1;
       for (int cc = 0; cc < nchains && ok; ++cc) {
        const bool first_chain = !MULTI || cc == 0, last_chain = !MULTI || cc == nchains - 1;
        const uint32_t buf = chain & 1u, aph = (chain >> 1) & 1u;
        // Everything the fused epilogue needs besides the accumulator is fetched before waiting for
        // the accumulator, so these global-memory latencies overlap the wait.
        const bool has_mask = FUSED && ep.wmask != nullptr;
        int hc_first = 0, hc_last = 0;
        bool bits_ok = true, tile_fast = false;
        float rci[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t mbits[4] = {0xFFu, 0xFFu, 0xFFu, 0xFFu};
        float *crow[4] = {nullptr, nullptr, nullptr, nullptr};
        float2 rcj_next[4];
        float lane_rcj_next = 0.f;
        long w_minus_c = 0;
        if constexpr (FUSED) {
          // per tile: reciprocal of Ci (0 = row below threshold), trace row pointers and the row's mask
          // bytes for every hypercolumn this half tile touches (bit k: hypercolumn hc_first + k)
          if (has_mask) {
            hc_first = hc_of(n_base < ep.cols ? n_base : ep.cols - 1);
            hc_last = hc_of(n_base + BN / 2 - 1 < ep.cols ? n_base + BN / 2 - 1 : ep.cols - 1);
          }
          bits_ok = hc_last - hc_first <= 7;
          const int nhc = hc_last - hc_first + 1;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const long i = ep.row0 + grow[j];
            rci[j] = rv[j] ? __ldg(ep.rci + i) : 0.f;
            crow[j] = ep.Cij + i * ep.cols + n_base + lc;
            if (has_mask && rv[j] && bits_ok) {
              // every byte is loaded (index clamped into the row's range) so that the loads go out together
              const uint8_t *mr = ep.wmask + i * ep.H + hc_first;
              uint32_t byte[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) byte[k] = __ldg(mr + (k < nhc ? k : 0));
              uint32_t bits = 0;
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (k < nhc && byte[k] != 0) bits |= 1u << k;
              mbits[j] = bits;
            }
          }
          // reciprocals of Cj for the first column group: this thread's pairs and, one per lane, the whole group
#pragma unroll
          for (int rep = 0; rep < 4; ++rep) {
            const long n = n_base + lc + rep * 8;
            rcj_next[rep] = n < ep.cols ? __ldg(reinterpret_cast<const float2 *>(ep.rcj + n)) : make_float2(0.f, 0.f);
          }
          lane_rcj_next = n_base + lane < ep.cols ? __ldg(ep.rcj + n_base + lane) : 0.f;
          tile_fast = ep.fast_ok && bits_ok && (long)mt * 128 + 128 <= ep.rows;
          w_minus_c = ep.W - ep.Cij;   // the weight of an element sits this far from its trace
        }
        if (!mbar_wait(bar_acc_full(buf), aph, abort_flag, status, kWaitAccFull)) { ok = false; break; }
        if (threadIdx.x == kConvWarps * 32) TC_TRACE(chain, 3);
        __syncwarp();
        tc_fence_after();
        // this warp's accumulator block: TMEM lanes 32q.., columns of its half tile
        const uint32_t tacc = tmem_base + buf * BN + ch * (BN / 2) + ((uint32_t)(32 * q) << 16);
        if constexpr (FUSED) {
          if (threadIdx.x == kConvWarps * 32) TC_TRACE(chain, 10);
#pragma unroll 1
          for (int g = 0; g < NG; ++g) {
            // This warp's 32 x 32 block of the trace matrix was fetched by TMA two blocks ago
            // (128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8); every row
            // of this thread has r % 8 == lane / 4).
            const uint32_t sb = slab & 1u;
            if (!mbar_wait(bar_slab(ew, sb), (slab >> 1) & 1u, abort_flag, status, kWaitSlab)) { ok = false; break; }
            const uint8_t *sl = smem + SM::SLAB_OFFSET + (ew * 2 + sb) * kSlabBytes + lr * 128;
            const long gs = n_base + g * 32;   // first column of the group
            float2 rcj[4];
#pragma unroll
            for (int rep = 0; rep < 4; ++rep) rcj[rep] = rcj_next[rep];
            const float lane_rcj = lane_rcj_next;
            if (g + 1 < NG) {   // the next group's values, in flight while this group is processed
#pragma unroll
              for (int rep = 0; rep < 4; ++rep) {
                const long nn = gs + 32 + lc + rep * 8;
                rcj_next[rep] = nn < ep.cols ? __ldg(reinterpret_cast<const float2 *>(ep.rcj + nn)) : make_float2(0.f, 0.f);
              }
              lane_rcj_next = gs + 32 + lane < ep.cols ? __ldg(ep.rcj + gs + 32 + lane) : 0.f;
            }
            // Fast groups (whole block inside the matrix, at most two hypercolumns per group): one
            // select word per row, bit 8*rep + e = "element e of column pair rep keeps its weight".
            const bool g_fast = tile_fast && gs + 32 <= ep.cols;
            uint32_t sel[4] = {0u, 0u, 0u, 0u};
            if (g_fast) {
              const uint32_t live32 = __ballot_sync(0xFFFFFFFFu, lane_rcj != 0.f);   // columns at or above the threshold
              uint32_t first32 = 0xFFFFFFFFu;   // columns of the group's first hypercolumn
              int k0 = 0;
              if (has_mask) {
                const int hc0 = hc_of(gs);
                const long bnd = (long)(hc0 + 1) * ep.Mc - gs;
                if (bnd < 32) first32 = (1u << bnd) - 1u;
                k0 = hc0 - hc_first;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t m0 = 0u - ((mbits[j] >> k0) & 1u), m1 = 0u - ((mbits[j] >> (k0 + 1)) & 1u);
                const uint32_t word = ((m0 & first32) | (m1 & ~first32)) & live32;
                sel[j] = rci[j] != 0.f ? (word >> lc) & 0x03030303u : 0u;
              }
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              // 16 of the warp's 32 TMEM lanes at a time keeps the live registers within budget
              float a[16];
              __syncwarp();  // tcgen05.ld is warp-collective
              tmem_ld_16x256b_x4(tacc + g * 32 + ((uint32_t)(16 * hh) << 16), a);
              float2 c[2][4];
#pragma unroll
              for (int rr = 0; rr < 2; ++rr)
#pragma unroll
                for (int rep = 0; rep < 4; ++rep)
                  c[rr][rep] = *reinterpret_cast<const float2 *>(sl + (16 * hh + 8 * rr) * 128 + swz[rep]);
              if (hh == 1) {
                // The buffer is about to be overwritten by the async proxy (TMA): every lane's
                // reads above must have been performed first, not merely issued.  With several chains the
                // block about to be fetched may be one this warp stored a moment ago: those global writes
                // are ordered before the fetch as well.
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                  // block slab+2: two column groups ahead in this tile, or the next tile's first groups.  With
                  // several chains the blocks of the next pass are fetched at the end of this one (below).
                  if (g + 2 < NG) issue_slab_at(slab + 2, mt, nt, g + 2);
                  else if (!MULTI && w + w_step < total) issue_slab_at(slab + 2, mt_next, nt_next, g + 2 - NG);
                }
              }
              if (g_fast) {
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                  const int j = 2 * hh + rr;
                  float *cp = crow[j] + g * 32;
                  const float r = rci[j];
                  const uint32_t sj = sel[j];
#pragma unroll
                  for (int rep = 0; rep < 4; ++rep) {
                    float2 c2 = c[rr][rep];
                    // the old trace decays once, in chain 0
                    c2.x = fmaf(c2.x, first_chain ? ep.p.one_minus : 1.f, a[rep * 4 + rr * 2 + 0] * ep.ema_scale);
                    c2.y = fmaf(c2.y, first_chain ? ep.p.one_minus : 1.f, a[rep * 4 + rr * 2 + 1] * ep.ema_scale);
                    if (!last_chain) {   // a partial sum: parked in the trace matrix (it stays in L2)
                      __stcg(reinterpret_cast<float2 *>(cp + rep * 8), c2);
                      continue;
                    }
                    c2.x = fmaxf(c2.x, 0.f);
                    c2.y = fmaxf(c2.y, 0.f);
                    const float wx = lg2_ftz(fmaxf(c2.x, ep.p.cthr4) * (r * rcj[rep].x)) * kLn2;
                    const float wy = lg2_ftz(fmaxf(c2.y, ep.p.cthr4) * (r * rcj[rep].y)) * kLn2;
                    __stcs(reinterpret_cast<float2 *>(cp + rep * 8), c2);
                    __stcs(reinterpret_cast<float2 *>(cp + w_minus_c + rep * 8),
                           make_float2((sj & (1u << (8 * rep))) ? wx : 0.f, (sj & (2u << (8 * rep))) ? wy : 0.f));
                  }
                }
              } else {
                // edge blocks and layouts the select words do not cover: every element checked
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                  const int j = 2 * hh + rr;
                  if (!rv[j]) continue;
                  float *cp = crow[j] + g * 32;
                  const uint8_t *mr = has_mask ? ep.wmask + (ep.row0 + grow[j]) * ep.H : nullptr;
#pragma unroll
                  for (int rep = 0; rep < 4; ++rep) {
                    const long n = gs + lc + rep * 8;
                    if (!(n < ep.cols)) continue;   // cols is even: n + 1 is in range too
                    float2 c2 = c[rr][rep];
                    // the old trace decays once, in chain 0
                    c2.x = fmaf(c2.x, first_chain ? ep.p.one_minus : 1.f, a[rep * 4 + rr * 2 + 0] * ep.ema_scale);
                    c2.y = fmaf(c2.y, first_chain ? ep.p.one_minus : 1.f, a[rep * 4 + rr * 2 + 1] * ep.ema_scale);
                    if (!last_chain) {
                      __stcg(reinterpret_cast<float2 *>(cp + rep * 8), c2);
                      continue;
                    }
                    c2.x = fmaxf(c2.x, 0.f);
                    c2.y = fmaxf(c2.y, 0.f);
                    bool on0 = rci[j] != 0.f && rcj[rep].x != 0.f, on1 = rci[j] != 0.f && rcj[rep].y != 0.f;
                    if (has_mask) {
                      const int h0 = hc_of(n), h1 = hc_of(n + 1);
                      if (bits_ok) {
                        on0 = on0 && ((mbits[j] >> (h0 - hc_first)) & 1u);
                        on1 = on1 && ((mbits[j] >> (h1 - hc_first)) & 1u);
                      } else {
                        on0 = on0 && __ldg(mr + h0) != 0;
                        on1 = on1 && __ldg(mr + h1) != 0;
                      }
                    }
                    const float wx = __logf(fmaxf(c2.x, ep.p.cthr4) * (rci[j] * rcj[rep].x));
                    const float wy = __logf(fmaxf(c2.y, ep.p.cthr4) * (rci[j] * rcj[rep].y));
                    __stcs(reinterpret_cast<float2 *>(cp + rep * 8), c2);
                    __stcs(reinterpret_cast<float2 *>(cp + w_minus_c + rep * 8), make_float2(on0 ? wx : 0.f, on1 ? wy : 0.f));
                  }
                }
              }
            }
            ++slab;
            if (threadIdx.x == kConvWarps * 32 && g < 3) TC_TRACE(chain, 13 + g);
          }
          if (MULTI && ok) {
            // The next pass re-reads blocks this warp has just stored (the running sums): one fence per pass
            // orders those global writes, and the shared-memory reads of both landing buffers, before the
            // async-proxy fetches of the next pass's first two blocks (or the next tile's).
            static_assert(!MULTI || NG >= 2, "two landing buffers are refilled at the end of a pass");
            fence_async_all();
            __syncwarp();
            if (lane == 0) {
              if (!last_chain) {
                issue_slab_at(slab, mt, nt, 0);
                issue_slab_at(slab + 1, mt, nt, 1);
              } else if (w + w_step < total) {
                issue_slab_at(slab, mt_next, nt_next, 0);
                issue_slab_at(slab + 1, mt_next, nt_next, 1);
              }
            }
          }
        } else {
#pragma unroll 1
          for (int g = 0; g < NG; ++g) {
            float a0[16], a1[16];
            const uint32_t t0 = tacc + g * 32;
            __syncwarp();  // tcgen05.ld is warp-collective
            tmem_ld_pair(t0, t0 + (16u << 16), a0, a1);
            if (!A_KMAJOR && !MULTI && ep.tma_store) {
              store_block(a0, a1, mt, nt, g);
              continue;
            }
            const long n0 = n_base + g * 32 + lc;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (!rv[j]) continue;
              const float *acc = (j >> 1) ? a1 : a0;
              float *orow = ep.out + ((long)sp * ep.rows + grow[j]) * ep.ld;
#pragma unroll
              for (int rep = 0; rep < 4; ++rep)
                if (n0 + rep * 8 < ep.cols) {   // cols is even: n+1 is in range too
                  float2 v = make_float2(acc[rep * 4 + (j & 1) * 2], acc[rep * 4 + (j & 1) * 2 + 1]);
                  float2 *dst = reinterpret_cast<float2 *>(orow + n0 + rep * 8);
                  if (!first_chain) {   // this thread stored the sum of the earlier chains at the same place
                    const float2 prev = __ldcg(dst);
                    v.x += prev.x;
                    v.y += prev.y;
                  }
                  if (last_chain) __stcs(dst, v); else __stcg(dst, v);
                }
            }
          }
        }
        if (!ok) break;
        if (threadIdx.x == kConvWarps * 32) TC_TRACE(chain, 4);
        tc_fence_before();
        // the accumulator buffer may be overwritten (PAIR: the leader's MMA warp waits for both CTAs' epilogues)
        if constexpr (PAIR) mbar_arrive_rank(bar_acc_empty(buf), 0);
        else mbar_arrive(bar_acc_empty(buf));
        ++chain;
       }   // chains of this tile
      }
    }
  }

  // stores this thread sent by TMA must have left shared memory (and landed) before the CTA retires
  if (!FUSED && !A_KMAJOR && warp >= kConvWarps && warp < kTmaWarp && lane == 0) bulk_wait_all();
  // ------------------------------------------------------------ tear-down
  __syncwarp();
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA retires while the other may still signal it or read its operands
  else __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, SM::TMEM_COLS);
    else tmem_dealloc(tmem_base, SM::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_mutex;
EncodeTiledFn g_encode = nullptr;
int g_available = -1;           // -1 unknown, 0 no, 1 yes
int *g_status[64] = {nullptr};  // per-device status word
int g_sm_count_tc[64] = {0};
std::atomic<int> g_reserved_sms{-1};   // -1: not set yet (the environment decides on first use)
std::atomic<long long> g_wait_limit{kWaitLimitCycles};
std::atomic<int> g_lose_arrive{0};     // launches that still have to lose one arrival (test hook)
long long wait_limit_now() { return g_wait_limit.load(); }
int take_lose_arrive() {
  int n = g_lose_arrive.load();
  while (n > 0 && !g_lose_arrive.compare_exchange_weak(n, n - 1)) {
  }
  return n > 0 ? 1 : 0;
}

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev < 0 || dev >= 64 ? 0 : dev;
}

bool init_once() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_available < 0) {
    g_available = 0;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess && fn != nullptr) {
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      g_available = 1;
    } else {
      (void)cudaGetLastError();
    }
  }
  return g_available == 1;
}

int *status_word() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status[dev] == nullptr) {
    int *p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_status[dev] = p;
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count_tc[dev] = n > 0 ? n : 148;
  }
  return g_status[dev];
}

// Encoded tensor maps are kept per host thread, keyed by everything that goes into them: a layer's step
// re-encodes the same handful of maps (same buffers, same shapes) every call, and the driver's encoder
// costs about a microsecond each, which is a tenth of the step of a small layer.
struct MapKey {
  const void *base;
  long inner, outer;
  int box_a, box_b, kind;
  bool operator==(const MapKey &o) const {
    return base == o.base && inner == o.inner && outer == o.outer && box_a == o.box_a && box_b == o.box_b && kind == o.kind;
  }
};
struct MapCache {
  static constexpr int kSlots = 128;
  MapKey key[kSlots];
  CUtensorMap map[kSlots];
  bool used[kSlots] = {false};
  static unsigned slot(const MapKey &k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (uint64_t)k.inner * 0xC2B2AE3D27D4EB4Full + (uint64_t)k.outer * 0x165667B19E3779F9ull +
         (uint64_t)(k.box_a * 131 + k.box_b * 17 + k.kind);
    return (unsigned)(h >> 40) % kSlots;
  }
  bool find(const MapKey &k, CUtensorMap *out) const {
    const unsigned s = slot(k);
    if (!used[s] || !(key[s] == k)) return false;
    *out = map[s];
    return true;
  }
  void put(const MapKey &k, const CUtensorMap &m) {
    const unsigned s = slot(k);
    key[s] = k;
    map[s] = m;
    used[s] = true;
  }
};
thread_local MapCache g_map_cache;

bool make_map_uncached(CUtensorMap *map, const float *base, long inner, long outer, int box_inner, int box_outer,
                       bool mn_major);
bool make_map_chunks_uncached(CUtensorMap *map, const float *base, long cols, long rows, int box_rows, int box_chunks);

// 2-D float32 tensor map over a row-major [outer, inner] matrix, zero fill.  `mn_major` selects the
// 32-byte-base flavour of the 128-byte swizzle that MN-major 32-bit operands need.
bool make_map(CUtensorMap *map, const float *base, long inner, long outer, int box_inner, int box_outer,
              bool mn_major) {
  const MapKey k{base, inner, outer, box_inner, box_outer, mn_major ? 1 : 0};
  if (g_map_cache.find(k, map)) return true;
  if (!make_map_uncached(map, base, inner, outer, box_inner, box_outer, mn_major)) return false;
  g_map_cache.put(k, *map);
  return true;
}
bool make_map_chunks(CUtensorMap *map, const float *base, long cols, long rows, int box_rows, int box_chunks) {
  const MapKey k{base, cols, rows, box_rows, box_chunks, 2};
  if (g_map_cache.find(k, map)) return true;
  if (!make_map_chunks_uncached(map, base, cols, rows, box_rows, box_chunks)) return false;
  g_map_cache.put(k, *map);
  return true;
}

bool make_map_uncached(CUtensorMap *map, const float *base, long inner, long outer, int box_inner, int box_outer,
                       bool mn_major) {
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)inner * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3-D view {32, rows, cols/32} of a row-major [rows, cols] float32 matrix (element (i, r, c) = m[r][32c + i]);
// a box {32, box_rows, box_chunks} lands in shared memory as [chunk][row][32], the MN-major stage layout.
bool make_map_chunks_uncached(CUtensorMap *map, const float *base, long cols, long rows, int box_rows, int box_chunks) {
  if (cols < 32) return false;
  cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)(cols / 32)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * sizeof(float), 128};
  cuuint32_t box[3] = {32, (cuuint32_t)box_rows, (cuuint32_t)box_chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Column tiles of width bn whose every 32-column group lies inside the matrix.
int full_chunk_tiles(long cols, int bn) { return (int)(((cols / 32) * 32) / bn); }

struct TcMaps {
  CUtensorMap a, b, a3, b3, c;
  CUtensorMap alo, blo, a3lo, b3lo;   // the operands' low-part planes (pre-split kernels)
};

template <bool A_KMAJOR, int BN, int BK, int STAGES, bool FUSED, int CHAIN, bool MULTI = false, bool PRESPLIT = false>
cudaError_t launch_tc(const TcMaps &tm, const TcWork &wk, const TcEpilogue &ep, cudaStream_t st,
                      bool leave_reserved_sms = false) {
  using SM = TcSmem<BN, BK, STAGES, FUSED || !A_KMAJOR, PRESPLIT>;
  int *status = status_word();
  if (status == nullptr) return cudaErrorMemoryAllocation;
  auto kernel = tc_contraction_kernel<A_KMAJOR, BN, BK, STAGES, FUSED, CHAIN, MULTI, PRESPLIT>;
  static std::atomic<bool> configured[64];   // per device; setting the attribute twice is harmless
  const int dev = current_device();
  if (!configured[dev].load()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) return e;
    configured[dev].store(true);
  }
  const long total = (long)wk.m_tiles * wk.n_tiles * wk.splits;
  if (total <= 0) return cudaSuccess;
  int sms = g_sm_count_tc[dev] - (leave_reserved_sms ? tc_get_reserved_sms() : 0);
  if (sms < 1) sms = 1;
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  kernel<<<grid, kThreads, SM::TOTAL, st>>>(tm.a, tm.b, tm.a3, tm.b3, tm.c, tm.alo, tm.blo, tm.a3lo, tm.b3lo, wk, ep,
                                            status);
  return cudaGetLastError();
}

// SBB_TC_PAIR=0 keeps one CTA per tile (read once).
bool pairs_enabled() {
  static const bool on = [] {
    const char *e = getenv("SBB_TC_PAIR");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// The CTA-pair form of a kernel: clusters of two CTAs, one 256 x BN tile per pair.
template <bool A_KMAJOR, int BN, int BK, int STAGES, bool FUSED, int CHAIN, bool MULTI = false>
cudaError_t launch_tc_pair(const TcMaps &tm, const TcWork &wk, const TcEpilogue &ep, cudaStream_t st) {
  using SM = TcSmem<BN, BK, STAGES, FUSED || !A_KMAJOR, false, true>;
  int *status = status_word();
  if (status == nullptr) return cudaErrorMemoryAllocation;
  auto kernel = tc_contraction_kernel<A_KMAJOR, BN, BK, STAGES, FUSED, CHAIN, MULTI, false, true>;
  static std::atomic<bool> configured[64];
  const int dev = current_device();
  if (!configured[dev].load()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) return e;
    configured[dev].store(true);
  }
  const long pairs = (long)((wk.m_tiles + 1) / 2) * wk.n_tiles * wk.splits;
  if (pairs <= 0) return cudaSuccess;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = SM::TOTAL;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // as many pairs as can be resident at once (one CTA per SM; pairs must share a GPC's SMs)
  static int max_clusters[64] = {0};
  if (max_clusters[dev] == 0) {
    cfg.gridDim = dim3((unsigned)(g_sm_count_tc[dev] / 2 * 2), 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) n = g_sm_count_tc[dev] / 2;
    max_clusters[dev] = n;
  }
  long clusters = max_clusters[dev] < g_sm_count_tc[dev] / 2 ? max_clusters[dev] : g_sm_count_tc[dev] / 2;
  if (clusters > pairs) clusters = pairs;
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  return cudaLaunchKernelEx(&cfg, kernel, tm.a, tm.b, tm.a3, tm.b3, tm.c, tm.alo, tm.blo, tm.a3lo, tm.b3lo, wk, ep,
                            status);
}

}  // namespace

// Launch counter shared with the general-shape kernels (defined in sbb_kernels.cu).
void count_launches(int n);

bool tc_available() {
  if (!init_once()) return false;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
  return major == 10;
}

bool tc_shape_ok(const void *x, const void *y_or_w, long N, long M) {
  return N % 4 == 0 && M % 4 == 0 && N >= 4 && M >= 4 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(y_or_w) & 15u) == 0 && N < 2147483647L && M < 2147483647L;
}

namespace {
constexpr int kFwdBN = 128, kFwdBK = 32, kFwdStages = 4;
constexpr int kFwdPrefetch = 0;  // k-blocks of W requested into L2 ahead of the shared-memory pipeline (measured: no gain at 4-16)
constexpr int kFwdChain = 4;  // 4 k-blocks of 32 = 128 k-values (48 MMAs) per tensor-memory accumulation chain
constexpr int kTrBN = 192, kTrBK = 16, kTrStages = 4;
// k-blocks per accumulation chain of the batch contractions: 16 x 16 = 256 samples (96 MMAs), after which the
// epilogue takes the partial sum over in float32.  Measured on B200: the tensor-memory accumulate truncates,
// so a chain's sum is low by about 1e-8 x (samples in the chain) relative; 256 keeps that below 4e-6.
constexpr int kTrChainKb = 16;
constexpr int kPairStages = 4;   // (tensor memory holds the A parts of four stages beside the two accumulators)
constexpr int kLongBN = 128, kLongStages = 5;   // tiles of the row-block product when the batch spans several chains

// k-blocks per split and the number of (non-empty) splits for the forward product: the split count
// that minimises (waves of CTAs) x (k-blocks per unit), plus the cost of writing and re-reading
// one more partial result.  A unit count just above a multiple of the SM count would otherwise
// run a nearly empty last wave (192 units on 148 SMs take as long as 296).
void forward_split_plan(long B, long N, long M, int &splits, int &k_per_split) {
  const long tiles = ((B + 127) / 128) * ((M + kFwdBN - 1) / kFwdBN);
  const long kblocks = (N + kFwdBK - 1) / kFwdBK;
  const int dev = current_device();
  const long sms = g_sm_count_tc[dev] > 0 ? g_sm_count_tc[dev] : 148;
  long max_splits = kblocks / 8 > 0 ? kblocks / 8 : 1;   // at least 8 k-blocks per split
  if (max_splits > 64) max_splits = 64;
  // one partial result costs B*M*8 bytes of traffic; in units of one k-block of one CTA (about 0.8 us
  // at 6.5 TB/s, spread over the SMs)
  const double partial_cost = (double)B * (double)M * 8.0 / 6.5e12 / 0.8e-6;
  double best_cost = 0.0;
  long best_per = kblocks;
  for (long want = 1; want <= max_splits; ++want) {
    const long per = (kblocks + want - 1) / want;
    const long actual = (kblocks + per - 1) / per;
    const long waves = (tiles * actual + sms - 1) / sms;
    const double cost = (double)waves * (double)per + (double)actual * partial_cost;
    if (want == 1 || cost < best_cost) {
      best_cost = cost;
      best_per = per;
    }
  }
  splits = (int)((kblocks + best_per - 1) / best_per);
  k_per_split = (int)best_per * kFwdBK;
}
}  // namespace

int forward_splits_tc(long B, long N, long M) {
  status_word();  // fills the SM count
  int s, k;
  forward_split_plan(B, N, M, s, k);
  return s;
}

cudaError_t launch_forward_product_tc(const float *x, const float *w, float *partial, long B, long N, long M,
                                      int splits, cudaStream_t st) {
  if (!tc_available() || !tc_shape_ok(x, w, N, M) || (reinterpret_cast<uintptr_t>(partial) & 7u)) return cudaErrorNotSupported;
  int plan_splits, k_per_split;
  status_word();
  forward_split_plan(B, N, M, plan_splits, k_per_split);
  if (plan_splits != splits) return cudaErrorInvalidValue;
  TcMaps tm;
  if (!make_map(&tm.a, x, N, B, 32, 128, false) || !make_map(&tm.b, w, M, N, 32, kFwdBK, true)) return cudaErrorInvalidValue;
  tm.a3 = tm.a;
  tm.c = tm.a;
  // CTA pairs when the row tiles pair up: the two CTAs that need the same tile of W each fetch half of it
  const bool pair = pairs_enabled() && ((B + 127) / 128) % 2 == 0;
  const bool b3 = make_map_chunks(&tm.b3, w, M, N, kFwdBK, (pair ? kFwdBN / 2 : kFwdBN) / 32);
  if (!b3) tm.b3 = tm.b;
  tm.alo = tm.blo = tm.a3lo = tm.b3lo = tm.a;
  TcWork wk{(int)((B + 127) / 128), (int)((M + kFwdBN - 1) / kFwdBN), splits, (int)N, k_per_split, 1, 0, 0,
            b3 ? full_chunk_tiles(M, kFwdBN) : 0, kFwdPrefetch, wait_limit_now(), take_lose_arrive(), 0};
#ifdef SBB_TC_TRACE
  if (const char *e = getenv("SBB_FWD_PREFETCH")) wk.b_prefetch = atoi(e);   // timeline builds may vary the distance
#endif
  TcEpilogue ep{};
  ep.out = partial;
  ep.rows = B;
  ep.cols = M;
  ep.ld = M;
  cudaError_t e = pair ? launch_tc_pair<true, kFwdBN, kFwdBK, kFwdStages, false, kFwdChain>(tm, wk, ep, st)
                       : launch_tc<true, kFwdBN, kFwdBK, kFwdStages, false, kFwdChain>(tm, wk, ep, st);
  if (e == cudaSuccess) count_launches(1);
  return e;
}

// Multiplier for n / d by multiply-high, or 0 if it is not exact for every n < limit.
static uint32_t exact_division_magic(long d, long limit) {
  if (d <= 1 || d >= (1L << 31) || limit >= (1L << 31)) return 0;
  const uint64_t magic = ((1ull << 32) + (uint64_t)d - 1) / (uint64_t)d;
  if (magic >> 32) return 0;
  for (long n = 0; n < limit; ++n)
    if ((long)(((uint64_t)n * magic) >> 32) != n / d) return 0;
  return (uint32_t)magic;
}

namespace {
// out = C < cthr ? 0 : 1 / C  for rows [row_begin, row_end) of Ci and every column of Cj: the
// epilogue multiplies by these and reads "below the threshold" off the zero.
__global__ void trace_reciprocals_kernel(const float *__restrict__ Ci, long row_begin, long row_end,
                                         const float *__restrict__ Cj, long M, float cthr, float *__restrict__ rci,
                                         float *__restrict__ rcj) {
  const long rows = row_end - row_begin;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < rows + M; t += (long)gridDim.x * blockDim.x) {
    if (t < rows) {
      const float c = Ci[row_begin + t];
      rci[row_begin + t] = c < cthr ? 0.f : 1.f / c;
    } else {
      const float c = Cj[t - rows];
      rcj[t - rows] = c < cthr ? 0.f : 1.f / c;
    }
  }
}
}  // namespace

namespace {
// Tensor maps of the two MN-major operands x[B, N] and y[B, M] of a batch contraction with `bn`-column tiles, and
// (pre != 0) of their low-part planes.  a3 / b3 report whether the one-box 3-D forms exist.
bool batch_operand_maps(TcMaps &tm, const float *x, const float *y, const float *x_lo, const float *y_lo, bool pre,
                        long B, long N, long M, int bn, bool &a3, bool &b3) {
  if (!make_map(&tm.a, x, N, B, 32, kTrBK, true) || !make_map(&tm.b, y, M, B, 32, kTrBK, true)) return false;
  a3 = N % 32 == 0 && make_map_chunks(&tm.a3, x, N, B, kTrBK, 4);
  if (!a3) tm.a3 = tm.a;
  b3 = make_map_chunks(&tm.b3, y, M, B, kTrBK, bn / 32);
  if (!b3) tm.b3 = tm.b;
  tm.alo = tm.a;
  tm.blo = tm.b;
  tm.a3lo = tm.a3;
  tm.b3lo = tm.b3;
  if (pre) {
    if (!make_map(&tm.alo, x_lo, N, B, 32, kTrBK, true) || !make_map(&tm.blo, y_lo, M, B, 32, kTrBK, true)) return false;
    if (a3 && !make_map_chunks(&tm.a3lo, x_lo, N, B, kTrBK, 4)) return false;
    if (b3 && !make_map_chunks(&tm.b3lo, y_lo, M, B, kTrBK, bn / 32)) return false;
  }
  return true;
}
bool lo_planes_usable(const float *x_lo, const float *y_lo) {
  return x_lo != nullptr && y_lo != nullptr && (reinterpret_cast<uintptr_t>(x_lo) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(y_lo) & 15u) == 0;
}
}  // namespace

size_t tc_trace_scratch_bytes(long N, long M) { return (size_t)(((N + 3) / 4) * 4 + M + 4) * sizeof(float); }

cudaError_t launch_trace_update_tc(const float *x, const float *y, long B, long N, long M, long H, const float *Ci,
                                   const float *Cj, float *Cij, float *w, const uint8_t *wmask, const int *col_hc,
                                   float *scratch, TraceParams<float> p, long row_begin, long row_end,
                                   cudaStream_t st) {
  // verified once per layer shape and host thread
  static thread_local long magic_for_mc = -1, magic_for_m = -1;
  static thread_local uint32_t magic_value = 0;
  uint32_t hc_magic = 0;
  if (wmask != nullptr && H > 0) {
    const long Mc = M / H;
    if (magic_for_mc != Mc || magic_for_m != M) {
      magic_value = exact_division_magic(Mc, M + 2);
      magic_for_mc = Mc;
      magic_for_m = M;
    }
    hc_magic = magic_value;
  }
  if (!tc_available() || !tc_shape_ok(x, y, N, M) || row_begin % 128 != 0) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(Cij) & 7u) || (reinterpret_cast<uintptr_t>(w) & 7u) ||
      scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 15u) ||
      (wmask && (col_hc == nullptr || (reinterpret_cast<uintptr_t>(col_hc) & 7u))))
    return cudaErrorNotSupported;
  if (row_end <= row_begin) return cudaSuccess;
  TcMaps tm;
  bool a3 = false, b3 = false;
  // The fused kernel splits its operands itself (A's parts go to tensor memory): with pre-split planes both
  // operands would come from shared memory, whose bandwidth the Cij blocks of the epilogue also need; measured
  // on the 55296 x 3000 layer the launch takes 0.608 ms that way against 0.587 ms.
  // a batch of more than one chain carries its running sum through the trace matrix (see the kernel)
  const bool multi = B > (long)kTrChainKb * kTrBK;
  // CTA pairs (one 256-row MMA over two SMs, each staging half of the tile's columns of y): single-chain batches
  const bool pair = pairs_enabled();
  // (pairs: y's one-box 3-D map covers half a tile's column chunks)
  if (!batch_operand_maps(tm, x, y, nullptr, nullptr, false, B, N, M, pair ? kTrBN / 2 : kTrBN, a3, b3))
    return cudaErrorInvalidValue;
  if (!make_map(&tm.c, Cij, M, N, 32, 32, false)) return cudaErrorInvalidValue;   // 32 x 32 blocks, 128-byte swizzle
  const long rows = row_end - row_begin;
  const int kper = (int)((B + kTrBK - 1) / kTrBK) * kTrBK;
  // tiles are walked so that the larger operand is the one re-used by consecutive tiles: column tiles
  // fastest when x (B x N) is the larger, row tiles fastest when y (B x M) is
  TcWork wk{(int)((rows + 127) / 128), (int)((M + kTrBN - 1) / kTrBN), 1, (int)B, kper, M > N ? 1 : 0, (int)row_begin,
            a3 ? 1 : 0, b3 ? full_chunk_tiles(M, kTrBN) : 0, 0, wait_limit_now(), take_lose_arrive(), kTrChainKb};
  TcEpilogue ep{};
  ep.rows = rows;
  ep.cols = M;
  float *rci = scratch, *rcj = scratch + ((N + 3) / 4) * 4;
  {
    const long n = rows + M;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    trace_reciprocals_kernel<<<blocks, 256, 0, st>>>(Ci, row_begin, row_end, Cj, M, p.cthr, rci, rcj);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    count_launches(1);
  }
  ep.rci = rci;
  ep.rcj = rcj;
  ep.Cij = Cij;
  ep.W = w;
  ep.wmask = wmask;
  ep.col_hc = col_hc;
  ep.hc_magic = hc_magic;
  ep.H = H;
  ep.Mc = H > 0 ? M / H : M;
  ep.fast_ok = (wmask == nullptr || ep.Mc >= 32) && p.cthr4 >= 1e-30f;
  ep.row0 = row_begin;
  ep.p = p;
  ep.ema_scale = p.taupdt / p.batch;
  cudaError_t e;
  if (pair)
    e = multi ? launch_tc_pair<false, kTrBN, kTrBK, kPairStages, true, 0, true>(tm, wk, ep, st)
              : launch_tc_pair<false, kTrBN, kTrBK, kPairStages, true, 0>(tm, wk, ep, st);
  else
    e = multi ? launch_tc<false, kTrBN, kTrBK, kTrStages, true, 0, true>(tm, wk, ep, st)
              : launch_tc<false, kTrBN, kTrBK, kTrStages, true, 0>(tm, wk, ep, st);
  if (e == cudaSuccess) count_launches(1);
  return e;
}

cudaError_t launch_outer_product_tc(const float *x, const float *y, long B, long N, long M, float *delta,
                                    long row_begin, long row_end, cudaStream_t st, const float *x_lo,
                                    const float *y_lo) {
  if (!tc_available() || !tc_shape_ok(x, y, N, M) || row_begin % 128 != 0 ||
      (reinterpret_cast<uintptr_t>(delta) & 7u))
    return cudaErrorNotSupported;
  if (row_end <= row_begin) return cudaSuccess;
  TcMaps tm;
  const bool pre = lo_planes_usable(x_lo, y_lo);
  const bool longb = B > (long)kTrChainKb * kTrBK;
  bool a3 = false, b3 = false;
  if (!batch_operand_maps(tm, x, y, x_lo, y_lo, pre, B, N, M, longb ? kLongBN : kTrBN, a3, b3)) return cudaErrorInvalidValue;
  tm.c = tm.a;
  const long rows = row_end - row_begin;
  const int kper = (int)((B + kTrBK - 1) / kTrBK) * kTrBK;
  if (longb) {
    // More than one accumulation chain: 128-column tiles whose running sums stay in the epilogue warps'
    // registers (as in the forward product), so no partial sum travels through memory.
    const bool b3n = b3;
    TcWork wk{(int)((rows + 127) / 128), (int)((M + kLongBN - 1) / kLongBN), 1, (int)B, kper, M > N ? 1 : 0,
              (int)row_begin, a3 ? 1 : 0, b3n ? full_chunk_tiles(M, kLongBN) : 0, 0, wait_limit_now(), 0, 0};
    TcEpilogue ep{};
    ep.out = delta + row_begin * M;
    ep.rows = rows;
    ep.cols = M;
    ep.ld = M;
    ep.tma_store = (reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0 && make_map(&tm.c, ep.out, M, rows, 32, 32, false);
    if (!ep.tma_store) tm.c = tm.a;
    cudaError_t e = pre ? launch_tc<false, kLongBN, kTrBK, kLongStages, false, kTrChainKb, false, true>(tm, wk, ep, st, true)
                        : launch_tc<false, kLongBN, kTrBK, kLongStages, false, kTrChainKb>(tm, wk, ep, st, true);
    if (e == cudaSuccess) count_launches(1);
    return e;
  }
  // tiles are walked so that the larger operand is the one re-used by consecutive tiles: column tiles
  // fastest when x (B x N) is the larger, row tiles fastest when y (B x M) is
  TcWork wk{(int)((rows + 127) / 128), (int)((M + kTrBN - 1) / kTrBN), 1, (int)B, kper, M > N ? 1 : 0, (int)row_begin,
            a3 ? 1 : 0, b3 ? full_chunk_tiles(M, kTrBN) : 0, 0, wait_limit_now(), take_lose_arrive(), kTrChainKb};
  TcEpilogue ep{};
  ep.out = delta + row_begin * M;
  ep.rows = rows;
  ep.cols = M;
  ep.ld = M;
  ep.tma_store = (reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0 && make_map(&tm.c, ep.out, M, rows, 32, 32, false);
  if (!ep.tma_store) tm.c = tm.a;
  // the one contraction that runs beside a collective (the reduction of the previous row block)
  cudaError_t e = pre ? launch_tc<false, kTrBN, kTrBK, kTrStages, false, 0, false, true>(tm, wk, ep, st, true)
                      : launch_tc<false, kTrBN, kTrBK, kTrStages, false, 0>(tm, wk, ep, st, true);
  if (e == cudaSuccess) count_launches(1);
  return e;
}


#ifdef SBB_TC_TRACE
extern "C" int sbb_tc_trace_read(unsigned long long *out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(unsigned long long) * 64 * 16);
}
#endif

void tc_set_wait_limit(long long cycles) { g_wait_limit.store(cycles > 0 ? cycles : kWaitLimitCycles); }
long long tc_get_wait_limit() { return g_wait_limit.load(); }
void tc_debug_lose_arrive(int launches) { g_lose_arrive.store(launches > 0 ? launches : 0); }

void tc_set_reserved_sms(int sms) { g_reserved_sms.store(sms < 0 ? 0 : sms); }
int tc_get_reserved_sms() {
  int v = g_reserved_sms.load();
  if (v < 0) {
    const char *e = getenv("SBB_COMM_SMS");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
    g_reserved_sms.store(v);
  }
  return v;
}

// The status word without synchronising the device: meaningful for work the caller has already waited for.
cudaError_t tc_peek_status(int *status) {
  *status = 0;
  const int dev = current_device();
  int *p = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    p = g_status[dev];
  }
  if (p == nullptr) return cudaSuccess;
  return cudaMemcpy(status, p, sizeof(int), cudaMemcpyDeviceToHost);
}

cudaError_t tc_clear_status() {
  const int dev = current_device();
  int *p = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    p = g_status[dev];
  }
  if (p == nullptr) return cudaSuccess;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return e;
  return cudaMemset(p, 0, sizeof(int));
}

cudaError_t tc_read_status(int *status) {
  *status = 0;
  const int dev = current_device();
  int *p = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    p = g_status[dev];
  }
  if (p == nullptr) return cudaSuccess;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return e;
  return cudaMemcpy(status, p, sizeof(int), cudaMemcpyDeviceToHost);
}

}  // namespace sbb
