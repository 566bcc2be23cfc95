// float64 contraction on the FP64 tensor-core instruction (mma.sync.m8n8k4.f64), for shapes whose
// rows start on 16-byte boundaries.  tcgen05 has no float64 kind; mma.sync peaks no higher than DFMA
// on this part, but one instruction carries 256 FMAs, so the issue slots, the shared-memory pipe and
// the register file (32 accumulators per thread instead of 64) are left with room to hide latencies:
// two CTAs of eight warps per SM instead of one.
//
// CTA tile 128 x 64 (eight warps, two CTAs per SM) or 64 x 64 (four warps, three CTAs per SM: for
// launches whose 128-row tiles would leave most of a last wave of CTAs empty), k-slabs of 16 in a
// three-stage cp.async pipeline, warp tile 32 x 32 (4 x 4 instruction tiles).  Shared-memory rows
// are padded so that a half-warp's fragment loads (four rows of four consecutive doubles) fall into
// 16 different bank pairs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sbb {
namespace f64mma {

constexpr int BN = 64, BK = 16, STAGES = 3;
constexpr int LDA_K = BK + 4;   // K-major A in shared memory: [m][k]
constexpr int LDB = BN + 4;     // B: [k][n]
constexpr int B_STAGE = BK * LDB;
template <int BM>
struct Cfg {
  static_assert(BM == 128 || BM == 64, "row tiles of 128 or 64");
  static constexpr int THREADS = BM * 2;        // (BM / 32) x 2 warps
  static constexpr int CTAS_PER_SM = BM == 128 ? 2 : 3;
  static constexpr int LDA_M = BM + 4;          // MN-major A: [k][m]
  static constexpr int A_STAGE = BM * LDA_K > BK * LDA_M ? BM * LDA_K : BK * LDA_M;   // doubles
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * (A_STAGE + B_STAGE) * sizeof(double);
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 16 : 0;   // 0: nothing is read, the destination is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void dmma(double &c0, double &c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// ----------------------------------------------------------------------------
// Natural logarithm of a positive, normal double in about a dozen FP64 instructions (the library's log costs
// several times that, and the fused trace epilogue takes one logarithm per element on the same FP64 pipe that
// feeds the tensor-core instruction).  x = 2^e * m, m in [1, 2); the top seven mantissa bits select c_i = 1 +
// (i + 0.5) / 128; with v_i = 1 / c_i rounded to double, r = m * v_i - 1 (one FMA, |r| < 2^-8) and
//     ln x = e * ln 2 - ln v_i + log1p(r),
// where -ln v_i is tabulated for the rounded v_i itself (so the rounding of v_i costs nothing) and log1p is its
// series up to r^6 (remainder below 2e-18).  Absolute error a few 1e-16 times max(1, |ln x|).  Anything else
// (zero, subnormal, negative, infinite, NaN) goes to the library function.
// ----------------------------------------------------------------------------
// {v_i, -ln v_i}
__device__ const double2 kLogTable[128] = {
    {0x1.fe01fe01fe020p-1, 0x1.ff00aa2b10ba0p-9},    {0x1.fa11caa01fa12p-1, 0x1.7dc475f810a69p-7},
    {0x1.f6310aca0dbb5p-1, 0x1.3cea44346a584p-6},    {0x1.f25f644230ab5p-1, 0x1.b9fc027af919ap-6},
    {0x1.ee9c7f8458e02p-1, 0x1.1b0d98923d97fp-5},    {0x1.eae807aba01ebp-1, 0x1.58a5bafc8e4d3p-5},
    {0x1.e741aa59750e4p-1, 0x1.95c830ec8e3f2p-5},    {0x1.e3a9179dc1a73p-1, 0x1.d276b8adb0b56p-5},
    {0x1.e01e01e01e01ep-1, 0x1.075983598e471p-4},    {0x1.dca01dca01dcap-1, 0x1.253f62f0a1417p-4},
    {0x1.d92f2231e7f8ap-1, 0x1.42edcbea646eep-4},    {0x1.d5cac807572b2p-1, 0x1.60658a93750c4p-4},
    {0x1.d272ca3fc5b1ap-1, 0x1.7da766d7b12d0p-4},    {0x1.cf26e5c44bfc6p-1, 0x1.9ab42462033aep-4},
    {0x1.cbe6d9601cbe7p-1, 0x1.b78c82bb0eda0p-4},    {0x1.c8b265afb8a42p-1, 0x1.d4313d66cb35dp-4},
    {0x1.c5894d10d4986p-1, 0x1.f0a30c01162a4p-4},    {0x1.c26b5392ea01cp-1, 0x1.0671512ca596fp-3},
    {0x1.bf583ee868d8bp-1, 0x1.14785846742acp-3},    {0x1.bc4fd65883e7bp-1, 0x1.2266f190a5acdp-3},
    {0x1.b951e2b18ff23p-1, 0x1.303d718e47fd5p-3},    {0x1.b65e2e3beee05p-1, 0x1.3dfc2b0ecc62ap-3},
    {0x1.b37484ad806cep-1, 0x1.4ba36f39a55e5p-3},    {0x1.b094b31d922a4p-1, 0x1.59338d9982085p-3},
    {0x1.adbe87f94905ep-1, 0x1.66acd4272ad51p-3},    {0x1.aaf1d2f87ebfdp-1, 0x1.740f8f54037a3p-3},
    {0x1.a82e65130e159p-1, 0x1.815c0a14357e9p-3},    {0x1.a574107688a4ap-1, 0x1.8e928de886d41p-3},
    {0x1.a2c2a87c51ca0p-1, 0x1.9bb362e7dfb85p-3},    {0x1.a01a01a01a01ap-1, 0x1.a8becfc882f19p-3},
    {0x1.9d79f176b682dp-1, 0x1.b5b519e8fb5a6p-3},    {0x1.9ae24ea5510dap-1, 0x1.c2968558c18c2p-3},
    {0x1.9852f0d8ec0ffp-1, 0x1.cf6354e09c5ddp-3},    {0x1.95cbb0be377aep-1, 0x1.dc1bca0abec7bp-3},
    {0x1.934c67f9b2ce6p-1, 0x1.e8c0252aa5a60p-3},    {0x1.90d4f120190d5p-1, 0x1.f550a564b7b37p-3},
    {0x1.8e6527af1373fp-1, 0x1.00e6c45ad501dp-2},    {0x1.8bfce8062ff3ap-1, 0x1.071b85fcd590dp-2},
    {0x1.899c0f601899cp-1, 0x1.0d46b579ab74bp-2},    {0x1.87427bcc092b9p-1, 0x1.136870293a8b0p-2},
    {0x1.84f00c2780614p-1, 0x1.1980d2dd4236fp-2},    {0x1.82a4a0182a4a0p-1, 0x1.1f8ff9e48a2f3p-2},
    {0x1.8060180601806p-1, 0x1.2596010df763ap-2},    {0x1.7e225515a4f1dp-1, 0x1.2b9303ab89d25p-2},
    {0x1.7beb3922e017cp-1, 0x1.31871c9544185p-2},    {0x1.79baa6bb6398bp-1, 0x1.3772662bfd85cp-2},
    {0x1.77908119ac60dp-1, 0x1.3d54fa5c1f710p-2},    {0x1.756cac201756dp-1, 0x1.432ef2a04e813p-2},
    {0x1.734f0c541fe8dp-1, 0x1.49006804009d0p-2},    {0x1.713786d9c7c09p-1, 0x1.4ec9732600269p-2},
    {0x1.6f26016f26017p-1, 0x1.548a2c3add263p-2},    {0x1.6d1a62681c861p-1, 0x1.5a42ab0f4cfe2p-2},
    {0x1.6b1490aa31a3dp-1, 0x1.5ff3070a793d4p-2},    {0x1.691473a88d0c0p-1, 0x1.659b57303e1f2p-2},
    {0x1.6719f3601671ap-1, 0x1.6b3bb2235943dp-2},    {0x1.6524f853b4aa3p-1, 0x1.70d42e2789236p-2},
    {0x1.63356b88ac0dep-1, 0x1.7664e1239dbcfp-2},    {0x1.614b36831ae94p-1, 0x1.7bede0a37afbfp-2},
    {0x1.5f66434292dfcp-1, 0x1.816f41da0d495p-2},    {0x1.5d867c3ece2a5p-1, 0x1.86e919a330ba1p-2},
    {0x1.5babcc647fa91p-1, 0x1.8c5b7c858b48bp-2},    {0x1.59d61f123ccaap-1, 0x1.91c67eb45a83ep-2},
    {0x1.5805601580560p-1, 0x1.972a341135159p-2},    {0x1.56397ba7c52e2p-1, 0x1.9c86b02dc0862p-2},
    {0x1.54725e6bb82fep-1, 0x1.a1dc064d5b995p-2},    {0x1.52aff56a8054bp-1, 0x1.a72a4966bd9e9p-2},
    {0x1.50f22e111c4c5p-1, 0x1.ac718c258b0e5p-2},    {0x1.4f38f62dd4c9bp-1, 0x1.b1b1e0ebdfc5ap-2},
    {0x1.4d843bedc2c4cp-1, 0x1.b6eb59d3cf35cp-2},    {0x1.4bd3edda68fe1p-1, 0x1.bc1e08b0dad0ap-2},
    {0x1.4a27fad76014ap-1, 0x1.c149ff115f027p-2},    {0x1.4880522014880p-1, 0x1.c66f4e3ff6ff9p-2},
    {0x1.46dce34596066p-1, 0x1.cb8e0744d7acap-2},    {0x1.453d9e2c776cap-1, 0x1.d0a63ae721e64p-2},
    {0x1.43a2730abee4dp-1, 0x1.d5b7f9ae2c684p-2},    {0x1.420b5265e5951p-1, 0x1.dac353e2c5955p-2},
    {0x1.40782d10e6566p-1, 0x1.dfc859906d5b5p-2},    {0x1.3ee8f42a5af07p-1, 0x1.e4c71a8687704p-2},
    {0x1.3d5d991aa75c6p-1, 0x1.e9bfa659861f5p-2},    {0x1.3bd60d9232955p-1, 0x1.eeb20c640ddf3p-2},
    {0x1.3a524387ac822p-1, 0x1.f39e5bc811e5dp-2},    {0x1.38d22d366088ep-1, 0x1.f884a36fe9ec1p-2},
    {0x1.3755bd1c945eep-1, 0x1.fd64f20f61571p-2},    {0x1.35dce5f9f2af8p-1, 0x1.011fab125ff8ap-1},
    {0x1.34679ace01346p-1, 0x1.0389eefce633cp-1},    {0x1.32f5ced6a1dfap-1, 0x1.05f14bd26459cp-1},
    {0x1.3187758e9ebb6p-1, 0x1.0855c884b450ep-1},    {0x1.301c82ac40260p-1, 0x1.0ab76bece14d2p-1},
    {0x1.2eb4ea1fed14bp-1, 0x1.0d163ccb9d6b8p-1},    {0x1.2d50a012d50a0p-1, 0x1.0f7241c9b497dp-1},
    {0x1.2bef98e5a3711p-1, 0x1.11cb81787ccf8p-1},    {0x1.2a91c92f3c105p-1, 0x1.1422025243d45p-1},
    {0x1.293725bb804a5p-1, 0x1.1675cababa60ep-1},    {0x1.27dfa38a1ce4dp-1, 0x1.18c6e0ff5cf07p-1},
    {0x1.268b37cd60127p-1, 0x1.1b154b57da29ep-1},    {0x1.2539d7e9177b2p-1, 0x1.1d610fe677003p-1},
    {0x1.23eb79717605bp-1, 0x1.1faa34b87094cp-1},    {0x1.22a0122a0122ap-1, 0x1.21f0bfc65beecp-1},
    {0x1.21579804855e6p-1, 0x1.2434b6f483934p-1},    {0x1.2012012012012p-1, 0x1.26762013430e0p-1},
    {0x1.1ecf43c7fb84cp-1, 0x1.28b500df60783p-1},    {0x1.1d8f5672e4abdp-1, 0x1.2af15f02640acp-1},
    {0x1.1c522fc1ce059p-1, 0x1.2d2b4012edc9dp-1},    {0x1.1b17c67f2bae3p-1, 0x1.2f62a99509546p-1},
    {0x1.19e0119e0119ep-1, 0x1.3197a0fa7fe6ap-1},    {0x1.18ab083902bdbp-1, 0x1.33ca2ba328994p-1},
    {0x1.1778a191bd684p-1, 0x1.35fa4edd36ea0p-1},    {0x1.1648d50fc3201p-1, 0x1.38280fe58797fp-1},
    {0x1.151b9a3fdd5c9p-1, 0x1.3a5373e7ebdf9p-1},    {0x1.13f0e8d344724p-1, 0x1.3c7c7fff73206p-1},
    {0x1.12c8b89edc0acp-1, 0x1.3ea33936b2f5bp-1},    {0x1.11a3019a74826p-1, 0x1.40c7a4880dceap-1},
    {0x1.107fbbe011080p-1, 0x1.42e9c6ddf80bfp-1},    {0x1.0f5edfab325a2p-1, 0x1.4509a5133bb0ap-1},
    {0x1.0e40655826011p-1, 0x1.472743f33aaadp-1},    {0x1.0d24456359e3ap-1, 0x1.4942a83a2fc07p-1},
    {0x1.0c0a7868b4171p-1, 0x1.4b5bd6956e273p-1},    {0x1.0af2f722eecb5p-1, 0x1.4d72d3a39fd01p-1},
    {0x1.09ddba6af8360p-1, 0x1.4f87a3f5026e9p-1},    {0x1.08cabb37565e2p-1, 0x1.519a4c0ba3446p-1},
    {0x1.07b9f29b8eae2p-1, 0x1.53aad05b99b7cp-1},    {0x1.06ab59c7912fbp-1, 0x1.55b9354b40bcep-1},
    {0x1.059eea0727586p-1, 0x1.57c57f336f191p-1},    {0x1.04949cc1664c5p-1, 0x1.59cfb25fae87fp-1},
    {0x1.038c6b78247fcp-1, 0x1.5bd7d30e71c73p-1},    {0x1.02864fc7729e9p-1, 0x1.5ddde57149923p-1},
    {0x1.0182436517a37p-1, 0x1.5fe1edad18919p-1},    {0x1.0080402010080p-1, 0x1.61e3efda46467p-1},
};

__device__ __forceinline__ double log_positive(double x) {
  const int hi = __double2hiint(x);
  if ((unsigned)hi - 0x00100000u >= 0x7FE00000u) return log(x);
  const int e = (hi >> 20) - 1023;
  const double m = __hiloint2double((hi & 0x000FFFFF) | 0x3FF00000, __double2loint(x));
  const double2 t = __ldg(&kLogTable[(hi >> 13) & 127]);
  const double r = fma(m, t.x, -1.0);
  double q = fma(r, -1.0 / 6.0, 1.0 / 5.0);
  q = fma(r, q, -1.0 / 4.0);
  q = fma(r, q, 1.0 / 3.0);
  q = fma(r, q, -1.0 / 2.0);
  q = fma(r * r, q, r);   // log1p(r)
  return fma((double)e, 0.693147180559945309417232, t.y + q);
}

// One k-slab of both operands into stage buffers As / Bs (zero-filled outside the operands).
// A is [K x Mdim] MN-major (element (k, m) at A[k*lda + m]) or, A_KMAJOR, [Mdim x K] (at A[m*lda + k]);
// B is [K x Ndim] MN-major.  All row starts and the 2-element chunks are 16-byte aligned (checked by the host).
template <bool A_KMAJOR, int BM>
__device__ __forceinline__ void load_slab(double *As, double *Bs, const double *__restrict__ A, long lda,
                                          const double *__restrict__ Bm, long ldb, long m0, long Mdim, long n0,
                                          long Ndim, int k0, int kend) {
  constexpr int THREADS = Cfg<BM>::THREADS, LDA_M = Cfg<BM>::LDA_M;
  const int tid = threadIdx.x;
  if constexpr (A_KMAJOR) {
#pragma unroll
    for (int t = 0; t < BM * (BK / 2) / THREADS; ++t) {
      const int v = tid + t * THREADS;
      const int r = v / (BK / 2), c = (v % (BK / 2)) * 2;
      const long m = m0 + r;
      const int k = k0 + c;
      const bool ok = m < Mdim && k < kend;
      cp_async16(As + r * LDA_K + c, ok ? A + m * lda + k : A, ok);
    }
  } else {
#pragma unroll
    for (int t = 0; t < BK * (BM / 2) / THREADS; ++t) {
      const int v = tid + t * THREADS;
      const int r = v / (BM / 2), c = (v % (BM / 2)) * 2;
      const int k = k0 + r;
      const long m = m0 + c;
      const bool ok = k < kend && m < Mdim;
      cp_async16(As + r * LDA_M + c, ok ? A + (long)k * lda + m : A, ok);
    }
  }
#pragma unroll
  for (int t = 0; t < BK * (BN / 2) / THREADS; ++t) {
    const int v = tid + t * THREADS;
    const int r = v / (BN / 2), c = (v % (BN / 2)) * 2;
    const int k = k0 + r;
    const long n = n0 + c;
    const bool ok = k < kend && n < Ndim;
    cp_async16(Bs + r * LDB + c, ok ? Bm + (long)k * ldb + n : Bm, ok);
  }
}

// grid.x = row tiles of the output, grid.y = column tiles (swapped when cols_fastest), grid.z = k-splits.
// k-split z covers [z*kper, min(K, (z+1)*kper)), kper a multiple of BK.  The epilogue receives the thread's
// accumulators: ep.tile(acc, m, n, z) with acc[mi][ni][e] = output element (m + 8*mi, n + 8*ni + e), n even;
// ep.prefetch(m, n, lane) is called before the main loop with the first element of the warp's 32 x 32 block.
template <bool A_KMAJOR, int BM, class Epilogue>
__global__ void __launch_bounds__(Cfg<BM>::THREADS, Cfg<BM>::CTAS_PER_SM)
    contraction_kernel(const double *__restrict__ A, long lda, const double *__restrict__ Bm, long ldb, long Mdim,
                       long Ndim, int K, int kper, bool cols_fastest, Epilogue ep) {
  constexpr int A_STAGE = Cfg<BM>::A_STAGE, LDA_M = Cfg<BM>::LDA_M;
  extern __shared__ __align__(16) double smem[];
  double *As = smem, *Bs = smem + STAGES * A_STAGE;
  const long m0 = (long)(cols_fastest ? blockIdx.y : blockIdx.x) * BM;
  const long n0 = (long)(cols_fastest ? blockIdx.x : blockIdx.y) * BN;
  const int kbeg = blockIdx.z * kper;
  const int kend = min(K, kbeg + kper);
  const int nk = kend > kbeg ? (kend - kbeg + BK - 1) / BK : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp % (BM / 32)) * 32, wn = (warp / (BM / 32)) * 32;   // the warp's 32 x 32 block of the tile
  const int g = lane >> 2, t = lane & 3;

  double acc[4][4][2];
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;

  ep.prefetch(m0 + wm, n0 + wn, lane);
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load_slab<A_KMAJOR, BM>(As + s * A_STAGE, Bs + s * B_STAGE, A, lda, Bm, ldb, m0, Mdim, n0, Ndim, kbeg + s * BK, kend);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();   // slab kt has landed (for this thread's copies; the barrier covers the others')
    __syncthreads();               // ... and everyone has finished with the stage refilled below
    {
      const int nx = kt + STAGES - 1;
      if (nx < nk) {
        const int s = nx % STAGES;
        load_slab<A_KMAJOR, BM>(As + s * A_STAGE, Bs + s * B_STAGE, A, lda, Bm, ldb, m0, Mdim, n0, Ndim, kbeg + nx * BK, kend);
      }
      cp_async_commit();
    }
    const double *as = As + (kt % STAGES) * A_STAGE;
    const double *bs = Bs + (kt % STAGES) * B_STAGE;
#pragma unroll
    for (int kk = 0; kk < BK / 4; ++kk) {
      double a[4], b[4];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
        a[mi] = A_KMAJOR ? as[(wm + mi * 8 + g) * LDA_K + kk * 4 + t] : as[(kk * 4 + t) * LDA_M + wm + mi * 8 + g];
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) b[ni] = bs[(kk * 4 + t) * LDB + wn + ni * 8 + g];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) dmma(acc[mi][ni][0], acc[mi][ni][1], a[mi], b[ni]);
    }
  }
  cp_async_wait<0>();
  ep.tile(acc, m0 + wm + g, n0 + wn + 2 * t, (int)blockIdx.z);
}

}  // namespace f64mma
}  // namespace sbb
