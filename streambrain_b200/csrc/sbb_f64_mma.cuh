// float64 contraction on the FP64 tensor-core instruction (mma.sync.m8n8k4.f64), for shapes whose
// rows start on 16-byte boundaries.  tcgen05 has no float64 kind; mma.sync peaks no higher than DFMA
// on this part, but one instruction carries 256 FMAs, so the issue slots, the shared-memory pipe and
// the register file (32 accumulators per thread instead of 64) are left with room to hide latencies:
// two CTAs of eight warps per SM instead of one.
//
// CTA tile 128 x 64, k-slabs of 16 in a three-stage cp.async pipeline, warp tile 32 x 32 (4 x 4
// instruction tiles).  Shared-memory rows are padded so that a half-warp's fragment loads (four
// rows of four consecutive doubles) fall into 16 different bank pairs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sbb {
namespace f64mma {

constexpr int BM = 128, BN = 64, BK = 16, STAGES = 3, THREADS = 256;
constexpr int LDA_K = BK + 4;   // K-major A in shared memory: [m][k]
constexpr int LDA_M = BM + 4;   // MN-major A: [k][m]
constexpr int LDB = BN + 4;     // B: [k][n]
constexpr int A_STAGE = BM * LDA_K > BK * LDA_M ? BM * LDA_K : BK * LDA_M;   // doubles
constexpr int B_STAGE = BK * LDB;
constexpr size_t SMEM_BYTES = (size_t)STAGES * (A_STAGE + B_STAGE) * sizeof(double);

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

// One k-slab of both operands into stage buffers As / Bs (zero-filled outside the operands).
// A is [K x Mdim] MN-major (element (k, m) at A[k*lda + m]) or, A_KMAJOR, [Mdim x K] (at A[m*lda + k]);
// B is [K x Ndim] MN-major.  All row starts and the 2-element chunks are 16-byte aligned (checked by the host).
template <bool A_KMAJOR>
__device__ __forceinline__ void load_slab(double *As, double *Bs, const double *__restrict__ A, long lda,
                                          const double *__restrict__ Bm, long ldb, long m0, long Mdim, long n0,
                                          long Ndim, int k0, int kend) {
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
// k-split z covers [z*kper, min(K, (z+1)*kper)), kper a multiple of BK.  The epilogue receives every
// accumulator pair: ep.pair(m, n, c0, c1, z) for output elements (m, n) and (m, n + 1), n even.
template <bool A_KMAJOR, class Epilogue>
__global__ void __launch_bounds__(THREADS, 2)
    contraction_kernel(const double *__restrict__ A, long lda, const double *__restrict__ Bm, long ldb, long Mdim,
                       long Ndim, int K, int kper, bool cols_fastest, Epilogue ep) {
  extern __shared__ __align__(16) double smem[];
  double *As = smem, *Bs = smem + STAGES * A_STAGE;
  const long m0 = (long)(cols_fastest ? blockIdx.y : blockIdx.x) * BM;
  const long n0 = (long)(cols_fastest ? blockIdx.x : blockIdx.y) * BN;
  const int kbeg = blockIdx.z * kper;
  const int kend = min(K, kbeg + kper);
  const int nk = kend > kbeg ? (kend - kbeg + BK - 1) / BK : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;   // the warp's 32 x 32 block of the tile
  const int g = lane >> 2, t = lane & 3;

  double acc[4][4][2];
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load_slab<A_KMAJOR>(As + s * A_STAGE, Bs + s * B_STAGE, A, lda, Bm, ldb, m0, Mdim, n0, Ndim, kbeg + s * BK, kend);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();   // slab kt has landed (for this thread's copies; the barrier covers the others')
    __syncthreads();               // ... and everyone has finished with the stage refilled below
    {
      const int nx = kt + STAGES - 1;
      if (nx < nk) {
        const int s = nx % STAGES;
        load_slab<A_KMAJOR>(As + s * A_STAGE, Bs + s * B_STAGE, A, lda, Bm, ldb, m0, Mdim, n0, Ndim, kbeg + nx * BK, kend);
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
  ep.begin(m0 + wm + g, n0 + wn + 2 * t);
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
      ep.pair(mi, ni, m0 + wm + mi * 8 + g, n0 + wn + ni * 8 + 2 * t, acc[mi][ni][0], acc[mi][ni][1], (int)blockIdx.z);
}

}  // namespace f64mma
}  // namespace sbb
