// General-shape CUDA kernels of the BCPNN layer train step (float and double).
//
// These are the kernels that accept any N, M, B (odd sizes, unaligned rows, the
// 10-column classifier) and the float64 path; the tcgen05 tile kernels for
// aligned float32 shapes live in their own translation unit and share the
// arithmetic helpers below.
//
// Data layout: every matrix is row-major and contiguous.  x[B,N], y[B,M],
// weights/Cij[N,M], wmask[N,H] bytes.  Both contractions of the step read their
// operands "MN-major" (contiguous along the output dimension) except the forward
// product's x, which is contiguous along the reduction dimension and is
// transposed on its way into shared memory.
#include "sbb_kernels.cuh"
#include "sbb_f64_mma.cuh"
#include "sbb_math.cuh"

#include <atomic>
#include <math.h>

namespace sbb {

static std::atomic<unsigned long long> g_launches{0};
unsigned long long kernel_launches() { return g_launches.load(); }
void count_launches(int n) { g_launches += (unsigned long long)n; }
static inline cudaError_t launched(int n = 1) {
  g_launches += (unsigned long long)n;
  return cudaGetLastError();
}

template <typename T>
TraceParams<T> make_trace_params(double taupdt, double cthr, long batch) {
  TraceParams<T> p;
  p.taupdt = (T)taupdt;
  // The reference forms (1.0 - taupdt) in double from the REAL-rounded taupdt and
  // rounds the result to REAL (kernels_openmp_internal.cc:101).
  p.one_minus = (T)(1.0 - (double)p.taupdt);
  p.batch = (T)batch;
  p.cthr = (T)cthr;
  p.cthr4 = p.cthr * p.cthr * p.cthr * p.cthr;
  return p;
}
template TraceParams<float> make_trace_params<float>(double, double, long);
template TraceParams<double> make_trace_params<double>(double, double, long);

// ----------------------------------------------------------------------------
// 16-byte vector helpers.
// ----------------------------------------------------------------------------
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  using type = float4;
  static constexpr int N = 4;
};
template <>
struct Vec16<double> {
  using type = double2;
  static constexpr int N = 2;
};

__device__ __forceinline__ void unpack(const float4 &v, float *r) {
  r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
}
__device__ __forceinline__ void unpack(const double2 &v, double *r) {
  r[0] = v.x; r[1] = v.y;
}
__device__ __forceinline__ float4 pack(const float *r) { return make_float4(r[0], r[1], r[2], r[3]); }
__device__ __forceinline__ double2 pack(const double *r) { return make_double2(r[0], r[1]); }

// Four consecutive elements from / to memory.  `vec` says the address is 16-byte
// aligned and all four are in range; otherwise `valid` (1..4) elements are touched.
__device__ __forceinline__ void load4(const float *p, float *r, bool vec, int valid) {
  if (vec && valid == 4) {
    unpack(*reinterpret_cast<const float4 *>(p), r);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) r[c] = c < valid ? p[c] : 0.f;
  }
}
__device__ __forceinline__ void load4(const double *p, double *r, bool vec, int valid) {
  if (vec && valid == 4) {
    unpack(*reinterpret_cast<const double2 *>(p), r);
    unpack(*reinterpret_cast<const double2 *>(p + 2), r + 2);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) r[c] = c < valid ? p[c] : 0.0;
  }
}
__device__ __forceinline__ void store4(float *p, const float *r, bool vec, int valid) {
  if (vec && valid == 4) {
    *reinterpret_cast<float4 *>(p) = pack(r);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (c < valid) p[c] = r[c];
  }
}
__device__ __forceinline__ void store4(double *p, const double *r, bool vec, int valid) {
  if (vec && valid == 4) {
    *reinterpret_cast<double2 *>(p) = pack(r);
    *reinterpret_cast<double2 *>(p + 2) = pack(r + 2);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (c < valid) p[c] = r[c];
  }
}

// One group of a micro-tile row (four floats / two doubles) from / to memory, same contract as load4 / store4.
__device__ __forceinline__ void loadg(const float *p, float *r, bool vec, int valid) { load4(p, r, vec, valid); }
__device__ __forceinline__ void storeg(float *p, const float *r, bool vec, int valid) { store4(p, r, vec, valid); }
__device__ __forceinline__ void loadg(const double *p, double *r, bool vec, int valid) {
  if (vec && valid == 2) {
    unpack(*reinterpret_cast<const double2 *>(p), r);
  } else {
#pragma unroll
    for (int c = 0; c < 2; ++c) r[c] = c < valid ? p[c] : 0.0;
  }
}
__device__ __forceinline__ void storeg(double *p, const double *r, bool vec, int valid) {
  if (vec && valid == 2) {
    *reinterpret_cast<double2 *>(p) = pack(r);
  } else {
#pragma unroll
    for (int c = 0; c < 2; ++c)
      if (c < valid) p[c] = r[c];
  }
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ----------------------------------------------------------------------------
// Tiled contraction core: C[Mdim, Ndim] (+)= A^T-or-A * B over k in [k0, k1).
// 128x128 output tile per 256-thread CTA, 8x8 micro-tile per thread split into
// two 4-wide halves in each dimension (rows ty*4+r and 64+ty*4+r; columns
// tx*4+c and 64+tx*4+c) so shared-memory reads are conflict-free 16-byte loads
// and global stores are 16 bytes per thread, 256 contiguous bytes per half-warp.
// The next k-slab is fetched into registers while the current one is multiplied.
// ----------------------------------------------------------------------------
template <typename T>
struct Tile {
  static constexpr int BM = 128, BN = 128, THREADS = 256;
  static constexpr int BK = sizeof(T) == 4 ? 16 : 8;
  static constexpr int LD = 128 + 4;                // shared row stride, elements
  static constexpr int EPT = BK * 128 / THREADS;    // elements per thread per operand slab
};

// Operand stored "MN-major": element (k, m) at p[k*ld + m].
template <typename T, int VEC>
__device__ __forceinline__ void load_mn(T (&r)[Tile<T>::EPT], const T *__restrict__ p, long ld, int k0, int k1,
                                        long m0, long mn) {
  constexpr int VPR = 128 / VEC;
#pragma unroll
  for (int t = 0; t < Tile<T>::EPT / VEC; ++t) {
    const int v = threadIdx.x + t * Tile<T>::THREADS;
    const int k = k0 + v / VPR;
    const long m = m0 + (long)(v % VPR) * VEC;
    const bool ok = k < k1 && m < mn;
    if constexpr (VEC == 1) {
      r[t] = ok ? __ldg(p + (long)k * ld + m) : (T)0;
    } else {
      using V = typename Vec16<T>::type;
      if (ok) {
        unpack(__ldg(reinterpret_cast<const V *>(p + (long)k * ld + m)), &r[t * VEC]);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) r[t * VEC + e] = (T)0;
      }
    }
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_mn(T *s, const T (&r)[Tile<T>::EPT]) {
  constexpr int VPR = 128 / VEC;
#pragma unroll
  for (int t = 0; t < Tile<T>::EPT / VEC; ++t) {
    const int v = threadIdx.x + t * Tile<T>::THREADS;
    const int k = v / VPR;
    const int m = (v % VPR) * VEC;
    if constexpr (VEC == 1) {
      s[k * Tile<T>::LD + m] = r[t];
    } else {
      using V = typename Vec16<T>::type;
      *reinterpret_cast<V *>(s + k * Tile<T>::LD + m) = pack(&r[t * VEC]);
    }
  }
}

// Operand stored "K-major": element (k, m) at p[m*ld + k]; transposed into shared.
template <typename T, int VEC>
__device__ __forceinline__ void load_km(T (&r)[Tile<T>::EPT], const T *__restrict__ p, long ld, int k0, int k1,
                                        long m0, long mn) {
  constexpr int VPR = Tile<T>::BK / VEC;
#pragma unroll
  for (int t = 0; t < Tile<T>::EPT / VEC; ++t) {
    const int v = threadIdx.x + t * Tile<T>::THREADS;
    const long m = m0 + v / VPR;
    const int k = k0 + (v % VPR) * VEC;
    const bool ok = m < mn && k < k1;
    if constexpr (VEC == 1) {
      r[t] = ok ? __ldg(p + m * ld + k) : (T)0;
    } else {
      using V = typename Vec16<T>::type;
      if (ok) {
        unpack(__ldg(reinterpret_cast<const V *>(p + m * ld + k)), &r[t * VEC]);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) r[t * VEC + e] = (T)0;
      }
    }
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_km(T *s, const T (&r)[Tile<T>::EPT]) {
  constexpr int VPR = Tile<T>::BK / VEC;
#pragma unroll
  for (int t = 0; t < Tile<T>::EPT / VEC; ++t) {
    const int v = threadIdx.x + t * Tile<T>::THREADS;
    const int m = v / VPR;
    const int k = (v % VPR) * VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) s[(k + e) * Tile<T>::LD + m] = r[t * VEC + e];
  }
}

__device__ __forceinline__ void lds4(const float *p, float *r) { unpack(*reinterpret_cast<const float4 *>(p), r); }
__device__ __forceinline__ void lds4(const double *p, double *r) {
  unpack(*reinterpret_cast<const double2 *>(p), r);
  unpack(*reinterpret_cast<const double2 *>(p + 2), r + 2);
}

// Columns of a thread's micro-tile.  A thread owns 8 columns as groups of one 16-byte vector each: float32
// two groups of four (columns g*64 + tx*4 ..), float64 four groups of two (columns g*32 + tx*2 ..), so that
// the 16 threads of a half-warp read (and later store) contiguous 16-byte pieces: 256 bytes per request, no
// shared-memory bank conflicts.  (With four doubles per thread and group the 16-byte reads of a half-warp sat
// 32 bytes apart: two-way conflicts on 40 % of the wavefronts of the float64 kernels.)
template <typename T>
struct MicroCols {
  static constexpr int GW = 16 / (int)sizeof(T);   // columns per group
  static constexpr int NG = 8 / GW;                // groups per thread
  static constexpr int STRIDE = 128 / NG;          // columns between the starts of a thread's groups
  __device__ static __forceinline__ int group_start(int tx, int g) { return g * STRIDE + tx * GW; }
  __device__ static __forceinline__ int col(int tx, int e) { return group_start(tx, e / GW) + e % GW; }
};
__device__ __forceinline__ void ldsv(const float *p, float *r) { unpack(*reinterpret_cast<const float4 *>(p), r); }
__device__ __forceinline__ void ldsv(const double *p, double *r) { unpack(*reinterpret_cast<const double2 *>(p), r); }

template <typename T>
__device__ __forceinline__ void multiply_slab(const T *As, const T *Bs, T (&acc)[8][8], int ty, int tx) {
  using MC = MicroCols<T>;
#pragma unroll
  for (int k = 0; k < Tile<T>::BK; ++k) {
    T a[8], b[8];
    lds4(As + k * Tile<T>::LD + ty * 4, a);
    lds4(As + k * Tile<T>::LD + 64 + ty * 4, a + 4);
#pragma unroll
    for (int g = 0; g < MC::NG; ++g) ldsv(Bs + k * Tile<T>::LD + MC::group_start(tx, g), b + g * MC::GW);
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[r][c] = fma(a[r], b[c], acc[r][c]);
  }
}

// Row / column of micro-tile entry e (0..7) inside the 128-wide tile.
__device__ __forceinline__ int micro_index(int t, int e) { return (e < 4 ? 0 : 64) + t * 4 + (e & 3); }

// grid.x = row tiles of the output, grid.y = column tiles (swapped when cols_fastest), grid.z = k-splits.
// A is [K x Mdim] MN-major (A_KMAJOR=false) or [Mdim x K] K-major (true); B is
// [K x Ndim] MN-major.  k-split z covers [z*kper, min(K,(z+1)*kper)), kper a
// multiple of the slab depth.
template <typename T, bool A_KMAJOR, int VEC, class Epilogue>
__global__ void __launch_bounds__(256, sizeof(T) == 4 ? 2 : 1)
    contraction_kernel(const T *__restrict__ A, long lda, const T *__restrict__ Bm, long ldb, long Mdim, long Ndim,
                       int K, int kper, bool cols_fastest, Epilogue ep) {
  using TL = Tile<T>;
  __shared__ __align__(16) T As[2][TL::BK * TL::LD];
  __shared__ __align__(16) T Bs[2][TL::BK * TL::LD];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // Rasterisation: the fastest grid dimension walks the tiles that share the larger re-used operand.
  const long m0 = (long)(cols_fastest ? blockIdx.y : blockIdx.x) * TL::BM;
  const long n0 = (long)(cols_fastest ? blockIdx.x : blockIdx.y) * TL::BN;
  const int kbeg = blockIdx.z * kper;
  const int kend = min(K, kbeg + kper);

  T acc[8][8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[r][c] = (T)0;

  T ra[TL::EPT], rb[TL::EPT];
  if (kbeg < kend) {
    if constexpr (A_KMAJOR) load_km<T, VEC>(ra, A, lda, kbeg, kend, m0, Mdim);
    else load_mn<T, VEC>(ra, A, lda, kbeg, kend, m0, Mdim);
    load_mn<T, VEC>(rb, Bm, ldb, kbeg, kend, n0, Ndim);
    if constexpr (A_KMAJOR) store_km<T, VEC>(As[0], ra);
    else store_mn<T, VEC>(As[0], ra);
    store_mn<T, VEC>(Bs[0], rb);
  }
  __syncthreads();
  int buf = 0;
  for (int k0 = kbeg; k0 < kend; k0 += TL::BK) {
    const int kn = k0 + TL::BK;
    const bool more = kn < kend;
    if (more) {
      if constexpr (A_KMAJOR) load_km<T, VEC>(ra, A, lda, kn, kend, m0, Mdim);
      else load_mn<T, VEC>(ra, A, lda, kn, kend, m0, Mdim);
      load_mn<T, VEC>(rb, Bm, ldb, kn, kend, n0, Ndim);
    }
    multiply_slab<T>(As[buf], Bs[buf], acc, ty, tx);
    if (more) {
      if constexpr (A_KMAJOR) store_km<T, VEC>(As[buf ^ 1], ra);
      else store_mn<T, VEC>(As[buf ^ 1], ra);
      store_mn<T, VEC>(Bs[buf ^ 1], rb);
    }
    __syncthreads();
    buf ^= 1;
  }
  ep(acc, m0, n0, ty, tx, (int)blockIdx.z);
}

// Epilogue: partial[z, m, n] = acc  (forward product) or delta[m, n] = acc.
template <typename T>
struct StoreEpilogue {
  T *out;
  long rows, cols;   // logical extent of one [rows, cols] slice
  long ld;           // row stride of out
  long zstride;      // elements between k-split slices
  bool vec;
  __device__ __forceinline__ void operator()(T (&acc)[8][8], long m0, long n0, int ty, int tx, int z) const {
    T *base = out + (long)z * zstride;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const long m = m0 + micro_index(ty, r);
      if (m >= rows) continue;
#pragma unroll
      for (int g = 0; g < MicroCols<T>::NG; ++g) {
        constexpr int GW = MicroCols<T>::GW;
        const long n = n0 + MicroCols<T>::group_start(tx, g);
        const long left = cols - n;
        if (left <= 0) continue;
        storeg(base + m * ld + n, &acc[r][g * GW], vec, left >= GW ? GW : (int)left);
      }
    }
  }
};

// Epilogue of the fused trace step: moving average of Cij, log-ratio weight,
// threshold and mask zeroing.  Each Cij element is read once and written once.
template <typename T>
struct TraceEpilogue {
  const T *Ci;
  const T *Cj;
  T *Cij;
  T *W;
  const uint8_t *wmask;  // [N, H] or null
  long row0;             // global row of tile row 0
  long row_end;          // global row limit
  long M, H, Mc;
  TraceParams<T> p;
  bool vec;
  __device__ __forceinline__ void operator()(T (&acc)[8][8], long m0, long n0, int ty, int tx, int) const {
    T cj[8];
    int hc[8];
    bool cj_low[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const long j = n0 + MicroCols<T>::col(tx, c);
      const bool in = j < M;
      cj[c] = in ? Cj[j] : (T)1;
      cj_low[c] = cj[c] < p.cthr;
      hc[c] = in ? (int)(j / Mc) : 0;
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const long i = row0 + m0 + micro_index(ty, r);
      if (i >= row_end) continue;
      const T ci = Ci[i];
      const bool skip = ci < p.cthr;
      const uint8_t *mrow = wmask ? wmask + i * H : nullptr;
#pragma unroll
      for (int g = 0; g < MicroCols<T>::NG; ++g) {
        constexpr int GW = MicroCols<T>::GW;
        const long j = n0 + MicroCols<T>::group_start(tx, g);
        const long left = M - j;
        if (left <= 0) continue;
        const int valid = left >= GW ? GW : (int)left;
        T c4[GW], w4[GW];
        loadg(Cij + i * M + j, c4, vec, valid);
#pragma unroll
        for (int c = 0; c < GW; ++c) {
          if (c < valid) {
            const T cij = trace_ema(c4[c], acc[r][g * GW + c], p);
            c4[c] = cij;
            T w = (T)0;
            if (!skip && !cj_low[g * GW + c] && (mrow == nullptr || mrow[hc[g * GW + c]] != 0))
              w = log_ratio(cij, ci, cj[g * GW + c], p.cthr4);
            w4[c] = w;
          }
        }
        storeg(Cij + i * M + j, c4, vec, valid);
        storeg(W + i * M + j, w4, vec, valid);
      }
    }
  }
};

// ----------------------------------------------------------------------------
// float64 on the FP64 tensor-core instruction (sbb_f64_mma.cuh): the same two epilogues, fed with the
// accumulator pairs of the mma.sync fragment layout (element (m, n) and (m, n + 1), n even).
// ----------------------------------------------------------------------------
struct StorePairs {
  double *out;
  long rows, cols, ld, zstride;
  bool vec;
  __device__ __forceinline__ void prefetch(long, long, int) const {}
  __device__ __forceinline__ void tile(const double (&acc)[4][4][2], long m_first, long n_first, int z) const {
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
      const long m = m_first + mi * 8;
      if (m >= rows) continue;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const long n = n_first + ni * 8;
        if (n >= cols) continue;
        double *p = out + (long)z * zstride + m * ld + n;
        if (vec) {
          *reinterpret_cast<double2 *>(p) = make_double2(acc[mi][ni][0], acc[mi][ni][1]);   // cols is even
        } else {
          p[0] = acc[mi][ni][0];
          if (n + 1 < cols) p[1] = acc[mi][ni][1];
        }
      }
    }
  }
};

// The fused trace epilogue on accumulator pairs.  Its memory accesses are what it waits for, so they are
// arranged in two phases: first every load the thread needs (its 16 pairs of the old trace, the mask bytes,
// Ci and Cj; the trace block was requested into L2 before the main loop), folded into the accumulators as
// they arrive; then the arithmetic and the stores.  With a load, a logarithm and two stores per pair in turn,
// the sixteen dependent memory round trips per thread left the tensor pipe idle half of the time.
struct TracePairs {
  const double *Ci, *Cj;
  double *Cij, *W;
  const uint8_t *wmask;
  long row0, row_end, M, H, Mc;
  TraceParams<double> p;
  double inv_batch;
  bool vec;
  __device__ __forceinline__ void prefetch(long m_warp, long n_warp, int lane) const {
    // the warp's 32 x 32 block of Cij: 256 bytes per row, two 128-byte lines, one request per line
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int line = lane + 32 * k;
      const long i = row0 + m_warp + (line >> 1), n = n_warp + (line & 1) * 16;
      if (i < row_end && n < M) asm volatile("prefetch.global.L2 [%0];" ::"l"(Cij + i * M + n));
    }
  }
  __device__ __forceinline__ void tile(double (&acc)[4][4][2], long m_first, long n_first, int) const {
    // ---- phase 1: loads
    double rci[4];
    unsigned on = 0;   // bit 8*mi + 2*ni + e: the element keeps a weight (row, column and mask allow it)
    double rcj[4][2];
    int hc[4][2];
    bool col_on[4][2];
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const long j = n_first + ni * 8 + e;
        const bool in = j < M;
        const double cj = in ? Cj[j] : 1.0;
        col_on[ni][e] = in && !(cj < p.cthr);
        rcj[ni][e] = col_on[ni][e] ? 1.0 / cj : 0.0;
        hc[ni][e] = in ? (int)(j / Mc) : 0;
      }
    const double scale = inv_batch * p.taupdt;
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
      const long i = row0 + m_first + mi * 8;
      const bool row_in = i < row_end;
      const double ci = row_in ? Ci[i] : 1.0;
      const bool row_on = row_in && !(ci < p.cthr);
      rci[mi] = row_on ? 1.0 / ci : 0.0;
      const uint8_t *mrow = wmask ? wmask + i * H : nullptr;
      double2 old[4];
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const long n = n_first + ni * 8;
        old[ni] = make_double2(0.0, 0.0);
        if (row_in && n < M) {
          const double *cp = Cij + i * M + n;
          if (vec) old[ni] = *reinterpret_cast<const double2 *>(cp);
          else old[ni] = make_double2(cp[0], n + 1 < M ? cp[1] : 0.0);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (row_on && col_on[ni][e] && (mrow == nullptr || mrow[hc[ni][e]] != 0)) on |= 1u << (8 * mi + 2 * ni + e);
      }
      // the moving average, with the batch mean and the averaging weight folded into one factor (the reciprocal
      // of the batch size is exact for powers of two, one rounding more otherwise); a NaN clamps to zero
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const double a0 = fma(old[ni].x, p.one_minus, acc[mi][ni][0] * scale);
        const double a1 = fma(old[ni].y, p.one_minus, acc[mi][ni][1] * scale);
        acc[mi][ni][0] = a0 > 0.0 ? a0 : 0.0;
        acc[mi][ni][1] = a1 > 0.0 ? a1 : 0.0;
      }
    }
    // ---- phase 2: weights and stores.  Cij / (Ci * Cj) by the reciprocals taken above: three roundings more
    // than the division, a few 1e-16 on the weight.
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
      const long i = row0 + m_first + mi * 8;
      if (i >= row_end) continue;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const long n = n_first + ni * 8;
        if (n >= M) continue;
        const double n0 = acc[mi][ni][0], n1 = acc[mi][ni][1];
        double w0 = 0.0, w1 = 0.0;
        if (on & (1u << (8 * mi + 2 * ni))) w0 = f64mma::log_positive((n0 < p.cthr4 ? p.cthr4 : n0) * (rci[mi] * rcj[ni][0]));
        if (on & (2u << (8 * mi + 2 * ni))) w1 = f64mma::log_positive((n1 < p.cthr4 ? p.cthr4 : n1) * (rci[mi] * rcj[ni][1]));
        double *cp = Cij + i * M + n, *wp = W + i * M + n;
        if (vec) {
          *reinterpret_cast<double2 *>(cp) = make_double2(n0, n1);
          *reinterpret_cast<double2 *>(wp) = make_double2(w0, w1);
        } else {
          cp[0] = n0;
          wp[0] = w0;
          if (n + 1 < M) {
            cp[1] = n1;
            wp[1] = w1;
          }
        }
      }
    }
  }
};

static StorePairs to_pairs(const StoreEpilogue<double> &e) { return StorePairs{e.out, e.rows, e.cols, e.ld, e.zstride, e.vec}; }
static TracePairs to_pairs(const TraceEpilogue<double> &e) {
  TracePairs t{};
  t.Ci = e.Ci;
  t.Cj = e.Cj;
  t.Cij = e.Cij;
  t.W = e.W;
  t.wmask = e.wmask;
  t.row0 = e.row0;
  t.row_end = e.row_end;
  t.M = e.M;
  t.H = e.H;
  t.Mc = e.Mc;
  t.p = e.p;
  t.inv_batch = 1.0 / e.p.batch;
  t.vec = e.vec;
  return t;
}
template <typename T>
static int to_pairs(const T &) { return 0; }   // float32 epilogues never take this path

// SBB_F64_CONTRACTION=dfma keeps float64 on the DFMA tile kernel (read once).
static bool f64_mma_enabled() {
  static const bool on = [] {
    const char *e = getenv("SBB_F64_CONTRACTION");
    return !(e != nullptr && strcmp(e, "dfma") == 0);
  }();
  return on;
}

static int sm_count();

template <bool A_KMAJOR, int BM, class Pairs>
static cudaError_t launch_f64_mma_tiles(const double *A, long lda, const double *Bm, long ldb, long Mdim, long Ndim,
                                        int K, int splits, bool cols_fastest, Pairs ep, cudaStream_t st) {
  namespace F = f64mma;
  using C = F::Cfg<BM>;
  auto kernel = F::contraction_kernel<A_KMAJOR, BM, Pairs>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const unsigned mt = (unsigned)((Mdim + BM - 1) / BM), nt = (unsigned)((Ndim + F::BN - 1) / F::BN);
  if (cols_fastest && mt > 65535u) cols_fastest = false;
  dim3 grid(cols_fastest ? nt : mt, cols_fastest ? mt : nt, (unsigned)splits);
  if (grid.y > 65535u || grid.z > 65535u) return cudaErrorInvalidConfiguration;
  const int slabs = (K + F::BK - 1) / F::BK;
  const int kper = (slabs + splits - 1) / splits * F::BK;
  kernel<<<grid, C::THREADS, C::SMEM_BYTES, st>>>(A, lda, Bm, ldb, Mdim, Ndim, K, kper, cols_fastest, ep);
  return launched();
}

// Row tiles of 128 unless 64 finishes in fewer waves of resident CTAs: time ~ waves x (rows of a tile) x (CTAs
// that share an SM).  1568 x 3000 outputs: 611 tiles of 128 rows are two full waves of 296 CTAs and a third with
// 19, 1175 tiles of 64 rows three waves of 444 half-sized CTAs.
template <bool A_KMAJOR, class Pairs>
static cudaError_t launch_f64_mma(const double *A, long lda, const double *Bm, long ldb, long Mdim, long Ndim, int K,
                                  int splits, bool cols_fastest, Pairs ep, cudaStream_t st) {
  namespace F = f64mma;
  const long nt = (Ndim + F::BN - 1) / F::BN, sms = sm_count();
  auto cost = [&](long bm, long ctas_per_sm) {
    const long tiles = ((Mdim + bm - 1) / bm) * nt * splits, slots = sms * ctas_per_sm;
    return ((tiles + slots - 1) / slots) * bm * ctas_per_sm;
  };
  if (cost(64, F::Cfg<64>::CTAS_PER_SM) < cost(128, F::Cfg<128>::CTAS_PER_SM))
    return launch_f64_mma_tiles<A_KMAJOR, 64>(A, lda, Bm, ldb, Mdim, Ndim, K, splits, cols_fastest, ep, st);
  return launch_f64_mma_tiles<A_KMAJOR, 128>(A, lda, Bm, ldb, Mdim, Ndim, K, splits, cols_fastest, ep, st);
}

template <typename T, bool A_KMAJOR, class Ep>
static cudaError_t launch_contraction(const T *A, long lda, const T *Bm, long ldb, long Mdim, long Ndim, int K,
                                      int splits, int kper, bool vec, bool cols_fastest, Ep ep, cudaStream_t st) {
  const unsigned mt = (unsigned)((Mdim + 127) / 128), nt = (unsigned)((Ndim + 127) / 128);
  if (mt == 0 || nt == 0 || K <= 0) return cudaSuccess;
  if constexpr (std::is_same<T, double>::value) {
    // `vec`: every operand row starts on a 16-byte boundary and holds an even number of elements
    if (vec && lda % 2 == 0 && ldb % 2 == 0 && f64_mma_enabled())
      return launch_f64_mma<A_KMAJOR>(A, lda, Bm, ldb, Mdim, Ndim, K, splits, cols_fastest, to_pairs(ep), st);
  }
  if (cols_fastest && mt > 65535u) cols_fastest = false;
  dim3 grid(cols_fastest ? nt : mt, cols_fastest ? mt : nt, (unsigned)splits);
  if (grid.y > 65535u || grid.z > 65535u) return cudaErrorInvalidConfiguration;
  constexpr int V = Vec16<T>::N;
  if (vec)
    contraction_kernel<T, A_KMAJOR, V, Ep><<<grid, 256, 0, st>>>(A, lda, Bm, ldb, Mdim, Ndim, K, kper, cols_fastest, ep);
  else
    contraction_kernel<T, A_KMAJOR, 1, Ep><<<grid, 256, 0, st>>>(A, lda, Bm, ldb, Mdim, Ndim, K, kper, cols_fastest, ep);
  return launched();
}

// ----------------------------------------------------------------------------
// Forward product (split over k so that small batches still fill the GPU).
// ----------------------------------------------------------------------------
static int g_sm_count = 0;
static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_sm_count = n;
    else
      g_sm_count = 148;
  }
  return g_sm_count;
}

template <typename T>
int forward_splits(long B, long N, long M) {
  // output tiles: 128 x 128 (float32 FFMA kernel), 128 x 64 (float64 tensor-core kernel)
  const long tiles = ((B + 127) / 128) * (sizeof(T) == 8 ? (M + 63) / 64 : (M + 127) / 128);
  const long want = 2L * sm_count();           // two resident CTAs per SM
  long s = tiles >= want ? 1 : want / (tiles > 0 ? tiles : 1);
  const long slabs = (N + Tile<T>::BK - 1) / Tile<T>::BK;
  const long max_s = slabs / 8 > 0 ? slabs / 8 : 1;  // at least 8 slabs per split
  if (s > max_s) s = max_s;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return (int)s;
}
template int forward_splits<float>(long, long, long);
template int forward_splits<double>(long, long, long);

template <typename T>
cudaError_t launch_forward_product(const T *x, const T *w, T *partial, long B, long N, long M, int splits,
                                   cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const long slabs = (N + Tile<T>::BK - 1) / Tile<T>::BK;
  const int kper = (int)((slabs + splits - 1) / splits) * Tile<T>::BK;
  const bool vec = (N % V == 0) && (M % V == 0) && aligned16(x) && aligned16(w);
  StoreEpilogue<T> ep{partial, B, M, M, B * M, (M % V == 0) && aligned16(partial)};
  return launch_contraction<T, true>(x, N, w, M, B, M, (int)N, splits, kper, vec, false, ep, st);
}
template cudaError_t launch_forward_product<float>(const float *, const float *, float *, long, long, long, int,
                                                   cudaStream_t);
template cudaError_t launch_forward_product<double>(const double *, const double *, double *, long, long, long, int,
                                                    cudaStream_t);

// ----------------------------------------------------------------------------
// out = sum_s partial[s] + bias, then softmax per hypercolumn.
// One sub-warp of `width` lanes per (row, hypercolumn) group.  A lane owns the
// entries sub, sub+width, ... of its group; with CACHE > 0 they stay in registers
// (Mc <= CACHE*width), otherwise they are re-read from `out`.
// ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T subwarp_max(T v, int width) {
  for (int off = width >> 1; off > 0; off >>= 1) {
    const T o = __shfl_xor_sync(0xffffffffu, v, off, width);
    v = o > v ? o : v;
  }
  return v;
}
template <typename T>
__device__ __forceinline__ T subwarp_sum(T v, int width) {
  for (int off = width >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off, width);
  return v;
}

template <typename T, int CACHE>
__global__ void __launch_bounds__(256)
    reduce_bias_softmax_kernel(const T *partial, int splits, long slice, const T *__restrict__ bias, T *out,
                               long groups, long H, long Mc, int width) {
  const int lane = threadIdx.x & 31;
  const int sub = lane % width;
  const long warp = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long g = warp * (32 / width) + lane / width;
  const bool live = g < groups;
  const long base = g * Mc;            // offset of the group inside [rows, H*Mc]
  const long col0 = (g % H) * Mc;      // first column of the group
  constexpr int NC = CACHE > 0 ? CACHE : 1;
  T v[NC];
  T mx = -INFINITY;
  if (CACHE > 0) {
#pragma unroll
    for (int e = 0; e < NC; ++e) {
      const long j = sub + (long)e * width;
      T s = -INFINITY;
      if (live && j < Mc) {
        s = partial[base + j];
        for (int z = 1; z < splits; ++z) s += partial[(long)z * slice + base + j];
        if (bias) s += bias[col0 + j];
      }
      v[e] = s;
      mx = s > mx ? s : mx;
    }
    mx = subwarp_max(mx, width);
    T sum = (T)0;
#pragma unroll
    for (int e = 0; e < NC; ++e) {
      const long j = sub + (long)e * width;
      if (live && j < Mc) {
        v[e] = sbb_exp(v[e] - mx);
        sum += v[e];
      }
    }
    sum = subwarp_sum(sum, width);
#pragma unroll
    for (int e = 0; e < NC; ++e) {
      const long j = sub + (long)e * width;
      if (live && j < Mc) out[base + j] = v[e] / sum;
    }
  } else {
    if (live)
      for (long j = sub; j < Mc; j += width) {
        T s = partial[base + j];
        for (int z = 1; z < splits; ++z) s += partial[(long)z * slice + base + j];
        if (bias) s += bias[col0 + j];
        out[base + j] = s;
        mx = s > mx ? s : mx;
      }
    mx = subwarp_max(mx, width);
    T sum = (T)0;
    if (live)
      for (long j = sub; j < Mc; j += width) {
        const T e = sbb_exp(out[base + j] - mx);
        out[base + j] = e;
        sum += e;
      }
    sum = subwarp_sum(sum, width);
    if (live)
      for (long j = sub; j < Mc; j += width) out[base + j] = out[base + j] / sum;
  }
}

// The same for groups of more than 16 entries (one whole warp per group) with every per-element index a
// compile-time multiple of 32 from three pointers formed once: the general kernel above spends most of its
// instructions on 64-bit index arithmetic (about 100 per element at Mc = 300, which made it issue-bound: 183 us
// for 246 MB at the 1568 -> 100 x 300 layer).
template <typename T, int NC, bool SPLIT>
__global__ void __launch_bounds__(256)
    softmax_warp_kernel(const T *partial, int splits, long slice, const T *__restrict__ bias, T *out, long groups,
                        int H, int Mc) {
  const int lane = threadIdx.x & 31;
  const long g = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= groups) return;   // whole warps leave together
  const T *src = partial + g * Mc + lane;
  const T *bs = bias ? bias + (g % H) * (long)Mc + lane : nullptr;
  T *dst = out + g * Mc + lane;
  const int left = Mc - lane;   // entry e of this lane exists when e * 32 < left
  T v[NC];
  T mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < NC; ++e) {
    T s = -INFINITY;
    if (e * 32 < left) {
      s = src[e * 32];
      if (SPLIT)
        for (int z = 1; z < splits; ++z) s += src[(long)z * slice + e * 32];
      if (bs) s += bs[e * 32];
    }
    v[e] = s;
    mx = s > mx ? s : mx;
  }
  mx = subwarp_max(mx, 32);
  T sum = (T)0;
#pragma unroll
  for (int e = 0; e < NC; ++e) {
    v[e] = e * 32 < left ? sbb_exp(v[e] - mx) : (T)0;
    sum += v[e];
  }
  sum = subwarp_sum(sum, 32);
#pragma unroll
  for (int e = 0; e < NC; ++e)
    if (e * 32 < left) dst[e * 32] = v[e] / sum;
}

// out[r, j] = sum_s partial[s, r, j] + bias[j]   (no softmax)
template <typename T>
__global__ void __launch_bounds__(256)
    reduce_bias_kernel(const T *partial, int splits, long slice, const T *__restrict__ bias, T *out, long total,
                       long M) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  T s = partial[idx];
  for (int z = 1; z < splits; ++z) s += partial[(long)z * slice + idx];
  if (bias) s += bias[idx % M];
  out[idx] = s;
}

template <typename T>
cudaError_t launch_reduce_bias_softmax(const T *partial, int splits, const T *bias, T *out, long rows, long H,
                                       long Mc, int softmax, cudaStream_t st) {
  const long M = H * Mc;
  const long total = rows * M;
  if (total == 0) return cudaSuccess;
  if (!softmax) {
    if (splits == 1 && bias == nullptr && partial == out) return cudaSuccess;
    reduce_bias_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(partial, splits, total, bias, out, total, M);
    return launched();
  }
  int width = 32;
  while (width > 1 && (width >> 1) >= Mc) width >>= 1;
  const long groups = rows * H;
  const long per_warp = 32 / width;
  const long warps = (groups + per_warp - 1) / per_warp;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  const long per_lane = (Mc + width - 1) / width;
  if (width == 32 && per_lane <= 16 && H < (1l << 31) && Mc < (1l << 31)) {
    // one warp per group: the lean kernel (same arithmetic, same summation order)
#define SBB_SOFTMAX_WARP(NC)                                                                                      \
  do {                                                                                                            \
    if (splits > 1)                                                                                               \
      softmax_warp_kernel<T, NC, true><<<(unsigned)((groups + 7) / 8), 256, 0, st>>>(partial, splits, total, bias, out, \
                                                                                    groups, (int)H, (int)Mc);    \
    else                                                                                                          \
      softmax_warp_kernel<T, NC, false><<<(unsigned)((groups + 7) / 8), 256, 0, st>>>(partial, splits, total, bias, out, \
                                                                                     groups, (int)H, (int)Mc);   \
  } while (0)
    if (per_lane <= 4) SBB_SOFTMAX_WARP(4);
    else if (per_lane <= 8) SBB_SOFTMAX_WARP(8);
    else if (per_lane <= 12) SBB_SOFTMAX_WARP(12);
    else SBB_SOFTMAX_WARP(16);
#undef SBB_SOFTMAX_WARP
    return launched();
  }
  if (per_lane <= 4)
    reduce_bias_softmax_kernel<T, 4><<<blocks, 256, 0, st>>>(partial, splits, total, bias, out, groups, H, Mc, width);
  else if (per_lane <= 8)
    reduce_bias_softmax_kernel<T, 8><<<blocks, 256, 0, st>>>(partial, splits, total, bias, out, groups, H, Mc, width);
  else if (per_lane <= 12)
    reduce_bias_softmax_kernel<T, 12><<<blocks, 256, 0, st>>>(partial, splits, total, bias, out, groups, H, Mc, width);
  else if (per_lane <= 16)
    reduce_bias_softmax_kernel<T, 16><<<blocks, 256, 0, st>>>(partial, splits, total, bias, out, groups, H, Mc, width);
  else
    reduce_bias_softmax_kernel<T, 0><<<blocks, 256, 0, st>>>(partial, splits, total, bias, out, groups, H, Mc, width);
  return launched();
}
template cudaError_t launch_reduce_bias_softmax<float>(const float *, int, const float *, float *, long, long, long,
                                                       int, cudaStream_t);
template cudaError_t launch_reduce_bias_softmax<double>(const double *, int, const double *, double *, long, long,
                                                        long, int, cudaStream_t);

// ----------------------------------------------------------------------------
// Column sums over the batch (and, fused, the Ci / Cj moving averages).
// Block = 32 columns x 8 row lanes; rows are summed in a fixed order.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    colsum_kernel(const T *__restrict__ a, long B, long cols, T *sums, T *c, TraceParams<T> p, int ema, T *lo) {
  __shared__ T part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long col = (long)blockIdx.x * 32 + tx;
  T s = (T)0;
  if (col < cols) {
    long b = ty;
    for (; b + 24 < B; b += 32) {
      const T v0 = __ldg(a + b * cols + col), v1 = __ldg(a + (b + 8) * cols + col);
      const T v2 = __ldg(a + (b + 16) * cols + col), v3 = __ldg(a + (b + 24) * cols + col);
      s += v0; s += v1; s += v2; s += v3;
      if (lo) {   // the operand's low parts for the split product of the tensor-core contraction that follows
        lo[b * cols + col] = tf32_lo(v0);
        lo[(b + 8) * cols + col] = tf32_lo(v1);
        lo[(b + 16) * cols + col] = tf32_lo(v2);
        lo[(b + 24) * cols + col] = tf32_lo(v3);
      }
    }
    for (; b < B; b += 8) {
      const T v = __ldg(a + b * cols + col);
      s += v;
      if (lo) lo[b * cols + col] = tf32_lo(v);
    }
  }
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < cols) {
    T t = part[0][tx];
#pragma unroll
    for (int r = 1; r < 8; ++r) t += part[r][tx];
    if (ema) c[col] = trace_ema(c[col], t, p);
    else sums[col] = t;
  }
}

template <typename T>
cudaError_t launch_colsum(const T *a, long B, long cols, T *sums, T *c, TraceParams<T> p, int ema, cudaStream_t st,
                          T *lo) {
  if (cols == 0) return cudaSuccess;
  colsum_kernel<T><<<(unsigned)((cols + 31) / 32), 256, 0, st>>>(a, B, cols, sums, c, p, ema, lo);
  return launched();
}
template cudaError_t launch_colsum<float>(const float *, long, long, float *, float *, TraceParams<float>, int,
                                          cudaStream_t, float *);
template cudaError_t launch_colsum<double>(const double *, long, long, double *, double *, TraceParams<double>, int,
                                           cudaStream_t, double *);

template <typename T>
__global__ void vector_ema_kernel(T *c, const T *__restrict__ sums, long n, TraceParams<T> p) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) c[i] = trace_ema(c[i], sums[i], p);
}
template <typename T>
cudaError_t launch_vector_ema(T *c, const T *sums, long n, TraceParams<T> p, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  vector_ema_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(c, sums, n, p);
  return launched();
}
template cudaError_t launch_vector_ema<float>(float *, const float *, long, TraceParams<float>, cudaStream_t);
template cudaError_t launch_vector_ema<double>(double *, const double *, long, TraceParams<double>, cudaStream_t);

// ----------------------------------------------------------------------------
// Trace step: fused (x^T y in the contraction, traces and weights in its
// epilogue) and split (raw x^T y, then an element-wise tail).
// ----------------------------------------------------------------------------
template <typename T>
cudaError_t launch_trace_update_fused(const T *x, const T *y, long B, long N, long M, long H, long Mc, const T *Ci,
                                      const T *Cj, T *Cij, T *w, const uint8_t *wmask, TraceParams<T> p,
                                      long row_begin, long row_end, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (row_end <= row_begin) return cudaSuccess;
  const bool vec = (N % V == 0) && (M % V == 0) && (row_begin % V == 0) && ((row_end - row_begin) % V == 0) &&
                   aligned16(x) && aligned16(y);
  TraceEpilogue<T> ep{Ci, Cj, Cij, w, wmask, row_begin, row_end, M, H, Mc, p,
                      (M % V == 0) && aligned16(Cij) && aligned16(w)};
  const int kper = (int)((B + Tile<T>::BK - 1) / Tile<T>::BK) * Tile<T>::BK;
  return launch_contraction<T, false>(x + row_begin, N, y, M, row_end - row_begin, M, (int)B, 1, kper, vec, true, ep, st);
}
template cudaError_t launch_trace_update_fused<float>(const float *, const float *, long, long, long, long, long,
                                                      const float *, const float *, float *, float *,
                                                      const uint8_t *, TraceParams<float>, long, long, cudaStream_t);
template cudaError_t launch_trace_update_fused<double>(const double *, const double *, long, long, long, long, long,
                                                       const double *, const double *, double *, double *,
                                                       const uint8_t *, TraceParams<double>, long, long,
                                                       cudaStream_t);

template <typename T>
cudaError_t launch_outer_product(const T *x, const T *y, long B, long N, long M, T *delta, long row_begin,
                                 long row_end, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (row_end <= row_begin) return cudaSuccess;
  const bool vec = (N % V == 0) && (M % V == 0) && (row_begin % V == 0) && ((row_end - row_begin) % V == 0) &&
                   aligned16(x) && aligned16(y);
  StoreEpilogue<T> ep{delta + row_begin * M, row_end - row_begin, M, M, 0, (M % V == 0) && aligned16(delta)};
  const int kper = (int)((B + Tile<T>::BK - 1) / Tile<T>::BK) * Tile<T>::BK;
  return launch_contraction<T, false>(x + row_begin, N, y, M, row_end - row_begin, M, (int)B, 1, kper, vec, true, ep, st);
}
template cudaError_t launch_outer_product<float>(const float *, const float *, long, long, long, float *, long, long,
                                                 cudaStream_t);
template cudaError_t launch_outer_product<double>(const double *, const double *, long, long, long, double *, long,
                                                  long, cudaStream_t);

// One thread per four consecutive columns, walking kApplyRows rows: the column data (Cj, the
// hypercolumn of each column) is set up once per thread, rows only add Ci and the mask byte.
constexpr int kApplyRows = 8;
// FAST (float32 only): the tensor-core path's arithmetic (see sbb_math.cuh), so that the data-parallel
// step and the fused single-device step of that path compute the same values from the same sums.
template <typename T, bool FAST>
__global__ void __launch_bounds__(256)
    trace_apply_kernel(const T *__restrict__ delta, long M, long H, long Mc, const T *__restrict__ Ci,
                       const T *__restrict__ Cj, T *Cij, T *W, const uint8_t *__restrict__ wmask, TraceParams<T> p,
                       int ema, long row_begin, long row_end, bool vec) {
  const long j = ((long)blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (j >= M) return;
  const long left = M - j;
  const int valid = left >= 4 ? 4 : (int)left;
  T cj[4];
  bool col_on[4];
  long hc[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    cj[c] = c < valid ? Cj[j + c] : (T)1;
    col_on[c] = c < valid && !(cj[c] < p.cthr);
    hc[c] = wmask ? (j + (c < valid ? c : 0)) / Mc : 0;
    if (FAST) cj[c] = (T)1 / cj[c];   // from here on the reciprocal
  }
  const T ema_scale = p.taupdt / p.batch;
  const bool one_hc = hc[0] == hc[3] && hc[0] == hc[1] && hc[0] == hc[2];
  const long r0 = row_begin + (long)blockIdx.x * kApplyRows;
  const long r1 = r0 + kApplyRows < row_end ? r0 + kApplyRows : row_end;
  for (long i = r0; i < r1; ++i) {
    T ci = Ci[i];
    const bool row_on = !(ci < p.cthr);
    if (FAST) ci = (T)1 / ci;
    bool on[4];
    if (wmask == nullptr) {
#pragma unroll
      for (int c = 0; c < 4; ++c) on[c] = row_on && col_on[c];
    } else if (one_hc) {
      const bool m = wmask[i * H + hc[0]] != 0;
#pragma unroll
      for (int c = 0; c < 4; ++c) on[c] = row_on && col_on[c] && m;
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) on[c] = row_on && col_on[c] && wmask[i * H + hc[c]] != 0;
    }
    T c4[4], d4[4], w4[4];
    load4(Cij + i * M + j, c4, vec, valid);
    if (ema) load4(delta + i * M + j, d4, vec, valid);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c < valid) {
        T cij = c4[c];
        if constexpr (FAST) {
          if (ema) cij = trace_ema_fast(c4[c], d4[c], p.one_minus, ema_scale);
          w4[c] = on[c] ? log_ratio_fast(cij, ci, cj[c], p.cthr4) : 0.f;
        } else {
          if (ema) cij = trace_ema(c4[c], d4[c], p);
          w4[c] = on[c] ? log_ratio(cij, ci, cj[c], p.cthr4) : (T)0;
        }
        c4[c] = cij;
      }
    }
    if (ema) store4(Cij + i * M + j, c4, vec, valid);
    store4(W + i * M + j, w4, vec, valid);
  }
}

template <typename T>
cudaError_t launch_trace_apply(const T *delta, long N, long M, long H, long Mc, const T *Ci, const T *Cj, T *Cij,
                               T *w, const uint8_t *wmask, TraceParams<T> p, int ema, long row_begin, long row_end,
                               cudaStream_t st, bool fast) {
  (void)N;
  constexpr int V = Vec16<T>::N;
  if (row_end <= row_begin || M == 0) return cudaSuccess;
  const long qpr = (M + 3) / 4;
  const bool vec = (M % V == 0) && aligned16(Cij) && aligned16(w) && (!ema || aligned16(delta));
  const long row_groups = (row_end - row_begin + kApplyRows - 1) / kApplyRows;
  const int threads = qpr >= 256 ? 256 : (int)((qpr + 31) / 32 * 32);
  const dim3 grid((unsigned)row_groups, (unsigned)((qpr + threads - 1) / threads));
  if constexpr (std::is_same<T, float>::value) {
    if (fast && p.cthr4 >= 1e-30f) {
      trace_apply_kernel<float, true><<<grid, threads, 0, st>>>(delta, M, H, Mc, Ci, Cj, Cij, w, wmask, p, ema, row_begin,
                                                                row_end, vec);
      return launched();
    }
  }
  trace_apply_kernel<T, false><<<grid, threads, 0, st>>>(delta, M, H, Mc, Ci, Cj, Cij, w, wmask, p, ema, row_begin,
                                                         row_end, vec);
  return launched();
}
template cudaError_t launch_trace_apply<float>(const float *, long, long, long, long, const float *, const float *,
                                               float *, float *, const uint8_t *, TraceParams<float>, int, long, long,
                                               cudaStream_t, bool);
template cudaError_t launch_trace_apply<double>(const double *, long, long, long, long, const double *,
                                                const double *, double *, double *, const uint8_t *,
                                                TraceParams<double>, int, long, long, cudaStream_t, bool);

// Un-fused trace update in the NumPy operation order: (1-t)*C + t*(sum/B).
template <typename T>
__global__ void counters_apply_kernel(T *c, const T *__restrict__ sums, long n, T taupdt, T batch) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const T v = ((T)1 - taupdt) * c[i] + taupdt * (sums[i] / batch);
  c[i] = v > (T)0 ? v : (T)0;
}
template <typename T>
cudaError_t launch_counters_apply(T *c, const T *sums, long n, T taupdt, T batch, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  counters_apply_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(c, sums, n, taupdt, batch);
  return launched();
}
template cudaError_t launch_counters_apply<float>(float *, const float *, long, float, float, cudaStream_t);
template cudaError_t launch_counters_apply<double>(double *, const double *, long, double, double, cudaStream_t);

// ----------------------------------------------------------------------------
// Bias kernels and small element-wise helpers.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void update_bias_kernel(T *bias, const T *__restrict__ Cj, T cthr, long M) {
  const long j = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j < M) bias[j] = Cj[j] < cthr ? sbb_log((T)2 * cthr) : sbb_log(Cj[j]);
}
template <typename T>
cudaError_t launch_update_bias(T *bias, const T *Cj, T cthr, long M, cudaStream_t st) {
  if (M == 0) return cudaSuccess;
  update_bias_kernel<T><<<(unsigned)((M + 255) / 256), 256, 0, st>>>(bias, Cj, cthr, M);
  return launched();
}
template cudaError_t launch_update_bias<float>(float *, const float *, float, long, cudaStream_t);
template cudaError_t launch_update_bias<double>(double *, const double *, double, long, cudaStream_t);

template <typename T>
__global__ void update_bias_regularized_kernel(T *bias, T *kbi, const T *__restrict__ Cj, T cthr, T khalf, T pmin4,
                                               T k, T taubdt, long M) {
  const long j = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= M) return;
  const T pj = Cj[j];
  T kb = (T)1 + k / ((pj - pmin4) * (pj - pmin4));
  if (pj < pmin4 || kb < khalf) kb = khalf;
  const T g = ((T)1 - taubdt) * kbi[j] + taubdt * kb;
  kbi[j] = g;
  bias[j] = pj < cthr ? g * sbb_log((T)2 * cthr) : g * sbb_log(pj);
}
template <typename T>
cudaError_t launch_update_bias_regularized(T *bias, T *kbi, const T *Cj, T cthr, T khalf, T pmin, T taubdt, long M,
                                           cudaStream_t st) {
  if (M == 0) return cudaSuccess;
  const T pmin4 = pmin / (T)4;
  const T k = (khalf - (T)1) * (pmin4 * pmin4);
  update_bias_regularized_kernel<T><<<(unsigned)((M + 255) / 256), 256, 0, st>>>(bias, kbi, Cj, cthr, khalf, pmin4, k,
                                                                                  taubdt, M);
  return launched();
}
template cudaError_t launch_update_bias_regularized<float>(float *, float *, const float *, float, float, float,
                                                           float, long, cudaStream_t);
template cudaError_t launch_update_bias_regularized<double>(double *, double *, const double *, double, double,
                                                            double, double, long, cudaStream_t);

template <typename T>
__global__ void add_bias_kernel(T *a, const T *__restrict__ bias, long total, long M) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) a[idx] += bias[idx % M];
}
template <typename T>
cudaError_t launch_add_bias(T *a, const T *bias, long rows, long M, cudaStream_t st) {
  const long total = rows * M;
  if (total == 0) return cudaSuccess;
  add_bias_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a, bias, total, M);
  return launched();
}
template cudaError_t launch_add_bias<float>(float *, const float *, long, long, cudaStream_t);
template cudaError_t launch_add_bias<double>(double *, const double *, long, long, cudaStream_t);

template <typename T>
__global__ void apply_mask_kernel(T *w, const uint8_t *__restrict__ wmask, long total, long M, long H, long Mc) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long i = idx / M, j = idx % M;
  if (!wmask[i * H + j / Mc]) w[idx] = (T)0;
}
template <typename T>
cudaError_t launch_apply_mask(T *w, const uint8_t *wmask, long N, long M, long H, long Mc, cudaStream_t st) {
  const long total = N * M;
  if (total == 0) return cudaSuccess;
  apply_mask_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w, wmask, total, M, H, Mc);
  return launched();
}
template cudaError_t launch_apply_mask<float>(float *, const uint8_t *, long, long, long, long, cudaStream_t);
template cudaError_t launch_apply_mask<double>(double *, const uint8_t *, long, long, long, long, cudaStream_t);

// ----------------------------------------------------------------------------
// Structural plasticity: score, swap, rewrite.
// ----------------------------------------------------------------------------
// One warp per input row: the mutual-information score numerator over the
// minicolumns of hypercolumn h (terms in REAL, accumulated in double) and the
// row's count of active connections.
template <typename T>
__global__ void __launch_bounds__(256)
    mask_score_kernel(const uint8_t *__restrict__ wmask, const T *__restrict__ weights, const T *__restrict__ Ci,
                      const T *__restrict__ Cj, const T *__restrict__ Cij, T cthr, T cthr4, long N, long M, long H,
                      long Mc, long h, T *score, int *csum, uint8_t *old_col) {
  const int lane = threadIdx.x & 31;
  const long i = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= N) return;  // whole warp leaves together
  // Every load of the row (its trace, the mask bytes, the trace block) is issued before the first use of any of
  // them: the loads do not depend on the row's trace value, only the arithmetic does, so the warp pays one
  // memory round trip instead of three.
  const T pi = Ci[i];
  int cnt = 0;
  for (long k = lane; k < H; k += 32) cnt += wmask[i * H + k];
  double s = 0.0;
  // four strided elements per lane at a time, all loads issued before the arithmetic
  for (long j0 = 0; j0 < Mc; j0 += 128) {
    T pj[4], pij[4], wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long jj = j0 + lane + 32 * u, col = h * Mc + jj;
      const bool in = jj < Mc;
      pj[u] = in ? Cj[col] : (T)0;
      pij[u] = in ? Cij[i * M + col] : (T)0;
      wv[u] = (in && weights) ? weights[i * M + col] : (T)0;
    }
    if (pi >= cthr) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j0 + lane + 32 * u < Mc && pj[u] >= cthr) {
          const T w = weights ? wv[u] : log_ratio(pij[u], pi, pj[u], cthr4);
          const T x = ((T)1 - pi) * pj[u];
          const T y = (pj[u] - pij[u]) / x;
          s += (double)(pij[u] * w + (pj[u] - pij[u]) * sbb_log(y));
        }
      }
    }
  }
  for (int off = 16; off > 0; off >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, off);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
  }
  if (lane == 0) {
    score[i] = (T)s;
    csum[i] = cnt;
    old_col[i] = wmask[i * H + h];   // the mask column before the swaps, for the weight rewrite
  }
}

template <typename T>
struct Pick {
  T v;
  long i;  // -1 = empty
};
// Maximum with ties to the larger index / minimum with ties to the larger index:
// the outcome of a front-to-back scan that replaces on >= (resp. <=).
template <typename T>
__device__ __forceinline__ Pick<T> pick_max(Pick<T> a, Pick<T> b) {
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  return (b.v > a.v || (b.v == a.v && b.i > a.i)) ? b : a;
}
template <typename T>
__device__ __forceinline__ Pick<T> pick_min(Pick<T> a, Pick<T> b) {
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  return (b.v < a.v || (b.v == a.v && b.i > a.i)) ? b : a;
}
template <typename T>
__device__ __forceinline__ Pick<T> shfl_pick(Pick<T> p, int off) {
  Pick<T> o;
  o.v = __shfl_xor_sync(0xffffffffu, p.v, off);
  o.i = __shfl_xor_sync(0xffffffffu, p.i, off);
  return o;
}

// Single CTA.  Every iteration scans all rows: among silent connections
// (mask 0) the highest score, among active ones (mask 1) the lowest, both with
// the reference's sequential-scan semantics: ties go to the last index, and a
// NaN score can only be selected when it belongs to the first candidate of its
// class (a scan never replaces its holder with a NaN, nor a NaN holder at all).
template <typename T>
__global__ void __launch_bounds__(1024)
    mask_swap_kernel(uint8_t *wmask, const T *__restrict__ nom, int *csum, long N, long M, long H, long Mc, long h,
                     long iterations, T *rewrite_w,
                     const uint8_t *__restrict__ old_col, const T *__restrict__ Ci, const T *__restrict__ Cj,
                     const T *__restrict__ Cij, T cthr, T cthr4) {
  __shared__ Pick<T> s_max[32], s_min[32];
  __shared__ long s_first0[32], s_first1[32];
  __shared__ int s_done;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) s_done = 0;
  __syncthreads();
  for (long it = 0; it < iterations; ++it) {
    Pick<T> bmax{(T)0, -1}, bmin{(T)0, -1};
    long first0 = N, first1 = N;
    for (long j = threadIdx.x; j < N; j += blockDim.x) {
      const uint8_t m = wmask[j * H + h];
      const T sc = (T)((double)nom[j] / (1.0 + (double)csum[j]));
      if (m == 0) {
        first0 = j < first0 ? j : first0;
        if (sc == sc) bmax = pick_max(bmax, Pick<T>{sc, j});
      } else if (m == 1) {
        first1 = j < first1 ? j : first1;
        if (sc == sc) bmin = pick_min(bmin, Pick<T>{sc, j});
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      bmax = pick_max(bmax, shfl_pick(bmax, off));
      bmin = pick_min(bmin, shfl_pick(bmin, off));
      const long f0 = __shfl_xor_sync(0xffffffffu, first0, off);
      const long f1 = __shfl_xor_sync(0xffffffffu, first1, off);
      first0 = f0 < first0 ? f0 : first0;
      first1 = f1 < first1 ? f1 : first1;
    }
    if (lane == 0) {
      s_max[wid] = bmax;
      s_min[wid] = bmin;
      s_first0[wid] = first0;
      s_first1[wid] = first1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < nwarps; ++w) {
        bmax = pick_max(bmax, s_max[w]);
        bmin = pick_min(bmin, s_min[w]);
        first0 = s_first0[w] < first0 ? s_first0[w] : first0;
        first1 = s_first1[w] < first1 ? s_first1[w] : first1;
      }
      long imax0 = N, imin1 = N;
      T vmax0 = (T)0, vmin1 = (T)0;
      if (first0 < N) {
        const T sf = (T)((double)nom[first0] / (1.0 + (double)csum[first0]));
        if (sf != sf) { imax0 = first0; vmax0 = sf; }
        else { imax0 = bmax.i; vmax0 = bmax.v; }
      }
      if (first1 < N) {
        const T sf = (T)((double)nom[first1] / (1.0 + (double)csum[first1]));
        if (sf != sf) { imin1 = first1; vmin1 = sf; }
        else { imin1 = bmin.i; vmin1 = bmin.v; }
      }
      if (imax0 == N || imin1 == N || vmax0 < vmin1) {
        s_done = 1;
      } else {
        wmask[imax0 * H + h] = 1;
        wmask[imin1 * H + h] = 0;
        csum[imax0] += 1;
        csum[imin1] -= 1;
      }
    }
    __syncthreads();
    if (s_done) break;
  }
  if (rewrite_w == nullptr) return;
  // rows whose mask bit changed get new weights in hypercolumn h (at most 2 * iterations rows)
  for (long j = threadIdx.x; j < N; j += blockDim.x) {
    const uint8_t now = wmask[j * H + h];
    if (now == old_col[j]) continue;
    const T ci = Ci[j];
    for (long jj = 0; jj < Mc; ++jj) {
      const long col = h * Mc + jj;
      const T cj = Cj[col];
      T v = (T)0;
      if (now != 0 && !(ci < cthr) && !(cj < cthr)) v = log_ratio(Cij[j * M + col], ci, cj, cthr4);
      rewrite_w[j * M + col] = v;
    }
  }
}

// ---- fast swap: per-chunk candidate lists, then a short exact simulation -------------------
// Only the two rows of a swap change their score, so the row chosen in iteration t is always
// among the t+1 best of its class in the initial ordering or a row moved by an earlier swap.
// Phase A extracts, per chunk of rows, the `iterations` best silent rows (highest score, ties
// to the larger index) and the `iterations` worst active rows (lowest score, ties to the
// larger index); phase B reduces the chunk lists to one list per class and replays the swaps
// exactly.  A NaN score makes the reference's scan order-dependent; phase B reproduces that too
// (see mask_replay_kernel).  Layers too small or too large for the lists, and more than
// kSwapMaxIter iterations, take the one-CTA full scan (mask_swap_kernel).
//
// Scores are mapped to unsigned keys whose integer order is the class order (silent rows: score
// descending first = larger key; active rows: the complement), so that one selection round is a
// register-local maximum, one warp-wide integer maximum (redux) for the key and one for the row
// index among equal keys (the reference's scans keep the last of equal scores), and a clear of the
// winner's register: no shuffle trees, no block barrier inside a round.
constexpr int kSwapMaxIter = 32;
constexpr int kSwapSlots = 1024;          // candidate slots per class handed from phase A to phase B
constexpr int kSwapCacheRows = 4096;      // rows per chunk whose score and class fit the chunk's shared memory
constexpr int kSwapThreads = 256;         // both phases: 8 warps = 2 classes x 4 slices

template <typename T>
__device__ __forceinline__ T swap_score(T nom, int csum) {
  return (T)((double)nom / (1.0 + (double)csum));
}

// Order-preserving keys: a < b  <=>  key(a) < key(b) for non-NaN scores (-0 counts as +0).
// Key 0 is never produced by a score and marks an empty slot, also after complementing.
template <typename T>
struct ScoreKey;
template <>
struct ScoreKey<float> {
  typedef uint32_t type;
  static __device__ __forceinline__ type make(float v) {
    const uint32_t u = __float_as_uint(v == 0.f ? 0.f : v);
    return (u >> 31) ? ~u : (u | 0x80000000u);
  }
  static __device__ __forceinline__ float value(type k) {
    return __uint_as_float((k >> 31) ? (k ^ 0x80000000u) : ~k);
  }
  static __device__ __forceinline__ type warp_max(type k) { return __reduce_max_sync(0xffffffffu, k); }
};
template <>
struct ScoreKey<double> {
  typedef unsigned long long type;
  static __device__ __forceinline__ type make(double v) {
    const unsigned long long u = (unsigned long long)__double_as_longlong(v == 0.0 ? 0.0 : v);
    return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
  }
  static __device__ __forceinline__ double value(type k) {
    return __longlong_as_double((long long)((k >> 63) ? (k ^ 0x8000000000000000ull) : ~k));
  }
  static __device__ __forceinline__ type warp_max(type k) {
    const uint32_t hi = __reduce_max_sync(0xffffffffu, (uint32_t)(k >> 32));
    const uint32_t lo = __reduce_max_sync(0xffffffffu, (uint32_t)(k >> 32) == hi ? (uint32_t)k : 0u);
    return ((type)hi << 32) | lo;
  }
};
// Class key: maximum = first in the class order.  cls 0 (silent): highest score; cls 1 (active): lowest.
template <typename T>
__device__ __forceinline__ typename ScoreKey<T>::type class_key(int cls, T v) {
  const typename ScoreKey<T>::type k = ScoreKey<T>::make(v);
  return cls == 0 ? k : ~k;
}
template <typename T>
__device__ __forceinline__ T class_key_value(int cls, typename ScoreKey<T>::type k) {
  return ScoreKey<T>::value(cls == 0 ? k : ~k);
}

// One warp: the first `rounds` of its R x 32 register-resident entries (key 0 = empty) in class
// order; lane 0 writes round k's (score, row) to out_v[k], out_i[k] (row -1 pads an exhausted list).
template <typename T, int R>
__device__ __forceinline__ void warp_select_regs(int cls, typename ScoreKey<T>::type (&key)[R], uint32_t (&row)[R],
                                                 int rounds, T *out_v, long *out_i) {
  typedef typename ScoreKey<T>::type K;
  const int lane = threadIdx.x & 31;
  for (int k = 0; k < rounds; ++k) {
    K mine = 0;
#pragma unroll
    for (int r = 0; r < R; ++r) mine = key[r] > mine ? key[r] : mine;
    const K best = ScoreKey<T>::warp_max(mine);
    if (best == 0) {   // exhausted (uniform)
      for (int kk = k + lane; kk < rounds; kk += 32) out_i[kk] = -1;
      break;
    }
    uint32_t my_row = 0;   // rows are stored + 1 so that 0 means "not holding the best key"
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (key[r] == best && row[r] + 1u > my_row) my_row = row[r] + 1u;
    const uint32_t win = __reduce_max_sync(0xffffffffu, my_row);
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (key[r] == best && row[r] + 1u == win) key[r] = 0;
    if (lane == 0) {
      out_v[k] = class_key_value<T>(cls, best);
      out_i[k] = (long)win - 1;
    }
  }
}

// Phase A.  lists: [class][chunk][iterations] of (value, row); row -1 = empty.
// CACHED: the chunk's scores and classes are first gathered into shared memory (coalesced).
template <typename T, int R>
__global__ void __launch_bounds__(kSwapThreads)
    mask_candidates_kernel(const uint8_t *__restrict__ wmask, const T *__restrict__ nom, const int *__restrict__ csum,
                           long N, long H, long h, int iterations, long rows_per_chunk, T *cand_v, long *cand_i) {
  typedef typename ScoreKey<T>::type K;
  __shared__ T s_lv[2][4 * kSwapMaxIter];
  __shared__ long s_li[2][4 * kSwapMaxIter];
  extern __shared__ __align__(16) unsigned char cand_dyn[];
  T *s_sc = reinterpret_cast<T *>(cand_dyn);
  uint8_t *s_cl = cand_dyn + rows_per_chunk * sizeof(T);
  const long r0 = (long)blockIdx.x * rows_per_chunk;
  const long r1 = r0 + rows_per_chunk < N ? r0 + rows_per_chunk : N;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (long j = r0 + threadIdx.x; j < r1; j += blockDim.x) {
    const uint8_t m = wmask[j * H + h];
    const T sc = swap_score(nom[j], csum[j]);
    uint8_t cl = m <= 1 ? m : 2;
    if (sc != sc) cl = 2;   // a NaN score is in no best list (the replay handles the one place it can matter)
    s_sc[j - r0] = sc;
    s_cl[j - r0] = cl;
  }
  __syncthreads();
  // level 1: warp (cls, slice) lists the first `iterations` rows of its class in its quarter of the chunk
  const int cls = wid & 1, slice = wid >> 1;
  {
    const long len = r1 - r0, q = (len + 3) / 4;
    const long b = slice * q, e = b + q < len ? b + q : len;   // chunk-relative
    K key[R];
    uint32_t row[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long j = b + lane + 32 * r;
      const bool mine = j < e && s_cl[j < e ? j : 0] == cls;
      key[r] = mine ? class_key<T>(cls, s_sc[j]) : (K)0;
      row[r] = (uint32_t)(r0 + j);
    }
    warp_select_regs<T, R>(cls, key, row, iterations, s_lv[cls] + slice * iterations, s_li[cls] + slice * iterations);
  }
  __syncthreads();
  // level 2: one warp per class merges the four slice lists (4 * iterations <= 128 entries) into the chunk's list
  if (wid < 2) {
    K key[4];
    uint32_t row[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int e = lane + 32 * r;
      const long i = e < 4 * iterations ? s_li[wid][e] : -1;
      key[r] = i >= 0 ? class_key<T>(wid, s_lv[wid][e]) : (K)0;
      row[r] = i >= 0 ? (uint32_t)i : 0u;
    }
    const long slot = ((long)wid * gridDim.x + blockIdx.x) * iterations;
    warp_select_regs<T, 4>(wid, key, row, iterations, cand_v + slot, cand_i + slot);
  }
}

// Phase B, one CTA: reduce the chunk lists to the first `iterations` rows of each class, replay
// the swaps on them (warp 0; every lane keeps one listed row and one moved row per class), then
// rewrite the weights of hypercolumn h for the rows a swap touched (rewrite_w != null).
//
// NaN scores follow the reference's front-to-back scan: the scan's first row of a class holds the
// pick until a row compares better, and nothing compares better than NaN, so a class whose
// lowest-index row has a NaN score picks that row; a NaN score anywhere else is never picked.
// Besides the best rows, the replay therefore tracks the `iterations + 1` lowest-index rows of
// each class (one row leaves a class per swap) with their NaN flags; NaN rows are in no best list.
constexpr int kLowSlots = 2 * 32;   // >= kSwapMaxIter + 1 lowest-index rows per class, two per lane
template <typename T>
__global__ void __launch_bounds__(kSwapThreads)
    mask_replay_kernel(uint8_t *wmask, const T *__restrict__ nom, int *csum, long N, long M, long H, long Mc, long h,
                       int iterations, int chunks, const T *__restrict__ cand_v, const long *__restrict__ cand_i,
                       T *rewrite_w, const T *__restrict__ Ci, const T *__restrict__ Cj, const T *__restrict__ Cij,
                       T cthr, T cthr4) {
  typedef typename ScoreKey<T>::type K;
  constexpr int R1 = kSwapSlots / 4 / 32;   // registers per lane for a quarter of one class's chunk lists
  constexpr uint32_t kNone = 0xFFFFFFFFu;
  __shared__ T l1_v[2][4 * kSwapMaxIter], top_v[2][kSwapMaxIter];
  __shared__ long l1_i[2][4 * kSwapMaxIter], top_i[2][kSwapMaxIter];
  __shared__ uint32_t low_row[2][kLowSlots];
  __shared__ int low_cs[2][kLowSlots];
  __shared__ uint8_t low_nan[2][kLowSlots];
  __shared__ int low_cnt[2], win_cnt[kSwapThreads / 32][2];
  __shared__ long touched[2 * kSwapMaxIter];
  __shared__ int n_touched;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int total = chunks * iterations;   // entries per class, <= kSwapSlots
  if (threadIdx.x == 0) {
    n_touched = 0;
    low_cnt[0] = low_cnt[1] = 0;
  }
  for (int e = threadIdx.x; e < 2 * kLowSlots; e += blockDim.x) low_row[e / kLowSlots][e % kLowSlots] = kNone;
  __syncthreads();
  // the lowest-index rows of each class: windows of blockDim rows from row 0 until both lists are full
  const int want = iterations + 1;
  for (long w0 = 0; w0 < N; w0 += blockDim.x) {
    const long j = w0 + threadIdx.x;
    const uint8_t m = j < N ? wmask[j * H + h] : (uint8_t)2;
    unsigned bal[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      bal[c] = __ballot_sync(0xffffffffu, m == c);
      if (lane == 0) win_cnt[wid][c] = __popc(bal[c]);
    }
    __syncthreads();
    if (m <= 1) {
      int pos = low_cnt[m] + __popc(bal[m] & ((1u << lane) - 1u));
      for (int w = 0; w < wid; ++w) pos += win_cnt[w][m];
      if (pos < want) {
        const T nm = nom[j];
        low_row[m][pos] = (uint32_t)j;
        low_nan[m][pos] = nm != nm ? 1 : 0;
        low_cs[m][pos] = csum[j];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0)
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        low_cnt[0] += win_cnt[w][0];
        low_cnt[1] += win_cnt[w][1];
      }
    __syncthreads();
    if (low_cnt[0] >= want && low_cnt[1] >= want) break;   // uniform: read after the barrier
  }
  {
    const int cls = wid & 1, slice = wid >> 1;
    const int q = (total + 3) / 4, b = slice * q, e = b + q < total ? b + q : total;
    K key[R1];
    uint32_t row[R1];
#pragma unroll
    for (int r = 0; r < R1; ++r) {
      const int t = b + lane + 32 * r;
      const long i = t < e ? cand_i[(long)cls * total + t] : -1;
      key[r] = i >= 0 ? class_key<T>(cls, cand_v[(long)cls * total + t]) : (K)0;
      row[r] = i >= 0 ? (uint32_t)i : 0u;
    }
    warp_select_regs<T, R1>(cls, key, row, iterations, l1_v[cls] + slice * iterations, l1_i[cls] + slice * iterations);
  }
  __syncthreads();
  if (wid < 2) {
    K key[4];
    uint32_t row[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int e = lane + 32 * r;
      const long i = e < 4 * iterations ? l1_i[wid][e] : -1;
      key[r] = i >= 0 ? class_key<T>(wid, l1_v[wid][e]) : (K)0;
      row[r] = i >= 0 ? (uint32_t)i : 0u;
    }
    warp_select_regs<T, 4>(wid, key, row, iterations, top_v[wid], top_i[wid]);
  }
  __syncthreads();
  if (wid == 0) {
    // per class c: slot A = listed best row number `lane`; slot B = the row moved into the class by swap
    // `lane` (it may carry a NaN score: key 0, but still a member); L0, L1 = listed lowest rows lane, lane + 32
    K ka[2], kb[2] = {0, 0};
    uint32_t ra[2], rb[2] = {kNone, kNone}, l0[2], l1[2];
    T na[2], nb[2] = {(T)0, (T)0};
    int ca[2], cb[2] = {0, 0}, c0[2], c1[2];
    bool nanb[2] = {false, false}, n0[2], n1[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const long i = lane < iterations ? top_i[c][lane] : -1;
      ka[c] = i >= 0 ? class_key<T>(c, top_v[c][lane]) : (K)0;
      ra[c] = i >= 0 ? (uint32_t)i : kNone;
      na[c] = i >= 0 ? nom[i] : (T)0;
      ca[c] = i >= 0 ? csum[i] : 0;
      l0[c] = low_row[c][lane];      n0[c] = low_nan[c][lane] != 0;      c0[c] = low_cs[c][lane];
      l1[c] = low_row[c][lane + 32]; n1[c] = low_nan[c][lane + 32] != 0; c1[c] = low_cs[c][lane + 32];
    }
    const T quiet_nan = (T)NAN;
    for (int it = 0; it < iterations; ++it) {
      K best[2];
      uint32_t pick[2];
      bool pick_nan[2];
      bool stop = false;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        // the class's first row in index order, and whether its score is NaN
        uint32_t f = l0[c] < l1[c] ? l0[c] : l1[c];
        f = rb[c] < f ? rb[c] : f;
        const uint32_t first = __reduce_min_sync(0xffffffffu, f);
        const bool first_is_nan = __any_sync(0xffffffffu, first != kNone && ((l0[c] == first && n0[c]) ||
                                                                           (l1[c] == first && n1[c]) ||
                                                                           (rb[c] == first && nanb[c])));
        // the best row among those with a number for a score
        best[c] = ScoreKey<T>::warp_max(ka[c] > kb[c] ? ka[c] : kb[c]);
        uint32_t mine = 0;
        if (best[c] != 0 && ka[c] == best[c]) mine = ra[c] + 1u;
        if (best[c] != 0 && kb[c] == best[c] && rb[c] + 1u > mine) mine = rb[c] + 1u;
        const uint32_t win = __reduce_max_sync(0xffffffffu, mine);
        pick_nan[c] = first_is_nan;
        pick[c] = first_is_nan ? first : win - 1u;
        if (first == kNone || (!first_is_nan && best[c] == 0)) stop = true;   // the class is empty
      }
      // the best silent row scores below the worst active one (never true with a NaN on either side)
      if (stop || (!pick_nan[0] && !pick_nan[1] &&
                   class_key_value<T>(0, best[0]) < class_key_value<T>(1, best[1])))
        break;   // uniform across the warp
      T mv_nom[2];
      int mv_cs[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t p = pick[c];
        const bool own_a = ka[c] != 0 && ra[c] == p;
        const bool own_b = rb[c] == p;
        const bool own_l0 = l0[c] == p, own_l1 = l1[c] == p;
        // the slots of the best lists know the numerator; a row picked for its NaN is only in L or B
        unsigned who = __ballot_sync(0xffffffffu, own_a || own_b);
        if (who == 0) who = __ballot_sync(0xffffffffu, own_l0 || own_l1);
        const int src = __ffs(who) - 1;
        const T my_nom = own_a ? na[c] : (own_b ? nb[c] : quiet_nan);
        const int my_cs = own_a ? ca[c] : (own_b ? cb[c] : (own_l0 ? c0[c] : c1[c]));
        mv_nom[c] = __shfl_sync(0xffffffffu, my_nom, src);
        mv_cs[c] = __shfl_sync(0xffffffffu, my_cs, src);
        if (own_a) ka[c] = 0;
        if (own_b) { kb[c] = 0; rb[c] = kNone; nanb[c] = false; }
        if (own_l0) l0[c] = kNone;
        if (own_l1) l1[c] = kNone;
      }
      if (lane == it) {
        // the silent row becomes active with one more connection, the active row silent with one fewer
        const long up = (long)pick[0], down = (long)pick[1];
        rb[1] = pick[0]; nb[1] = mv_nom[0]; cb[1] = mv_cs[0] + 1; nanb[1] = pick_nan[0];
        kb[1] = nanb[1] ? (K)0 : class_key<T>(1, swap_score(nb[1], cb[1]));
        rb[0] = pick[1]; nb[0] = mv_nom[1]; cb[0] = mv_cs[1] - 1; nanb[0] = pick_nan[1];
        kb[0] = nanb[0] ? (K)0 : class_key<T>(0, swap_score(nb[0], cb[0]));
        wmask[up * H + h] = 1;
        wmask[down * H + h] = 0;
        csum[up] = cb[1];
        csum[down] = cb[0];
        touched[2 * it] = up;
        touched[2 * it + 1] = down;
        n_touched = 2 * it + 2;
      }
    }
  }
  __syncthreads();
  if (rewrite_w == nullptr) return;
  // a touched row's weights in hypercolumn h follow its final mask bit (idempotent when a row was touched
  // twice).  Row data first (one thread per touched row), so that the element loop has independent loads only.
  __shared__ T t_ci[2 * kSwapMaxIter];
  __shared__ uint8_t t_on[2 * kSwapMaxIter];
  const int nt = n_touched;
  if ((int)threadIdx.x < nt) {
    const long i = touched[threadIdx.x];
    const T ci = Ci[i];
    t_ci[threadIdx.x] = ci;
    t_on[threadIdx.x] = wmask[i * H + h] != 0 && !(ci < cthr);
  }
  __syncthreads();
  const long total_elems = (long)nt * Mc;
#pragma unroll 4
  for (long t = threadIdx.x; t < total_elems; t += blockDim.x) {
    const int r = (int)(t / Mc);
    const long i = touched[r], col = h * Mc + t % Mc;
    const T cj = Cj[col];
    const T cij = Cij[i * M + col];
    T v = (T)0;
    if (t_on[r] && !(cj < cthr)) v = log_ratio(cij, t_ci[r], cj, cthr4);
    rewrite_w[i * M + col] = v;
  }
}

__host__ __device__ static inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }
static constexpr size_t kSwapListBytes = 256 + (size_t)2 * kSwapSlots * (sizeof(double) + sizeof(long));

size_t mask_scratch_bytes(long N, size_t elem) {
  return align256((size_t)N * elem) + align256((size_t)N * sizeof(int)) + align256((size_t)N) + kSwapListBytes;
}

// Scratch layout: [score N x T][active count N x int][old mask column N bytes][nan flag, candidate lists].
template <typename T>
struct MaskScratch {
  T *score;
  int *csum;
  uint8_t *old_col;
  int *nan_flag;
  long *cand_i;
  T *cand_v;
  __host__ __device__ MaskScratch(void *scratch, long N) {
    unsigned char *p = static_cast<unsigned char *>(scratch);
    score = reinterpret_cast<T *>(p);
    p += align256((size_t)N * sizeof(T));
    csum = reinterpret_cast<int *>(p);
    p += align256((size_t)N * sizeof(int));
    old_col = p;
    p += align256((size_t)N);
    nan_flag = reinterpret_cast<int *>(p);
    cand_i = reinterpret_cast<long *>(p + 256);
    cand_v = reinterpret_cast<T *>(p + 256 + (size_t)2 * kSwapSlots * sizeof(long));
  }
};

template <typename T>
cudaError_t launch_mask_update(uint8_t *wmask, const T *weights, const T *Ci, const T *Cj, const T *Cij, T cthr,
                               long N, long M, long H, long Mc, long h, long iterations, void *scratch,
                               cudaStream_t st, T *rewrite_w) {
  if (N == 0) return cudaSuccess;
  MaskScratch<T> ms(scratch, N);
  const T cthr4 = cthr * cthr * cthr * cthr;
  mask_score_kernel<T><<<(unsigned)((N + 7) / 8), 256, 0, st>>>(wmask, weights, Ci, Cj, Cij, cthr, cthr4, N, M, H, Mc,
                                                                 h, ms.score, ms.csum, ms.old_col);
  cudaError_t e = launched();
  if (e != cudaSuccess) return e;
  return launch_mask_select<T>(wmask, Ci, Cj, Cij, cthr, N, M, H, Mc, h, iterations, scratch, st, rewrite_w);
}

// The swaps alone, from per-row scores, active counts and the old mask column already in `scratch`.
template <typename T>
cudaError_t launch_mask_select(uint8_t *wmask, const T *Ci, const T *Cj, const T *Cij, T cthr, long N, long M, long H,
                               long Mc, long h, long iterations, void *scratch, cudaStream_t st, T *rewrite_w) {
  if (N == 0) return cudaSuccess;
  MaskScratch<T> ms(scratch, N);
  const T cthr4 = cthr * cthr * cthr * cthr;
  cudaError_t e = cudaSuccess;
  // candidate lists: rows fit 32-bit indices and a chunk (<= kSwapCacheRows rows) fits shared memory
  const int max_chunks = iterations >= 1 && iterations <= kSwapMaxIter ? kSwapSlots / (int)iterations : 0;
  if (max_chunks > 0 && N >= 1024 && N < (1l << 31) && (N + max_chunks - 1) / max_chunks <= kSwapCacheRows) {
    int chunks = (int)((N + 767) / 768);
    if (chunks > max_chunks) chunks = max_chunks;
    const long rows_per_chunk = (N + chunks - 1) / chunks;
    chunks = (int)((N + rows_per_chunk - 1) / rows_per_chunk);
    const size_t dyn = (size_t)rows_per_chunk * (sizeof(T) + 1);
    const long slice = (rows_per_chunk + 3) / 4;   // rows one warp keeps in registers, 32 per register
#define SBB_CAND(R)                                                                                              \
  mask_candidates_kernel<T, R><<<chunks, kSwapThreads, dyn, st>>>(wmask, ms.score, ms.csum, N, H, h, (int)iterations, \
                                                                  rows_per_chunk, ms.cand_v, ms.cand_i)
    if (slice <= 4 * 32) SBB_CAND(4);
    else if (slice <= 8 * 32) SBB_CAND(8);
    else if (slice <= 16 * 32) SBB_CAND(16);
    else SBB_CAND(32);
#undef SBB_CAND
    e = launched();
    if (e != cudaSuccess) return e;
    mask_replay_kernel<T><<<1, kSwapThreads, 0, st>>>(wmask, ms.score, ms.csum, N, M, H, Mc, h, (int)iterations, chunks,
                                                     ms.cand_v, ms.cand_i, rewrite_w, Ci, Cj, Cij, cthr, cthr4);
    return launched();
  }
  mask_swap_kernel<T><<<1, 1024, 0, st>>>(wmask, ms.score, ms.csum, N, M, H, Mc, h, iterations, rewrite_w,
                                          ms.old_col, Ci, Cj, Cij, cthr, cthr4);
  return launched();
}
template cudaError_t launch_mask_select<float>(uint8_t *, const float *, const float *, const float *, float, long, long,
                                               long, long, long, long, void *, cudaStream_t, float *);
template cudaError_t launch_mask_select<double>(uint8_t *, const double *, const double *, const double *, double, long,
                                                long, long, long, long, long, void *, cudaStream_t, double *);
template cudaError_t launch_mask_update<float>(uint8_t *, const float *, const float *, const float *, const float *,
                                               float, long, long, long, long, long, long, void *, cudaStream_t,
                                               float *);
template cudaError_t launch_mask_update<double>(uint8_t *, const double *, const double *, const double *,
                                                const double *, double, long, long, long, long, long, long, void *,
                                                cudaStream_t, double *);


// ----------------------------------------------------------------------------
// Evaluation helper: rows whose predicted class equals the labelled class
// (first maximum wins, as numpy.argmax).
// ----------------------------------------------------------------------------
template <typename T>
__global__ void count_correct_kernel(const T *__restrict__ pred, const T *__restrict__ labels, long rows, long classes,
                                     unsigned long long *count) {
  const long r = (long)blockIdx.x * blockDim.x + threadIdx.x;
  bool hit = false;
  if (r < rows) {
    long ap = 0, al = 0;
    T vp = pred[r * classes], vl = labels[r * classes];
    for (long c = 1; c < classes; ++c) {
      const T p = pred[r * classes + c], l = labels[r * classes + c];
      if (p > vp) { vp = p; ap = c; }
      if (l > vl) { vl = l; al = c; }
    }
    hit = ap == al;
  }
  const unsigned ballot = __ballot_sync(0xffffffffu, hit);
  if ((threadIdx.x & 31) == 0 && ballot) atomicAdd(count, (unsigned long long)__popc(ballot));
}
template <typename T>
cudaError_t launch_count_correct(const T *pred, const T *labels, long rows, long classes, unsigned long long *count,
                                 cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  count_correct_kernel<T><<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(pred, labels, rows, classes, count);
  return launched();
}
template cudaError_t launch_count_correct<float>(const float *, const float *, long, long, unsigned long long *,
                                                 cudaStream_t);
template cudaError_t launch_count_correct<double>(const double *, const double *, long, long, unsigned long long *,
                                                  cudaStream_t);

// ----------------------------------------------------------------------------
// Batch assembly: dst[r, :] = src[order[first + r], :] (order null: the identity).  One
// warp copies one row in 16-byte pieces when the row pitch allows, else element-wise.
// HBM-bound: rows * cols * sizeof(T) read and written.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const T *__restrict__ src, const long *__restrict__ order, long first, long rows, long cols,
                       T *__restrict__ dst, int vec16) {
  const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long r = warp; r < rows; r += nwarps) {
    const long from = order ? order[first + r] : first + r;
    const T *s = src + from * cols;
    T *d = dst + r * cols;
    if (vec16) {
      const long pieces = cols * (long)sizeof(T) / 16;
      const uint4 *s4 = reinterpret_cast<const uint4 *>(s);
      uint4 *d4 = reinterpret_cast<uint4 *>(d);
      for (long k = lane; k < pieces; k += 32) d4[k] = __ldg(s4 + k);
    } else {
      for (long k = lane; k < cols; k += 32) d[k] = s[k];
    }
  }
}
template <typename T>
cudaError_t launch_gather_rows(const T *src, const long *order, long first, long rows, long cols, T *dst,
                               cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  const int vec16 = (cols * (long)sizeof(T)) % 16 == 0 && aligned16(src) && aligned16(dst);
  const long blocks = (rows + 7) / 8;   // eight warps per block, one row per warp and pass
  const int cap = sm_count() * 8;
  gather_rows_kernel<T><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(src, order, first, rows, cols, dst,
                                                                                 vec16);
  return launched();
}
template cudaError_t launch_gather_rows<float>(const float *, const long *, long, long, long, float *, cudaStream_t);
template cudaError_t launch_gather_rows<double>(const double *, const long *, long, long, long, double *,
                                                cudaStream_t);

// ----------------------------------------------------------------------------
// Row-sharded layer over peer-mapped memory.  Every rank owns a block of input rows of
// the layer (those rows of the weights, of Cij and of Ci).  Per step the ranks exchange the
// matching COLUMNS of their input batches, so that every owner holds its columns of the
// whole global batch; each owner then forms its part of every sample's support, the parts
// are summed across the ranks, and the owner updates its rows from the global batch.
// The pointer tables below hold, per destination rank, an address in that rank's memory
// (the rank's own entry is a local address).
// ----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) peer_broadcast_kernel(const T *__restrict__ src, long n, PeerTable dst) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const T v = src[i];
    for (int d = 0; d < dst.n; ++d) static_cast<T *>(dst.ptr[d])[i] = v;
  }
}
template <typename T>
cudaError_t launch_peer_broadcast(const T *src, long n, const PeerTable &dst, cudaStream_t st) {
  if (n <= 0 || dst.n <= 0) return cudaSuccess;
  const long blocks = (n + 255) / 256;
  peer_broadcast_kernel<T><<<(unsigned)(blocks < 1184 ? blocks : 1184), 256, 0, st>>>(src, n, dst);
  return launched();
}
template cudaError_t launch_peer_broadcast<float>(const float *, long, const PeerTable &, cudaStream_t);
template cudaError_t launch_peer_broadcast<double>(const double *, long, const PeerTable &, cudaStream_t);
template cudaError_t launch_peer_broadcast<uint4>(const uint4 *, long, const PeerTable &, cudaStream_t);

// Column block o of x[B, N] (columns [o * block, min(N, (o + 1) * block))) goes to rank o as a dense
// [B, width_o] matrix at dst.ptr[o].  V = elements moved per thread (a 16-byte vector when the shapes allow).
// Blocks of 128 threads with few registers, so that the kernel can run on a side stream beside a
// tensor-core contraction, whose one CTA per SM leaves room for little else.
template <typename T, int V>
__global__ void __launch_bounds__(128)
    scatter_columns_kernel(const T *__restrict__ x, long B, long N, long block, PeerTable dst) {
  struct alignas(sizeof(T) * V) Pack {
    T v[V];
  };
  const long per_row = N / V;
  const long total = B * per_row;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
    const long b = t / per_row;
    const long c = (t - b * per_row) * V;
    const long o = c / block;
    const long first = o * block;
    const long width = first + block <= N ? block : N - first;
    const Pack v = *reinterpret_cast<const Pack *>(x + b * N + c);
    *reinterpret_cast<Pack *>(static_cast<T *>(dst.ptr[o]) + b * width + (c - first)) = v;
  }
}
template <typename T>
cudaError_t launch_scatter_columns(const T *x, long B, long N, long block, const PeerTable &dst, cudaStream_t st) {
  if (B <= 0 || N <= 0) return cudaSuccess;
  constexpr int V = Vec16<T>::N;
  // a vector never straddles two owners when both N and the block width are multiples of V
  bool vec = N % V == 0 && block % V == 0 && aligned16(x);
  for (int d = 0; d < dst.n; ++d) vec = vec && aligned16(dst.ptr[d]);
  const long total = vec ? B * (N / V) : B * N;
  const long blocks = (total + 127) / 128;
  const unsigned grid = (unsigned)(blocks < 2368 ? blocks : 2368);
  if (vec) scatter_columns_kernel<T, V><<<grid, 128, 0, st>>>(x, B, N, block, dst);
  else scatter_columns_kernel<T, 1><<<grid, 128, 0, st>>>(x, B, N, block, dst);
  return launched();
}
template cudaError_t launch_scatter_columns<float>(const float *, long, long, long, const PeerTable &, cudaStream_t);
template cudaError_t launch_scatter_columns<double>(const double *, long, long, long, const PeerTable &, cudaStream_t);

// out[i] = sum over s (in order) of partial[s * n + i]
template <typename T>
__global__ void __launch_bounds__(256) sum_partials_kernel(const T *__restrict__ partial, int splits, long n, T *out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    T s = partial[i];
    for (int k = 1; k < splits; ++k) s += partial[(long)k * n + i];
    out[i] = s;
  }
}
template <typename T>
cudaError_t launch_sum_partials(const T *partial, int splits, long n, T *out, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const long blocks = (n + 255) / 256;
  sum_partials_kernel<T><<<(unsigned)(blocks < 2368 ? blocks : 2368), 256, 0, st>>>(partial, splits, n, out);
  return launched();
}
template cudaError_t launch_sum_partials<float>(const float *, int, long, float *, cudaStream_t);
template cudaError_t launch_sum_partials<double>(const double *, int, long, double *, cudaStream_t);

// Mask scores of the rows [row_begin, row_end) this rank owns, written into every rank's work arrays
// (scratch_tab: base of each rank's mask scratch, laid out for N rows).
template <typename T>
__global__ void __launch_bounds__(256)
    mask_score_rows_kernel(const uint8_t *__restrict__ wmask, const T *__restrict__ Ci, const T *__restrict__ Cj,
                           const T *__restrict__ Cij, T cthr, T cthr4, long N, long M, long H, long Mc, long h,
                           long row_begin, long row_end, PeerTable scratch_tab) {
  const int lane = threadIdx.x & 31;
  const long i = row_begin + (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= row_end) return;
  const T pi = Ci[i];
  double s = 0.0;
  if (pi >= cthr) {
    for (long jj = lane; jj < Mc; jj += 32) {
      const long col = h * Mc + jj;
      const T pj = Cj[col];
      if (pj >= cthr) {
        const T pij = Cij[i * M + col];
        const T w = log_ratio(pij, pi, pj, cthr4);
        const T x = ((T)1 - pi) * pj;
        const T y = (pj - pij) / x;
        s += (double)(pij * w + (pj - pij) * sbb_log(y));
      }
    }
  }
  int cnt = 0;
  for (long k = lane; k < H; k += 32) cnt += wmask[i * H + k];
  for (int off = 16; off > 0; off >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, off);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
  }
  if (lane == 0) {
    const uint8_t bit = wmask[i * H + h];
    for (int d = 0; d < scratch_tab.n; ++d) {
      MaskScratch<T> ms(scratch_tab.ptr[d], N);
      ms.score[i] = (T)s;
      ms.csum[i] = cnt;
      ms.old_col[i] = bit;
    }
  }
}
template <typename T>
cudaError_t launch_mask_score_rows(const uint8_t *wmask, const T *Ci, const T *Cj, const T *Cij, T cthr, long N, long M,
                                   long H, long Mc, long h, long row_begin, long row_end, const PeerTable &scratch_tab,
                                   cudaStream_t st) {
  if (row_end <= row_begin) return cudaSuccess;
  const T cthr4 = cthr * cthr * cthr * cthr;
  mask_score_rows_kernel<T><<<(unsigned)((row_end - row_begin + 7) / 8), 256, 0, st>>>(
      wmask, Ci, Cj, Cij, cthr, cthr4, N, M, H, Mc, h, row_begin, row_end, scratch_tab);
  return launched();
}
template cudaError_t launch_mask_score_rows<float>(const uint8_t *, const float *, const float *, const float *, float,
                                                   long, long, long, long, long, long, long, const PeerTable &,
                                                   cudaStream_t);
template cudaError_t launch_mask_score_rows<double>(const uint8_t *, const double *, const double *, const double *,
                                                    double, long, long, long, long, long, long, long, const PeerTable &,
                                                    cudaStream_t);

// After the swaps: owned rows whose mask bit changed get hypercolumn h's weights recomputed from the owner's
// traces, in every rank's weight matrix.  One warp per owned row.
template <typename T>
__global__ void __launch_bounds__(256)
    mask_rewrite_rows_kernel(const uint8_t *__restrict__ wmask, const uint8_t *__restrict__ old_col,
                             const T *__restrict__ Ci, const T *__restrict__ Cj, const T *__restrict__ Cij, T cthr,
                             T cthr4, long M, long H, long Mc, long h, long row_begin, long row_end, PeerTable wtab) {
  const int lane = threadIdx.x & 31;
  const long i = row_begin + (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= row_end) return;
  const uint8_t now = wmask[i * H + h];
  if (now == old_col[i]) return;
  const T ci = Ci[i];
  for (long jj = lane; jj < Mc; jj += 32) {
    const long col = h * Mc + jj;
    const T cj = Cj[col];
    T v = (T)0;
    if (now != 0 && !(ci < cthr) && !(cj < cthr)) v = log_ratio(Cij[i * M + col], ci, cj, cthr4);
    for (int d = 0; d < wtab.n; ++d) static_cast<T *>(wtab.ptr[d])[i * M + col] = v;
  }
}
template <typename T>
cudaError_t launch_mask_rewrite_rows(const uint8_t *wmask, const void *scratch, const T *Ci, const T *Cj, const T *Cij,
                                     T cthr, long N, long M, long H, long Mc, long h, long row_begin, long row_end,
                                     const PeerTable &wtab, cudaStream_t st) {
  if (row_end <= row_begin) return cudaSuccess;
  MaskScratch<T> ms(const_cast<void *>(scratch), N);
  const T cthr4 = cthr * cthr * cthr * cthr;
  mask_rewrite_rows_kernel<T><<<(unsigned)((row_end - row_begin + 7) / 8), 256, 0, st>>>(
      wmask, ms.old_col, Ci, Cj, Cij, cthr, cthr4, M, H, Mc, h, row_begin, row_end, wtab);
  return launched();
}
template cudaError_t launch_mask_rewrite_rows<float>(const uint8_t *, const void *, const float *, const float *,
                                                     const float *, float, long, long, long, long, long, long, long,
                                                     const PeerTable &, cudaStream_t);
template cudaError_t launch_mask_rewrite_rows<double>(const uint8_t *, const void *, const double *, const double *,
                                                      const double *, double, long, long, long, long, long, long, long,
                                                      const PeerTable &, cudaStream_t);

}  // namespace sbb

// ----------------------------------------------------------------------------
// Measured float64 rates of the device, for the roofline of the float64 kernels:
// a register-resident DFMA loop and a loop of mma.sync.m8n8k4 (the float64 tensor-core
// instruction).  Both keep every operand in registers; the result is stored once so
// that the loops are not removed.
// ----------------------------------------------------------------------------
namespace sbb {
namespace {
__global__ void __launch_bounds__(256) dfma_rate_kernel(double *out, int iters) {
  double a[8];
  const double x = 1.0 + 1e-9 * threadIdx.x, y = 1e-9;
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = (double)k;
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = fma(a[k], x, y);
  }
  double s = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += a[k];
  if (s == 12345.678) out[0] = s;   // never true: keeps the loop alive
}
__global__ void __launch_bounds__(256) dmma_rate_kernel(double *out, int iters) {
  double c[4][2];
  const double a = 1.0 + 1e-9 * threadIdx.x, b = 1e-9;
#pragma unroll
  for (int k = 0; k < 4; ++k) c[k][0] = c[k][1] = (double)k;
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                   : "+d"(c[k][0]), "+d"(c[k][1])
                   : "d"(a), "d"(b));
  }
  double s = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) s += c[k][0] + c[k][1];
  if (s == 12345.678) out[0] = s;
}
}  // namespace

// TFLOP/s of both loops on the current device (CUDA events, best of three launches).
cudaError_t measure_fp64_rates(double *dfma_tflops, double *dmma_tflops) {
  double *out = nullptr;
  cudaError_t e = cudaMalloc(&out, sizeof(double));
  if (e != cudaSuccess) return e;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const int blocks = sm_count() * 4, iters = 20000;
  double best[2] = {0.0, 0.0};
  for (int which = 0; which < 2; ++which)
    for (int rep = 0; rep < 4; ++rep) {
      cudaEventRecord(e0, 0);
      if (which == 0) dfma_rate_kernel<<<blocks, 256>>>(out, iters);
      else dmma_rate_kernel<<<blocks, 256>>>(out, iters);
      cudaEventRecord(e1, 0);
      e = cudaEventSynchronize(e1);
      if (e != cudaSuccess) break;
      launched();
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      // DFMA: 8 FMAs per thread and iteration; DMMA: 4 instructions of 8 x 8 x 4 FMAs per warp and iteration
      const double flops = which == 0 ? 2.0 * 8 * iters * 256.0 * blocks : 2.0 * 4 * 256 * iters * 8.0 * blocks;
      const double tf = flops / (ms * 1e-3) / 1e12;
      if (rep > 0 && tf > best[which]) best[which] = tf;
    }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(out);
  if (e != cudaSuccess) return e;
  *dfma_tflops = best[0];
  *dmma_tflops = best[1];
  return cudaGetLastError();
}
}  // namespace sbb
