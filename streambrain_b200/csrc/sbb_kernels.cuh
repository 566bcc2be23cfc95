// Launch interface of the BCPNN layer kernels (device pointers, asynchronous on
// the given stream).  Every launcher returns cudaSuccess or the launch error and
// bumps the process-wide launch counter once per kernel launched.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sbb {

// Scalars of the trace / weight arithmetic, already rounded to REAL.
template <typename T>
struct TraceParams {
  T taupdt;     // trace time constant
  T one_minus;  // (REAL)(1.0 - (double)taupdt)
  T batch;      // divisor of the batch sums (global batch under data parallelism)
  T cthr;       // taupdt / 2
  T cthr4;      // cthr^4, floor of Cij inside the logarithm
};

template <typename T>
TraceParams<T> make_trace_params(double taupdt, double cthr, long batch);

unsigned long long kernel_launches();

// Number of K-splits the forward product uses for a [B,N]x[N,M] problem and the
// number of REALs of scratch (splits*B*M) it needs.
template <typename T>
int forward_splits(long B, long N, long M);

// partial[s, B, M] = x[B, N(k-range s)] * w[N, M]   (s = 0..splits-1)
template <typename T>
cudaError_t launch_forward_product(const T *x, const T *w, T *partial, long B, long N, long M, int splits,
                                   cudaStream_t st);

// out[r, :] = sum_s partial[s, r, :] + bias, then (softmax != 0) the softmax over
// every group of Mc entries.  partial may alias out when splits == 1; bias may be null.
template <typename T>
cudaError_t launch_reduce_bias_softmax(const T *partial, int splits, const T *bias, T *out, long rows, long H,
                                       long Mc, int softmax, cudaStream_t st);

// sums[j] = sum_b a[b, j]                       (ema == 0)
// c[j]    = EMA(c[j], sum_b a[b, j])            (ema != 0; sums unused)
// lo != nullptr (float32): also writes lo[b, j] = the low part of a[b, j] for a split TF32 product (sbb_math.cuh).
template <typename T>
cudaError_t launch_colsum(const T *a, long B, long cols, T *sums, T *c, TraceParams<T> p, int ema, cudaStream_t st,
                          T *lo = nullptr);

// c[j] = EMA(c[j], sums[j])
template <typename T>
cudaError_t launch_vector_ema(T *c, const T *sums, long n, TraceParams<T> p, cudaStream_t st);

// Fused trace step for rows [row_begin,row_end) of Cij: acc = x^T y over the batch,
// Cij = EMA(Cij, acc), w = log-ratio(Cij, Ci, Cj) with rows/columns below cthr and
// masked connections (wmask may be null) set to zero.  Ci, Cj hold the NEW values.
template <typename T>
cudaError_t launch_trace_update_fused(const T *x, const T *y, long B, long N, long M, long H, long Mc, const T *Ci,
                                      const T *Cj, T *Cij, T *w, const uint8_t *wmask, TraceParams<T> p,
                                      long row_begin, long row_end, cudaStream_t st);

// delta[i, j] = sum_b x[b, i] y[b, j] for rows [row_begin,row_end)  (delta is [N, M])
template <typename T>
cudaError_t launch_outer_product(const T *x, const T *y, long B, long N, long M, T *delta, long row_begin,
                                 long row_end, cudaStream_t st);

// Element-wise tail of the trace step from precomputed sums (delta may be null when
// only the weights are to be recomputed from the current traces: ema == 0).
template <typename T>
cudaError_t launch_trace_apply(const T *delta, long N, long M, long H, long Mc, const T *Ci, const T *Cj, T *Cij,
                               T *w, const uint8_t *wmask, TraceParams<T> p, int ema, long row_begin, long row_end,
                               cudaStream_t st, bool fast = false);

// Un-fused Cij update with the numpy operation order: (1-t)*C + t*(sum/B).
template <typename T>
cudaError_t launch_counters_apply(T *c, const T *sums, long n, T taupdt, T batch, cudaStream_t st);

template <typename T>
cudaError_t launch_update_bias(T *bias, const T *Cj, T cthr, long M, cudaStream_t st);

template <typename T>
cudaError_t launch_update_bias_regularized(T *bias, T *kbi, const T *Cj, T cthr, T khalf, T pmin, T taubdt, long M,
                                           cudaStream_t st);

template <typename T>
cudaError_t launch_add_bias(T *a, const T *bias, long rows, long M, cudaStream_t st);

template <typename T>
cudaError_t launch_apply_mask(T *w, const uint8_t *wmask, long N, long M, long H, long Mc, cudaStream_t st);

// Mask update for hypercolumn h.  `weights` null => the un-masked weight is
// recomputed from the traces.  `scratch` holds mask_scratch_bytes(N, sizeof(T))
// bytes (256-byte aligned): per-row score, active count and previous mask bit, candidate lists.
// `rewrite_w` non-null => the weights of hypercolumn h are recomputed from the traces, under the
// new mask, for every row whose mask bit a swap changed.
size_t mask_scratch_bytes(long N, size_t elem);
template <typename T>
cudaError_t launch_mask_update(uint8_t *wmask, const T *weights, const T *Ci, const T *Cj, const T *Cij, T cthr,
                               long N, long M, long H, long Mc, long h, long iterations, void *scratch,
                               cudaStream_t st, T *rewrite_w = nullptr);

template <typename T>
cudaError_t launch_count_correct(const T *pred, const T *labels, long rows, long classes, unsigned long long *count,
                                 cudaStream_t st);

// The swaps of a mask update alone, from per-row scores / active counts / old mask column already in `scratch`.
template <typename T>
cudaError_t launch_mask_select(uint8_t *wmask, const T *Ci, const T *Cj, const T *Cij, T cthr, long N, long M, long H,
                               long Mc, long h, long iterations, void *scratch, cudaStream_t st, T *rewrite_w);

// Row-sharded layer over peer-mapped memory (see sbb_kernels.cu): one address per destination rank.
constexpr int kMaxPeers = 8;
struct PeerTable {
  void *ptr[kMaxPeers];
  int n;
};
template <typename T>
cudaError_t launch_peer_broadcast(const T *src, long n, const PeerTable &dst, cudaStream_t st);
// Column block o (of width `block`, the last one clipped to N) of x[B, N] -> dense [B, width_o] matrix at dst.ptr[o].
template <typename T>
cudaError_t launch_scatter_columns(const T *x, long B, long N, long block, const PeerTable &dst, cudaStream_t st);
// out[i] = sum_s partial[s * n + i]
template <typename T>
cudaError_t launch_sum_partials(const T *partial, int splits, long n, T *out, cudaStream_t st);
template <typename T>
cudaError_t launch_mask_score_rows(const uint8_t *wmask, const T *Ci, const T *Cj, const T *Cij, T cthr, long N, long M,
                                   long H, long Mc, long h, long row_begin, long row_end, const PeerTable &scratch_tab,
                                   cudaStream_t st);
template <typename T>
cudaError_t launch_mask_rewrite_rows(const uint8_t *wmask, const void *scratch, const T *Ci, const T *Cj, const T *Cij,
                                     T cthr, long N, long M, long H, long Mc, long h, long row_begin, long row_end,
                                     const PeerTable &wtab, cudaStream_t st);

// Measured float64 rates (TFLOP/s) of the current device: a register-resident DFMA loop and a loop of the
// float64 tensor-core instruction mma.sync.m8n8k4.  Synchronises; takes a few milliseconds.
cudaError_t measure_fp64_rates(double *dfma_tflops, double *dmma_tflops);

// dst[r, :] = src[order[first + r], :] for r in [0, rows); order == nullptr means the identity.
template <typename T>
cudaError_t launch_gather_rows(const T *src, const long *order, long first, long rows, long cols, T *dst,
                               cudaStream_t st);

}  // namespace sbb
