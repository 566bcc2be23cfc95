// Device arithmetic shared by every kernel that touches a trace or a weight, so
// that the general-shape kernels and the tensor-core kernels produce the same
// values from the same batch sums.
#pragma once
#include "sbb_kernels.cuh"

#include <math.h>

namespace sbb {

__device__ __forceinline__ float sbb_log(float x) { return logf(x); }
__device__ __forceinline__ double sbb_log(double x) { return log(x); }
__device__ __forceinline__ float sbb_exp(float x) { return expf(x); }
__device__ __forceinline__ double sbb_exp(double x) { return exp(x); }

// One moving-average step from a batch sum: sum/B, *taupdt, old*(1-taupdt), add,
// clamp at zero (a NaN clamps to zero, as std::max(0, NaN) does).
template <typename T>
__device__ __forceinline__ T trace_ema(T old, T sum, const TraceParams<T> &p) {
  T tmp = sum / p.batch;
  tmp = tmp * p.taupdt;
  T c = old * p.one_minus;
  c = c + tmp;
  return c > (T)0 ? c : (T)0;
}

template <typename T>
__device__ __forceinline__ T log_ratio(T cij, T ci, T cj, T cthr4) {
  const T num = cij < cthr4 ? cthr4 : cij;
  return sbb_log(num / (ci * cj));
}

// The arithmetic of the tensor-core path (fused epilogue, and the element-wise tail of the
// data-parallel step when that path is selected): the batch mean and the moving-average weight
// folded into one factor taupdt / batch, the ratio by IEEE reciprocals of Ci and Cj formed once per
// row / column, the logarithm by lg2.approx (relative error below 2^-22) -- about a quarter of the
// instructions of the IEEE forms above, and well inside the tolerance of the weights (which are a
// logarithm of a ratio of noisy traces).
__device__ __forceinline__ float trace_ema_fast(float old, float sum, float one_minus, float ema_scale) {
  return fmaxf(fmaf(old, one_minus, sum * ema_scale), 0.f);
}
__device__ __forceinline__ float log_ratio_fast(float cij, float rci, float rcj, float cthr4) {
  return __log2f(fmaxf(cij, cthr4) * (rci * rcj)) * 0.693147180559945309f;
}

// The "lo" part of a float32 value v for a product carried by TF32 tensor cores.  The tensor core reads
// only the upper 19 bits of a 32-bit operand, so the untouched value already acts as hi = v truncated to TF32
// and only lo = v - hi (exact) has to be produced; it is rounded to the 11 significant bits of TF32 (Veltkamp
// split with 2^13 + 1, all on the FMA pipe), so that what the tensor core drops of it is zero.  hi + lo then
// differs from v by at most 2^-22 |v|.  Inf / NaN give a NaN lo.
__device__ __forceinline__ float tf32_lo(float v) {
  const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  const float lo = __fsub_rn(v, hi);
  const float c = __fmul_rn(lo, 8193.f);
  return __fsub_rn(c, __fsub_rn(c, lo));
}
__device__ __forceinline__ double tf32_lo(double v) { return v; }   // never used: float64 has no tensor path

}  // namespace sbb
