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

// Variants used in the tensor-core epilogue, where eight warps per SM do the arithmetic of a
// whole 128 x 256 tile: the batch mean by reciprocal multiply, the ratio by the hardware
// reciprocal (2 ulp) and the logarithm by lg2.approx (absolute error below 2^-21 near 1,
// 3 ulp elsewhere) -- about a quarter of the instructions of the IEEE forms above, and well
// inside the tolerance of the weights (which are a logarithm of a ratio of noisy traces).
__device__ __forceinline__ float trace_ema_fast(float old, float sum, const TraceParams<float> &p, float inv_batch) {
  const float tmp = (sum * inv_batch) * p.taupdt;
  return fmaxf(fmaf(old, p.one_minus, tmp), 0.f);
}
__device__ __forceinline__ float log_ratio_fast(float cij, float ci, float cj, float cthr4) {
  return __logf(__fdividef(fmaxf(cij, cthr4), ci * cj));
}

}  // namespace sbb
