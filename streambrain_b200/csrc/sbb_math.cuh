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

}  // namespace sbb
