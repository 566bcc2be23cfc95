// Launch interface of the tcgen05 (5th-generation tensor core) contraction
// kernels: float32 operands multiplied as three TF32 products with float32
// accumulation in tensor memory, operands fetched by TMA.  Only shapes whose
// row pitches are multiples of 16 bytes are eligible; callers fall back to the
// general-shape kernels otherwise.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sbb_kernels.cuh"

namespace sbb {

// True when the current device is compute capability 10.x and the driver's
// tensor-map encoder could be resolved.
bool tc_available();

// Row pitches of x[B,N], y[B,M] / w[N,M] must be multiples of 16 bytes and the
// base pointers 16-byte aligned.
bool tc_shape_ok(const void *x, const void *y_or_w, long N, long M);

// Number of k-splits the tensor-core forward product uses (scratch = splits*B*M floats).
int forward_splits_tc(long B, long N, long M);

// partial[s, B, M] = x[B, k-range s] * w[N, M]
cudaError_t launch_forward_product_tc(const float *x, const float *w, float *partial, long B, long N, long M,
                                      int splits, cudaStream_t st);

// Fused trace step (same contract as launch_trace_update_fused); col_hc[j] = j / Mc.
// `scratch` holds tc_trace_scratch_bytes(N, M) bytes, 16-byte aligned (threshold-gated
// reciprocals of Ci and Cj, written by a small kernel ahead of the contraction).
size_t tc_trace_scratch_bytes(long N, long M);
cudaError_t launch_trace_update_tc(const float *x, const float *y, long B, long N, long M, long H,
                                   const float *Ci, const float *Cj, float *Cij, float *w, const uint8_t *wmask,
                                   const int *col_hc, float *scratch, TraceParams<float> p, long row_begin,
                                   long row_end, cudaStream_t st);

// delta[i, j] = sum_b x[b, i] y[b, j] for rows [row_begin,row_end)
// x_lo / y_lo (both or neither): planes of the operands' low parts as launch_colsum writes them; with them the
// kernel takes both halves of both operands by TMA and converts nothing itself.
cudaError_t launch_outer_product_tc(const float *x, const float *y, long B, long N, long M, float *delta,
                                    long row_begin, long row_end, cudaStream_t st, const float *x_lo = nullptr,
                                    const float *y_lo = nullptr);

// Multiprocessors launch_outer_product_tc leaves free for kernels of other streams.
void tc_set_reserved_sms(int sms);
int tc_get_reserved_sms();

// Time limit of one device-side wait in SM clock cycles (default 4e9, about two seconds), process-wide.
void tc_set_wait_limit(long long cycles);
long long tc_get_wait_limit();
// Test hook: each of the next `launches` tensor-core launches that convert operands inside the kernel loses one
// barrier arrival in its first CTA, so that a wait there runs into its time limit.
void tc_debug_lose_arrive(int launches);

// Status word of the bounded device-side waits on the current device: 0 = all
// waits completed, otherwise the code of the first wait that gave up.
// Synchronises the device.
cudaError_t tc_read_status(int *status);
// The same word read without synchronising (for callers that have just waited for their own work),
// and reset to 0 (synchronises the device first).
cudaError_t tc_peek_status(int *status);
cudaError_t tc_clear_status();

}  // namespace sbb
