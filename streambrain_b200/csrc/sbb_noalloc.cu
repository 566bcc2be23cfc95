// Mask update for callers that are not allowed to allocate device memory.
//
// Some hosts of this library own every byte of the GPU themselves: a training
// framework that hands out memory from one pre-sized arena, or a step loop where
// the implicit device-wide synchronisation of cudaMalloc / cudaFree would stall
// other streams.  The ordinary mask update needs two per-row work arrays (a
// score and an active-connection count per input row).  Here they live in a
// fixed array inside the library image, so the call touches no allocator at all:
// no cudaMalloc, no cudaFree, no library routine that allocates.
//
// Cost and limits
//   * The array is SBB_NOALLOC_MAX_ROWS * 13 bytes plus 40 KiB (1.7 MiB) and is resident on
//     every GPU that loads the library, from load until the process exits.
//   * Layers with more than SBB_NOALLOC_MAX_ROWS input rows are refused with
//     SBB_ERR_UNSUPPORTED; nothing is launched in that case.
//   * All calls on a device share the one array.  Both work arrays are fully
//     rewritten for rows [0, N) before they are read, so stale contents from an
//     earlier (larger) call are harmless, but two calls that overlap in time on
//     the same GPU (different streams or threads) race on it.  Serialise them.
//   * The first call on each device resolves the array's device address (see
//     scratch_for_current_device).  Make that first call outside any stream
//     capture; later calls only launch kernels.
#include "../../include/sbb200.h"
#include "sbb_kernels.cuh"

#include <cstdio>
#include <mutex>

namespace sbb {
void set_last_error(const char *message);   // sbb_api.cu: the text sbb_last_error() returns on this thread
}

namespace {

constexpr long kMaxRows = SBB_NOALLOC_MAX_ROWS;
constexpr size_t kScoreBytes = (size_t)kMaxRows * sizeof(double);  // REAL score per row, sized for double
constexpr size_t kCountBytes = (size_t)kMaxRows * sizeof(int);     // active connections per row
constexpr size_t kColBytes = (size_t)kMaxRows;                     // previous mask bit per row
constexpr size_t kListBytes = 40 * 1024;                           // candidate lists of the swap search

// In host code this name is only a handle for the runtime; it is NOT a device
// address and must never be passed to a kernel.  The address a kernel can use
// comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_mask_scratch[kScoreBytes + kCountBytes + kColBytes + kListBytes];

constexpr int kMaxDevices = 64;
void *g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;
thread_local char g_noalloc_error[256];

int scratch_for_current_device(void **out) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    (void)cudaGetLastError();
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "update_mask_noalloc: no CUDA device is available; this library has no CPU path");
    return SBB_ERR_NO_DEVICE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "update_mask_noalloc: cannot identify the current device (%s)",
             cudaGetErrorString(e));
    return SBB_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_mask_scratch);  // resolved with `dev` current, kept for later calls
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_noalloc_error, sizeof(g_noalloc_error),
               "update_mask_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
      return SBB_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return SBB_OK;
}

}  // namespace

extern "C" {

const char *sbb_noalloc_last_error(void) { return g_noalloc_error; }

static int update_mask_noalloc_impl(int dtype, uint8_t *wmask_dev, const void *weights_dev, const void *Ci_dev,
                                    const void *Cj_dev, const void *Cij_dev, double cthr, long N, long M, long H,
                                    long Mc, long h, long iterations, void *stream);

int sbb_update_mask_noalloc(int dtype, uint8_t *wmask_dev, const void *weights_dev, const void *Ci_dev,
                            const void *Cj_dev, const void *Cij_dev, double cthr, long N, long M, long H, long Mc,
                            long h, long iterations, void *stream) {
  const int rc = update_mask_noalloc_impl(dtype, wmask_dev, weights_dev, Ci_dev, Cj_dev, Cij_dev, cthr, N, M, H, Mc, h,
                                          iterations, stream);
  // the message is also what sbb_last_error() returns, like every other entry point's
  if (rc != SBB_OK) sbb::set_last_error(g_noalloc_error);
  return rc;
}

static int update_mask_noalloc_impl(int dtype, uint8_t *wmask_dev, const void *weights_dev, const void *Ci_dev,
                                    const void *Cj_dev, const void *Cij_dev, double cthr, long N, long M, long H,
                                    long Mc, long h, long iterations, void *stream) {
  g_noalloc_error[0] = 0;
  if (dtype != SBB_F32 && dtype != SBB_F64) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "update_mask_noalloc: invalid dtype %d", dtype);
    return SBB_ERR_INVALID;
  }
  if (!wmask_dev || !Ci_dev || !Cj_dev || !Cij_dev) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "update_mask_noalloc: null pointer");
    return SBB_ERR_INVALID;
  }
  if (N <= 0 || H <= 0 || Mc <= 0 || M != H * Mc || h < 0 || h >= H || iterations < 0) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "update_mask_noalloc: bad shape N=%ld M=%ld H=%ld Mc=%ld h=%ld iterations=%ld", N, M, H, Mc, h,
             iterations);
    return SBB_ERR_INVALID;
  }
  if (N > kMaxRows) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "update_mask_noalloc: %ld input rows exceed the built-in work area of %ld rows; use sbb_update_mask or "
             "a layer handle, which allocate their own", N, kMaxRows);
    return SBB_ERR_UNSUPPORTED;
  }
  void *scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != SBB_OK) return rc;
  if (sbb::mask_scratch_bytes(N, dtype == SBB_F32 ? 4 : 8) > kScoreBytes + kCountBytes + kColBytes + kListBytes) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "update_mask_noalloc: built-in work area too small");
    return SBB_ERR_UNSUPPORTED;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (dtype == SBB_F32)
    e = sbb::launch_mask_update<float>(wmask_dev, (const float *)weights_dev, (const float *)Ci_dev,
                                       (const float *)Cj_dev, (const float *)Cij_dev, (float)cthr, N, M, H, Mc, h,
                                       iterations, scratch, st);
  else
    e = sbb::launch_mask_update<double>(wmask_dev, (const double *)weights_dev, (const double *)Ci_dev,
                                        (const double *)Cj_dev, (const double *)Cij_dev, cthr, N, M, H, Mc, h,
                                        iterations, scratch, st);
  if (e != cudaSuccess) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "update_mask_noalloc: launch failed (%s)",
             cudaGetErrorString(e));
    return SBB_ERR_CUDA;
  }
  return SBB_OK;
}

}  // extern "C"
