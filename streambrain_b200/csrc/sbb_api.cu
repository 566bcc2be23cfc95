// C ABI of libsbb200.so: the device-resident layer object, the stateless
// host-buffer kernel mirrors and the data-parallel split step.  See
// include/sbb200.h for the contract of every entry point.
#include "../../include/sbb200.h"
#include "sbb_kernels.cuh"
#include "sbb_tc.cuh"

#include <cstdarg>
#include <cstdlib>
#include <type_traits>
#include <vector>
#include <cstdio>
#include <cstring>
#include <string>

namespace {

thread_local std::string g_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  return fail(SBB_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

#define SBB_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e__ = (call);                            \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

#define SBB_TRY(call)               \
  do {                              \
    int rc__ = (call);              \
    if (rc__ != SBB_OK) return rc__; \
  } while (0)

int device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

int need_device() {
  if (device_count() <= 0) return fail(SBB_ERR_NO_DEVICE, "no CUDA device is available; this library has no CPU path");
  return SBB_OK;
}

size_t esize(int dtype) { return dtype == SBB_F32 ? 4 : 8; }

// Process-wide choice of contraction kernels (see sbb_set_contraction_path).
int initial_path() {
  const char *e = std::getenv("SBB_CONTRACTION");
  if (e && std::strcmp(e, "general") == 0) return SBB_PATH_GENERAL;
  return SBB_PATH_TENSOR;
}
int g_path = initial_path();

template <typename T>
bool tensor_path(const void *x, const void *other, long N, long M) {
  if (!std::is_same<T, float>::value || g_path != SBB_PATH_TENSOR) return false;
  return sbb::tc_shape_ok(x, other, N, M) && sbb::tc_available();
}

int check_dtype(int dtype) {
  if (dtype != SBB_F32 && dtype != SBB_F64) return fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  return SBB_OK;
}

// Device buffer that lives for one host-buffer call.
struct Staged {
  void *d = nullptr;
  size_t bytes = 0;
  ~Staged() {
    if (d) cudaFree(d);
  }
  int alloc(size_t n) {
    bytes = n;
    if (n == 0) return SBB_OK;
    SBB_CUDA(cudaMalloc(&d, n));
    return SBB_OK;
  }
  int upload(const void *h, size_t n) {
    SBB_TRY(alloc(n));
    if (n) SBB_CUDA(cudaMemcpy(d, h, n, cudaMemcpyHostToDevice));
    return SBB_OK;
  }
  int download(void *h) const {
    if (bytes) SBB_CUDA(cudaMemcpy(h, d, bytes, cudaMemcpyDeviceToHost));
    return SBB_OK;
  }
  template <typename T>
  T *as() const {
    return static_cast<T *>(d);
  }
};

// Scratch that grows on demand and is kept (no allocation in steady state).
struct Scratch {
  void *d = nullptr;
  size_t cap = 0;
  int reserve(size_t n) {
    if (n <= cap) return SBB_OK;
    if (d) SBB_CUDA(cudaFree(d));
    d = nullptr;
    cap = 0;
    SBB_CUDA(cudaMalloc(&d, n));
    cap = n;
    return SBB_OK;
  }
  void release() {
    if (d) cudaFree(d);
    d = nullptr;
    cap = 0;
  }
};

// Planes for the low parts of x[B, N] and y[B, M] (float32 tensor path only): written by the column-sum
// kernels, read by the contraction that follows them in the same step.
struct LoPlanes {
  float *x = nullptr, *y = nullptr;
};
template <typename T>
int reserve_lo(Scratch &buf, long B, long N, long M, bool wanted, LoPlanes *out) {
  *out = LoPlanes{};
  if (!wanted || !std::is_same<T, float>::value) return SBB_OK;
  SBB_TRY(buf.reserve((size_t)B * (size_t)(N + M) * sizeof(float)));
  out->x = static_cast<float *>(buf.d);
  out->y = out->x + (size_t)B * N;
  return SBB_OK;
}
template <typename T>
T *lo_as(float *p) {
  return reinterpret_cast<T *>(p);   // only dereferenced for T = float (null otherwise)
}

#define ARG(cond, ...) \
  do {                 \
    if (!(cond)) return fail(SBB_ERR_INVALID, __VA_ARGS__); \
  } while (0)

}  // namespace

namespace sbb {
void set_last_error(const char *message) { g_error = message ? message : ""; }
}  // namespace sbb

struct sbb_layer {
  sbb_layer_desc desc;
  long N, H, Mc, M;
  int device;
  void *state[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t state_bytes[7] = {0, 0, 0, 0, 0, 0, 0};
  Scratch fwd_partial;   // k-split partial sums of the forward product
  Scratch score;         // mask-update scratch: per-row score, active count, candidate lists
  Scratch hx, hy, ht;    // staging for the host-buffer entry points
  Scratch col_hc;        // M ints: hypercolumn of every output column (j / Mc)
  Scratch rc;            // threshold-gated reciprocals of Ci and Cj for the tensor-core trace update
  Scratch lo;            // low parts of x[B, N] and y[B, M] for the split TF32 products of the batch contractions
  long lo_batch = 0;     // batch rows the planes in `lo` were written for (0 = none)
  cudaStream_t own_stream = nullptr;
  // sbb_layer_step_host_async: two staging slots, copies on their own streams
  Scratch ax[2], ay[2], at[2];
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  cudaEvent_t ev_copied[2] = {nullptr, nullptr};    // slot's inputs have landed
  cudaEvent_t ev_stepped[2] = {nullptr, nullptr};   // the step that used the slot has finished
  cudaEvent_t ev_read[2] = {nullptr, nullptr};      // the slot's activation has been copied out
  unsigned long long async_calls = 0;
  bool async_open = false;
  // optional per-phase event ring (sbb_layer_profile)
  bool profiling = false;
  cudaEvent_t ev_begin[2][SBB_PROFILE_SLOTS];
  cudaEvent_t ev_end[2][SBB_PROFILE_SLOTS];
  bool ev_created = false;
  long phase_calls[2] = {0, 0};
  bool dp_fast = false;  // the last sbb_layer_dp_local ran the tensor-core product
  // row-sharded layer over peer-mapped memory (sbb_layer_shard_*)
  struct Shard {
    bool on = false, attached = false;
    long rank = 0, world = 1;
    long rows_per_rank = 0;            // multiple of 128; rank r owns rows [r * rows_per_rank, ...) clipped to N
    long max_batch = 0;                // largest local batch the gathered-input buffers hold
    // The own columns of the global batch, [world * B, own rows] with rank s's samples at rows [s * B, (s + 1) * B).
    // Three buffers used in turn: while this rank's step t reads one, the peers may already fill the next with
    // batch t + 1, and a peer that is still inside step t - 1 reads the third.
    Scratch xg[3];
    int cur = 0;                       // buffer of the step in flight
    int staged = 0;                    // batches scattered but not yet taken by a forward pass (0..2)
    long slot_batch[3] = {0, 0, 0};    // local batch each buffer was filled with
    long batch = 0;                    // local batch of the step in flight (0: no forward pass yet)
    Scratch yg;                        // activations of the global batch, [world * B, M]
    void *peer[SBB_SHARD_BUFFERS][8];  // per buffer kind and rank: that rank's buffer, mapped here (own rank: local)
    bool opened[SBB_SHARD_BUFFERS][8];
  } shard;
};

namespace {

// Brackets one kernel launch with events when profiling is on.
struct PhaseTimer {
  sbb_layer *L;
  int phase;
  cudaStream_t st;
  long slot = -1;
  PhaseTimer(sbb_layer *l, int ph, cudaStream_t s) : L(l), phase(ph), st(s) {
    if (L->profiling) {
      slot = L->phase_calls[phase] % SBB_PROFILE_SLOTS;
      cudaEventRecord(L->ev_begin[phase][slot], st);
    }
  }
  void stop() {
    if (slot >= 0) {
      cudaEventRecord(L->ev_end[phase][slot], st);
      L->phase_calls[phase] += 1;
      slot = -1;
    }
  }
};

template <typename T>
int layer_forward(sbb_layer *L, const T *x, long B, T *y, cudaStream_t st) {
  const T *W = static_cast<const T *>(L->state[SBB_STATE_WEIGHTS]);
  bool tc = tensor_path<T>(x, W, L->N, L->M);
  // an unsplit tensor-core product writes straight into y, which must then be 8-byte aligned
  if (tc && sbb::forward_splits_tc(B, L->N, L->M) == 1 && (reinterpret_cast<uintptr_t>(y) & 7u)) tc = false;
  const int splits = tc ? sbb::forward_splits_tc(B, L->N, L->M) : sbb::forward_splits<T>(B, L->N, L->M);
  T *partial = y;
  if (splits > 1) {
    SBB_TRY(L->fwd_partial.reserve((size_t)splits * B * L->M * sizeof(T)));
    partial = static_cast<T *>(L->fwd_partial.d);
  }
  PhaseTimer timer(L, SBB_PHASE_FORWARD, st);
  if (tc) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_forward_product_tc(x, W, partial, B, L->N, L->M, splits, st));
  } else {
    SBB_CUDA(sbb::launch_forward_product<T>(x, W, partial, B, L->N, L->M, splits, st));
  }
  timer.stop();
  SBB_CUDA(sbb::launch_reduce_bias_softmax<T>(partial, splits, static_cast<const T *>(L->state[SBB_STATE_BIAS]), y, B,
                                              L->H, L->Mc, 1, st));
  return SBB_OK;
}

template <typename T>
int layer_finish(sbb_layer *L, long h, cudaStream_t st) {
  if (L->desc.kind != SBB_LAYER_PLASTIC) return SBB_OK;
  const double cthr = L->desc.taupdt / 2;
  T *W = static_cast<T *>(L->state[SBB_STATE_WEIGHTS]);
  T *Ci = static_cast<T *>(L->state[SBB_STATE_CI]);
  T *Cj = static_cast<T *>(L->state[SBB_STATE_CJ]);
  T *Cij = static_cast<T *>(L->state[SBB_STATE_CIJ]);
  uint8_t *wmask = static_cast<uint8_t *>(L->state[SBB_STATE_WMASK]);
  SBB_CUDA(sbb::launch_update_bias_regularized<T>(static_cast<T *>(L->state[SBB_STATE_BIAS]),
                                                  static_cast<T *>(L->state[SBB_STATE_KBI]), Cj, (T)cthr,
                                                  (T)L->desc.khalf, (T)L->desc.pmin, (T)L->desc.taubdt, L->M, st));
  if (h >= 0) {
    // The score uses the freshly recomputed, un-masked weight of every connection,
    // which is a function of the traces alone; the masked weights already written
    // for hypercolumn h are then rewritten under the updated mask.
    SBB_CUDA(sbb::launch_mask_update<T>(wmask, nullptr, Ci, Cj, Cij, (T)cthr, L->N, L->M, L->H, L->Mc, h,
                                        L->desc.mask_iterations, L->score.d, st, W));
  }
  return SBB_OK;
}

template <typename T>
int layer_train_step(sbb_layer *L, const T *x, const T *y, long B, long h, cudaStream_t st) {
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(L->desc.taupdt, L->desc.taupdt / 2, B);
  T *Ci = static_cast<T *>(L->state[SBB_STATE_CI]);
  T *Cj = static_cast<T *>(L->state[SBB_STATE_CJ]);
  const bool tc = tensor_path<T>(x, y, L->N, L->M);
  SBB_CUDA(sbb::launch_colsum<T>(x, B, L->N, nullptr, Ci, p, 1, st));
  SBB_CUDA(sbb::launch_colsum<T>(y, B, L->M, nullptr, Cj, p, 1, st));
  PhaseTimer timer(L, SBB_PHASE_TRACE, st);
  if (tc) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_trace_update_tc(x, y, B, L->N, L->M, L->H, Ci, Cj, static_cast<T *>(L->state[SBB_STATE_CIJ]),
                                           static_cast<T *>(L->state[SBB_STATE_WEIGHTS]),
                                           static_cast<const uint8_t *>(L->state[SBB_STATE_WMASK]),
                                           static_cast<const int *>(L->col_hc.d), static_cast<float *>(L->rc.d), p,
                                           0, L->N, st));
  } else {
    SBB_CUDA(sbb::launch_trace_update_fused<T>(x, y, B, L->N, L->M, L->H, L->Mc, Ci, Cj,
                                               static_cast<T *>(L->state[SBB_STATE_CIJ]),
                                               static_cast<T *>(L->state[SBB_STATE_WEIGHTS]),
                                               static_cast<const uint8_t *>(L->state[SBB_STATE_WMASK]), p, 0, L->N,
                                               st));
  }
  timer.stop();
  return layer_finish<T>(L, h, st);
}

template <typename T>
int layer_dp_local(sbb_layer *L, const T *x, const T *y, long B, T *delta, long rb, long re, cudaStream_t st) {
  sbb::TraceParams<T> p = sbb::make_trace_params<T>(L->desc.taupdt, L->desc.taupdt / 2, B);
  T *xty = delta + L->N + L->M;
  // remembered for sbb_layer_dp_apply_rows: the element-wise tail uses the arithmetic of the path that formed the sums
  L->dp_fast = tensor_path<T>(x, y, L->N, L->M) && (reinterpret_cast<uintptr_t>(xty) & 7u) == 0;
  LoPlanes lo;
  if (rb == 0) {
    // the first row block of a step also forms the column sums and, for the tensor path, the operands' low parts,
    // which the later row blocks of the same step (same x, y, B) re-use
    SBB_TRY(reserve_lo<T>(L->lo, B, L->N, L->M, L->dp_fast, &lo));
    SBB_CUDA(sbb::launch_colsum<T>(x, B, L->N, delta, nullptr, p, 0, st, lo_as<T>(lo.x)));
    SBB_CUDA(sbb::launch_colsum<T>(y, B, L->M, delta + L->N, nullptr, p, 0, st, lo_as<T>(lo.y)));
    L->lo_batch = lo.x ? B : 0;
  } else if (L->dp_fast && L->lo_batch == B) {
    lo.x = static_cast<float *>(L->lo.d);
    lo.y = lo.x + (size_t)B * L->N;
  }
  PhaseTimer timer(L, SBB_PHASE_TRACE, st);
  if (L->dp_fast) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_outer_product_tc(x, y, B, L->N, L->M, xty, rb, re, st, lo.x, lo.y));
  } else {
    SBB_CUDA(sbb::launch_outer_product<T>(x, y, B, L->N, L->M, xty, rb, re, st));
  }
  timer.stop();
  return SBB_OK;
}

template <typename T>
int layer_dp_apply_vectors(sbb_layer *L, const T *delta, long Bg, cudaStream_t st) {
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(L->desc.taupdt, L->desc.taupdt / 2, Bg);
  SBB_CUDA(sbb::launch_vector_ema<T>(static_cast<T *>(L->state[SBB_STATE_CI]), delta, L->N, p, st));
  SBB_CUDA(sbb::launch_vector_ema<T>(static_cast<T *>(L->state[SBB_STATE_CJ]), delta + L->N, L->M, p, st));
  return SBB_OK;
}

template <typename T>
int layer_dp_apply_rows(sbb_layer *L, const T *delta, long Bg, long rb, long re, cudaStream_t st) {
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(L->desc.taupdt, L->desc.taupdt / 2, Bg);
  SBB_CUDA(sbb::launch_trace_apply<T>(delta + L->N + L->M, L->N, L->M, L->H, L->Mc,
                                      static_cast<const T *>(L->state[SBB_STATE_CI]),
                                      static_cast<const T *>(L->state[SBB_STATE_CJ]),
                                      static_cast<T *>(L->state[SBB_STATE_CIJ]),
                                      static_cast<T *>(L->state[SBB_STATE_WEIGHTS]),
                                      static_cast<const uint8_t *>(L->state[SBB_STATE_WMASK]), p, 1, rb, re, st,
                                      // the arithmetic of the path that formed the sums (see sbb_math.cuh)
                                      L->dp_fast));
  return SBB_OK;
}

int check_layer(const sbb_layer *L) {
  if (!L) return fail(SBB_ERR_INVALID, "null layer handle");
  int dev = -1;
  SBB_CUDA(cudaGetDevice(&dev));
  if (dev != L->device)
    return fail(SBB_ERR_INVALID, "layer lives on device %d but device %d is current", L->device, dev);
  return SBB_OK;
}

int check_batch(const sbb_layer *L, long B) {
  ARG(B > 0, "batch must be positive, got %ld", B);
  ARG(B <= 2147483647L / 2 && L->N <= 2147483647L / 2, "batch %ld or in_features %ld out of range", B, L->N);
  return SBB_OK;
}

#define DISPATCH(dtype, expr_f32, expr_f64) ((dtype) == SBB_F32 ? (expr_f32) : (expr_f64))

// Called by entry points right after they have waited for their own work: a bounded device-side wait
// that gave up leaves the step half done, which the caller must learn from the return code.
int check_wait_status() {
  int st = 0;
  SBB_CUDA(sbb::tc_peek_status(&st));
  if (st != 0)
    return fail(SBB_ERR_TIMEOUT,
                "a bounded device-side wait gave up (code %d): the state of layers stepped since the last check is "
                "undefined; reload it and call sbb_device_clear_wait_status",
                st);
  return SBB_OK;
}

}  // namespace

extern "C" {

int sbb_version(void) { return 100; }
const char *sbb_last_error(void) { return g_error.c_str(); }
int sbb_device_count(void) { return device_count(); }
unsigned long long sbb_kernel_launches(void) { return sbb::kernel_launches(); }

int sbb_set_contraction_path(int path) {
  ARG(path == SBB_PATH_GENERAL || path == SBB_PATH_TENSOR, "invalid contraction path %d", path);
  g_path = path;
  return SBB_OK;
}
int sbb_get_contraction_path(void) { return g_path; }

int sbb_set_reserved_sms(int sms) {
  if (sms < 0) return fail(SBB_ERR_INVALID, "sbb_set_reserved_sms: negative count");
  sbb::tc_set_reserved_sms(sms);
  return SBB_OK;
}
int sbb_get_reserved_sms(void) { return sbb::tc_get_reserved_sms(); }
int sbb_tensor_path_available(void) { return device_count() > 0 && sbb::tc_available() ? 1 : 0; }
int sbb_device_wait_status(int *status) {
  ARG(status, "device_wait_status: null pointer");
  SBB_TRY(need_device());
  SBB_CUDA(sbb::tc_read_status(status));
  if (*status != 0) return fail(SBB_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d)", *status);
  return SBB_OK;
}

int sbb_set_wait_limit_cycles(long long cycles) {
  if (cycles <= 0) return fail(SBB_ERR_INVALID, "sbb_set_wait_limit_cycles: the limit must be positive");
  sbb::tc_set_wait_limit(cycles);
  return SBB_OK;
}
long long sbb_get_wait_limit_cycles(void) { return sbb::tc_get_wait_limit(); }
int sbb_debug_lose_arrival(int launches) {
  sbb::tc_debug_lose_arrive(launches);
  return SBB_OK;
}

int sbb_measure_fp64_rates(double *dfma_tflops, double *dmma_tflops) {
  ARG(dfma_tflops && dmma_tflops, "measure_fp64_rates: null pointer");
  SBB_TRY(need_device());
  SBB_CUDA(sbb::measure_fp64_rates(dfma_tflops, dmma_tflops));
  return SBB_OK;
}

int sbb_device_clear_wait_status(void) {
  SBB_TRY(need_device());
  SBB_CUDA(sbb::tc_clear_status());
  return SBB_OK;
}

int sbb_stream_sync(void *stream) {
  SBB_TRY(need_device());
  SBB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return check_wait_status();
}

// ---------------------------------------------------------------- stateless
int sbb_update_state(int dtype, void *activation, const void *inputs, const void *weights, const void *bias, long B,
                     long N, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(activation && inputs && weights && bias, "update_state: null pointer");
  ARG(B > 0 && N > 0 && M > 0, "update_state: non-positive shape B=%ld N=%ld M=%ld", B, N, M);
  SBB_TRY(need_device());
  const size_t s = esize(dtype);
  Staged x, w, b, out, part;
  SBB_TRY(x.upload(inputs, B * N * s));
  SBB_TRY(w.upload(weights, N * M * s));
  SBB_TRY(b.upload(bias, M * s));
  SBB_TRY(out.alloc(B * M * s));
  const bool tc = dtype == SBB_F32 && tensor_path<float>(x.d, w.d, N, M);
  const int splits = tc ? sbb::forward_splits_tc(B, N, M)
                        : DISPATCH(dtype, sbb::forward_splits<float>(B, N, M), sbb::forward_splits<double>(B, N, M));
  void *partial = out.d;
  if (splits > 1) {
    SBB_TRY(part.alloc((size_t)splits * B * M * s));
    partial = part.d;
  }
  if (dtype == SBB_F32) {
    if (tc)
      SBB_CUDA(sbb::launch_forward_product_tc(x.as<float>(), w.as<float>(), (float *)partial, B, N, M, splits, 0));
    else
      SBB_CUDA(sbb::launch_forward_product<float>(x.as<float>(), w.as<float>(), (float *)partial, B, N, M, splits, 0));
    SBB_CUDA(sbb::launch_reduce_bias_softmax<float>((float *)partial, splits, b.as<float>(), out.as<float>(), B, 1, M,
                                                    0, 0));
  } else {
    SBB_CUDA(sbb::launch_forward_product<double>(x.as<double>(), w.as<double>(), (double *)partial, B, N, M, splits, 0));
    SBB_CUDA(sbb::launch_reduce_bias_softmax<double>((double *)partial, splits, b.as<double>(), out.as<double>(), B, 1,
                                                     M, 0, 0));
  }
  SBB_CUDA(cudaDeviceSynchronize());
  return out.download(activation);
}

int sbb_add_bias(int dtype, void *a, const void *bias, long rows, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(a && bias, "add_bias: null pointer");
  ARG(rows > 0 && M > 0, "add_bias: non-positive shape");
  SBB_TRY(need_device());
  const size_t s = esize(dtype);
  Staged da, db;
  SBB_TRY(da.upload(a, rows * M * s));
  SBB_TRY(db.upload(bias, M * s));
  if (dtype == SBB_F32) SBB_CUDA(sbb::launch_add_bias<float>(da.as<float>(), db.as<float>(), rows, M, 0));
  else SBB_CUDA(sbb::launch_add_bias<double>(da.as<double>(), db.as<double>(), rows, M, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return da.download(a);
}

int sbb_softmax_minicolumns(int dtype, void *a, long rows, long H, long Mc) {
  SBB_TRY(check_dtype(dtype));
  ARG(a, "softmax_minicolumns: null pointer");
  ARG(rows > 0 && H > 0 && Mc > 0, "softmax_minicolumns: non-positive shape");
  SBB_TRY(need_device());
  Staged da;
  SBB_TRY(da.upload(a, rows * H * Mc * esize(dtype)));
  if (dtype == SBB_F32)
    SBB_CUDA(sbb::launch_reduce_bias_softmax<float>(da.as<float>(), 1, nullptr, da.as<float>(), rows, H, Mc, 1, 0));
  else
    SBB_CUDA(sbb::launch_reduce_bias_softmax<double>(da.as<double>(), 1, nullptr, da.as<double>(), rows, H, Mc, 1, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return da.download(a);
}

}  // extern "C"

namespace {
template <typename T>
int update_counters_t(void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o, double taupdt, long B, long N,
                      long M) {
  const size_t s = sizeof(T);
  Staged dci, dcj, dcij, dx, dy, sums;
  SBB_TRY(dci.upload(Ci, N * s));
  SBB_TRY(dcj.upload(Cj, M * s));
  SBB_TRY(dcij.upload(Cij, N * M * s));
  SBB_TRY(dx.upload(a_i, B * N * s));
  SBB_TRY(dy.upload(a_o, B * M * s));
  SBB_TRY(sums.alloc((size_t)(N + M + N * M + 4) * s));
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(taupdt, taupdt / 2, B);
  T *sx = sums.as<T>();
  T *sy = sx + N;
  // keep the [N, M] block 16-byte aligned whatever N + M is
  T *sxy = sx + ((N + M + 3) / 4) * 4;
  const bool tc = tensor_path<T>(dx.d, dy.d, N, M);
  Scratch lo_buf;
  LoPlanes lo;
  int lo_rc = reserve_lo<T>(lo_buf, B, N, M, tc, &lo);
  struct Release { Scratch &s; ~Release() { s.release(); } } release_lo{lo_buf};
  SBB_TRY(lo_rc);
  SBB_CUDA(sbb::launch_colsum<T>(dx.as<T>(), B, N, sx, nullptr, p, 0, 0, lo_as<T>(lo.x)));
  SBB_CUDA(sbb::launch_colsum<T>(dy.as<T>(), B, M, sy, nullptr, p, 0, 0, lo_as<T>(lo.y)));
  if (tc) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_outer_product_tc(dx.as<T>(), dy.as<T>(), B, N, M, sxy, 0, N, 0, lo.x, lo.y));
  } else {
    SBB_CUDA(sbb::launch_outer_product<T>(dx.as<T>(), dy.as<T>(), B, N, M, sxy, 0, N, 0));
  }
  SBB_CUDA(sbb::launch_counters_apply<T>(dci.as<T>(), sx, N, (T)taupdt, (T)B, 0));
  SBB_CUDA(sbb::launch_counters_apply<T>(dcj.as<T>(), sy, M, (T)taupdt, (T)B, 0));
  SBB_CUDA(sbb::launch_counters_apply<T>(dcij.as<T>(), sxy, N * M, (T)taupdt, (T)B, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_TRY(dci.download(Ci));
  SBB_TRY(dcj.download(Cj));
  return dcij.download(Cij);
}

template <typename T>
int update_weights_t(void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o, double taupdt, long B, long N,
                     long M, void *weights, double cthr) {
  const size_t s = sizeof(T);
  Staged dci, dcj, dcij, dx, dy, dw;
  SBB_TRY(dci.upload(Ci, N * s));
  SBB_TRY(dcj.upload(Cj, M * s));
  SBB_TRY(dcij.upload(Cij, N * M * s));
  SBB_TRY(dx.upload(a_i, B * N * s));
  SBB_TRY(dy.upload(a_o, B * M * s));
  SBB_TRY(dw.alloc(N * M * s));
  Staged drc;
  SBB_TRY(drc.alloc(sbb::tc_trace_scratch_bytes(N, M)));
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(taupdt, cthr, B);
  const bool tc = tensor_path<T>(dx.d, dy.d, N, M);
  SBB_CUDA(sbb::launch_colsum<T>(dx.as<T>(), B, N, nullptr, dci.as<T>(), p, 1, 0));
  SBB_CUDA(sbb::launch_colsum<T>(dy.as<T>(), B, M, nullptr, dcj.as<T>(), p, 1, 0));
  if (tc) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_trace_update_tc(dx.as<T>(), dy.as<T>(), B, N, M, 1, dci.as<T>(), dcj.as<T>(), dcij.as<T>(),
                                           dw.as<T>(), nullptr, nullptr, drc.as<float>(), p, 0, N, 0));
  } else {
    SBB_CUDA(sbb::launch_trace_update_fused<T>(dx.as<T>(), dy.as<T>(), B, N, M, 1, M, dci.as<T>(), dcj.as<T>(),
                                               dcij.as<T>(), dw.as<T>(), nullptr, p, 0, N, 0));
  }
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_TRY(dci.download(Ci));
  SBB_TRY(dcj.download(Cj));
  SBB_TRY(dcij.download(Cij));
  return dw.download(weights);
}

template <typename T>
int recompute_weights_t(void *weights, const void *Ci, const void *Cj, const void *Cij, double cthr, long N, long M) {
  const size_t s = sizeof(T);
  Staged dci, dcj, dcij, dw;
  SBB_TRY(dci.upload(Ci, N * s));
  SBB_TRY(dcj.upload(Cj, M * s));
  SBB_TRY(dcij.upload(Cij, N * M * s));
  SBB_TRY(dw.alloc(N * M * s));
  sbb::TraceParams<T> p = sbb::make_trace_params<T>(2 * cthr, cthr, 1);
  SBB_CUDA(sbb::launch_trace_apply<T>(nullptr, N, M, 1, M, dci.as<T>(), dcj.as<T>(), dcij.as<T>(), dw.as<T>(), nullptr,
                                      p, 0, 0, N, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return dw.download(weights);
}

template <typename T>
int update_mask_t(uint8_t *wmask, const void *weights, const void *Ci, const void *Cj, const void *Cij, double cthr,
                  long N, long M, long H, long Mc, long h, long iterations) {
  const size_t s = sizeof(T);
  Staged dm, dw, dci, dcj, dcij, score;
  SBB_TRY(dm.upload(wmask, N * H));
  SBB_TRY(dw.upload(weights, N * M * s));
  SBB_TRY(dci.upload(Ci, N * s));
  SBB_TRY(dcj.upload(Cj, M * s));
  SBB_TRY(dcij.upload(Cij, N * M * s));
  SBB_TRY(score.alloc(sbb::mask_scratch_bytes(N, s)));
  SBB_CUDA(sbb::launch_mask_update<T>(dm.as<uint8_t>(), dw.as<T>(), dci.as<T>(), dcj.as<T>(), dcij.as<T>(), (T)cthr, N,
                                      M, H, Mc, h, iterations, score.d, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return dm.download(wmask);
}
}  // namespace

extern "C" {

int sbb_update_counters(int dtype, void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o, double taupdt,
                        long B, long N, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(Ci && Cj && Cij && a_i && a_o, "update_counters: null pointer");
  ARG(B > 0 && N > 0 && M > 0, "update_counters: non-positive shape");
  SBB_TRY(need_device());
  return DISPATCH(dtype, update_counters_t<float>(Ci, Cj, Cij, a_i, a_o, taupdt, B, N, M),
                  update_counters_t<double>(Ci, Cj, Cij, a_i, a_o, taupdt, B, N, M));
}

int sbb_update_weights(int dtype, void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o, double taupdt,
                       long B, long N, long M, void *weights, double cthr) {
  SBB_TRY(check_dtype(dtype));
  ARG(Ci && Cj && Cij && a_i && a_o && weights, "update_weights: null pointer");
  ARG(B > 0 && N > 0 && M > 0, "update_weights: non-positive shape");
  SBB_TRY(need_device());
  return DISPATCH(dtype, update_weights_t<float>(Ci, Cj, Cij, a_i, a_o, taupdt, B, N, M, weights, cthr),
                  update_weights_t<double>(Ci, Cj, Cij, a_i, a_o, taupdt, B, N, M, weights, cthr));
}

int sbb_recompute_weights(int dtype, void *weights, const void *Ci, const void *Cj, const void *Cij, double cthr,
                          long N, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(weights && Ci && Cj && Cij, "recompute_weights: null pointer");
  ARG(N > 0 && M > 0, "recompute_weights: non-positive shape");
  SBB_TRY(need_device());
  return DISPATCH(dtype, recompute_weights_t<float>(weights, Ci, Cj, Cij, cthr, N, M),
                  recompute_weights_t<double>(weights, Ci, Cj, Cij, cthr, N, M));
}

int sbb_update_bias(int dtype, void *bias, const void *Cj, double cthr, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(bias && Cj, "update_bias: null pointer");
  ARG(M > 0, "update_bias: non-positive size");
  SBB_TRY(need_device());
  const size_t s = esize(dtype);
  Staged db, dc;
  SBB_TRY(db.alloc(M * s));
  SBB_TRY(dc.upload(Cj, M * s));
  if (dtype == SBB_F32) SBB_CUDA(sbb::launch_update_bias<float>(db.as<float>(), dc.as<float>(), (float)cthr, M, 0));
  else SBB_CUDA(sbb::launch_update_bias<double>(db.as<double>(), dc.as<double>(), cthr, M, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return db.download(bias);
}

int sbb_update_bias_regularized(int dtype, void *bias, void *kbi, const void *Cj, double cthr, double khalf,
                                double pmin, double taubdt, long M) {
  SBB_TRY(check_dtype(dtype));
  ARG(bias && kbi && Cj, "update_bias_regularized: null pointer");
  ARG(M > 0, "update_bias_regularized: non-positive size");
  SBB_TRY(need_device());
  const size_t s = esize(dtype);
  Staged db, dk, dc;
  SBB_TRY(db.alloc(M * s));
  SBB_TRY(dk.upload(kbi, M * s));
  SBB_TRY(dc.upload(Cj, M * s));
  if (dtype == SBB_F32)
    SBB_CUDA(sbb::launch_update_bias_regularized<float>(db.as<float>(), dk.as<float>(), dc.as<float>(), (float)cthr,
                                                        (float)khalf, (float)pmin, (float)taubdt, M, 0));
  else
    SBB_CUDA(sbb::launch_update_bias_regularized<double>(db.as<double>(), dk.as<double>(), dc.as<double>(), cthr, khalf,
                                                         pmin, taubdt, M, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_TRY(db.download(bias));
  return dk.download(kbi);
}

int sbb_update_mask(int dtype, uint8_t *wmask, const void *weights, const void *Ci, const void *Cj, const void *Cij,
                    double cthr, long N, long M, long H, long Mc, long h, long iterations) {
  SBB_TRY(check_dtype(dtype));
  ARG(wmask && weights && Ci && Cj && Cij, "update_mask: null pointer");
  ARG(N > 0 && H > 0 && Mc > 0 && M == H * Mc, "update_mask: shape mismatch N=%ld M=%ld H=%ld Mc=%ld", N, M, H, Mc);
  ARG(h >= 0 && h < H, "update_mask: hypercolumn %ld outside [0,%ld)", h, H);
  ARG(iterations >= 0, "update_mask: negative iteration count");
  SBB_TRY(need_device());
  return DISPATCH(dtype, update_mask_t<float>(wmask, weights, Ci, Cj, Cij, cthr, N, M, H, Mc, h, iterations),
                  update_mask_t<double>(wmask, weights, Ci, Cj, Cij, cthr, N, M, H, Mc, h, iterations));
}

int sbb_apply_mask(int dtype, void *weights, const uint8_t *wmask, long N, long M, long H, long Mc) {
  SBB_TRY(check_dtype(dtype));
  ARG(weights && wmask, "apply_mask: null pointer");
  ARG(N > 0 && H > 0 && Mc > 0 && M == H * Mc, "apply_mask: shape mismatch N=%ld M=%ld H=%ld Mc=%ld", N, M, H, Mc);
  SBB_TRY(need_device());
  Staged dw, dm;
  SBB_TRY(dw.upload(weights, N * M * esize(dtype)));
  SBB_TRY(dm.upload(wmask, N * H));
  if (dtype == SBB_F32) SBB_CUDA(sbb::launch_apply_mask<float>(dw.as<float>(), dm.as<uint8_t>(), N, M, H, Mc, 0));
  else SBB_CUDA(sbb::launch_apply_mask<double>(dw.as<double>(), dm.as<uint8_t>(), N, M, H, Mc, 0));
  SBB_CUDA(cudaDeviceSynchronize());
  return dw.download(weights);
}

// -------------------------------------------------------------------- layer
int sbb_layer_create(const sbb_layer_desc *desc, sbb_layer **out) {
  ARG(desc && out, "layer_create: null pointer");
  *out = nullptr;
  SBB_TRY(check_dtype(desc->dtype));
  ARG(desc->kind == SBB_LAYER_DENSE || desc->kind == SBB_LAYER_PLASTIC, "layer_create: invalid kind %d", desc->kind);
  ARG(desc->in_features > 0 && desc->hypercolumns > 0 && desc->minicolumns > 0,
      "layer_create: non-positive shape N=%ld H=%ld Mc=%ld", desc->in_features, desc->hypercolumns, desc->minicolumns);
  ARG(desc->mask_iterations >= 0, "layer_create: negative mask_iterations");
  SBB_TRY(need_device());
  sbb_layer *L = new sbb_layer();
  L->desc = *desc;
  L->N = desc->in_features;
  L->H = desc->hypercolumns;
  L->Mc = desc->minicolumns;
  L->M = L->H * L->Mc;
  const size_t s = esize(desc->dtype);
  L->state_bytes[SBB_STATE_WEIGHTS] = (size_t)L->N * L->M * s;
  L->state_bytes[SBB_STATE_BIAS] = (size_t)L->M * s;
  L->state_bytes[SBB_STATE_CI] = (size_t)L->N * s;
  L->state_bytes[SBB_STATE_CJ] = (size_t)L->M * s;
  L->state_bytes[SBB_STATE_CIJ] = (size_t)L->N * L->M * s;
  if (desc->kind == SBB_LAYER_PLASTIC) {
    L->state_bytes[SBB_STATE_KBI] = (size_t)L->M * s;
    L->state_bytes[SBB_STATE_WMASK] = (size_t)L->N * L->H;
  }
  int rc = SBB_OK;
  cudaError_t e = cudaGetDevice(&L->device);
  for (int k = 0; k < 7 && e == cudaSuccess; ++k)
    if (L->state_bytes[k]) {
      e = cudaMalloc(&L->state[k], L->state_bytes[k]);
      if (e == cudaSuccess) e = cudaMemset(L->state[k], 0, L->state_bytes[k]);
    }
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) rc = cuda_fail(e, "layer_create");
  if (rc == SBB_OK) rc = L->rc.reserve(sbb::tc_trace_scratch_bytes(L->N, L->M));
  if (rc == SBB_OK && desc->kind == SBB_LAYER_PLASTIC) {
    rc = L->score.reserve(sbb::mask_scratch_bytes(L->N, s));
    if (rc == SBB_OK) rc = L->col_hc.reserve((size_t)(L->M + 4) * sizeof(int));
    if (rc == SBB_OK) {
      std::vector<int> hc((size_t)L->M);
      for (long j = 0; j < L->M; ++j) hc[(size_t)j] = (int)(j / L->Mc);
      e = cudaMemcpy(L->col_hc.d, hc.data(), hc.size() * sizeof(int), cudaMemcpyHostToDevice);
      if (e != cudaSuccess) rc = cuda_fail(e, "layer_create");
    }
  }
  if (rc != SBB_OK) {
    std::string keep = g_error;
    sbb_layer_destroy(L);
    g_error = keep;
    return rc;
  }
  *out = L;
  return SBB_OK;
}

int sbb_layer_destroy(sbb_layer *L) {
  if (!L) return SBB_OK;
  for (int k = 0; k < 7; ++k)
    if (L->state[k]) cudaFree(L->state[k]);
  L->fwd_partial.release();
  L->score.release();
  L->hx.release();
  L->hy.release();
  L->ht.release();
  L->col_hc.release();
  L->rc.release();
  L->lo.release();
  if (L->shard.on) {
    for (int b = 0; b < SBB_SHARD_BUFFERS; ++b)
      for (int r = 0; r < 8; ++r)
        if (L->shard.opened[b][r]) cudaIpcCloseMemHandle(L->shard.peer[b][r]);
    for (auto &b : L->shard.xg) b.release();
    L->shard.yg.release();
  }
  if (L->own_stream) cudaStreamDestroy(L->own_stream);
  if (L->h2d_stream) cudaStreamDestroy(L->h2d_stream);
  if (L->d2h_stream) cudaStreamDestroy(L->d2h_stream);
  for (int k = 0; k < 2; ++k) {
    if (L->ev_copied[k]) cudaEventDestroy(L->ev_copied[k]);
    if (L->ev_stepped[k]) cudaEventDestroy(L->ev_stepped[k]);
    if (L->ev_read[k]) cudaEventDestroy(L->ev_read[k]);
    L->ax[k].release();
    L->ay[k].release();
    L->at[k].release();
  }
  if (L->ev_created)
    for (int ph = 0; ph < 2; ++ph)
      for (int k = 0; k < SBB_PROFILE_SLOTS; ++k) {
        cudaEventDestroy(L->ev_begin[ph][k]);
        cudaEventDestroy(L->ev_end[ph][k]);
      }
  delete L;
  return SBB_OK;
}

static int state_slot(const sbb_layer *L, int which, size_t bytes, bool check_bytes) {
  if (!L) return fail(SBB_ERR_INVALID, "null layer handle");
  ARG(which >= 0 && which < 7, "invalid state index %d", which);
  ARG(L->state_bytes[which] != 0, "state %d does not exist for this layer kind", which);
  if (check_bytes)
    ARG(bytes == L->state_bytes[which], "state %d holds %zu bytes, caller passed %zu", which, L->state_bytes[which],
        bytes);
  return SBB_OK;
}

int sbb_layer_set_state(sbb_layer *L, int which, const void *host, size_t bytes) {
  SBB_TRY(state_slot(L, which, bytes, true));
  ARG(host, "set_state: null pointer");
  SBB_TRY(check_layer(L));
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_CUDA(cudaMemcpy(L->state[which], host, bytes, cudaMemcpyHostToDevice));
  return SBB_OK;
}

int sbb_layer_get_state(sbb_layer *L, int which, void *host, size_t bytes) {
  SBB_TRY(state_slot(L, which, bytes, true));
  ARG(host, "get_state: null pointer");
  SBB_TRY(check_layer(L));
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_CUDA(cudaMemcpy(host, L->state[which], bytes, cudaMemcpyDeviceToHost));
  return check_wait_status();
}

int sbb_layer_state_ptr(sbb_layer *L, int which, void **device_ptr) {
  SBB_TRY(state_slot(L, which, 0, false));
  ARG(device_ptr, "state_ptr: null pointer");
  *device_ptr = L->state[which];
  return SBB_OK;
}

int sbb_layer_info(const sbb_layer *L, sbb_layer_desc *out) {
  ARG(L && out, "layer_info: null pointer");
  *out = L->desc;
  return SBB_OK;
}

int sbb_layer_profile(sbb_layer *L, int enable) {
  SBB_TRY(check_layer(L));
  if (enable && !L->ev_created) {
    for (int ph = 0; ph < 2; ++ph)
      for (int k = 0; k < SBB_PROFILE_SLOTS; ++k) {
        SBB_CUDA(cudaEventCreate(&L->ev_begin[ph][k]));
        SBB_CUDA(cudaEventCreate(&L->ev_end[ph][k]));
      }
    L->ev_created = true;
  }
  L->profiling = enable != 0;
  L->phase_calls[0] = L->phase_calls[1] = 0;
  return SBB_OK;
}

int sbb_layer_phase_calls(sbb_layer *L, int phase, long *calls) {
  SBB_TRY(check_layer(L));
  ARG(phase == SBB_PHASE_FORWARD || phase == SBB_PHASE_TRACE, "invalid phase %d", phase);
  ARG(calls, "phase_calls: null pointer");
  *calls = L->phase_calls[phase];
  return SBB_OK;
}

int sbb_layer_phase_ms(sbb_layer *L, int phase, long index, float *ms) {
  SBB_TRY(check_layer(L));
  ARG(phase == SBB_PHASE_FORWARD || phase == SBB_PHASE_TRACE, "invalid phase %d", phase);
  ARG(ms, "phase_ms: null pointer");
  ARG(L->ev_created, "profiling was never enabled on this layer");
  ARG(index >= 0 && index < L->phase_calls[phase] && index >= L->phase_calls[phase] - SBB_PROFILE_SLOTS,
      "call %ld is not in the ring (calls so far: %ld)", index, L->phase_calls[phase]);
  const long slot = index % SBB_PROFILE_SLOTS;
  SBB_CUDA(cudaEventSynchronize(L->ev_end[phase][slot]));
  SBB_CUDA(cudaEventElapsedTime(ms, L->ev_begin[phase][slot], L->ev_end[phase][slot]));
  return SBB_OK;
}

int sbb_layer_forward(sbb_layer *L, const void *x_dev, long B, void *y_dev, void *stream) {
  SBB_TRY(check_layer(L));
  ARG(x_dev && y_dev, "layer_forward: null pointer");
  SBB_TRY(check_batch(L, B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, layer_forward<float>(L, (const float *)x_dev, B, (float *)y_dev, st),
                  layer_forward<double>(L, (const double *)x_dev, B, (double *)y_dev, st));
}

int sbb_layer_train_step(sbb_layer *L, const void *x_dev, const void *y_dev, long B, long hypercolumn, void *stream) {
  SBB_TRY(check_layer(L));
  ARG(x_dev && y_dev, "layer_train_step: null pointer");
  SBB_TRY(check_batch(L, B));
  ARG(hypercolumn < L->H, "layer_train_step: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  if (L->desc.kind != SBB_LAYER_PLASTIC) hypercolumn = -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype,
                  layer_train_step<float>(L, (const float *)x_dev, (const float *)y_dev, B, hypercolumn, st),
                  layer_train_step<double>(L, (const double *)x_dev, (const double *)y_dev, B, hypercolumn, st));
}

int sbb_layer_train_finalize(sbb_layer *L, void *stream) {
  SBB_TRY(check_layer(L));
  if (L->desc.kind != SBB_LAYER_DENSE) return SBB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const double cthr = L->desc.taupdt / 2;
  if (L->desc.dtype == SBB_F32)
    SBB_CUDA(sbb::launch_update_bias<float>((float *)L->state[SBB_STATE_BIAS], (const float *)L->state[SBB_STATE_CJ],
                                            (float)cthr, L->M, st));
  else
    SBB_CUDA(sbb::launch_update_bias<double>((double *)L->state[SBB_STATE_BIAS],
                                             (const double *)L->state[SBB_STATE_CJ], cthr, L->M, st));
  return SBB_OK;
}

int sbb_layer_forward_host(sbb_layer *L, const void *x_host, long B, void *y_host) {
  SBB_TRY(check_layer(L));
  ARG(x_host && y_host, "layer_forward_host: null pointer");
  SBB_TRY(check_batch(L, B));
  const size_t s = esize(L->desc.dtype);
  SBB_TRY(L->hx.reserve((size_t)B * L->N * s));
  SBB_TRY(L->hy.reserve((size_t)B * L->M * s));
  cudaStream_t st = L->own_stream;
  // Work queued earlier on other streams (a device-buffer call) must have landed
  // before this call reads or rewrites the layer state on its own stream.
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_CUDA(cudaMemcpyAsync(L->hx.d, x_host, (size_t)B * L->N * s, cudaMemcpyHostToDevice, st));
  SBB_TRY(DISPATCH(L->desc.dtype, layer_forward<float>(L, (const float *)L->hx.d, B, (float *)L->hy.d, st),
                   layer_forward<double>(L, (const double *)L->hx.d, B, (double *)L->hy.d, st)));
  SBB_CUDA(cudaMemcpyAsync(y_host, L->hy.d, (size_t)B * L->M * s, cudaMemcpyDeviceToHost, st));
  SBB_CUDA(cudaStreamSynchronize(st));
  return check_wait_status();
}

int sbb_layer_train_step_host(sbb_layer *L, const void *x_host, const void *y_host, long B, long hypercolumn) {
  SBB_TRY(check_layer(L));
  ARG(x_host && y_host, "layer_train_step_host: null pointer");
  SBB_TRY(check_batch(L, B));
  ARG(hypercolumn < L->H, "layer_train_step_host: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  if (L->desc.kind != SBB_LAYER_PLASTIC) hypercolumn = -1;
  const size_t s = esize(L->desc.dtype);
  SBB_TRY(L->hx.reserve((size_t)B * L->N * s));
  SBB_TRY(L->ht.reserve((size_t)B * L->M * s));
  cudaStream_t st = L->own_stream;
  // Work queued earlier on other streams (a device-buffer call) must have landed
  // before this call reads or rewrites the layer state on its own stream.
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_CUDA(cudaMemcpyAsync(L->hx.d, x_host, (size_t)B * L->N * s, cudaMemcpyHostToDevice, st));
  SBB_CUDA(cudaMemcpyAsync(L->ht.d, y_host, (size_t)B * L->M * s, cudaMemcpyHostToDevice, st));
  SBB_TRY(DISPATCH(L->desc.dtype,
                   layer_train_step<float>(L, (const float *)L->hx.d, (const float *)L->ht.d, B, hypercolumn, st),
                   layer_train_step<double>(L, (const double *)L->hx.d, (const double *)L->ht.d, B, hypercolumn, st)));
  SBB_CUDA(cudaStreamSynchronize(st));
  return check_wait_status();
}

int sbb_layer_step_host(sbb_layer *L, const void *x_host, const void *target_host, long B, long hypercolumn,
                        void *y_host) {
  SBB_TRY(check_layer(L));
  ARG(x_host, "layer_step_host: null pointer");
  SBB_TRY(check_batch(L, B));
  ARG(hypercolumn < L->H, "layer_step_host: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  if (L->desc.kind != SBB_LAYER_PLASTIC) hypercolumn = -1;
  const size_t s = esize(L->desc.dtype);
  SBB_TRY(L->hx.reserve((size_t)B * L->N * s));
  SBB_TRY(L->hy.reserve((size_t)B * L->M * s));
  if (target_host) SBB_TRY(L->ht.reserve((size_t)B * L->M * s));
  cudaStream_t st = L->own_stream;
  // Work queued earlier on other streams (a device-buffer call) must have landed
  // before this call reads or rewrites the layer state on its own stream.
  SBB_CUDA(cudaDeviceSynchronize());
  SBB_CUDA(cudaMemcpyAsync(L->hx.d, x_host, (size_t)B * L->N * s, cudaMemcpyHostToDevice, st));
  if (target_host)
    SBB_CUDA(cudaMemcpyAsync(L->ht.d, target_host, (size_t)B * L->M * s, cudaMemcpyHostToDevice, st));
  const void *train_on = target_host ? L->ht.d : L->hy.d;
  if (L->desc.dtype == SBB_F32) {
    SBB_TRY(layer_forward<float>(L, (const float *)L->hx.d, B, (float *)L->hy.d, st));
    SBB_TRY(layer_train_step<float>(L, (const float *)L->hx.d, (const float *)train_on, B, hypercolumn, st));
  } else {
    SBB_TRY(layer_forward<double>(L, (const double *)L->hx.d, B, (double *)L->hy.d, st));
    SBB_TRY(layer_train_step<double>(L, (const double *)L->hx.d, (const double *)train_on, B, hypercolumn, st));
  }
  if (y_host) SBB_CUDA(cudaMemcpyAsync(y_host, L->hy.d, (size_t)B * L->M * s, cudaMemcpyDeviceToHost, st));
  SBB_CUDA(cudaStreamSynchronize(st));
  return check_wait_status();
}

int sbb_layer_step_host_async(sbb_layer *L, const void *x_host, const void *target_host, long B, long hypercolumn,
                              void *y_host) {
  SBB_TRY(check_layer(L));
  ARG(x_host, "layer_step_host_async: null pointer");
  SBB_TRY(check_batch(L, B));
  ARG(hypercolumn < L->H, "layer_step_host_async: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  if (L->desc.kind != SBB_LAYER_PLASTIC) hypercolumn = -1;
  const size_t s = esize(L->desc.dtype);
  if (!L->h2d_stream) {
    SBB_CUDA(cudaStreamCreateWithFlags(&L->h2d_stream, cudaStreamNonBlocking));
    SBB_CUDA(cudaStreamCreateWithFlags(&L->d2h_stream, cudaStreamNonBlocking));
    for (int k = 0; k < 2; ++k) {
      SBB_CUDA(cudaEventCreateWithFlags(&L->ev_copied[k], cudaEventDisableTiming));
      SBB_CUDA(cudaEventCreateWithFlags(&L->ev_stepped[k], cudaEventDisableTiming));
      SBB_CUDA(cudaEventCreateWithFlags(&L->ev_read[k], cudaEventDisableTiming));
    }
  }
  if (!L->async_open) {
    // Work queued earlier on other streams must have landed before this pipeline touches the layer.
    SBB_CUDA(cudaDeviceSynchronize());
    L->async_open = true;
  }
  const int slot = (int)(L->async_calls & 1ull);
  // growing a staging buffer allocates (and so waits for the device): only the first calls do
  SBB_TRY(L->ax[slot].reserve((size_t)B * L->N * s));
  SBB_TRY(L->ay[slot].reserve((size_t)B * L->M * s));
  if (target_host) SBB_TRY(L->at[slot].reserve((size_t)B * L->M * s));
  cudaStream_t st = L->own_stream;
  // inputs: after the step that last read this slot, beside the step now running
  SBB_CUDA(cudaStreamWaitEvent(L->h2d_stream, L->ev_stepped[slot], 0));
  SBB_CUDA(cudaMemcpyAsync(L->ax[slot].d, x_host, (size_t)B * L->N * s, cudaMemcpyHostToDevice, L->h2d_stream));
  if (target_host)
    SBB_CUDA(cudaMemcpyAsync(L->at[slot].d, target_host, (size_t)B * L->M * s, cudaMemcpyHostToDevice,
                             L->h2d_stream));
  SBB_CUDA(cudaEventRecord(L->ev_copied[slot], L->h2d_stream));
  // the step: behind its inputs and behind the read-out of the activation this slot held two calls ago
  SBB_CUDA(cudaStreamWaitEvent(st, L->ev_copied[slot], 0));
  SBB_CUDA(cudaStreamWaitEvent(st, L->ev_read[slot], 0));
  const void *train_on = target_host ? L->at[slot].d : L->ay[slot].d;
  if (L->desc.dtype == SBB_F32) {
    SBB_TRY(layer_forward<float>(L, (const float *)L->ax[slot].d, B, (float *)L->ay[slot].d, st));
    SBB_TRY(layer_train_step<float>(L, (const float *)L->ax[slot].d, (const float *)train_on, B, hypercolumn, st));
  } else {
    SBB_TRY(layer_forward<double>(L, (const double *)L->ax[slot].d, B, (double *)L->ay[slot].d, st));
    SBB_TRY(layer_train_step<double>(L, (const double *)L->ax[slot].d, (const double *)train_on, B, hypercolumn, st));
  }
  SBB_CUDA(cudaEventRecord(L->ev_stepped[slot], st));
  if (y_host) {
    SBB_CUDA(cudaStreamWaitEvent(L->d2h_stream, L->ev_stepped[slot], 0));
    SBB_CUDA(cudaMemcpyAsync(y_host, L->ay[slot].d, (size_t)B * L->M * s, cudaMemcpyDeviceToHost, L->d2h_stream));
    SBB_CUDA(cudaEventRecord(L->ev_read[slot], L->d2h_stream));
  }
  L->async_calls += 1;
  return SBB_OK;
}

int sbb_layer_wait(sbb_layer *L) {
  SBB_TRY(check_layer(L));
  if (L->h2d_stream) {
    SBB_CUDA(cudaStreamSynchronize(L->h2d_stream));
    SBB_CUDA(cudaStreamSynchronize(L->own_stream));
    SBB_CUDA(cudaStreamSynchronize(L->d2h_stream));
  }
  L->async_open = false;
  return check_wait_status();
}

// ------------------------------------------------------------ data parallel
size_t sbb_layer_delta_elems(const sbb_layer *L) {
  if (!L) return 0;
  return (size_t)L->N + (size_t)L->M + (size_t)L->N * L->M;
}

static int check_rows(const sbb_layer *L, long rb, long re) {
  ARG(rb >= 0 && re <= L->N && rb <= re, "row range [%ld,%ld) outside [0,%ld)", rb, re, L->N);
  ARG(rb % 128 == 0, "row_begin %ld is not a multiple of 128", rb);
  return SBB_OK;
}

int sbb_layer_dp_local(sbb_layer *L, const void *x_dev, const void *y_dev, long B_local, void *delta_dev,
                       long row_begin, long row_end, void *stream) {
  SBB_TRY(check_layer(L));
  ARG(x_dev && y_dev && delta_dev, "dp_local: null pointer");
  SBB_TRY(check_batch(L, B_local));
  SBB_TRY(check_rows(L, row_begin, row_end));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype,
                  layer_dp_local<float>(L, (const float *)x_dev, (const float *)y_dev, B_local, (float *)delta_dev,
                                        row_begin, row_end, st),
                  layer_dp_local<double>(L, (const double *)x_dev, (const double *)y_dev, B_local,
                                         (double *)delta_dev, row_begin, row_end, st));
}

int sbb_layer_dp_apply_vectors(sbb_layer *L, const void *delta_dev, long B_global, void *stream) {
  SBB_TRY(check_layer(L));
  ARG(delta_dev, "dp_apply_vectors: null pointer");
  ARG(B_global > 0, "dp_apply_vectors: non-positive global batch");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, layer_dp_apply_vectors<float>(L, (const float *)delta_dev, B_global, st),
                  layer_dp_apply_vectors<double>(L, (const double *)delta_dev, B_global, st));
}

int sbb_layer_dp_apply_rows(sbb_layer *L, const void *delta_dev, long B_global, long row_begin, long row_end,
                            void *stream) {
  SBB_TRY(check_layer(L));
  ARG(delta_dev, "dp_apply_rows: null pointer");
  ARG(B_global > 0, "dp_apply_rows: non-positive global batch");
  SBB_TRY(check_rows(L, row_begin, row_end));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype,
                  layer_dp_apply_rows<float>(L, (const float *)delta_dev, B_global, row_begin, row_end, st),
                  layer_dp_apply_rows<double>(L, (const double *)delta_dev, B_global, row_begin, row_end, st));
}

int sbb_layer_dp_finish(sbb_layer *L, long hypercolumn, void *stream) {
  SBB_TRY(check_layer(L));
  ARG(hypercolumn < L->H, "dp_finish: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, layer_finish<float>(L, hypercolumn, st), layer_finish<double>(L, hypercolumn, st));
}

}  // extern "C"

// ------------------------------------------------- row-sharded layer over peer-mapped memory
namespace {

enum { kShardX0 = 0, kShardX1 = 1, kShardX2 = 2, kShardMask = 3, kShardW = 4, kShardCij = 5, kShardCi = 6 };

void *shard_local_buffer(sbb_layer *L, int which) {
  switch (which) {
    case kShardX0: return L->shard.xg[0].d;
    case kShardX1: return L->shard.xg[1].d;
    case kShardX2: return L->shard.xg[2].d;
    case kShardMask: return L->score.d;
    case kShardW: return L->state[SBB_STATE_WEIGHTS];
    case kShardCij: return L->state[SBB_STATE_CIJ];
    default: return L->state[SBB_STATE_CI];
  }
}

long shard_begin(const sbb_layer *L, long r) {
  const long b = r * L->shard.rows_per_rank;
  return b < L->N ? b : L->N;
}

// Table of one address per rank: that rank's buffer `which` plus a byte offset.
sbb::PeerTable shard_table(sbb_layer *L, int which, size_t byte_offset) {
  sbb::PeerTable t{};
  t.n = (int)L->shard.world;
  for (int r = 0; r < t.n; ++r) t.ptr[r] = static_cast<char *>(L->shard.peer[which][r]) + byte_offset;
  return t;
}

int check_shard(sbb_layer *L, bool need_peers) {
  SBB_TRY(check_layer(L));
  ARG(L->shard.on, "the layer is not row-sharded (sbb_layer_shard_init)");
  ARG(!need_peers || L->shard.attached, "the peers' buffers are not attached yet (sbb_layer_shard_attach)");
  return SBB_OK;
}

// The step in flight was opened by sbb_layer_shard_forward with the same local batch.
int check_shard_step(sbb_layer *L, long B, const char *what) {
  SBB_TRY(check_shard(L, true));
  ARG(B > 0 && B == L->shard.batch, "%s: local batch %ld, but the step in flight (sbb_layer_shard_forward) has %ld", what,
      B, L->shard.batch);
  return SBB_OK;
}

template <typename T>
int shard_scatter(sbb_layer *L, const T *x, long B, cudaStream_t st) {
  auto &S = L->shard;
  const int slot = (S.cur + 1 + S.staged) % 3;   // every rank makes the same calls, so the slots agree
  // rank o receives this rank's samples as rows [rank * B, (rank + 1) * B) of its [world * B, rows of o] buffer
  sbb::PeerTable t{};
  t.n = (int)S.world;
  for (long o = 0; o < S.world; ++o) {
    const long width = shard_begin(L, o + 1) - shard_begin(L, o);
    t.ptr[o] = static_cast<T *>(S.peer[kShardX0 + slot][o]) + (size_t)S.rank * B * width;
  }
  if (S.world == 1) {
    SBB_CUDA(sbb::launch_scatter_columns<T>(x, B, L->N, S.rows_per_rank, t, st));
    S.staged += 1;   // (recorded only once everything is queued: a failed call stages nothing)
    S.slot_batch[slot] = B;
    return SBB_OK;
  }
  // Across ranks the column blocks travel by copy engines (strided 2-D copies over NVLink): the exchange of a
  // batch staged ahead then runs beside the current step's contractions without taking issue slots or
  // shared-memory bandwidth from them (a store kernel on a side stream cost the forward product 7 %).
  // Owners are visited starting after this rank, so that at any time every rank sends to a different owner.
  for (long k = 1; k <= S.world; ++k) {
    const long o = (S.rank + k) % S.world;
    const long rb = shard_begin(L, o), width = shard_begin(L, o + 1) - rb;
    if (width <= 0) continue;
    SBB_CUDA(cudaMemcpy2DAsync(t.ptr[o], (size_t)width * sizeof(T), x + rb, (size_t)L->N * sizeof(T),
                               (size_t)width * sizeof(T), (size_t)B, cudaMemcpyDeviceToDevice, st));
  }
  S.staged += 1;
  S.slot_batch[slot] = B;
  return SBB_OK;
}

template <typename T>
int shard_forward(sbb_layer *L, long B, T *support, cudaStream_t st) {
  auto &S = L->shard;
  const long rb = shard_begin(L, S.rank), re = shard_begin(L, S.rank + 1);
  const long nr = re - rb, Bg = B * S.world, M = L->M;
  if (nr <= 0) {   // more ranks than 128-row blocks: this rank owns nothing and adds nothing
    SBB_CUDA(cudaMemsetAsync(support, 0, (size_t)Bg * M * sizeof(T), st));
    return SBB_OK;
  }
  const T *xg = static_cast<const T *>(S.xg[S.cur].d);
  const T *W = static_cast<const T *>(L->state[SBB_STATE_WEIGHTS]) + rb * M;
  bool tc = tensor_path<T>(xg, W, nr, M) && (reinterpret_cast<uintptr_t>(support) & 7u) == 0;
  const int splits = tc ? sbb::forward_splits_tc(Bg, nr, M) : sbb::forward_splits<T>(Bg, nr, M);
  T *partial = support;
  if (splits > 1) {
    SBB_TRY(L->fwd_partial.reserve((size_t)splits * Bg * M * sizeof(T)));
    partial = static_cast<T *>(L->fwd_partial.d);
  }
  PhaseTimer timer(L, SBB_PHASE_FORWARD, st);
  if (tc) {
    if constexpr (std::is_same<T, float>::value)
      SBB_CUDA(sbb::launch_forward_product_tc(xg, W, partial, Bg, nr, M, splits, st));
  } else {
    SBB_CUDA(sbb::launch_forward_product<T>(xg, W, partial, Bg, nr, M, splits, st));
  }
  timer.stop();
  if (splits > 1) SBB_CUDA(sbb::launch_sum_partials<T>(partial, splits, Bg * M, support, st));
  return SBB_OK;
}

template <typename T>
int shard_activate(sbb_layer *L, long B, const T *support, T *y_local, cudaStream_t st) {
  auto &S = L->shard;
  const long Bg = B * S.world, M = L->M;
  SBB_TRY(S.yg.reserve((size_t)Bg * M * sizeof(T)));
  T *yg = static_cast<T *>(S.yg.d);
  SBB_CUDA(sbb::launch_reduce_bias_softmax<T>(support, 1, static_cast<const T *>(L->state[SBB_STATE_BIAS]), yg, Bg, L->H,
                                              L->Mc, 1, st));
  if (y_local)
    SBB_CUDA(cudaMemcpyAsync(y_local, yg + (size_t)S.rank * B * M, (size_t)B * M * sizeof(T), cudaMemcpyDeviceToDevice, st));
  return SBB_OK;
}

template <typename T>
int shard_train(sbb_layer *L, long B, long h, cudaStream_t st) {
  auto &S = L->shard;
  const long rb = shard_begin(L, S.rank), re = shard_begin(L, S.rank + 1);
  const long nr = re - rb, Bg = B * S.world, N = L->N, M = L->M;
  ARG(S.yg.d != nullptr && S.yg.cap >= (size_t)Bg * M * sizeof(T), "shard_train: no activations (sbb_layer_shard_activate)");
  const sbb::TraceParams<T> p = sbb::make_trace_params<T>(L->desc.taupdt, L->desc.taupdt / 2, Bg);
  const T *xg = static_cast<const T *>(S.xg[S.cur].d);
  const T *yg = static_cast<const T *>(S.yg.d);
  T *Ci = static_cast<T *>(L->state[SBB_STATE_CI]);
  T *Cj = static_cast<T *>(L->state[SBB_STATE_CJ]);
  T *Cij = static_cast<T *>(L->state[SBB_STATE_CIJ]);
  T *W = static_cast<T *>(L->state[SBB_STATE_WEIGHTS]);
  const uint8_t *wmask = static_cast<const uint8_t *>(L->state[SBB_STATE_WMASK]);
  // Cj from the whole batch on every rank (identical inputs, identical results); Ci, Cij and the weights for the
  // own rows only, addressed as a layer of `nr` inputs that starts at row rb
  SBB_CUDA(sbb::launch_colsum<T>(yg, Bg, M, nullptr, Cj, p, 1, st));
  if (nr > 0) {
    SBB_CUDA(sbb::launch_colsum<T>(xg, Bg, nr, nullptr, Ci + rb, p, 1, st));
    PhaseTimer timer(L, SBB_PHASE_TRACE, st);
    if (tensor_path<T>(xg, yg, nr, M)) {
      if constexpr (std::is_same<T, float>::value)
        SBB_CUDA(sbb::launch_trace_update_tc(xg, yg, Bg, nr, M, L->H, Ci + rb, Cj, Cij + rb * M, W + rb * M,
                                             wmask ? wmask + rb * L->H : nullptr, static_cast<const int *>(L->col_hc.d),
                                             static_cast<float *>(L->rc.d), p, 0, nr, st));
    } else {
      SBB_CUDA(sbb::launch_trace_update_fused<T>(xg, yg, Bg, nr, M, L->H, L->Mc, Ci + rb, Cj, Cij + rb * M, W + rb * M,
                                                 wmask ? wmask + rb * L->H : nullptr, p, 0, nr, st));
    }
    timer.stop();
  }
  if (L->desc.kind != SBB_LAYER_PLASTIC) return SBB_OK;
  const double cthr = L->desc.taupdt / 2;
  SBB_CUDA(sbb::launch_update_bias_regularized<T>(static_cast<T *>(L->state[SBB_STATE_BIAS]),
                                                  static_cast<T *>(L->state[SBB_STATE_KBI]), Cj, (T)cthr,
                                                  (T)L->desc.khalf, (T)L->desc.pmin, (T)L->desc.taubdt, M, st));
  if (h >= 0 && nr > 0)   // scores of the owned rows, into every rank's work arrays
    SBB_CUDA(sbb::launch_mask_score_rows<T>(wmask, Ci, Cj, Cij, (T)cthr, N, M, L->H, L->Mc, h, rb, re,
                                            shard_table(L, kShardMask, 0), st));
  return SBB_OK;
}

template <typename T>
int shard_mask(sbb_layer *L, long h, cudaStream_t st) {
  auto &S = L->shard;
  const double cthr = L->desc.taupdt / 2;
  const T *Ci = static_cast<const T *>(L->state[SBB_STATE_CI]);
  const T *Cj = static_cast<const T *>(L->state[SBB_STATE_CJ]);
  const T *Cij = static_cast<const T *>(L->state[SBB_STATE_CIJ]);
  uint8_t *wmask = static_cast<uint8_t *>(L->state[SBB_STATE_WMASK]);
  // the swaps, identically on every rank (all hold all scores); every owner rewrites the weights of its own rows
  SBB_CUDA(sbb::launch_mask_select<T>(wmask, Ci, Cj, Cij, (T)cthr, L->N, L->M, L->H, L->Mc, h, L->desc.mask_iterations,
                                      L->score.d, st, nullptr));
  const long rb = shard_begin(L, S.rank), re = shard_begin(L, S.rank + 1);
  sbb::PeerTable own{};
  own.n = 1;
  own.ptr[0] = L->state[SBB_STATE_WEIGHTS];
  SBB_CUDA(sbb::launch_mask_rewrite_rows<T>(wmask, L->score.d, Ci, Cj, Cij, (T)cthr, L->N, L->M, L->H, L->Mc, h, rb, re,
                                            own, st));
  return SBB_OK;
}

// Copies `bytes` at `offset` of this rank's buffer `which` to the same place in every other rank's.
int shard_share(sbb_layer *L, int which, size_t offset, size_t bytes, cudaStream_t st) {
  auto &S = L->shard;
  if (bytes == 0) return SBB_OK;
  const char *src = static_cast<const char *>(S.peer[which][S.rank]) + offset;
  sbb::PeerTable others{};
  for (long r = 0; r < S.world; ++r)
    if (r != S.rank) others.ptr[others.n++] = static_cast<char *>(S.peer[which][r]) + offset;
  if (bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0)
    SBB_CUDA(sbb::launch_peer_broadcast<uint4>(reinterpret_cast<const uint4 *>(src), (long)(bytes / 16), others, st));
  else if (bytes % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 7u) == 0)
    SBB_CUDA(sbb::launch_peer_broadcast<double>(reinterpret_cast<const double *>(src), (long)(bytes / 8), others, st));
  else
    SBB_CUDA(sbb::launch_peer_broadcast<float>(reinterpret_cast<const float *>(src), (long)(bytes / 4), others, st));
  return SBB_OK;
}

}  // namespace

extern "C" {

int sbb_layer_shard_init(sbb_layer *L, long rank, long world_size, long max_local_batch, unsigned char *handles_out) {
  SBB_TRY(check_layer(L));
  ARG(handles_out, "shard_init: null pointer");
  ARG(world_size >= 1 && world_size <= 8 && rank >= 0 && rank < world_size, "shard_init: rank %ld of %ld (at most 8)",
      rank, world_size);
  ARG(max_local_batch > 0, "shard_init: non-positive batch");
  SBB_TRY(check_batch(L, max_local_batch * world_size));
  ARG(!L->shard.on, "shard_init: the layer is already sharded");
  auto &S = L->shard;
  const size_t s = esize(L->desc.dtype);
  const long tiles = (L->N + 127) / 128;
  S.rank = rank;
  S.world = world_size;
  S.max_batch = max_local_batch;
  S.rows_per_rank = ((tiles + world_size - 1) / world_size) * 128;
  // every rank allocates a full block's width, so that the buffers have one size everywhere
  const size_t xg_bytes = (size_t)world_size * max_local_batch * S.rows_per_rank * s;
  for (auto &b : S.xg) SBB_TRY(b.reserve(xg_bytes));
  if (L->score.d == nullptr) SBB_TRY(L->score.reserve(sbb::mask_scratch_bytes(L->N, s)));
  for (int b = 0; b < SBB_SHARD_BUFFERS; ++b)
    for (int r = 0; r < 8; ++r) {
      S.peer[b][r] = nullptr;
      S.opened[b][r] = false;
    }
  for (int b = 0; b < SBB_SHARD_BUFFERS; ++b) {
    S.peer[b][rank] = shard_local_buffer(L, b);
    cudaIpcMemHandle_t hnd;
    SBB_CUDA(cudaIpcGetMemHandle(&hnd, S.peer[b][rank]));
    static_assert(sizeof(hnd) == SBB_SHARD_HANDLE_BYTES, "IPC handle size");
    std::memcpy(handles_out + (size_t)b * SBB_SHARD_HANDLE_BYTES, &hnd, sizeof(hnd));
  }
  S.cur = 0;
  S.staged = 0;
  S.batch = 0;
  S.on = true;
  S.attached = world_size == 1;
  return SBB_OK;
}

int sbb_layer_shard_attach(sbb_layer *L, const unsigned char *all_handles) {
  SBB_TRY(check_shard(L, false));
  ARG(all_handles, "shard_attach: null pointer");
  auto &S = L->shard;
  for (long r = 0; r < S.world; ++r) {
    if (r == S.rank) continue;
    for (int b = 0; b < SBB_SHARD_BUFFERS; ++b) {
      if (S.opened[b][r]) continue;
      cudaIpcMemHandle_t hnd;
      std::memcpy(&hnd, all_handles + ((size_t)r * SBB_SHARD_BUFFERS + b) * SBB_SHARD_HANDLE_BYTES, sizeof(hnd));
      void *p = nullptr;
      SBB_CUDA(cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess));
      S.peer[b][r] = p;
      S.opened[b][r] = true;
    }
  }
  S.attached = true;
  return SBB_OK;
}

int sbb_layer_shard_scatter(sbb_layer *L, const void *x_dev, long B_local, void *stream) {
  SBB_TRY(check_shard(L, true));
  ARG(x_dev, "shard_scatter: null pointer");
  ARG(B_local > 0 && B_local <= L->shard.max_batch, "shard_scatter: local batch %ld outside [1, %ld] (sbb_layer_shard_init)",
      B_local, L->shard.max_batch);
  ARG(L->shard.staged < 2, "shard_scatter: two batches are already staged; run a step (sbb_layer_shard_forward) first");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, shard_scatter<float>(L, (const float *)x_dev, B_local, st),
                  shard_scatter<double>(L, (const double *)x_dev, B_local, st));
}

int sbb_layer_shard_forward(sbb_layer *L, long B_local, void *support_dev, void *stream) {
  SBB_TRY(check_shard(L, true));
  ARG(support_dev, "shard_forward: null pointer");
  {
    auto &S = L->shard;
    ARG(S.staged >= 1, "shard_forward: no batch is staged (sbb_layer_shard_scatter)");
    const int next = (S.cur + 1) % 3;
    ARG(B_local == S.slot_batch[next], "shard_forward: local batch %ld, but the staged batch has %ld", B_local,
        S.slot_batch[next]);
    S.cur = next;   // the oldest staged batch becomes the step in flight
    S.staged -= 1;
    S.batch = B_local;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = DISPATCH(L->desc.dtype, shard_forward<float>(L, B_local, (float *)support_dev, st),
                          shard_forward<double>(L, B_local, (double *)support_dev, st));
  if (rc != SBB_OK) {   // nothing was consumed: the batch stays staged
    auto &S = L->shard;
    S.cur = (S.cur + 2) % 3;
    S.staged += 1;
    S.batch = 0;
  }
  return rc;
}

int sbb_layer_shard_activate(sbb_layer *L, long B_local, const void *support_dev, void *y_local_dev, void *stream) {
  SBB_TRY(check_shard_step(L, B_local, "shard_activate"));
  ARG(support_dev, "shard_activate: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, shard_activate<float>(L, B_local, (const float *)support_dev, (float *)y_local_dev, st),
                  shard_activate<double>(L, B_local, (const double *)support_dev, (double *)y_local_dev, st));
}

int sbb_layer_shard_train(sbb_layer *L, long B_local, long hypercolumn, void *stream) {
  SBB_TRY(check_shard_step(L, B_local, "shard_train"));
  ARG(hypercolumn < L->H, "shard_train: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  if (L->desc.kind != SBB_LAYER_PLASTIC) hypercolumn = -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, shard_train<float>(L, B_local, hypercolumn, st),
                  shard_train<double>(L, B_local, hypercolumn, st));
}

int sbb_layer_shard_mask(sbb_layer *L, long hypercolumn, void *stream) {
  SBB_TRY(check_shard(L, true));
  ARG(L->desc.kind == SBB_LAYER_PLASTIC, "shard_mask: the layer has no mask");
  ARG(hypercolumn >= 0 && hypercolumn < L->H, "shard_mask: hypercolumn %ld outside [0,%ld)", hypercolumn, L->H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return DISPATCH(L->desc.dtype, shard_mask<float>(L, hypercolumn, st), shard_mask<double>(L, hypercolumn, st));
}

int sbb_layer_shard_drop_staged(sbb_layer *L) {
  SBB_TRY(check_shard(L, false));
  L->shard.staged = 0;
  return SBB_OK;
}

int sbb_layer_shard_share_rows(sbb_layer *L, void *stream) {
  SBB_TRY(check_shard(L, true));
  auto &S = L->shard;
  const size_t s = esize(L->desc.dtype);
  const long rb = shard_begin(L, S.rank), re = shard_begin(L, S.rank + 1);
  if (re <= rb) return SBB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SBB_TRY(shard_share(L, kShardCij, (size_t)rb * L->M * s, (size_t)(re - rb) * L->M * s, st));
  SBB_TRY(shard_share(L, kShardW, (size_t)rb * L->M * s, (size_t)(re - rb) * L->M * s, st));
  SBB_TRY(shard_share(L, kShardCi, (size_t)rb * s, (size_t)(re - rb) * s, st));
  return SBB_OK;
}

long sbb_layer_shard_world(const sbb_layer *L) { return L != nullptr && L->shard.on && L->shard.attached ? L->shard.world : 0; }

int sbb_layer_shard_rows(const sbb_layer *L, long rank, long *row_begin, long *row_end) {
  ARG(L && row_begin && row_end, "shard_rows: null pointer");
  ARG(L->shard.on, "shard_rows: the layer is not sharded");
  ARG(rank >= 0 && rank < L->shard.world, "shard_rows: rank %ld outside [0,%ld)", rank, L->shard.world);
  *row_begin = shard_begin(L, rank);
  *row_end = shard_begin(L, rank + 1);
  return SBB_OK;
}

int sbb_count_correct(int dtype, const void *pred_dev, const void *labels_dev, long rows, long classes,
                      long *correct_host, void *stream) {
  SBB_TRY(check_dtype(dtype));
  ARG(pred_dev && labels_dev && correct_host, "count_correct: null pointer");
  ARG(rows >= 0 && classes > 0, "count_correct: bad shape");
  SBB_TRY(need_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Staged cnt;
  SBB_TRY(cnt.alloc(sizeof(unsigned long long)));
  SBB_CUDA(cudaMemsetAsync(cnt.d, 0, sizeof(unsigned long long), st));
  if (dtype == SBB_F32)
    SBB_CUDA(sbb::launch_count_correct<float>((const float *)pred_dev, (const float *)labels_dev, rows, classes,
                                              cnt.as<unsigned long long>(), st));
  else
    SBB_CUDA(sbb::launch_count_correct<double>((const double *)pred_dev, (const double *)labels_dev, rows, classes,
                                               cnt.as<unsigned long long>(), st));
  unsigned long long h = 0;
  SBB_CUDA(cudaMemcpyAsync(&h, cnt.d, sizeof(h), cudaMemcpyDeviceToHost, st));
  SBB_CUDA(cudaStreamSynchronize(st));
  *correct_host = (long)h;
  return check_wait_status();
}

}  // extern "C"
