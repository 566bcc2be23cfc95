/* sbb200.h -- C ABI of the B200 BCPNN layer backend (libsbb200.so).
 *
 * Every function returns SBB_OK (0) or an SBB_ERR_* code; sbb_last_error() gives
 * the message of the calling thread's last failure.  Nothing here calls exit(),
 * traps on the device, or falls back to the CPU: without a CUDA device every
 * compute entry point returns SBB_ERR_NO_DEVICE.
 *
 * All matrices are row-major and C-contiguous.  N = in_features, H =
 * hypercolumns, Mc = minicolumns, M = H*Mc = out_features, B = batch rows.
 * `dtype` selects float (SBB_F32) or double (SBB_F64) for every REAL pointer.
 * Scalars are passed as double and rounded to REAL inside, as pybind11 does for
 * the reference's Python floats.
 *
 * Citations name the StreamBrain interface each entry point replaces, by path
 * inside the StreamBrain repository (K/ = BCPNN/backend/_kernels/).
 */
#ifndef SBB200_H
#define SBB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SBB_OK 0
#define SBB_ERR_INVALID 1     /* bad argument (null pointer, size, dtype, range) */
#define SBB_ERR_CUDA 2        /* a CUDA runtime call or kernel launch failed */
#define SBB_ERR_NO_DEVICE 3   /* no usable CUDA device */
#define SBB_ERR_UNSUPPORTED 4 /* shape or mode this build does not handle */
#define SBB_ERR_TIMEOUT 5     /* a bounded device-side wait gave up */

#define SBB_F32 0
#define SBB_F64 1

#define SBB_LAYER_DENSE 0   /* DenseLayer: traces + weights each step, bias at finalize */
#define SBB_LAYER_PLASTIC 1 /* StructuralPlasticityLayer: + regularised bias + mask */

/* Which state array sbb_layer_{set,get}_state / sbb_layer_state_ptr address. */
#define SBB_STATE_WEIGHTS 0 /* REAL [N, M] */
#define SBB_STATE_BIAS 1    /* REAL [M]    */
#define SBB_STATE_CI 2      /* REAL [N]    */
#define SBB_STATE_CJ 3      /* REAL [M]    */
#define SBB_STATE_CIJ 4     /* REAL [N, M] */
#define SBB_STATE_KBI 5     /* REAL [M]     (plastic only) */
#define SBB_STATE_WMASK 6   /* uint8 [N, H] (plastic only) */

int sbb_version(void);
const char *sbb_last_error(void);
/* Number of CUDA devices visible (0 without a driver); never fails. */
int sbb_device_count(void);

/* ------------------------------------------------------------------------
 * Stateless kernels on HOST buffers.  Each call stages its operands to the
 * current CUDA device, runs the kernels, copies the mutated arrays back and
 * synchronises -- the calling convention of the reference's native kernel
 * modules, whose pybind11 functions take numpy arrays and mutate them in place.
 * ---------------------------------------------------------------------- */

/* activation[B,M] = inputs[B,N] * weights[N,M] + bias[M].
 * Replaces update_state_float{32,64}: K/kernels_openmp_internal.cc:342-358, 464-465. */
int sbb_update_state(int dtype, void *activation, const void *inputs, const void *weights,
                     const void *bias, long B, long N, long M);

/* a[rows,M] += bias[M].  Replaces add_bias_float{32,64}: K/kernels_cuda_internal.cu:915-936
 * (wrapper K/kernels_cuda.py:18-26). */
int sbb_add_bias(int dtype, void *a, const void *bias, long rows, long M);

/* Softmax over each group of Mc consecutive entries of a[rows, H*Mc], in place.
 * Replaces softmax_minicolumns: K/kernels_numpy.py:13-25 (used by the cpu backend,
 * BCPNN/backend/cpu_backend.py:10,24) and K/kernels_cuda.py:29-37. */
int sbb_softmax_minicolumns(int dtype, void *a, long rows, long H, long Mc);

/* Un-fused trace update C = max(0, (1-t)C + t*mean_b(.)) for Ci, Cj, Cij.
 * Replaces update_counters: K/kernels_numpy.py:28-49, K/kernels_cuda.py:40-48. */
int sbb_update_counters(int dtype, void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o,
                        double taupdt, long B, long N, long M);

/* Fused trace update + log-ratio weights (new Ci, Cj, Cij, weights in place).
 * Replaces update_weights_float{32,64} of the OpenMP module:
 * K/kernels_openmp_internal.cc:89-205, 361-383, 461-462 (wrapper K/kernels_openmp.py:16-25). */
int sbb_update_weights(int dtype, void *Ci, void *Cj, void *Cij, const void *a_i, const void *a_o,
                       double taupdt, long B, long N, long M, void *weights, double cthr);

/* weights = 0 where Ci<cthr or Cj<cthr, else log(max(Cij,cthr^4)/(Ci*Cj)).
 * Replaces the un-fused update_weights: K/kernels_numpy.py:52-64, K/kernels_cuda.py:51-59. */
int sbb_recompute_weights(int dtype, void *weights, const void *Ci, const void *Cj, const void *Cij,
                          double cthr, long N, long M);

/* bias = log(Cj), or log(2 cthr) where Cj < cthr.
 * Replaces update_bias_float{32,64}: K/kernels_openmp_internal.cc:207-220, 386-396. */
int sbb_update_bias(int dtype, void *bias, const void *Cj, double cthr, long M);

/* Regularised bias with the gain trace kbi.
 * Replaces update_bias_regularized_float{32,64}: K/kernels_openmp_internal.cc:222-246, 399-415. */
int sbb_update_bias_regularized(int dtype, void *bias, void *kbi, const void *Cj, double cthr,
                                double khalf, double pmin, double taubdt, long M);

/* Structural-plasticity swap for hypercolumn h: up to `iterations` times the
 * silent connection with the highest score replaces the active one with the lowest.
 * Replaces update_mask_float{32,64}: K/kernels_openmp_internal.cc:248-320, 418-441. */
int sbb_update_mask(int dtype, uint8_t *wmask, const void *weights, const void *Ci, const void *Cj,
                    const void *Cij, double cthr, long N, long M, long H, long Mc, long h,
                    long iterations);

/* weights[i,j] = 0 where wmask[i, j/Mc] == 0.
 * Replaces apply_mask_float{32,64}: K/kernels_openmp_internal.cc:322-335, 444-458. */
int sbb_apply_mask(int dtype, void *weights, const uint8_t *wmask, long N, long M, long H, long Mc);

/* ------------------------------------------------------------------------
 * Device-resident layer.  State lives in HBM for the life of the handle; a train
 * step allocates nothing after the first call at a given batch size.  Handles
 * are bound to the device current at creation and are not thread-safe.
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 * calls enqueue work and return without synchronising unless stated.
 * Replaces the layer objects of BCPNN/backend/_cpu_base_backend.py:7-172 as
 * specialised by BCPNN/backend/cpu_backend.py:7-52.
 * ---------------------------------------------------------------------- */
typedef struct sbb_layer sbb_layer;

typedef struct sbb_layer_desc {
  int dtype;            /* SBB_F32 / SBB_F64 */
  int kind;             /* SBB_LAYER_DENSE / SBB_LAYER_PLASTIC */
  long in_features;     /* N */
  long hypercolumns;    /* H */
  long minicolumns;     /* Mc */
  double taupdt;        /* trace time constant; cthr = taupdt/2 */
  double khalf, pmin, taubdt; /* regularised-bias parameters (plastic) */
  long mask_iterations; /* swaps attempted per mask update (the cpu backend uses 16) */
} sbb_layer_desc;

int sbb_layer_create(const sbb_layer_desc *desc, sbb_layer **out);
int sbb_layer_destroy(sbb_layer *layer);

/* The description the layer was created with (its shape attributes in_features, hypercolumns,
 * minicolumns and hyper-parameters: BCPNN/backend/_cpu_base_backend.py:22-30, 93-105). */
int sbb_layer_info(const sbb_layer *layer, sbb_layer_desc *out);

/* Copy one state array from / to host memory (synchronous).  `bytes` must equal
 * the array's size.  These are the lazy attribute views (weights, bias, Ci, Cj,
 * Cij, kbi, wmask) of the reference's layer objects. */
int sbb_layer_set_state(sbb_layer *layer, int which, const void *host, size_t bytes);
int sbb_layer_get_state(sbb_layer *layer, int which, void *host, size_t bytes);
/* Device address of a state array (for callers that keep tensors on the device). */
int sbb_layer_state_ptr(sbb_layer *layer, int which, void **device_ptr);

/* y[B,M] = softmax_minicolumns(x[B,N] * weights + bias); x, y on the device.
 * compute_activation: BCPNN/backend/_cpu_base_backend.py:44-51, 126-133. */
int sbb_layer_forward(sbb_layer *layer, const void *x_dev, long B, void *y_dev, void *stream);

/* One train step from device buffers x[B,N] (layer input) and y[B,M] (layer
 * output, or the one-hot labels for the classifier).  `hypercolumn` >= 0 also
 * runs the mask update for that hypercolumn (plastic only); pass -1 for none.
 * train_step: BCPNN/backend/cpu_backend.py:13-15, 29-52. */
int sbb_layer_train_step(sbb_layer *layer, const void *x_dev, const void *y_dev, long B,
                         long hypercolumn, void *stream);

/* Dense: bias = log(Cj).  Plastic: no-op.  train_finalize: cpu_backend.py:17-18. */
int sbb_layer_train_finalize(sbb_layer *layer, void *stream);

/* Same two calls with HOST buffers: inputs are copied to the device, results
 * copied back (y_host may be NULL for sbb_layer_step_host) and the call returns
 * after synchronising.  sbb_layer_step_host runs forward + train step, the body
 * of the reference's training loop (BCPNN/backend/_cpu_base_backend.py:290-309);
 * `target_host` is NULL for a hidden layer (it trains on its own activation) or
 * the labels [B,M] for the classifier. */
int sbb_layer_forward_host(sbb_layer *layer, const void *x_host, long B, void *y_host);
/* train_step alone from host buffers x[B,N], y[B,M] (the reference signature
 * train_step(inputs, outputs[, hypercolumn]): cpu_backend.py:13, 29). */
int sbb_layer_train_step_host(sbb_layer *layer, const void *x_host, const void *y_host, long B,
                              long hypercolumn);
int sbb_layer_step_host(sbb_layer *layer, const void *x_host, const void *target_host, long B,
                        long hypercolumn, void *y_host);
/* The same step without waiting for it: the inputs are copied on a copy stream into one of
 * two staging buffers, the step runs on the layer's own stream behind the copy, the activation
 * is copied to y_host (may be NULL) on a third stream, and the call returns at once.  The
 * copy of call k+1 therefore runs beside the step of call k (the loop body of
 * _cpu_base_backend.py:290-309 with its host-device traffic double-buffered).  Host buffers
 * should be page-locked, must stay untouched until sbb_layer_wait returns (x_host, target_host)
 * and hold the result only after it (y_host).  Between the first such call and sbb_layer_wait
 * no other entry point may be used on this layer. */
int sbb_layer_step_host_async(sbb_layer *layer, const void *x_host, const void *target_host, long B,
                              long hypercolumn, void *y_host);
/* Waits for every sbb_layer_step_host_async issued so far (copies included). */
int sbb_layer_wait(sbb_layer *layer);

/* ------------------------------------------------------------------------
 * Batch data-parallel step, split around the one exchange the path has.
 * `delta` is a device buffer of N + M + N*M REALs laid out [sum_b x | sum_b y |
 * x^T y].  Each rank calls sbb_layer_dp_local on its slice of the batch, the
 * caller sum-reduces `delta` across ranks (NCCL), then every rank calls
 * sbb_layer_dp_apply_vectors once, sbb_layer_dp_apply_rows over all rows and
 * sbb_layer_dp_finish.  Row ranges let the caller pipeline the reduction of one
 * block of rows behind the product of the next; row_begin must be a multiple of
 * 128.  Semantics: K/kernels_mpi_internal.cc:71-250 (per-rank partial sums,
 * Allreduce, update with divisor batch*world_size).
 * ---------------------------------------------------------------------- */
size_t sbb_layer_delta_elems(const sbb_layer *layer);
/* x^T y for rows [row_begin,row_end) of the trace matrix into delta; with
 * row_begin == 0 also the two column sums. */
int sbb_layer_dp_local(sbb_layer *layer, const void *x_dev, const void *y_dev, long B_local,
                       void *delta_dev, long row_begin, long row_end, void *stream);
/* Ci, Cj moving averages from the reduced sums (divisor B_global). */
int sbb_layer_dp_apply_vectors(sbb_layer *layer, const void *delta_dev, long B_global, void *stream);
/* Cij moving average + weights (+ mask) for rows [row_begin,row_end). */
int sbb_layer_dp_apply_rows(sbb_layer *layer, const void *delta_dev, long B_global, long row_begin,
                            long row_end, void *stream);
/* Regularised bias and, with hypercolumn >= 0, the mask update (plastic only). */
int sbb_layer_dp_finish(sbb_layer *layer, long hypercolumn, void *stream);

/* ------------------------------------------------------------------------
 * Row-sharded data-parallel step over peer-mapped memory (one process per GPU, at
 * most 8 GPUs of one node).  Every rank owns an equal block of input rows of the
 * layer (multiples of 128): those rows of the weights, of Cij, of Ci and of the mask
 * work.  The batch stays split by samples on the way in and out (rank r feeds and
 * receives samples [r*B, (r+1)*B) of the global batch of world_size*B), and one step
 * is forward + train of an unsupervised layer, which learns from its own activations:
 *   1. sbb_layer_shard_scatter: column block o of this rank's input batch goes to
 *      rank o over NVLink (plain peer stores), so that every owner holds its columns
 *      of the whole global batch;
 *   -- barrier over the ranks (the caller's: any collective on `stream`) --
 *   2. sbb_layer_shard_forward: the owner's part of every sample's support,
 *      x[:, own rows] * W[own rows, :], into support_dev [world_size*B, M];
 *   -- the caller sums support_dev over the ranks in place (one all-reduce of
 *      world_size*B*M elements: the only collective that carries data) --
 *   3. sbb_layer_shard_activate: bias + softmax of the summed supports, identically on
 *      every rank; this rank's B rows are copied to y_local_dev when it is not NULL;
 *   4. sbb_layer_shard_train: Ci of the own rows, Cj, the own rows of Cij and of the
 *      weights from the global batch (one fused launch, as on one GPU), bias; with
 *      hypercolumn >= 0 also the mask scores of the own rows into every rank's work
 *      arrays, and then  -- barrier --  5. sbb_layer_shard_mask: the swaps, identically
 *      on every rank, and the owner rewrites the weights of its swapped rows.
 * The result is the single-GPU step at the global batch, which is also what the
 * reduce-then-update scheme of the reference's MPI backend computes
 * (K/kernels_mpi_internal.cc:100-250; its own row-sharded tail kernels with
 * Allgatherv: :263-286, 352-404, 453-484).  Per rank and step about
 * (world_size-1)/world_size * B*N elements cross NVLink on the way out plus the
 * all-reduce of the supports, instead of two passes over an N x M matrix, and every
 * rank does 1/world_size of the global step's arithmetic and memory traffic.
 * Between barriers no kernel waits on another rank.
 * Staging ahead.  The gathered inputs live in three buffers used in turn, so a rank may scatter
 * batch t+1 while step t is still running: sbb_layer_shard_scatter stages a batch (at most two
 * staged at a time) and sbb_layer_shard_forward takes the oldest staged one.  The rules that keep
 * this free of races: (i) a rank starts the scatter of batch t+1 only after the all-reduce of step
 * t-1's supports has completed on its stream (every rank entered it, so every rank has finished
 * step t-2, the last reader of the buffer being refilled); (ii) between every rank's scatter of
 * batch t+1 and any rank's forward pass on it lies a collective that each rank enters after its
 * own scatter has completed -- the all-reduce of step t's supports serves when the scatter ran on
 * a side stream that `stream` waited for before that all-reduce, and then step t+1 needs no
 * barrier of its own; the first step of a run uses the explicit barrier of point 1.
 * While a layer is sharded a rank
 * holds current values only for its own rows of the weights, Cij and Ci;
 * sbb_layer_shard_share_rows copies them to all ranks (then a barrier) when the whole
 * layer is wanted everywhere: the plain forward pass, checkpoints, tests.
 * ---------------------------------------------------------------------- */
#define SBB_SHARD_BUFFERS 7        /* three gathered-input buffers, mask work arrays, weights, Cij, Ci */
#define SBB_SHARD_HANDLE_BYTES 64  /* one CUDA IPC memory handle */
/* Allocates the gathered-input buffers for local batches of up to max_local_batch samples and writes
 * this rank's SBB_SHARD_BUFFERS IPC handles to handles_out (SBB_SHARD_BUFFERS * SBB_SHARD_HANDLE_BYTES
 * bytes), to be exchanged by the caller. */
int sbb_layer_shard_init(sbb_layer *layer, long rank, long world_size, long max_local_batch,
                         unsigned char *handles_out);
/* all_handles: the handles of ranks 0..world_size-1, concatenated in rank order. */
int sbb_layer_shard_attach(sbb_layer *layer, const unsigned char *all_handles);
/* Stages x_dev, this rank's [B_local, in_features] slice of a global batch, for the oldest step not yet
 * started; every rank passes the same B_local and makes the same sequence of calls. */
int sbb_layer_shard_scatter(sbb_layer *layer, const void *x_dev, long B_local, void *stream);
/* Starts the step on the oldest staged batch.  support_dev: [world_size * B_local, M] REALs, written in
 * full (the caller then sums it over the ranks). */
int sbb_layer_shard_forward(sbb_layer *layer, long B_local, void *support_dev, void *stream);
/* support_dev: the summed supports; y_local_dev: NULL or [B_local, M] for this rank's activations. */
int sbb_layer_shard_activate(sbb_layer *layer, long B_local, const void *support_dev, void *y_local_dev,
                             void *stream);
int sbb_layer_shard_train(sbb_layer *layer, long B_local, long hypercolumn, void *stream);
int sbb_layer_shard_mask(sbb_layer *layer, long hypercolumn, void *stream);
int sbb_layer_shard_share_rows(sbb_layer *layer, void *stream);
/* Forgets the batches that are staged but that no step will consume (every rank alike; host state only). */
int sbb_layer_shard_drop_staged(sbb_layer *layer);
/* Number of ranks the layer is sharded over (peers attached), 0 if it is not. */
long sbb_layer_shard_world(const sbb_layer *layer);
/* Input rows [row_begin, row_end) of the layer that `rank` owns. */
int sbb_layer_shard_rows(const sbb_layer *layer, long rank, long *row_begin, long *row_end);

/* ------------------------------------------------------------------------
 * The fit / evaluate loops of a stack of layers, run below the host language:
 * the dataset is kept on the device, batches are assembled there from the
 * epoch's sample order, all kernels of all batches are queued on one stream
 * without host synchronisation, and evaluation hits are counted on the device.
 * Replaces Network of BCPNN/backend/_cpu_base_backend.py:174-314 (and the
 * device-side shuffled batching of BCPNN/backend/full_cuda_backend/dataloader.h:70-132).
 * Layers are borrowed: the caller creates and destroys them.  Random orders are
 * drawn by the caller (the reference draws them from NumPy's global stream:
 * _cpu_base_backend.py:258-264), so seeded runs reproduce the reference's.
 * ---------------------------------------------------------------------- */
typedef struct sbb_network sbb_network;

/* How a data-parallel network sums the batch deltas over ranks (the reference's
 * mpi backend calls MPI_Allreduce inside its kernel: K/kernels_mpi_internal.cc:153-161).
 * reduce_begin starts an in-place sum over ranks of `elems` REALs at device_ptr, ordered
 * after the work already queued on `stream`, and returns a token >= 0 (< 0 on failure);
 * reduce_wait makes `stream` wait for that reduction and returns 0 on success. */
typedef struct sbb_comm {
  void *user;
  long (*reduce_begin)(void *user, void *device_ptr, size_t elems, int dtype, void *stream);
  int (*reduce_wait)(void *user, long token, void *stream);
} sbb_comm;

/* The schedule of one batch of an epoch, as pure arithmetic (no device): the slice
 * [first, first + count) of the epoch's sample order that `rank` of `world_size` takes of batch
 * number `batch` (count = floor(batch size / world_size); _cpu_base_backend.py:279-288), and
 * the position `mask_slot` in the epoch's hypercolumn order of the hypercolumn whose mask is
 * updated with this batch, or -1 for none (_cpu_base_backend.py:297-302).  epoch > 0 with fewer
 * batches than hypercolumns + 1 returns SBB_ERR_UNSUPPORTED (the reference's ZeroDivisionError).
 * sbb_network_train_batches and sbb_network_evaluate follow exactly this plan. */
int sbb_network_batch_plan(long samples, long maximal_batch_size, long world_size, long rank, long hypercolumns,
                           long epoch, long batch, long *first, long *count, long *mask_slot);

int sbb_network_create(int dtype, sbb_network **out);
int sbb_network_destroy(sbb_network *net);
/* Network.add_layer: _cpu_base_backend.py:182-186 (the caller converts the layer's dtype first). */
int sbb_network_add_layer(sbb_network *net, sbb_layer *layer);
/* world_rank / world_size of the slice rule (_cpu_base_backend.py:179-180, 223-233, 279-288);
 * `comm` may be NULL (ranks then train independently on their slices, as the cpu backend would);
 * with `comm` every train step is the split data-parallel step, whatever world_size is: the
 * row-sharded one (sbb_layer_shard_*; the reduction callbacks sum the supports and serve as the
 * barrier) for unsupervised layers sharded over world_size ranks, else reduce-and-replicate
 * (sbb_layer_dp_*).  At the end of an epoch a sharded layer's rows are shared with all ranks. */
int sbb_network_set_data_parallel(sbb_network *net, long rank, long world_size, const sbb_comm *comm);
/* Copies images[samples, features] and labels[samples, classes] (host, REAL) to the device. */
int sbb_network_set_dataset(sbb_network *net, const void *images_host, const void *labels_host, long samples,
                            long features, long classes);
/* The epoch's sample order (a permutation of [0, samples), host): _cpu_base_backend.py:258-260. */
int sbb_network_set_epoch_order(sbb_network *net, const long *order_host);
/* Batches [batch_begin, batch_end) of one epoch of training layer `layer_index`
 * (_cpu_base_backend.py:266-312).  `epoch` counts from 0 inside one fit call: mask updates
 * happen only for epoch > 0, for hypercolumn hypercolumn_order_host[i / period] at batches
 * i % period == 0 with period = batches_per_epoch / (H + 1); period == 0 is the reference's
 * ZeroDivisionError and returns SBB_ERR_UNSUPPORTED.  The call that includes the epoch's last
 * batch also runs train_finalize and waits for the device; earlier calls only queue work. */
int sbb_network_train_batches(sbb_network *net, long layer_index, long maximal_batch_size,
                              const long *hypercolumn_order_host, long epoch, long batch_begin, long batch_end);
/* Network.evaluate over the dataset in stored order: _cpu_base_backend.py:205-245.  Returns this
 * rank's counts; the caller sums them over ranks (mpi_backend.py:63-69). */
int sbb_network_evaluate(sbb_network *net, long maximal_batch_size, long *correct, long *total);

/* Count argmax(pred[r,:]) == argmax(labels[r,:]) over rows, device buffers;
 * writes the count to *correct_host after synchronising the stream.
 * Network.evaluate: BCPNN/backend/_cpu_base_backend.py:239-240. */
int sbb_count_correct(int dtype, const void *pred_dev, const void *labels_dev, long rows, long classes,
                      long *correct_host, void *stream);

/* Mask update that allocates nothing: for hosts that own all device memory
 * themselves (one pre-sized arena) or cannot accept the device-wide stall of
 * cudaMalloc/cudaFree inside their step loop.  Same arithmetic and result as
 * sbb_update_mask, but every array is a DEVICE pointer supplied by the caller
 * (wmask is updated in place; weights_dev may be NULL, the un-masked weights are
 * then recomputed from the traces) and the two per-row work arrays live in a
 * fixed 1.7 MiB array inside the library, resident on every GPU that loads it
 * until the process exits.  More than SBB_NOALLOC_MAX_ROWS input rows returns
 * SBB_ERR_UNSUPPORTED without launching.  All calls on a device share that
 * array: calls that overlap in time on one GPU race and must be serialised by
 * the caller.  The first call on each device looks up the array's address
 * (cudaGetSymbolAddress) and should be made outside any stream capture.  The
 * work is enqueued on `stream`; the call does not synchronise.  The message of a
 * failure is returned by sbb_noalloc_last_error() and by sbb_last_error().
 * This entry point has no counterpart in the reference. */
#define SBB_NOALLOC_MAX_ROWS 131072
int sbb_update_mask_noalloc(int dtype, uint8_t *wmask_dev, const void *weights_dev, const void *Ci_dev,
                            const void *Cj_dev, const void *Cij_dev, double cthr, long N, long M, long H,
                            long Mc, long h, long iterations, void *stream);
const char *sbb_noalloc_last_error(void);

/* Per-phase device timing of a layer.  With profiling enabled every forward and
 * every train step brackets its dominant kernel (phase 0: forward product,
 * phase 1: trace update) with CUDA events on the launching stream, in a ring of
 * SBB_PROFILE_SLOTS slots per phase.  sbb_layer_phase_ms returns the duration of
 * call number `index` (0 = first call after enabling) once that work has
 * finished; it synchronises on the slot's end event.  No counterpart in the
 * reference, which only takes wall-clock times around fit/evaluate (train.py:181-193). */
#define SBB_PROFILE_SLOTS 64
#define SBB_PHASE_FORWARD 0
#define SBB_PHASE_TRACE 1
int sbb_layer_profile(sbb_layer *layer, int enable);
int sbb_layer_phase_calls(sbb_layer *layer, int phase, long *calls);
int sbb_layer_phase_ms(sbb_layer *layer, int phase, long index, float *ms);

/* Which kernels carry the two contractions (forward product, x^T y) of float32
 * layers: SBB_PATH_GENERAL = the general-shape FFMA kernels, SBB_PATH_TENSOR =
 * the tcgen05 tensor-core kernels (three TF32 products per float32 product)
 * wherever the shape is eligible (row pitches multiples of 16 bytes, device of
 * compute capability 10.x), the general-shape kernels otherwise.  float64 and
 * ineligible shapes always take the general-shape kernels.  The initial value is
 * SBB_PATH_TENSOR unless the environment variable SBB_CONTRACTION is "general".
 * Process-wide. */
#define SBB_PATH_GENERAL 0
#define SBB_PATH_TENSOR 1
int sbb_set_contraction_path(int path);
int sbb_get_contraction_path(void);
/* Multiprocessors the persistent tensor-core kernel of sbb_layer_dp_local (the batch
 * outer product of one row block) leaves free: it launches one CTA per remaining
 * multiprocessor.  A data-parallel step sets this so that the kernels of the collective
 * reducing the previous row block, which run beside it on another stream, find room
 * at once instead of waiting for a resident CTA to retire.  0 (the initial value, or the
 * environment variable SBB_COMM_SMS) uses every multiprocessor.  Process-wide.
 * No counterpart in the reference (its MPI backend reduces on the host). */
int sbb_set_reserved_sms(int sms);
int sbb_get_reserved_sms(void);
/* 1 when the tensor-core kernels can run on the current device. */
int sbb_tensor_path_available(void);
/* Status of the bounded device-side waits of the tensor-core kernels on the
 * current device: *status = 0 when every wait completed, else the code of the
 * first wait that gave up (SBB_ERR_TIMEOUT is returned as well).  Synchronises
 * the device. */
int sbb_device_wait_status(int *status);
/* The status word is sticky: once a wait has given up, every entry point that waits for device work
 * (sbb_layer_get_state, sbb_layer_wait, the *_host calls, sbb_count_correct, sbb_stream_sync,
 * sbb_network_*) returns SBB_ERR_TIMEOUT after its own wait, because the kernel that gave up left its
 * step half done: the traces and weights of the layers stepped since the last clean check are undefined
 * and must be reloaded (sbb_layer_set_state).  This call then resets the word so that work can go on.
 * Synchronises the device.  No counterpart in the reference (its kernels have no waits). */
int sbb_device_clear_wait_status(void);
/* Time limit of one device-side wait, in SM clock cycles (initially 4e9, about two seconds).  Process-wide. */
int sbb_set_wait_limit_cycles(long long cycles);
long long sbb_get_wait_limit_cycles(void);
/* Test hook: each of the next `launches` tensor-core launches of the forward product or the fused trace update
 * loses one barrier arrival in its first CTA, so that a wait inside the kernel runs into its time limit, the CTA
 * gives up in order (no trap, no endless loop) and the status word reports it.  Used with a short time limit to
 * check that path; results of such a launch are undefined. */
int sbb_debug_lose_arrival(int launches);

/* ------------------------------------------------------------------------
 * Dataset files (host code; no device needed).  Images are unsigned bytes scaled
 * to [0, 1] as REAL, labels unsigned bytes expanded to one-hot REAL rows.
 * ---------------------------------------------------------------------- */
/* Rank and dimensions of an IDX file (MNIST / Fashion-MNIST), validated against the
 * file size.  Replaces the header handling of train.py:10-18 (which skips 16 / 8 bytes
 * unchecked) and BCPNN/backend/full_cuda_backend/dataset.cpp:30-47. */
int sbb_idx_info(const char *path, int *ndim, long dims[4]);
/* out[samples, features] = bytes / 255.  train.py:9-15, dataset.cpp:49-60. */
int sbb_read_idx_images(const char *path, int dtype, void *out, long samples, long features);
/* out[samples, classes] one-hot.  train.py:17-21. */
int sbb_read_idx_labels(const char *path, int dtype, void *out, long samples, long classes);
/* Size in bytes of a headerless file (the STL-10 binaries). */
int sbb_raw_u8_count(const char *path, long *bytes);
/* out[samples, features] = bytes / 255 in file order.  load_stl_10_images: train.py:26-31. */
int sbb_read_raw_u8_images(const char *path, int dtype, void *out, long samples, long features);
/* out[samples, classes] one-hot of (byte - first_label).  load_stl_10_labels: train.py:34-41
 * (first_label = 1). */
int sbb_read_raw_u8_labels(const char *path, int dtype, void *out, long samples, long classes, long first_label);

/* Measured float64 rates of the current device in TFLOP/s: a register-resident DFMA loop and a loop of the
 * float64 tensor-core instruction (mma.sync.m8n8k4): the denominators of the float64 kernels' roofline, and the
 * evidence for running them on the FP64 pipe (on B200 the two rates are equal).  Synchronises the device.  No
 * counterpart in the reference. */
int sbb_measure_fp64_rates(double *dfma_tflops, double *dmma_tflops);

/* Number of kernels this library has launched in this process (all threads). */
unsigned long long sbb_kernel_launches(void);

/* Block until all work on `stream` has finished. */
int sbb_stream_sync(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SBB200_H */
