// The training / evaluation loop of a layer stack, behind the C ABI (sbb_network_*).
//
// What the loop does is fixed by StreamBrain's Network class (BCPNN/backend/_cpu_base_backend.py:205-314):
// batches of `maximal_batch_size` consecutive positions of the epoch's sample order (the last one partial),
// of which rank r of w takes the r-th slice of floor(size / w) samples; a forward pass through the layers up
// to the one being trained; from the second epoch of a fit call on, a mask update every nb / (H + 1) batches
// for the hypercolumn the epoch's hypercolumn order names; the last layer trains on the labels; train_finalize
// after every epoch.  How it is done here: the dataset lives on the device, a batch is assembled by a gather
// kernel from the epoch's order (uploaded once per epoch; the order itself comes from the caller's random
// stream, so seeded runs reproduce the reference's), every kernel of every batch is queued on one stream with
// no host synchronisation in between, and evaluation hits are counted on the device and read once.
// The file uses the layer objects only through the public C ABI.
#include "../../include/sbb200.h"
#include "sbb_kernels.cuh"

#include <cstdarg>
#include <cstdio>
#include <string>
#include <vector>

namespace sbb {
void set_last_error(const char *message);
}

namespace {

int net_fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  sbb::set_last_error(buf);
  return code;
}

#define NET_CUDA(call)                                                                       \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return net_fail(SBB_ERR_CUDA, "%s: %s (%s)", #call, cudaGetErrorName(e__), cudaGetErrorString(e__)); \
  } while (0)

#define NET_TRY(call)               \
  do {                              \
    int rc__ = (call);              \
    if (rc__ != SBB_OK) return rc__; \
  } while (0)

struct DeviceBuffer {
  void *d = nullptr;
  size_t cap = 0;
  int reserve(size_t bytes) {
    if (bytes <= cap) return SBB_OK;
    if (d) NET_CUDA(cudaFree(d));
    d = nullptr;
    cap = 0;
    NET_CUDA(cudaMalloc(&d, bytes));
    cap = bytes;
    return SBB_OK;
  }
  void release() {
    if (d) cudaFree(d);
    d = nullptr;
    cap = 0;
  }
};

// Row blocks of the batch outer product whose reductions are pipelined: at most `blocks` ranges of
// [0, rows) whose starts are multiples of 128.
std::vector<std::pair<long, long>> row_blocks(long rows, long blocks) {
  const long tiles = (rows + 127) / 128;
  if (blocks > tiles) blocks = tiles;
  if (blocks < 1) blocks = 1;
  std::vector<std::pair<long, long>> out;
  long start = 0;
  for (long k = 0; k < blocks; ++k) {
    long end = ((tiles * (k + 1)) / blocks) * 128;
    if (end > rows) end = rows;
    if (end > start) {
      out.emplace_back(start, end);
      start = end;
    }
  }
  return out;
}

}  // namespace

struct sbb_network {
  int dtype = SBB_F32;
  int device = 0;
  std::vector<sbb_layer *> layers;
  std::vector<sbb_layer_desc> desc;
  long rank = 0, world = 1;
  sbb_comm comm{};
  bool have_comm = false;
  // dataset
  DeviceBuffer images, labels, order;
  long samples = 0, features = 0, classes = 0;
  bool have_order = false;
  // per-batch buffers
  DeviceBuffer batch_x, batch_t;
  std::vector<DeviceBuffer> act;   // activation of every layer
  DeviceBuffer delta;              // data-parallel batch sums of the layer being trained
  DeviceBuffer hits;               // evaluation counter
  DeviceBuffer token;              // one float: the barrier of the row-sharded step
  DeviceBuffer support;            // row-sharded step: supports of the global batch, summed over the ranks in place
  DeviceBuffer ahead_x[2];         // row-sharded step: the batch staged ahead is assembled here, in turn
  cudaStream_t side = nullptr;     // row-sharded step: assembles and exchanges the next batch beside the current step
  cudaEvent_t ev_step = nullptr, ev_staged = nullptr;
  cudaStream_t stream = nullptr;
  size_t esize() const { return dtype == SBB_F32 ? 4 : 8; }
  long out_features(size_t k) const { return desc[k].hypercolumns * desc[k].minicolumns; }
};

namespace {

int check_net(const sbb_network *net) {
  if (!net) return net_fail(SBB_ERR_INVALID, "null network handle");
  int dev = -1;
  NET_CUDA(cudaGetDevice(&dev));
  if (dev != net->device)
    return net_fail(SBB_ERR_INVALID, "network lives on device %d but device %d is current", net->device, dev);
  return SBB_OK;
}

// Assembles rows [first, first + count) of the current order into the batch buffers (labels when wanted).
int assemble(sbb_network *net, long first, long count, bool shuffled, bool want_labels, const void **x,
             const void **t) {
  const size_t s = net->esize();
  const long *order = shuffled ? static_cast<const long *>(net->order.d) : nullptr;
  if (!shuffled) {   // consecutive samples: used in place
    *x = static_cast<const char *>(net->images.d) + (size_t)first * net->features * s;
    *t = static_cast<const char *>(net->labels.d) + (size_t)first * net->classes * s;
    return SBB_OK;
  }
  NET_TRY(net->batch_x.reserve((size_t)count * net->features * s));
  if (net->dtype == SBB_F32)
    NET_CUDA(sbb::launch_gather_rows<float>((const float *)net->images.d, order, first, count, net->features,
                                            (float *)net->batch_x.d, net->stream));
  else
    NET_CUDA(sbb::launch_gather_rows<double>((const double *)net->images.d, order, first, count, net->features,
                                             (double *)net->batch_x.d, net->stream));
  *x = net->batch_x.d;
  *t = nullptr;
  if (want_labels) {
    NET_TRY(net->batch_t.reserve((size_t)count * net->classes * s));
    if (net->dtype == SBB_F32)
      NET_CUDA(sbb::launch_gather_rows<float>((const float *)net->labels.d, order, first, count, net->classes,
                                              (float *)net->batch_t.d, net->stream));
    else
      NET_CUDA(sbb::launch_gather_rows<double>((const double *)net->labels.d, order, first, count, net->classes,
                                               (double *)net->batch_t.d, net->stream));
    *t = net->batch_t.d;
  }
  return SBB_OK;
}

// Forward pass through layers [0, upto]; returns the input and the output of layer `upto`.
int forward_through(sbb_network *net, const void *x, long count, size_t upto, const void **in_last,
                    const void **out_last) {
  const size_t s = net->esize();
  const void *cur = x;
  for (size_t k = 0; k <= upto; ++k) {
    NET_TRY(net->act[k].reserve((size_t)count * net->out_features(k) * s));
    NET_TRY(sbb_layer_forward(net->layers[k], cur, count, net->act[k].d, net->stream));
    *in_last = cur;
    cur = net->act[k].d;
  }
  *out_last = cur;
  return SBB_OK;
}

// A one-element reduction on the network's stream: orders the stream after every rank's earlier work.
int rank_barrier(sbb_network *net) {
  NET_TRY(net->token.reserve(sizeof(float)));
  const long t = net->comm.reduce_begin(net->comm.user, net->token.d, 1, SBB_F32, net->stream);
  if (t < 0 || net->comm.reduce_wait(net->comm.user, t, net->stream) != 0)
    return net_fail(SBB_ERR_INVALID, "the reduction callback failed (barrier of the row-sharded step)");
  return SBB_OK;
}

bool row_sharded(const sbb_network *net, const sbb_layer *layer) {
  return net->have_comm && net->world > 0 && sbb_layer_shard_world(layer) == net->world;
}

// Shuffled rows [first, first + count) of the dataset, assembled into `buf` on `stream`.
int assemble_images(sbb_network *net, long first, long count, DeviceBuffer &buf, cudaStream_t stream, const void **x) {
  NET_TRY(buf.reserve((size_t)count * net->features * net->esize()));
  const long *order = static_cast<const long *>(net->order.d);
  if (net->dtype == SBB_F32)
    NET_CUDA(sbb::launch_gather_rows<float>((const float *)net->images.d, order, first, count, net->features,
                                            (float *)buf.d, stream));
  else
    NET_CUDA(sbb::launch_gather_rows<double>((const double *)net->images.d, order, first, count, net->features,
                                             (double *)buf.d, stream));
  *x = buf.d;
  return SBB_OK;
}

// The part of the row-sharded step after the exchange of the inputs: forward product of the staged batch, sum of
// the supports over the ranks, activation into `y`, train step, mask update.  `staged_ahead`: the next batch was
// scattered on the side stream, which the network's stream joins before the all-reduce (so that the all-reduce
// also tells every rank that all exchanges of the next batch are complete).
int sharded_step(sbb_network *net, sbb_layer *layer, const sbb_layer_desc &d, void *y, long count, long hypercolumn,
                 bool staged_ahead) {
  const long M = d.hypercolumns * d.minicolumns;
  const size_t elems = (size_t)count * net->world * M;
  NET_TRY(net->support.reserve(elems * net->esize()));
  NET_TRY(sbb_layer_shard_forward(layer, count, net->support.d, net->stream));
  if (staged_ahead) NET_CUDA(cudaStreamWaitEvent(net->stream, net->ev_staged, 0));
  const long t = net->comm.reduce_begin(net->comm.user, net->support.d, elems, net->dtype, net->stream);
  if (t < 0 || net->comm.reduce_wait(net->comm.user, t, net->stream) != 0)
    return net_fail(SBB_ERR_INVALID, "the reduction callback failed (supports of the row-sharded step)");
  NET_TRY(sbb_layer_shard_activate(layer, count, net->support.d, y, net->stream));
  const bool mask = hypercolumn >= 0 && d.kind == SBB_LAYER_PLASTIC;
  NET_TRY(sbb_layer_shard_train(layer, count, mask ? hypercolumn : -1, net->stream));
  if (mask) {
    NET_TRY(rank_barrier(net));
    NET_TRY(sbb_layer_shard_mask(layer, hypercolumn, net->stream));
  }
  return SBB_OK;
}

// One data-parallel train step of `layer`: the reduction of one row block of x^T y runs beside the product of
// the next (BCPNN/backend/_kernels/kernels_mpi_internal.cc:100-161 with the Allreduce pipelined by rows).
int dp_train_step(sbb_network *net, sbb_layer *layer, const sbb_layer_desc &d, const void *x, const void *y,
                  long count, long hypercolumn) {
  const long N = d.in_features, M = d.hypercolumns * d.minicolumns;
  const size_t s = net->esize();
  NET_TRY(net->delta.reserve(sbb_layer_delta_elems(layer) * s));
  char *delta = static_cast<char *>(net->delta.d);
  const auto blocks = row_blocks(N, 4);
  std::vector<long> tokens;
  for (const auto &b : blocks) {
    NET_TRY(sbb_layer_dp_local(layer, x, y, count, delta, b.first, b.second, net->stream));
    // block 0 also owns the two column sums at the head of the buffer
    const size_t lo = b.first == 0 ? 0 : (size_t)(N + M) + (size_t)b.first * M;
    const size_t hi = (size_t)(N + M) + (size_t)b.second * M;
    const long token = net->comm.reduce_begin(net->comm.user, delta + lo * s, hi - lo, net->dtype, net->stream);
    if (token < 0) return net_fail(SBB_ERR_INVALID, "the reduction callback failed to start (block at row %ld)", b.first);
    tokens.push_back(token);
  }
  const long global = count * net->world;
  for (size_t k = 0; k < blocks.size(); ++k) {
    if (net->comm.reduce_wait(net->comm.user, tokens[k], net->stream) != 0)
      return net_fail(SBB_ERR_INVALID, "the reduction callback failed to complete (block %zu)", k);
    if (k == 0) NET_TRY(sbb_layer_dp_apply_vectors(layer, delta, global, net->stream));
    NET_TRY(sbb_layer_dp_apply_rows(layer, delta, global, blocks[k].first, blocks[k].second, net->stream));
  }
  return sbb_layer_dp_finish(layer, hypercolumn, net->stream);
}

}  // namespace

extern "C" {

int sbb_network_batch_plan(long samples, long maximal_batch_size, long world_size, long rank, long hypercolumns,
                           long epoch, long batch, long *first, long *count, long *mask_slot) {
  if (!first || !count || !mask_slot) return net_fail(SBB_ERR_INVALID, "batch_plan: null pointer");
  if (samples <= 0 || maximal_batch_size <= 0 || world_size < 1 || rank < 0 || rank >= world_size || hypercolumns < 1 ||
      epoch < 0)
    return net_fail(SBB_ERR_INVALID, "batch_plan: bad arguments");
  const long nb = (samples + maximal_batch_size - 1) / maximal_batch_size;
  if (batch < 0 || batch >= nb) return net_fail(SBB_ERR_INVALID, "batch_plan: batch %ld outside [0, %ld)", batch, nb);
  const long begin = batch * maximal_batch_size;
  const long end = begin + maximal_batch_size < samples ? begin + maximal_batch_size : samples;
  const long local = (end - begin) / world_size;   // the remainder of an uneven split is dropped
  *first = begin + rank * local;
  *count = local;
  *mask_slot = -1;
  if (epoch > 0) {
    const long period = nb / (hypercolumns + 1);
    // the reference computes batch % (nb // (H + 1)) here and fails with a division by zero
    if (period == 0)
      return net_fail(SBB_ERR_UNSUPPORTED,
                      "division by zero in the mask schedule: %ld batches per epoch are fewer than hypercolumns + 1 = %ld",
                      nb, hypercolumns + 1);
    if (batch % period == 0 && batch / period < hypercolumns) *mask_slot = batch / period;
  }
  return SBB_OK;
}

int sbb_network_create(int dtype, sbb_network **out) {
  if (!out) return net_fail(SBB_ERR_INVALID, "network_create: null pointer");
  *out = nullptr;
  if (dtype != SBB_F32 && dtype != SBB_F64) return net_fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  if (sbb_device_count() <= 0)
    return net_fail(SBB_ERR_NO_DEVICE, "no CUDA device is available; this library has no CPU path");
  sbb_network *net = new sbb_network();
  net->dtype = dtype;
  cudaError_t e = cudaGetDevice(&net->device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&net->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete net;
    return net_fail(SBB_ERR_CUDA, "network_create: %s", cudaGetErrorString(e));
  }
  *out = net;
  return SBB_OK;
}

int sbb_network_destroy(sbb_network *net) {
  if (!net) return SBB_OK;
  net->images.release();
  net->labels.release();
  net->order.release();
  net->batch_x.release();
  net->batch_t.release();
  net->delta.release();
  net->hits.release();
  net->token.release();
  net->support.release();
  net->ahead_x[0].release();
  net->ahead_x[1].release();
  if (net->side) cudaStreamDestroy(net->side);
  if (net->ev_step) cudaEventDestroy(net->ev_step);
  if (net->ev_staged) cudaEventDestroy(net->ev_staged);
  for (auto &a : net->act) a.release();
  if (net->stream) cudaStreamDestroy(net->stream);
  delete net;
  return SBB_OK;
}

int sbb_network_add_layer(sbb_network *net, sbb_layer *layer) {
  NET_TRY(check_net(net));
  sbb_layer_desc d;
  NET_TRY(sbb_layer_info(layer, &d));
  if (d.dtype != net->dtype) return net_fail(SBB_ERR_INVALID, "layer dtype %d differs from the network's %d", d.dtype, net->dtype);
  if (!net->layers.empty() && d.in_features != net->out_features(net->layers.size() - 1))
    return net_fail(SBB_ERR_INVALID, "layer takes %ld inputs but the layer before it has %ld units", d.in_features,
                    net->out_features(net->layers.size() - 1));
  net->layers.push_back(layer);
  net->desc.push_back(d);
  net->act.emplace_back();
  return SBB_OK;
}

int sbb_network_set_data_parallel(sbb_network *net, long rank, long world_size, const sbb_comm *comm) {
  NET_TRY(check_net(net));
  if (world_size < 1 || rank < 0 || rank >= world_size)
    return net_fail(SBB_ERR_INVALID, "rank %ld outside [0, %ld)", rank, world_size);
  if (comm && (!comm->reduce_begin || !comm->reduce_wait))
    return net_fail(SBB_ERR_INVALID, "set_data_parallel: both reduction callbacks are required");
  net->rank = rank;
  net->world = world_size;
  net->have_comm = comm != nullptr;
  if (comm) net->comm = *comm;
  return SBB_OK;
}

int sbb_network_set_dataset(sbb_network *net, const void *images_host, const void *labels_host, long samples,
                            long features, long classes) {
  NET_TRY(check_net(net));
  if (!images_host || !labels_host) return net_fail(SBB_ERR_INVALID, "set_dataset: null pointer");
  if (samples <= 0 || features <= 0 || classes <= 0)
    return net_fail(SBB_ERR_INVALID, "set_dataset: non-positive shape %ld x %ld / %ld", samples, features, classes);
  const size_t s = net->esize();
  NET_CUDA(cudaStreamSynchronize(net->stream));
  NET_TRY(net->images.reserve((size_t)samples * features * s));
  NET_TRY(net->labels.reserve((size_t)samples * classes * s));
  NET_CUDA(cudaMemcpy(net->images.d, images_host, (size_t)samples * features * s, cudaMemcpyHostToDevice));
  NET_CUDA(cudaMemcpy(net->labels.d, labels_host, (size_t)samples * classes * s, cudaMemcpyHostToDevice));
  net->samples = samples;
  net->features = features;
  net->classes = classes;
  net->have_order = false;
  return SBB_OK;
}

int sbb_network_set_epoch_order(sbb_network *net, const long *order_host) {
  NET_TRY(check_net(net));
  if (!order_host) return net_fail(SBB_ERR_INVALID, "set_epoch_order: null pointer");
  if (net->samples <= 0) return net_fail(SBB_ERR_INVALID, "set_epoch_order: no dataset");
  for (long k = 0; k < net->samples; ++k)
    if (order_host[k] < 0 || order_host[k] >= net->samples)
      return net_fail(SBB_ERR_INVALID, "set_epoch_order: entry %ld = %ld outside [0, %ld)", k, order_host[k], net->samples);
  NET_CUDA(cudaStreamSynchronize(net->stream));   // batches of the previous epoch may still read the old order
  NET_TRY(net->order.reserve((size_t)net->samples * sizeof(long)));
  NET_CUDA(cudaMemcpy(net->order.d, order_host, (size_t)net->samples * sizeof(long), cudaMemcpyHostToDevice));
  net->have_order = true;
  return SBB_OK;
}

int sbb_network_train_batches(sbb_network *net, long layer_index, long maximal_batch_size,
                              const long *hypercolumn_order_host, long epoch, long batch_begin, long batch_end) {
  NET_TRY(check_net(net));
  if (layer_index < 0 || (size_t)layer_index >= net->layers.size())
    return net_fail(SBB_ERR_INVALID, "train_batches: layer %ld outside [0, %zu)", layer_index, net->layers.size());
  if (maximal_batch_size <= 0) return net_fail(SBB_ERR_INVALID, "train_batches: non-positive batch size");
  if (net->samples <= 0 || !net->have_order)
    return net_fail(SBB_ERR_INVALID, "train_batches: set the dataset and the epoch's sample order first");
  if (net->features != net->desc[0].in_features)
    return net_fail(SBB_ERR_INVALID, "train_batches: samples have %ld features, the first layer takes %ld",
                    net->features, net->desc[0].in_features);
  const size_t li = (size_t)layer_index;
  const bool last = li + 1 == net->layers.size();
  if (last && net->classes != net->out_features(li))
    return net_fail(SBB_ERR_INVALID, "train_batches: labels have %ld columns, the last layer has %ld units",
                    net->classes, net->out_features(li));
  const long nb = (net->samples + maximal_batch_size - 1) / maximal_batch_size;
  if (batch_begin < 0 || batch_end > nb || batch_begin > batch_end)
    return net_fail(SBB_ERR_INVALID, "train_batches: batches [%ld, %ld) outside [0, %ld)", batch_begin, batch_end, nb);
  const long H = net->desc[li].hypercolumns;
  if (epoch > 0) {
    if (!hypercolumn_order_host) return net_fail(SBB_ERR_INVALID, "train_batches: null hypercolumn order");
    for (long k = 0; k < H; ++k)
      if (hypercolumn_order_host[k] < 0 || hypercolumn_order_host[k] >= H)
        return net_fail(SBB_ERR_INVALID, "train_batches: hypercolumn order entry %ld = %ld outside [0, %ld)", k,
                        hypercolumn_order_host[k], H);
  }
  const bool dp = net->have_comm;   // with callbacks the split step runs even for one rank (a sum over one)
  // a layer that learns from its own activations and is sharded over the ranks takes the row-sharded step
  const bool sharded = !last && row_sharded(net, net->layers[li]);
  bool staged_ahead = false;   // the batch of this iteration was already exchanged during the previous one
  if (sharded && net->side == nullptr) {
    NET_CUDA(cudaStreamCreateWithFlags(&net->side, cudaStreamNonBlocking));
    NET_CUDA(cudaEventCreateWithFlags(&net->ev_step, cudaEventDisableTiming));
    NET_CUDA(cudaEventCreateWithFlags(&net->ev_staged, cudaEventDisableTiming));
  }
  if (batch_begin == 0) NET_CUDA(cudaDeviceSynchronize());   // state written through other streams has landed
  for (long i = batch_begin; i < batch_end; ++i) {
    long first = 0, count = 0, slot = -1;
    NET_TRY(sbb_network_batch_plan(net->samples, maximal_batch_size, net->world, net->rank, H, epoch, i, &first, &count,
                                   &slot));
    if (count <= 0) continue;
    const void *x = nullptr, *t = nullptr, *in_last = nullptr, *out_last = nullptr;
    if (!staged_ahead) NET_TRY(assemble(net, first, count, true, last, &x, &t));
    const long h = slot >= 0 ? hypercolumn_order_host[slot] : -1;
    if (sharded) {   // the layer's own forward pass is part of its sharded step
      if (!staged_ahead) {
        in_last = x;
        if (li > 0) {
          const void *unused = nullptr;
          NET_TRY(forward_through(net, x, count, li - 1, &unused, &in_last));
        }
        NET_TRY(sbb_layer_shard_scatter(net->layers[li], in_last, count, net->stream));
        NET_TRY(rank_barrier(net));
      }
      // The first layer's next batch is assembled and exchanged on the side stream beside this step's forward
      // product; it starts once the previous step has finished here (every rank is then past the step before it).
      staged_ahead = false;
      long first2 = 0, count2 = 0, slot2 = -1;
      if (li == 0 && i + 1 < batch_end) {
        NET_TRY(sbb_network_batch_plan(net->samples, maximal_batch_size, net->world, net->rank, H, epoch, i + 1, &first2,
                                       &count2, &slot2));
        if (count2 > 0) {
          const void *x2 = nullptr;
          NET_CUDA(cudaEventRecord(net->ev_step, net->stream));
          NET_CUDA(cudaStreamWaitEvent(net->side, net->ev_step, 0));
          NET_TRY(assemble_images(net, first2, count2, net->ahead_x[(i + 1) & 1], net->side, &x2));
          NET_TRY(sbb_layer_shard_scatter(net->layers[li], x2, count2, net->side));
          NET_CUDA(cudaEventRecord(net->ev_staged, net->side));
          staged_ahead = true;
        }
      }
      NET_TRY(net->act[li].reserve((size_t)count * net->out_features(li) * net->esize()));
      NET_TRY(sharded_step(net, net->layers[li], net->desc[li], net->act[li].d, count, h, staged_ahead));
      continue;
    }
    NET_TRY(forward_through(net, x, count, li, &in_last, &out_last));
    const void *target = last ? t : out_last;
    if (dp) NET_TRY(dp_train_step(net, net->layers[li], net->desc[li], in_last, target, count, last ? -1 : h));
    else NET_TRY(sbb_layer_train_step(net->layers[li], in_last, target, count, last ? -1 : h, net->stream));
  }
  if (batch_end == nb) {
    if (sharded) {   // every rank gets the whole layer: the plain forward pass and checkpoints need it
      NET_TRY(sbb_layer_shard_share_rows(net->layers[li], net->stream));
      NET_TRY(rank_barrier(net));
    }
    NET_TRY(sbb_layer_train_finalize(net->layers[li], net->stream));
    return sbb_stream_sync(net->stream);   // one wait per epoch; also surfaces a device-side wait that gave up
  }
  return SBB_OK;
}

int sbb_network_evaluate(sbb_network *net, long maximal_batch_size, long *correct, long *total) {
  NET_TRY(check_net(net));
  if (!correct || !total) return net_fail(SBB_ERR_INVALID, "evaluate: null pointer");
  if (maximal_batch_size <= 0) return net_fail(SBB_ERR_INVALID, "evaluate: non-positive batch size");
  if (net->layers.empty() || net->samples <= 0) return net_fail(SBB_ERR_INVALID, "evaluate: no layers or no dataset");
  if (net->features != net->desc[0].in_features || net->classes != net->out_features(net->layers.size() - 1))
    return net_fail(SBB_ERR_INVALID, "evaluate: dataset is %ld -> %ld, the network %ld -> %ld", net->features,
                    net->classes, net->desc[0].in_features, net->out_features(net->layers.size() - 1));
  NET_TRY(net->hits.reserve(sizeof(unsigned long long)));
  NET_CUDA(cudaDeviceSynchronize());
  NET_CUDA(cudaMemsetAsync(net->hits.d, 0, sizeof(unsigned long long), net->stream));
  const long nb = (net->samples + maximal_batch_size - 1) / maximal_batch_size;
  long seen = 0;
  for (long i = 0; i < nb; ++i) {
    long first = 0, count = 0, slot = -1;
    NET_TRY(sbb_network_batch_plan(net->samples, maximal_batch_size, net->world, net->rank, 1, 0, i, &first, &count, &slot));
    if (count <= 0) continue;
    const void *x = nullptr, *t = nullptr, *in_last = nullptr, *out_last = nullptr;
    NET_TRY(assemble(net, first, count, false, true, &x, &t));
    NET_TRY(forward_through(net, x, count, net->layers.size() - 1, &in_last, &out_last));
    if (net->dtype == SBB_F32)
      NET_CUDA(sbb::launch_count_correct<float>((const float *)out_last, (const float *)t, count, net->classes,
                                                (unsigned long long *)net->hits.d, net->stream));
    else
      NET_CUDA(sbb::launch_count_correct<double>((const double *)out_last, (const double *)t, count, net->classes,
                                                 (unsigned long long *)net->hits.d, net->stream));
    seen += count;
  }
  unsigned long long hits = 0;
  NET_CUDA(cudaMemcpyAsync(&hits, net->hits.d, sizeof(hits), cudaMemcpyDeviceToHost, net->stream));
  NET_TRY(sbb_stream_sync(net->stream));
  *correct = (long)hits;
  *total = seen;
  return SBB_OK;
}

}  // extern "C"
