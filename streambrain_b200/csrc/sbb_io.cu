// Dataset file readers of the C ABI (host code only; nothing here touches the GPU).
//
// Two formats feed the reference's training driver:
//   * IDX (MNIST, Fashion-MNIST): big-endian header  [0, 0, type, ndim] [dim_0] ... [dim_{ndim-1}]
//     followed by the raw elements; images are unsigned bytes scaled to [0, 1], labels are
//     unsigned bytes turned into one-hot rows.
//     StreamBrain: train.py:9-23 (skips 16 / 8 header bytes), full_cuda_backend/dataset.cpp:7-64.
//   * STL-10 binaries: headerless unsigned bytes, 3*96*96 per image in file order, labels 1..10.
//     StreamBrain: train.py:26-41.
// Unlike the reference (which trusts the files and calls exit() on a mismatch) every header field is
// validated against the file size and the caller's buffer, and failures are returned as status codes.
#include "../../include/sbb200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

namespace sbb {
void set_last_error(const char *message);
}

namespace {

int io_fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  sbb::set_last_error(buf);
  return code;
}

struct File {
  FILE *f = nullptr;
  explicit File(const char *path) { f = path ? std::fopen(path, "rb") : nullptr; }
  ~File() {
    if (f) std::fclose(f);
  }
  long size() {
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    return n;
  }
};

uint32_t be32(const unsigned char *p) {
  return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | (uint32_t)p[3];
}

// Parses an IDX header; leaves the file positioned at the first element.
int idx_header(File &fh, const char *path, int *ndim, long dims[4], long *elements) {
  unsigned char magic[4];
  if (std::fread(magic, 1, 4, fh.f) != 4) return io_fail(SBB_ERR_INVALID, "%s: shorter than an IDX header", path);
  if (magic[0] != 0 || magic[1] != 0) return io_fail(SBB_ERR_INVALID, "%s: not an IDX file (bad magic)", path);
  if (magic[2] != 0x08)
    return io_fail(SBB_ERR_UNSUPPORTED, "%s: IDX element type 0x%02x, only unsigned bytes (0x08) are read", path,
                   magic[2]);
  *ndim = magic[3];
  if (*ndim < 1 || *ndim > 4) return io_fail(SBB_ERR_UNSUPPORTED, "%s: IDX rank %d outside [1, 4]", path, *ndim);
  long total = 1;
  for (int d = 0; d < 4; ++d) dims[d] = 1;
  for (int d = 0; d < *ndim; ++d) {
    unsigned char b[4];
    if (std::fread(b, 1, 4, fh.f) != 4) return io_fail(SBB_ERR_INVALID, "%s: truncated IDX header", path);
    dims[d] = (long)be32(b);
    total *= dims[d];
  }
  *elements = total;
  return SBB_OK;
}

template <typename T>
void scale_bytes(const unsigned char *src, T *dst, long n, double divisor) {
  const T d = (T)divisor;
  for (long i = 0; i < n; ++i) dst[i] = (T)src[i] / d;
}

template <typename T>
int one_hot(const unsigned char *lab, T *dst, long n, long classes, long base, const char *path) {
  std::memset(dst, 0, sizeof(T) * (size_t)n * (size_t)classes);
  for (long i = 0; i < n; ++i) {
    const long c = (long)lab[i] - base;
    if (c < 0 || c >= classes)
      return io_fail(SBB_ERR_INVALID, "%s: label %d of sample %ld outside [%ld, %ld)", path, (int)lab[i], i, base,
                     base + classes);
    dst[i * classes + c] = (T)1;
  }
  return SBB_OK;
}

int read_payload(File &fh, const char *path, long n, std::vector<unsigned char> &buf) {
  buf.resize((size_t)n);
  if (n > 0 && std::fread(buf.data(), 1, (size_t)n, fh.f) != (size_t)n)
    return io_fail(SBB_ERR_INVALID, "%s: file ends before its %ld elements", path, n);
  return SBB_OK;
}

}  // namespace

extern "C" {

int sbb_idx_info(const char *path, int *ndim, long dims[4]) {
  if (!path || !ndim || !dims) return io_fail(SBB_ERR_INVALID, "idx_info: null pointer");
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  const long size = fh.size();
  long elements = 0;
  int rc = idx_header(fh, path, ndim, dims, &elements);
  if (rc != SBB_OK) return rc;
  if (size != 4 + 4L * *ndim + elements)
    return io_fail(SBB_ERR_INVALID, "%s: %ld bytes on disk, header promises %ld", path, size, 4 + 4L * *ndim + elements);
  return SBB_OK;
}

int sbb_read_idx_images(const char *path, int dtype, void *out, long samples, long features) {
  if (!path || !out) return io_fail(SBB_ERR_INVALID, "read_idx_images: null pointer");
  if (dtype != SBB_F32 && dtype != SBB_F64) return io_fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  int ndim = 0;
  long dims[4], elements = 0;
  int rc = idx_header(fh, path, &ndim, dims, &elements);
  if (rc != SBB_OK) return rc;
  if (dims[0] != samples || elements != samples * features)
    return io_fail(SBB_ERR_INVALID, "%s holds %ld samples of %ld values, caller expects %ld x %ld", path, dims[0],
                   dims[0] ? elements / dims[0] : 0, samples, features);
  std::vector<unsigned char> buf;
  rc = read_payload(fh, path, elements, buf);
  if (rc != SBB_OK) return rc;
  if (dtype == SBB_F32) scale_bytes(buf.data(), static_cast<float *>(out), elements, 255.0);
  else scale_bytes(buf.data(), static_cast<double *>(out), elements, 255.0);
  return SBB_OK;
}

int sbb_read_idx_labels(const char *path, int dtype, void *out, long samples, long classes) {
  if (!path || !out) return io_fail(SBB_ERR_INVALID, "read_idx_labels: null pointer");
  if (dtype != SBB_F32 && dtype != SBB_F64) return io_fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  if (classes <= 0) return io_fail(SBB_ERR_INVALID, "read_idx_labels: non-positive class count");
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  int ndim = 0;
  long dims[4], elements = 0;
  int rc = idx_header(fh, path, &ndim, dims, &elements);
  if (rc != SBB_OK) return rc;
  if (ndim != 1 || elements != samples)
    return io_fail(SBB_ERR_INVALID, "%s holds %ld labels (rank %d), caller expects %ld", path, elements, ndim, samples);
  std::vector<unsigned char> buf;
  rc = read_payload(fh, path, elements, buf);
  if (rc != SBB_OK) return rc;
  return dtype == SBB_F32 ? one_hot(buf.data(), static_cast<float *>(out), samples, classes, 0, path)
                          : one_hot(buf.data(), static_cast<double *>(out), samples, classes, 0, path);
}

int sbb_raw_u8_count(const char *path, long *bytes) {
  if (!path || !bytes) return io_fail(SBB_ERR_INVALID, "raw_u8_count: null pointer");
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  *bytes = fh.size();
  return SBB_OK;
}

int sbb_read_raw_u8_images(const char *path, int dtype, void *out, long samples, long features) {
  if (!path || !out) return io_fail(SBB_ERR_INVALID, "read_raw_u8_images: null pointer");
  if (dtype != SBB_F32 && dtype != SBB_F64) return io_fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  const long size = fh.size();
  if (samples < 0 || features <= 0 || size != samples * features)
    return io_fail(SBB_ERR_INVALID, "%s holds %ld bytes, caller expects %ld x %ld", path, size, samples, features);
  std::vector<unsigned char> buf;
  int rc = read_payload(fh, path, size, buf);
  if (rc != SBB_OK) return rc;
  if (dtype == SBB_F32) scale_bytes(buf.data(), static_cast<float *>(out), size, 255.0);
  else scale_bytes(buf.data(), static_cast<double *>(out), size, 255.0);
  return SBB_OK;
}

int sbb_read_raw_u8_labels(const char *path, int dtype, void *out, long samples, long classes, long first_label) {
  if (!path || !out) return io_fail(SBB_ERR_INVALID, "read_raw_u8_labels: null pointer");
  if (dtype != SBB_F32 && dtype != SBB_F64) return io_fail(SBB_ERR_INVALID, "invalid dtype %d", dtype);
  if (classes <= 0) return io_fail(SBB_ERR_INVALID, "read_raw_u8_labels: non-positive class count");
  File fh(path);
  if (!fh.f) return io_fail(SBB_ERR_INVALID, "cannot open %s", path);
  const long size = fh.size();
  if (size != samples) return io_fail(SBB_ERR_INVALID, "%s holds %ld labels, caller expects %ld", path, size, samples);
  std::vector<unsigned char> buf;
  int rc = read_payload(fh, path, size, buf);
  if (rc != SBB_OK) return rc;
  return dtype == SBB_F32 ? one_hot(buf.data(), static_cast<float *>(out), samples, classes, first_label, path)
                          : one_hot(buf.data(), static_cast<double *>(out), samples, classes, first_label, path);
}

}  // extern "C"
