// pybind11 kernel module _bcpnn_kernels_b200_internal: the reference's native-module interface on top of the
// C ABI of libsbb200.so.
//
// StreamBrain's backends reach their kernels through pybind11 modules whose functions carry a dtype suffix
// (BCPNN/backend/_kernels/kernels_openmp_internal.cc:460-478 for the cpu backend,
// BCPNN/backend/_kernels/kernels_cuda_internal.cu:915-936 for the gpu backend).  This module exports the union
// of both sets under the same names and argument orders, so the reference's wrapper files bind it like their own
// (`import _bcpnn_kernels_b200_internal as _i`).  Arrays are borrowed for the call and mutated in place.
//
// One deliberate difference: pybind11's array_t arguments silently convert (and so copy) an array of the wrong
// dtype or layout, and the in-place result is then lost (the reference's own test passes an int8 mask this way,
// _kernels/test_openmp.py:243).  Here every array is checked and a mismatch raises TypeError; only a mask that
// is merely read may be any 1-byte integer or bool type.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>

#include "sbb200.h"

namespace py = pybind11;

namespace {

template <typename T>
struct Code;
template <>
struct Code<float> {
  static constexpr int value = SBB_F32;
};
template <>
struct Code<double> {
  static constexpr int value = SBB_F64;
};

void ok(int rc) {
  if (rc != SBB_OK) throw std::runtime_error(sbb_last_error());
}

template <typename T>
T *real(py::array &a, const char *name, int ndim, bool writeable) {
  if (!py::dtype::of<T>().is(a.dtype()))
    throw py::type_error(std::string(name) + ": expected dtype " + std::string(py::str(py::dtype::of<T>())) + ", got " +
                         std::string(py::str(a.dtype())));
  if (!(a.flags() & py::array::c_style)) throw py::type_error(std::string(name) + ": array must be C-contiguous");
  if (a.ndim() != ndim) throw py::value_error(std::string(name) + ": wrong number of dimensions");
  if (writeable && !a.writeable()) throw py::type_error(std::string(name) + ": array is read-only");
  return static_cast<T *>(a.mutable_data());
}

uint8_t *mask(py::array &a, const char *name, bool writeable) {
  if (a.itemsize() != 1 || (a.dtype().kind() != 'u' && a.dtype().kind() != 'i' && a.dtype().kind() != 'b'))
    throw py::type_error(std::string(name) + ": expected a one-byte integer mask");
  if (writeable && a.dtype().kind() != 'u') throw py::type_error(std::string(name) + ": a mask updated in place must be uint8");
  if (!(a.flags() & py::array::c_style)) throw py::type_error(std::string(name) + ": array must be C-contiguous");
  if (a.ndim() != 2) throw py::value_error(std::string(name) + ": wrong number of dimensions");
  return static_cast<uint8_t *>(a.mutable_data());
}

template <typename T>
void update_state(py::array activation, py::array inputs, py::array weights, py::array bias) {
  T *out = real<T>(activation, "activation", 2, true);
  const T *x = real<T>(inputs, "inputs", 2, false);
  const T *w = real<T>(weights, "weights", 2, false);
  const T *b = real<T>(bias, "bias", 1, false);
  const long B = inputs.shape(0), N = inputs.shape(1), M = weights.shape(1);
  if (weights.shape(0) != N || activation.shape(0) != B || activation.shape(1) != M || bias.shape(0) != M)
    throw py::value_error("update_state: shape mismatch");
  ok(sbb_update_state(Code<T>::value, out, x, w, b, B, N, M));
}

// The gpu module's argument order: (state, weight, bias, inputs), kernels_cuda_internal.cu:533.
template <typename T>
void update_state_cuda_order(py::array state, py::array weights, py::array bias, py::array inputs) {
  update_state<T>(state, inputs, weights, bias);
}

template <typename T>
T update_weights(T C, py::array Ci, py::array Cj, py::array Cij, py::array a_i, py::array a_o, T taupdt,
                 py::array weights, T cthr) {
  T *ci = real<T>(Ci, "Ci", 1, true), *cj = real<T>(Cj, "Cj", 1, true), *cij = real<T>(Cij, "Cij", 2, true);
  const T *x = real<T>(a_i, "a_i", 2, false), *y = real<T>(a_o, "a_o", 2, false);
  T *w = real<T>(weights, "weights", 2, true);
  const long B = a_i.shape(0), N = a_i.shape(1), M = a_o.shape(1);
  if (a_o.shape(0) != B || Ci.shape(0) != N || Cj.shape(0) != M || Cij.shape(0) != N || Cij.shape(1) != M ||
      weights.shape(0) != N || weights.shape(1) != M)
    throw py::value_error("update_weights: shape mismatch");
  ok(sbb_update_weights(Code<T>::value, ci, cj, cij, x, y, (double)taupdt, B, N, M, w, (double)cthr));
  C = ((T)1 - taupdt) * C + taupdt;   // the scalar trace the reference returns (kernels_openmp_internal.cc:98-99)
  return C > (T)0 ? C : (T)0;
}

template <typename T>
void recompute_weights(py::array weights, py::array Ci, py::array Cj, py::array Cij, T cthr) {
  T *w = real<T>(weights, "weights", 2, true);
  const T *ci = real<T>(Ci, "Ci", 1, false), *cj = real<T>(Cj, "Cj", 1, false), *cij = real<T>(Cij, "Cij", 2, false);
  const long N = weights.shape(0), M = weights.shape(1);
  if (Ci.shape(0) != N || Cj.shape(0) != M || Cij.shape(0) != N || Cij.shape(1) != M)
    throw py::value_error("update_weights: shape mismatch");
  ok(sbb_recompute_weights(Code<T>::value, w, ci, cj, cij, (double)cthr, N, M));
}

template <typename T>
void update_counters(py::array Ci, py::array Cj, py::array Cij, py::array a_i, py::array a_o, T taupdt) {
  T *ci = real<T>(Ci, "Ci", 1, true), *cj = real<T>(Cj, "Cj", 1, true), *cij = real<T>(Cij, "Cij", 2, true);
  const T *x = real<T>(a_i, "inputs", 2, false), *y = real<T>(a_o, "outputs", 2, false);
  const long B = a_i.shape(0), N = a_i.shape(1), M = a_o.shape(1);
  if (a_o.shape(0) != B || Ci.shape(0) != N || Cj.shape(0) != M || Cij.shape(0) != N || Cij.shape(1) != M)
    throw py::value_error("update_counters: shape mismatch");
  ok(sbb_update_counters(Code<T>::value, ci, cj, cij, x, y, (double)taupdt, B, N, M));
}

template <typename T>
void update_bias(py::array bias, py::array Cj, T cthr) {
  T *b = real<T>(bias, "bias", 1, true);
  const T *cj = real<T>(Cj, "Cj", 1, false);
  if (Cj.shape(0) != bias.shape(0)) throw py::value_error("update_bias: shape mismatch");
  ok(sbb_update_bias(Code<T>::value, b, cj, (double)cthr, bias.shape(0)));
}

template <typename T>
void update_bias_regularized(py::array bias, py::array kbi, py::array Cj, T cthr, T khalf, T pmin, T taubdt) {
  T *b = real<T>(bias, "bias", 1, true), *k = real<T>(kbi, "kbi", 1, true);
  const T *cj = real<T>(Cj, "Cj", 1, false);
  if (Cj.shape(0) != bias.shape(0) || kbi.shape(0) != bias.shape(0))
    throw py::value_error("update_bias_regularized: shape mismatch");
  ok(sbb_update_bias_regularized(Code<T>::value, b, k, cj, (double)cthr, (double)khalf, (double)pmin, (double)taubdt,
                                 bias.shape(0)));
}

template <typename T>
void update_mask(py::array wmask, py::array weights, py::array Ci, py::array Cj, py::array Cij, T cthr, long H, long Mc,
                 long h, long iterations) {
  uint8_t *m = mask(wmask, "wmask", true);
  const T *w = real<T>(weights, "weights", 2, false), *ci = real<T>(Ci, "Ci", 1, false), *cj = real<T>(Cj, "Cj", 1, false),
          *cij = real<T>(Cij, "Cij", 2, false);
  const long N = weights.shape(0), M = weights.shape(1);
  if (wmask.shape(0) != N || wmask.shape(1) != H || Ci.shape(0) != N || Cj.shape(0) != M || Cij.shape(0) != N ||
      Cij.shape(1) != M)
    throw py::value_error("update_mask: shape mismatch");
  ok(sbb_update_mask(Code<T>::value, m, w, ci, cj, cij, (double)cthr, N, M, H, Mc, h, iterations));
}

template <typename T>
void apply_mask(py::array weights, py::array wmask, long H, long Mc) {
  T *w = real<T>(weights, "weights", 2, true);
  const uint8_t *m = mask(wmask, "wmask", false);
  const long N = weights.shape(0), M = weights.shape(1);
  if (wmask.shape(0) != N || wmask.shape(1) != H) throw py::value_error("apply_mask: shape mismatch");
  ok(sbb_apply_mask(Code<T>::value, w, m, N, M, H, Mc));
}

template <typename T>
void add_bias(py::array a, py::array bias) {
  T *p = real<T>(a, "matrix", 2, true);
  const T *b = real<T>(bias, "bias", 1, false);
  if (bias.shape(0) != a.shape(1)) throw py::value_error("add_bias: shape mismatch");
  ok(sbb_add_bias(Code<T>::value, p, b, a.shape(0), a.shape(1)));
}

template <typename T>
void softmax_minicolumns(py::array a, long H, long Mc) {
  T *p = real<T>(a, "matrix", 2, true);
  if (a.shape(1) != H * Mc) throw py::value_error("softmax_minicolumns: shape mismatch");
  ok(sbb_softmax_minicolumns(Code<T>::value, p, a.shape(0), H, Mc));
}

template <typename T>
void bind(py::module_ &m, const std::string &suffix) {
  m.def(("update_state" + suffix).c_str(), &update_state<T>);
  m.def(("update_state_cuda_order" + suffix).c_str(), &update_state_cuda_order<T>);
  m.def(("update_weights" + suffix).c_str(), &update_weights<T>);        // fused, openmp module
  m.def(("update_weights" + suffix).c_str(), &recompute_weights<T>);     // un-fused, gpu module (overload by arity)
  m.def(("update_counters" + suffix).c_str(), &update_counters<T>);
  m.def(("update_bias" + suffix).c_str(), &update_bias<T>);
  m.def(("update_bias_regularized" + suffix).c_str(), &update_bias_regularized<T>);
  m.def(("update_mask" + suffix).c_str(), &update_mask<T>);
  m.def(("apply_mask" + suffix).c_str(), &apply_mask<T>);
  m.def(("add_bias" + suffix).c_str(), &add_bias<T>);
  m.def(("softmax_minicolumns" + suffix).c_str(), &softmax_minicolumns<T>);
}

}  // namespace

PYBIND11_MODULE(_bcpnn_kernels_b200_internal, m) {
  m.doc() = "BCPNN layer kernels on B200 (C ABI of libsbb200.so) under the reference's pybind11 names";
  // the gpu module's one-time set-up (kernels_cuda_internal.cu:905-913): nothing to prepare here
  m.def("initialize", []() { return sbb_device_count(); });
  bind<float>(m, "_float32");
  bind<double>(m, "_float64");
}
