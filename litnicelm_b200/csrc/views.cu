// Host-side decoding of the plugin contract's tensor views
// (backend_plugin_api.hpp:7-18) into the compact forms the kernels take.
#include "common.cuh"

namespace lb {

thread_local bool g_pdl_enabled = false;

static void check_view(const BackendTensorView *t, const char *who) {
  if (t == nullptr) throw std::invalid_argument(std::string(who) + ": null tensor view");
  if (t->rank == 0 || t->rank > LITNICE_TENSOR_MAX_RANK)
    throw std::invalid_argument(std::string(who) + ": unsupported rank " + std::to_string(t->rank));
  for (uint32_t i = 0; i < t->rank; ++i)
    if (t->dims[i] <= 0)
      throw std::runtime_error(std::string(who) + ": invalid non-positive dimension");
  if (t->data == nullptr) throw std::invalid_argument(std::string(who) + ": null data pointer");
}

long long view_numel(const BackendTensorView *t) {
  long long n = 1;
  for (uint32_t i = 0; i < t->rank; ++i) n *= t->dims[i];
  return n;
}

// Same rule as TensorView::is_contiguous in the reference (tensor.hpp): the
// byte strides must equal those of a dense row-major tensor, axis by axis
// (an axis of extent 1 is NOT exempt there, which is why prefix-slice views of
// the inference buffers count as non-contiguous).
bool view_is_contiguous(const BackendTensorView *t) {
  long long expect = 4;
  for (int i = (int)t->rank - 1; i >= 0; --i) {
    if (t->strides_bytes[i] != expect) return false;
    expect *= t->dims[i];
  }
  return true;
}

// Collapses a list of (extent, stride) axes: extent-1 axes vanish, and an
// outer axis merges with the next inner one when outer.stride ==
// inner.extent * inner.stride.
static int collapse(const long long *dims, const long long *strides, int n, long long *od,
                    long long *os) {
  int m = 0;
  for (int i = 0; i < n; ++i) {
    if (dims[i] == 1) continue;
    if (m > 0 && os[m - 1] == dims[i] * strides[i]) {
      od[m - 1] *= dims[i];
      os[m - 1] = strides[i];
    } else {
      od[m] = dims[i];
      os[m] = strides[i];
      ++m;
    }
  }
  return m;
}

RowView make_row_view(const BackendTensorView *t, const char *who) {
  check_view(t, who);
  RowView v{};
  v.data = static_cast<char *>(t->data);
  const int r = (int)t->rank;
  v.cols = t->dims[r - 1];
  v.cs = t->strides_bytes[r - 1];
  long long d[6], s[6];
  for (int i = 0; i < r - 1; ++i) {
    d[i] = t->dims[i];
    s[i] = t->strides_bytes[i];
  }
  v.np = collapse(d, s, r - 1, v.pd, v.ps);
  v.rows = 1;
  for (int i = 0; i < v.np; ++i) v.rows *= v.pd[i];
  return v;
}

MatView make_mat_view(const BackendTensorView *t, const char *who) {
  check_view(t, who);
  if (t->rank < 2) throw std::invalid_argument(std::string(who) + ": rank >= 2 required");
  MatView v{};
  v.data = static_cast<char *>(t->data);
  const int r = (int)t->rank;
  v.rows = t->dims[r - 2];
  v.cols = t->dims[r - 1];
  v.rs = t->strides_bytes[r - 2];
  v.cs = t->strides_bytes[r - 1];
  long long d[6], s[6];
  for (int i = 0; i < r - 2; ++i) {
    d[i] = t->dims[i];
    s[i] = t->strides_bytes[i];
  }
  v.nb = collapse(d, s, r - 2, v.bd, v.bs);
  v.batch = 1;
  for (int i = 0; i < v.nb; ++i) v.batch *= v.bd[i];
  return v;
}

}  // namespace lb
