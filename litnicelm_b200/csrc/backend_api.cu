// The litnicelm `backend.library` plugin table (BackendApiV1, version 16)
// implemented on CUDA. Each entry mirrors the behaviour of DefaultCpuBackend
// (litnicelm src/model/backend/device_backend.cpp:657-1775) for the views the
// host builds, and reports failures as C++ exceptions, which is the contract of
// the loader (device_backend.cpp:182-230, main.cpp:37-40).
//
// All work of one backend instance is issued on one stream. The only host
// synchronisation points are the host<->device copies, which the host requires
// to be complete on return (host_tensor_stage.hpp:120-124, checkpoint.cpp:214-218).
// Nothing falls back to the CPU.
#include "common.cuh"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace lb {

namespace {

struct Backend {
  int device = 0;
  cudaStream_t st = nullptr;
  DevErr *err_host = nullptr;  // host-mapped; kernels write, host reads after a sync
  DevErr *err_dev = nullptr;
  std::unordered_map<void *, void *> over_aligned;  // user pointer -> cudaMalloc base
  std::map<uintptr_t, uint64_t> allocs;             // user pointer -> bytes, for every live allocation
  int ctx_iteration = 0, ctx_group = 0;
  long long launches = 0;
  void *scratch = nullptr;  // partial sums and row statistics of the training entries
  size_t scratch_bytes = 0;

  // Deferred operators. The host issues one table call per operator and per attention head
  // (self_attention_fused_inplace.cpp:82-94: three calls per head; transformer_layer.cpp:79-86 and
  // the FFN variants: a product, then its bias). Calls that can be merged with their neighbours are
  // recorded instead of launched and issued together at the next call that is anything else:
  // a projection with the bias (and ReLU) that follows it becomes one launch, and the score product,
  // causal softmax and context product of all heads of a layer become three launches instead of
  // three per head. Nothing is reordered against other calls and every buffer the host's sequence
  // writes is written with the same values, so the host cannot tell the difference
  // (LITNICE_B200_ABI_QUEUE=0 issues every call at once).
  struct Pending {
    enum Kind { PROJECTION, BIAS, BIAS_RELU, SCORES, SOFTMAX, CONTEXT } kind;
    BackendTensorView a, b, c;  // copies: the host's views are only valid during its call
    float scale = 0.f;
  };
  std::vector<Pending> queue;
  bool queue_on = true;
  float *queue_scratch = nullptr;  // scores of all heads when the host gives every head the same buffer
  size_t queue_scratch_floats = 0;
  long long fused_projections = 0, grouped_heads = 0;

  // Read-ahead for row-by-row read-back. The host reads logits one row per
  // copy_device2host call (host_tensor_stage.hpp:101-125: s calls of V floats per
  // token). When two small copies in a row walk forward through one allocation
  // with nothing written to the device in between, the rest of that walk is
  // fetched in one transfer into pinned memory and later calls are answered
  // from there. `epoch` counts the table calls that may write device memory;
  // the mirror is valid only for the epoch it was filled in.
  unsigned long long epoch = 0;
  bool read_ahead = true;        // LITNICE_B200_READ_AHEAD=0 turns it off
  char *shadow = nullptr;        // pinned
  uint64_t shadow_cap = 0;
  uintptr_t shadow_src = 0;      // device range mirrored: [shadow_src, shadow_src + shadow_len)
  uint64_t shadow_len = 0;
  unsigned long long shadow_epoch = ~0ull;
  uintptr_t last_src = 0;        // previous small copy
  uint64_t last_bytes = 0;
  unsigned long long last_epoch = ~0ull;
  uint64_t next_window = 0;
  long long d2h_calls = 0, d2h_served_from_shadow = 0;
};

constexpr uint64_t SHADOW_SMALL = 1ull << 20;    // copies up to this size are candidates
constexpr uint64_t SHADOW_FIRST = 1ull << 20;    // first read-ahead window
constexpr uint64_t SHADOW_MAX = 64ull << 20;     // largest window (pinned buffer size)

// Every table entry except the read-only ones comes through here: whatever it
// does may write device memory, which invalidates the read-back mirror.
void flush_queue(Backend *b);

Backend *self(void *h) {
  if (h == nullptr) throw std::invalid_argument("litnice_b200: null backend handle");
  Backend *b = static_cast<Backend *>(h);
  ++b->epoch;
  if (!b->queue.empty()) flush_queue(b);
  return b;
}
Backend *self_reader(void *h) {  // entries that only read (they see every earlier call's effect)
  if (h == nullptr) throw std::invalid_argument("litnice_b200: null backend handle");
  Backend *b = static_cast<Backend *>(h);
  if (!b->queue.empty()) flush_queue(b);
  return b;
}
Backend *self_recording(void *h) {  // entries that may record instead of launching, and pure bookkeeping
  if (h == nullptr) throw std::invalid_argument("litnice_b200: null backend handle");
  Backend *b = static_cast<Backend *>(h);
  ++b->epoch;
  return b;
}

void bind(Backend *b) { LB_CUDA(cudaSetDevice(b->device)); }

void raise_device_error(Backend *b) {
  if (b->err_host->code == DEVERR_NONE) return;
  const int code = b->err_host->code, detail = b->err_host->detail;
  b->err_host->code = DEVERR_NONE;
  if (code == DEVERR_BAD_TOKEN_ID)
    throw std::runtime_error("litnice_b200::embedding_lookup: embedding id out of range (id=" +
                             std::to_string(detail) + ")");
  if (code == DEVERR_BAD_TARGET)
    throw std::runtime_error("litnice_b200::cross_entropy: target out of range (target=" + std::to_string(detail) +
                             ")");
  throw std::runtime_error("litnice_b200: device error code " + std::to_string(code));
}

void sync_and_check(Backend *b) {
  LB_CUDA(cudaStreamSynchronize(b->st));
  raise_device_error(b);
}

void require_gpu_f32(LitniceView t, const char *who) {
  if (t == nullptr) throw std::invalid_argument(std::string(who) + ": null view");
  if (t->device != 1u) throw std::runtime_error(std::string(who) + " requires a GPU tensor");
  if (t->dtype != 0u) throw std::runtime_error(std::string(who) + " requires an f32 tensor");
}

RowView flat_view(LitniceView t) {
  RowView v{};
  v.data = static_cast<char *>(t->data);
  v.np = 0;
  v.rows = 1;
  v.cols = view_numel(t);
  v.cs = 4;
  return v;
}

// ---- lifecycle ---------------------------------------------------------------

void *api_create(uint32_t device_kind) {
  // The loader tries GPU (1) first, then CPU (0) (device_backend.cpp:208-220).
  if (device_kind != 1u) return nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    throw std::runtime_error(std::string("litnice_b200: no CUDA device: ") + cudaGetErrorString(e));
  int dev = 0;
  if (const char *env = std::getenv("LITNICE_B200_DEVICE")) dev = std::atoi(env);
  if (dev < 0 || dev >= count) throw std::runtime_error("litnice_b200: LITNICE_B200_DEVICE out of range");
  auto *b = new Backend();
  try {
    b->device = dev;
    if (const char *env = std::getenv("LITNICE_B200_READ_AHEAD")) b->read_ahead = env[0] != '0';
    if (const char *env = std::getenv("LITNICE_B200_ABI_QUEUE")) b->queue_on = env[0] != '0';
    bind(b);
    cudaDeviceProp prop{};
    LB_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      throw std::runtime_error("litnice_b200: this plugin is built for sm_100a (B200) only; found sm_" +
                               std::to_string(prop.major) + std::to_string(prop.minor));
    LB_CUDA(cudaStreamCreateWithFlags(&b->st, cudaStreamNonBlocking));
    LB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&b->err_host), sizeof(DevErr), cudaHostAllocMapped));
    b->err_host->code = DEVERR_NONE;
    b->err_host->detail = 0;
    LB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&b->err_dev), b->err_host, 0));
  } catch (...) {
    delete b;
    throw;
  }
  return b;
}

void api_destroy(void *h) {
  if (h == nullptr) return;
  Backend *b = static_cast<Backend *>(h);
  cudaSetDevice(b->device);
  b->queue.clear();  // nothing can observe recorded work once the instance is gone
  if (b->st) {
    cudaStreamSynchronize(b->st);
    cudaStreamDestroy(b->st);
  }
  if (b->err_host) cudaFreeHost(b->err_host);
  if (b->shadow) cudaFreeHost(b->shadow);
  if (b->scratch) cudaFree(b->scratch);
  if (b->queue_scratch) cudaFree(b->queue_scratch);
  delete b;
}

uint32_t api_device(void *h) {
  self_reader(h);
  return 1u;
}

void *api_alloc(void *h, uint64_t bytes, uint32_t alignment) {
  Backend *b = self(h);
  if (bytes == 0) return nullptr;
  if (alignment == 0 || (alignment & (alignment - 1)) != 0)
    throw std::invalid_argument("litnice_b200::alloc: invalid alignment");
  bind(b);
  void *p = nullptr;
  if (alignment <= 256) {  // cudaMalloc returns 256-byte aligned memory
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("litnice_b200::alloc failed: ") + cudaGetErrorString(e));
    b->allocs[reinterpret_cast<uintptr_t>(p)] = bytes;
    return p;
  }
  cudaError_t e = cudaMalloc(&p, bytes + alignment);
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("litnice_b200::alloc failed: ") + cudaGetErrorString(e));
  const uintptr_t a = (reinterpret_cast<uintptr_t>(p) + alignment - 1) & ~(uintptr_t)(alignment - 1);
  b->over_aligned[reinterpret_cast<void *>(a)] = p;
  b->allocs[a] = bytes;
  return reinterpret_cast<void *>(a);
}

void api_free(void *h, void *ptr) {
  Backend *b = self(h);
  if (ptr == nullptr) return;
  bind(b);
  LB_CUDA(cudaStreamSynchronize(b->st));
  b->allocs.erase(reinterpret_cast<uintptr_t>(ptr));
  auto it = b->over_aligned.find(ptr);
  if (it != b->over_aligned.end()) {
    LB_CUDA(cudaFree(it->second));
    b->over_aligned.erase(it);
  } else {
    LB_CUDA(cudaFree(ptr));
  }
}

void api_h2d(void *h, void *dst, const void *src, uint64_t bytes) {
  Backend *b = self(h);
  if (bytes == 0) return;
  if (dst == nullptr || src == nullptr)
    throw std::invalid_argument("litnice_b200::copy_host2device: null pointer");
  bind(b);
  LB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, b->st));
  LB_CUDA(cudaStreamSynchronize(b->st));
}

void api_d2h(void *h, void *dst, const void *src, uint64_t bytes) {
  Backend *b = self_reader(h);
  if (bytes == 0) return;
  if (dst == nullptr || src == nullptr)
    throw std::invalid_argument("litnice_b200::copy_device2host: null pointer");
  ++b->d2h_calls;
  const uintptr_t a = reinterpret_cast<uintptr_t>(src);
  if (b->shadow_epoch == b->epoch && a >= b->shadow_src && a + bytes <= b->shadow_src + b->shadow_len) {
    std::memcpy(dst, b->shadow + (a - b->shadow_src), bytes);  // mirrored since the last device write
    ++b->d2h_served_from_shadow;
    b->last_src = a;
    b->last_bytes = bytes;
    b->last_epoch = b->epoch;
    return;
  }
  bind(b);
  // Second small copy of a forward walk with no device write in between: fetch
  // ahead, up to the end of the allocation the walk is in.
  const bool walking = b->read_ahead && bytes <= SHADOW_SMALL && b->last_epoch == b->epoch &&
                       b->last_bytes == bytes && a > b->last_src;
  if (walking) {
    auto it = b->allocs.upper_bound(a);
    if (it != b->allocs.begin()) {
      --it;
      const uintptr_t end = it->first + it->second;
      if (a + bytes <= end && b->last_src >= it->first) {
        // a walk that outruns its window doubles the next one
        uint64_t want = b->shadow_epoch == b->epoch ? b->next_window : SHADOW_FIRST;
        if (want > SHADOW_MAX) want = SHADOW_MAX;
        uint64_t len = end - a < want ? end - a : want;
        if (len >= 2 * bytes) {
          if (b->shadow_cap < len) {
            if (b->shadow) cudaFreeHost(b->shadow);
            b->shadow = nullptr;
            b->shadow_cap = 0;
            const uint64_t cap = len > SHADOW_FIRST ? SHADOW_MAX : SHADOW_FIRST;
            if (cudaHostAlloc(reinterpret_cast<void **>(&b->shadow), cap, cudaHostAllocDefault) == cudaSuccess)
              b->shadow_cap = cap;
            else
              (void)cudaGetLastError();
          }
          if (b->shadow_cap >= len) {
            LB_CUDA(cudaMemcpyAsync(b->shadow, src, len, cudaMemcpyDeviceToHost, b->st));
            sync_and_check(b);
            b->shadow_src = a;
            b->shadow_len = len;
            b->shadow_epoch = b->epoch;
            b->next_window = 2 * want;
            std::memcpy(dst, b->shadow, bytes);
            b->last_src = a;
            b->last_bytes = bytes;
            b->last_epoch = b->epoch;
            return;
          }
        }
      }
    }
  }
  LB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, b->st));
  sync_and_check(b);
  b->last_src = a;
  b->last_bytes = bytes;
  b->last_epoch = b->epoch;
}

BackendMemoryInfo api_memory_info(void *h) {
  Backend *b = self_reader(h);
  bind(b);
  size_t fr = 0, tot = 0;
  LB_CUDA(cudaMemGetInfo(&fr, &tot));
  return BackendMemoryInfo{1u, fr, tot};
}

// ---- elementwise -------------------------------------------------------------

// device_backend.cpp:715-732. Dense f32 views are copied flat; any other view
// is copied element by element over its full logical shape. (For a rank-3
// non-dense view the CPU backend walks only dims 0 and 1; every element it
// writes receives the same value here, and the remaining elements of the
// logical shape are copied as well.)
void api_copy(void *h, LitniceView src, LitniceView dst) {
  Backend *b = self(h);
  require_gpu_f32(src, "litnice_b200::copy(src)");
  require_gpu_f32(dst, "litnice_b200::copy(dst)");
  bind(b);
  if (view_is_contiguous(src) && view_is_contiguous(dst)) {
    if (view_numel(src) != view_numel(dst)) throw std::runtime_error("litnice_b200::copy: numel mismatch");
    launch_rowwise(EW_COPY, flat_view(src), nullptr, 0, 0.f, flat_view(dst), b->st);
  } else {
    RowView s = make_row_view(src, "copy(src)"), d = make_row_view(dst, "copy(dst)");
    if (s.rows != d.rows || s.cols != d.cols) throw std::runtime_error("litnice_b200::copy: shape mismatch");
    launch_rowwise(EW_COPY, s, nullptr, 0, 0.f, d, b->st);
  }
  ++b->launches;
}

void api_fill(void *h, LitniceView t, float v) {
  Backend *b = self(h);
  require_gpu_f32(t, "litnice_b200::fill");
  bind(b);
  RowView o = view_is_contiguous(t) ? flat_view(t) : make_row_view(t, "fill");
  launch_rowwise(EW_FILL, o, nullptr, 0, v, o, b->st);
  ++b->launches;
}

bool is_pos_broadcast(LitniceView a, LitniceView bb, LitniceView out) {
  return a->rank == 3 && bb->rank == 2 && out->rank == 3 && a->dims[1] == bb->dims[0] &&
         a->dims[2] == bb->dims[1] && out->dims[0] == a->dims[0] && out->dims[1] == a->dims[1] &&
         out->dims[2] == a->dims[2];
}

// device_backend.cpp:752-813, including the rank-3 + rank-2 broadcast used for
// X += pos_emb[0:s] (transformer.cpp:93-94).
void api_add(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(a, "litnice_b200::add(a)");
  require_gpu_f32(bb, "litnice_b200::add(b)");
  require_gpu_f32(out, "litnice_b200::add(out)");
  bind(b);
  const long long na = view_numel(a), nb = view_numel(bb), no = view_numel(out);
  if (na == nb && na == no) {
    if (view_is_contiguous(a) && view_is_contiguous(bb) && view_is_contiguous(out)) {
      RowView fb = flat_view(bb);
      launch_rowwise(EW_ADD, flat_view(a), &fb, 0, 0.f, flat_view(out), b->st);
    } else {
      RowView ra = make_row_view(a, "add(a)"), rb = make_row_view(bb, "add(b)"),
              ro = make_row_view(out, "add(out)");
      if (ra.cols != rb.cols || ra.cols != ro.cols)
        throw std::runtime_error("litnice_b200::add: last-axis mismatch");
      launch_rowwise(EW_ADD, ra, &rb, 0, 0.f, ro, b->st);
    }
  } else if (is_pos_broadcast(a, bb, out)) {
    RowView ra = make_row_view(a, "add(a)"), ro = make_row_view(out, "add(out)");
    RowView rb{};
    rb.data = static_cast<char *>(bb->data);
    rb.np = 1;
    rb.pd[0] = bb->dims[0];
    rb.ps[0] = bb->strides_bytes[0];
    rb.rows = bb->dims[0];
    rb.cols = bb->dims[1];
    rb.cs = bb->strides_bytes[1];
    launch_rowwise(EW_ADD, ra, &rb, a->dims[1], 0.f, ro, b->st);
  } else {
    throw std::runtime_error("litnice_b200::add: numel or broadcast shape mismatch");
  }
  ++b->launches;
}

void api_add_inplace(void *h, LitniceView a, LitniceView bb) {
  api_add(h, a, bb, a);
}

bool same_view(const BackendTensorView &p, const BackendTensorView &q) {
  if (p.data != q.data || p.rank != q.rank || p.dtype != q.dtype || p.device != q.device) return false;
  for (uint32_t i = 0; i < p.rank; ++i)
    if (p.dims[i] != q.dims[i] || p.strides_bytes[i] != q.strides_bytes[i]) return false;
  return true;
}

void bias_op(void *h, EwOp op, LitniceView x, LitniceView bias, LitniceView out, const char *who) {
  Backend *b = self_recording(h);
  require_gpu_f32(x, who);
  require_gpu_f32(bias, who);
  require_gpu_f32(out, who);
  {
    RowView rx = make_row_view(x, who), ro = make_row_view(out, who);
    if (view_numel(bias) != rx.cols || ro.cols != rx.cols || ro.rows != rx.rows)
      throw std::runtime_error(std::string(who) + ": semantic shape mismatch");
  }
  // In place on the result of the projection recorded just before: joins it as its epilogue.
  if (b->queue.size() == 1 && b->queue[0].kind == Backend::Pending::PROJECTION && (op == EW_ADD_BIAS || op == EW_ADD_BIAS_RELU) && same_view(*x, *out) && same_view(b->queue[0].c, *x) &&
      bias->strides_bytes[bias->rank - 1] == 4 && (reinterpret_cast<uintptr_t>(bias->data) & 3) == 0) {
    Backend::Pending p;
    p.kind = op == EW_ADD_BIAS ? Backend::Pending::BIAS : Backend::Pending::BIAS_RELU;
    p.a = *bias;
    p.c = *out;
    b->queue.push_back(p);
    flush_queue(b);  // a projection with its epilogue is complete
    return;
  }
  if (!b->queue.empty()) flush_queue(b);
  bind(b);
  RowView rx = make_row_view(x, who), ro = make_row_view(out, who);
  RowView rb{};
  rb.data = static_cast<char *>(bias->data);
  rb.np = 0;
  rb.rows = 1;
  rb.cols = rx.cols;
  rb.cs = bias->strides_bytes[bias->rank - 1];
  launch_rowwise(op, rx, &rb, 1, 0.f, ro, b->st);
  ++b->launches;
}

// device_backend.cpp:840-940
void api_add_bias(void *h, LitniceView x, LitniceView bias, LitniceView out) {
  bias_op(h, EW_ADD_BIAS, x, bias, out, "litnice_b200::add_bias_rowwise");
}
void api_add_bias_relu(void *h, LitniceView x, LitniceView bias, LitniceView out) {
  bias_op(h, EW_ADD_BIAS_RELU, x, bias, out, "litnice_b200::add_bias_relu_rowwise");
}
void api_add_bias_relu_inplace(void *h, LitniceView x, LitniceView bias) {
  bias_op(h, EW_ADD_BIAS_RELU, x, bias, x, "litnice_b200::add_bias_relu_rowwise_inplace");
}

void unary_op(void *h, EwOp op, LitniceView x, float s, LitniceView out, const char *who) {
  Backend *b = self(h);
  require_gpu_f32(x, who);
  require_gpu_f32(out, who);
  bind(b);
  if (view_numel(x) != view_numel(out)) throw std::runtime_error(std::string(who) + ": numel mismatch");
  if (view_is_contiguous(x) && view_is_contiguous(out)) {
    launch_rowwise(op, flat_view(x), nullptr, 0, s, flat_view(out), b->st);
  } else {
    RowView rx = make_row_view(x, who), ro = make_row_view(out, who);
    if (rx.cols != ro.cols || rx.rows != ro.rows) throw std::runtime_error(std::string(who) + ": shape mismatch");
    launch_rowwise(op, rx, nullptr, 0, s, ro, b->st);
  }
  ++b->launches;
}

// device_backend.cpp:942-964, :978-1001
void api_mul_scalar(void *h, LitniceView x, float s, LitniceView out) {
  unary_op(h, EW_MUL_SCALAR, x, s, out, "litnice_b200::mul_scalar");
}
void api_relu(void *h, LitniceView x, LitniceView out) {
  unary_op(h, EW_RELU, x, 0.f, out, "litnice_b200::relu");
}

// device_backend.cpp:1675-1697
void api_causal_mask(void *h, LitniceView scores, float neg_inf) {
  Backend *b = self(h);
  require_gpu_f32(scores, "litnice_b200::apply_causal_mask_inplace");
  bind(b);
  MatView m = make_mat_view(scores, "apply_causal_mask_inplace");
  if (m.rows != m.cols)
    throw std::runtime_error("litnice_b200::apply_causal_mask_inplace: scores must end with [T,T]");
  launch_causal_mask(m, neg_inf, b->st);
  ++b->launches;
}

// device_backend.cpp:1345-1366
void api_embedding(void *h, LitniceView table, LitniceView ids, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(table, "litnice_b200::embedding_lookup(table)");
  require_gpu_f32(out, "litnice_b200::embedding_lookup(out)");
  if (ids == nullptr || ids->device != 1u || ids->dtype > 1u)
    throw std::runtime_error("litnice_b200::embedding_lookup: unsupported index dtype");
  if (table->rank != 2) throw std::runtime_error("litnice_b200::embedding_lookup: table must be rank 2");
  bind(b);
  RowView tv{};
  tv.data = static_cast<char *>(table->data);
  tv.np = 1;
  tv.pd[0] = table->dims[0];
  tv.ps[0] = table->strides_bytes[0];
  tv.rows = table->dims[0];
  tv.cols = table->dims[1];
  tv.cs = table->strides_bytes[1];
  RowView iv = make_row_view(ids, "embedding_lookup(ids)");
  RowView ov = make_row_view(out, "embedding_lookup(out)");
  if (ov.rows != iv.rows * iv.cols || ov.cols != tv.cols)
    throw std::runtime_error("litnice_b200::embedding_lookup: shape mismatch");
  launch_embedding(tv, static_cast<const char *>(ids->data), ids->dtype == 0u ? 1 : 0, iv, ov,
                   b->err_dev, b->st);
  ++b->launches;
}

void api_transpose(void *h, LitniceView x, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(x, "litnice_b200::transpose(x)");
  require_gpu_f32(out, "litnice_b200::transpose(out)");
  bind(b);
  launch_transpose(make_mat_view(x, "transpose(x)"), make_mat_view(out, "transpose(out)"), b->st);
  ++b->launches;
}

// ---- norm / softmax ------------------------------------------------------------

// device_backend.cpp:1247-1279
void api_layernorm(void *h, LitniceView x, LitniceView gamma, LitniceView beta, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(x, "litnice_b200::layernorm_forward(x)");
  require_gpu_f32(gamma, "litnice_b200::layernorm_forward(gamma)");
  require_gpu_f32(beta, "litnice_b200::layernorm_forward(beta)");
  require_gpu_f32(out, "litnice_b200::layernorm_forward(out)");
  bind(b);
  RowView rx = make_row_view(x, "layernorm_forward(x)"), ro = make_row_view(out, "layernorm_forward(out)");
  if (rx.rows != ro.rows || rx.cols != ro.cols || view_numel(gamma) != rx.cols || view_numel(beta) != rx.cols)
    throw std::runtime_error("litnice_b200::layernorm_forward: shape mismatch");
  launch_layernorm(rx, static_cast<const float *>(gamma->data), gamma->strides_bytes[gamma->rank - 1],
                   static_cast<const float *>(beta->data), beta->strides_bytes[beta->rank - 1], ro, b->st);
  ++b->launches;
}

// device_backend.cpp:1466-1517
void api_softmax_rows(void *h, LitniceView x, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(x, "litnice_b200::softmax_rows(x)");
  require_gpu_f32(out, "litnice_b200::softmax_rows(out)");
  bind(b);
  RowView rx = make_row_view(x, "softmax_rows(x)"), ro = make_row_view(out, "softmax_rows(out)");
  if (rx.rows != ro.rows || rx.cols != ro.cols) throw std::runtime_error("litnice_b200::softmax_rows: shape mismatch");
  launch_softmax_rows(rx, ro, 0, 1.0f, b->st);
  ++b->launches;
}

// device_backend.cpp:1554-1592
void run_causal_softmax(Backend *b, const BackendTensorView *scores, float scale, const BackendTensorView *out) {
  bind(b);
  RowView rx = make_row_view(scores, "scaled_causal_softmax_rows(scores)"),
          ro = make_row_view(out, "scaled_causal_softmax_rows(out)");
  launch_softmax_rows(rx, ro, 1, scale, b->st);
  ++b->launches;
}

void api_causal_softmax(void *h, LitniceView scores, float scale, LitniceView out) {
  Backend *b = self_recording(h);
  require_gpu_f32(scores, "litnice_b200::scaled_causal_softmax_rows(scores)");
  require_gpu_f32(out, "litnice_b200::scaled_causal_softmax_rows(out)");
  {
    RowView rx = make_row_view(scores, "scaled_causal_softmax_rows(scores)"),
            ro = make_row_view(out, "scaled_causal_softmax_rows(out)");
    if (rx.rows != ro.rows || rx.cols != ro.cols)
      throw std::runtime_error("litnice_b200::scaled_causal_softmax_rows: shape mismatch");
  }
  // the softmax of the score product recorded just before: part of a head's three calls
  if (!b->queue.empty() && b->queue.back().kind == Backend::Pending::SCORES && same_view(b->queue.back().c, *scores)) {
    Backend::Pending p;
    p.kind = Backend::Pending::SOFTMAX;
    p.a = *scores;
    p.c = *out;
    p.scale = scale;
    b->queue.push_back(p);
    return;
  }
  if (!b->queue.empty()) flush_queue(b);
  run_causal_softmax(b, scores, scale, out);
}

// ---- matrix products -------------------------------------------------------------

MatView transposed(MatView v) {
  std::swap(v.rows, v.cols);
  std::swap(v.rs, v.cs);
  return v;
}

MatView shared_matrix(LitniceView t, const char *who) {  // rank-2 operand used by every batch
  MatView v = make_mat_view(t, who);
  if (t->rank != 2) throw std::runtime_error(std::string(who) + ": rank-2 matrix required");
  return v;
}

void check_gemm(const MatView &a, const MatView &bm, const MatView &c, const char *who) {
  if (a.cols != bm.rows || c.rows != a.rows || c.cols != bm.cols)
    throw std::runtime_error(std::string(who) + ": inner or output dimension mismatch");
  if (a.batch != c.batch || (bm.batch != 1 && bm.batch != c.batch))
    throw std::runtime_error(std::string(who) + ": batch mismatch");
}

void run_gemm(Backend *b, const MatView &a, const MatView &bm, const MatView &c, const char *who,
              const GemmEpilogue &ep = GemmEpilogue{}) {
  check_gemm(a, bm, c, who);
  bind(b);
  launch_gemm_simt(a, bm, c, c.rows, c.cols, a.cols, ep, b->st);
  ++b->launches;
}

// device_backend.cpp:1096-1110
void api_gemm(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(a, "litnice_b200::gemm(a)");
  require_gpu_f32(bb, "litnice_b200::gemm(b)");
  require_gpu_f32(out, "litnice_b200::gemm(out)");
  run_gemm(b, make_mat_view(a, "gemm(a)"), make_mat_view(bb, "gemm(b)"), make_mat_view(out, "gemm(out)"),
           "litnice_b200::gemm");
}

// device_backend.cpp:1112-1131
void api_gemm_ranked_matrix_rhs(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self_recording(h);
  if (!b->queue.empty()) flush_queue(b);
  require_gpu_f32(a, "litnice_b200::gemm_ranked_matrix_rhs(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_ranked_matrix_rhs(b)");
  require_gpu_f32(out, "litnice_b200::gemm_ranked_matrix_rhs(out)");
  const MatView av = make_mat_view(a, "gemm_ranked_matrix_rhs(a)"), bv = shared_matrix(bb, "gemm_ranked_matrix_rhs(b)"),
                ov = make_mat_view(out, "gemm_ranked_matrix_rhs(out)");
  if (b->queue_on) {  // recorded: the bias call that usually follows becomes its epilogue
    check_gemm(av, bv, ov, "litnice_b200::gemm_ranked_matrix_rhs");
    Backend::Pending p;
    p.kind = Backend::Pending::PROJECTION;
    p.a = *a;
    p.b = *bb;
    p.c = *out;
    b->queue.push_back(p);
    return;
  }
  run_gemm(b, av, bv, ov, "litnice_b200::gemm_ranked_matrix_rhs");
}

// device_backend.cpp:1175-1193
void api_gemm_batched(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self_recording(h);
  require_gpu_f32(a, "litnice_b200::gemm_batched(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_batched(b)");
  require_gpu_f32(out, "litnice_b200::gemm_batched(out)");
  const MatView av = make_mat_view(a, "gemm_batched(a)"), bv = make_mat_view(bb, "gemm_batched(b)"),
                ov = make_mat_view(out, "gemm_batched(out)");
  // the context product of the softmax recorded just before: completes a head's three calls
  if (!b->queue.empty() && b->queue.back().kind == Backend::Pending::SOFTMAX && same_view(b->queue.back().c, *a)) {
    check_gemm(av, bv, ov, "litnice_b200::gemm_batched");
    Backend::Pending p;
    p.kind = Backend::Pending::CONTEXT;
    p.a = *a;
    p.b = *bb;
    p.c = *out;
    b->queue.push_back(p);
    return;
  }
  if (!b->queue.empty()) flush_queue(b);
  run_gemm(b, av, bv, ov, "litnice_b200::gemm_batched");
}

// device_backend.cpp:1216-1235: out[r,c] = sum_k a[r,k] * b[c,k]
void api_gemm_batched_rhs_t(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self_recording(h);
  require_gpu_f32(a, "litnice_b200::gemm_batched_rhs_t(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_batched_rhs_t(b)");
  require_gpu_f32(out, "litnice_b200::gemm_batched_rhs_t(out)");
  const MatView av = make_mat_view(a, "gemm_batched_rhs_t(a)"),
                bv = transposed(make_mat_view(bb, "gemm_batched_rhs_t(b)")),
                ov = make_mat_view(out, "gemm_batched_rhs_t(out)");
  // a score product opens a head's three calls; it may follow the completed calls of earlier heads
  const bool heads_pending = !b->queue.empty() && b->queue.back().kind == Backend::Pending::CONTEXT;
  if (!b->queue.empty() && !heads_pending) flush_queue(b);
  if (b->queue_on) {
    check_gemm(av, bv, ov, "litnice_b200::gemm_batched_rhs_t");
    Backend::Pending p;
    p.kind = Backend::Pending::SCORES;
    p.a = *a;
    p.b = *bb;
    p.c = *out;
    b->queue.push_back(p);
    return;
  }
  run_gemm(b, av, bv, ov, "litnice_b200::gemm_batched_rhs_t");
}

// ---- the deferred operators, issued ---------------------------------------------------------

MatView with_heads(MatView v, long long n, long long delta) {  // one more (outermost) batch axis
  for (int i = v.nb; i > 0; --i) {
    v.bd[i] = v.bd[i - 1];
    v.bs[i] = v.bs[i - 1];
  }
  v.bd[0] = n;
  v.bs[0] = delta;
  ++v.nb;
  v.batch *= n;
  return v;
}
RowView with_heads(RowView v, long long n, long long delta) {
  for (int i = v.np; i > 0; --i) {
    v.pd[i] = v.pd[i - 1];
    v.ps[i] = v.ps[i - 1];
  }
  v.pd[0] = n;
  v.ps[0] = delta;
  ++v.np;
  v.rows *= n;
  return v;
}

bool same_shape(const BackendTensorView &p, const BackendTensorView &q) {
  if (p.rank != q.rank) return false;
  for (uint32_t i = 0; i < p.rank; ++i)
    if (p.dims[i] != q.dims[i] || p.strides_bytes[i] != q.strides_bytes[i]) return false;
  return true;
}

void issue_one(Backend *b, const Backend::Pending &p) {
  switch (p.kind) {
    case Backend::Pending::PROJECTION:
      run_gemm(b, make_mat_view(&p.a, "gemm_ranked_matrix_rhs(a)"), shared_matrix(&p.b, "gemm_ranked_matrix_rhs(b)"),
               make_mat_view(&p.c, "gemm_ranked_matrix_rhs(out)"), "litnice_b200::gemm_ranked_matrix_rhs");
      break;
    case Backend::Pending::SCORES:
      run_gemm(b, make_mat_view(&p.a, "gemm_batched_rhs_t(a)"), transposed(make_mat_view(&p.b, "gemm_batched_rhs_t(b)")),
               make_mat_view(&p.c, "gemm_batched_rhs_t(out)"), "litnice_b200::gemm_batched_rhs_t");
      break;
    case Backend::Pending::SOFTMAX:
      run_causal_softmax(b, &p.a, p.scale, &p.c);
      break;
    case Backend::Pending::CONTEXT:
      run_gemm(b, make_mat_view(&p.a, "gemm_batched(a)"), make_mat_view(&p.b, "gemm_batched(b)"),
               make_mat_view(&p.c, "gemm_batched(out)"), "litnice_b200::gemm_batched");
      break;
    default:
      throw std::logic_error("litnice_b200: a recorded bias has no projection");
  }
}

// The three calls of heads [0, n) starting at queue index `at` as three launches over all heads, when
// every head's views have the same shape and their addresses advance by one constant per operand.
bool issue_heads_grouped(Backend *b, size_t at, long long n) {
  const Backend::Pending *q = b->queue.data() + at;
  auto delta = [&](int op, int which) -> long long {  // address step from head 0 to head 1
    auto pick = [&](const Backend::Pending &p) { return which == 0 ? p.a.data : which == 1 ? p.b.data : p.c.data; };
    return (long long)(static_cast<char *>(pick(q[3 + op])) - static_cast<char *>(pick(q[op])));
  };
  const long long dq = delta(0, 0), dk = delta(0, 1), ds = delta(0, 2), dw = delta(1, 2), dv = delta(2, 1),
                  dc = delta(2, 2);
  for (long long h = 0; h < n; ++h)
    for (int op = 0; op < 3; ++op) {
      const Backend::Pending &p = q[3 * h + op], &p0 = q[op];
      if (!same_shape(p.a, p0.a) || !same_shape(p.c, p0.c) || (op != 1 && !same_shape(p.b, p0.b))) return false;
      if (op == 1 && p.scale != p0.scale) return false;
      auto at_step = [&](void *ptr, void *base, long long d) {
        return static_cast<char *>(ptr) == static_cast<char *>(base) + h * d;
      };
      if (op == 0 && !(at_step(p.a.data, p0.a.data, dq) && at_step(p.b.data, p0.b.data, dk) &&
                       at_step(p.c.data, p0.c.data, ds)))
        return false;
      if (op == 1 && !at_step(p.c.data, p0.c.data, dw)) return false;
      if (op == 2 && !(at_step(p.b.data, p0.b.data, dv) && at_step(p.c.data, p0.c.data, dc))) return false;
    }
  if (dw == 0 || dc == 0) return false;  // heads must not share their outputs
  MatView qa = make_mat_view(&q[0].a, "gemm_batched_rhs_t(a)"),
          kb = transposed(make_mat_view(&q[0].b, "gemm_batched_rhs_t(b)")),
          sc = make_mat_view(&q[0].c, "gemm_batched_rhs_t(out)");
  RowView sx = make_row_view(&q[1].a, "scaled_causal_softmax_rows(scores)"),
          so = make_row_view(&q[1].c, "scaled_causal_softmax_rows(out)");
  MatView wa = make_mat_view(&q[2].a, "gemm_batched(a)"), vb = make_mat_view(&q[2].b, "gemm_batched(b)"),
          co = make_mat_view(&q[2].c, "gemm_batched(out)");
  if (qa.nb > 2 || sx.np > 3) return false;
  bind(b);
  const bool shared_scores = ds == 0;  // every head's scores land in one buffer of the host
  MatView sc_all = with_heads(sc, n, ds);
  RowView sx_all = with_heads(sx, n, ds);
  if (shared_scores) {
    // Scores of all heads side by side in scratch; the host's buffer receives the last head's, which is
    // what it holds after the host's own sequence.
    if (sc.batch != 1) return false;
    const size_t per_head = (size_t)sc.rows * sc.cols;
    if (per_head * n > b->queue_scratch_floats) {
      LB_CUDA(cudaStreamSynchronize(b->st));
      if (b->queue_scratch) cudaFree(b->queue_scratch);
      b->queue_scratch = nullptr;
      b->queue_scratch_floats = 0;
      if (cudaMalloc(reinterpret_cast<void **>(&b->queue_scratch), per_head * n * 4) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
      }
      b->queue_scratch_floats = per_head * n;
    }
    MatView dense_sc{};
    dense_sc.data = reinterpret_cast<char *>(b->queue_scratch);
    dense_sc.nb = 0;
    dense_sc.batch = 1;
    dense_sc.rows = sc.rows;
    dense_sc.cols = sc.cols;
    dense_sc.rs = sc.cols * 4;
    dense_sc.cs = 4;
    sc_all = with_heads(dense_sc, n, (long long)per_head * 4);
    RowView dense_sx{};
    dense_sx.data = reinterpret_cast<char *>(b->queue_scratch);
    dense_sx.np = 1;
    dense_sx.pd[0] = sc.rows;
    dense_sx.ps[0] = sc.cols * 4;
    dense_sx.rows = sc.rows;
    dense_sx.cols = sc.cols;
    dense_sx.cs = 4;
    sx_all = with_heads(dense_sx, n, (long long)per_head * 4);
  }
  launch_gemm_simt(with_heads(qa, n, dq), with_heads(kb, n, dk), sc_all, sc.rows, sc.cols, qa.cols, GemmEpilogue{},
                   b->st);
  launch_softmax_rows(sx_all, with_heads(so, n, dw), 1, q[1].scale, b->st);
  launch_gemm_simt(with_heads(wa, n, dw), with_heads(vb, n, dv), with_heads(co, n, dc), co.rows, co.cols, wa.cols,
                   GemmEpilogue{}, b->st);
  b->launches += 3;
  if (shared_scores) {
    RowView last{};
    last.data = reinterpret_cast<char *>(b->queue_scratch + (size_t)(n - 1) * sc.rows * sc.cols);
    last.np = 1;
    last.pd[0] = sc.rows;
    last.ps[0] = sc.cols * 4;
    last.rows = sc.rows;
    last.cols = sc.cols;
    last.cs = 4;
    launch_rowwise(EW_COPY, last, nullptr, 0, 0.f, sx, b->st);
    ++b->launches;
  }
  b->grouped_heads += n;
  return true;
}

void flush_queue(Backend *b) {
  std::vector<Backend::Pending> q;
  q.swap(b->queue);  // whatever happens below, nothing stays recorded
  if (q.empty()) return;
  if (q[0].kind == Backend::Pending::PROJECTION) {
    if (q.size() == 2) {  // a projection and its bias (+ ReLU) in one launch
      GemmEpilogue ep;
      ep.bias = static_cast<const float *>(q[1].a.data);
      ep.relu = q[1].kind == Backend::Pending::BIAS_RELU ? 1 : 0;
      run_gemm(b, make_mat_view(&q[0].a, "gemm_ranked_matrix_rhs(a)"),
               shared_matrix(&q[0].b, "gemm_ranked_matrix_rhs(b)"), make_mat_view(&q[0].c, "gemm_ranked_matrix_rhs(out)"),
               "litnice_b200::gemm_ranked_matrix_rhs", ep);
      ++b->fused_projections;
    } else {
      issue_one(b, q[0]);
    }
    return;
  }
  const long long heads = (long long)(q.size() / 3);  // complete (scores, softmax, context) triples
  size_t done = 0;
  if (heads >= 2) {
    b->queue.swap(q);  // issue_heads_grouped reads the recorded calls through the instance
    bool grouped = false;
    try {
      grouped = issue_heads_grouped(b, 0, heads);
    } catch (...) {
      b->queue.clear();
      throw;
    }
    q.swap(b->queue);
    if (grouped) done = (size_t)heads * 3;
  }
  for (size_t i = done; i < q.size(); ++i) issue_one(b, q[i]);
}

// ---- exec-context lanes ------------------------------------------------------------
// The multistream attention variant brackets per-head work with these calls
// (self_attention_fused_inplace_multistream.cpp:71-87). One in-order stream
// already keeps the GPU busy for these shapes, so the lanes are serial aliases;
// only the nesting is validated.

uint32_t api_supports_ctx(void *h) {
  self_recording(h);
  return 1u;
}
void api_start_iter(void *h) {
  Backend *b = self_recording(h);
  if (b->ctx_iteration) throw std::runtime_error("litnice_b200: exec context iteration already started");
  b->ctx_iteration = 1;
}
void api_finish_iter(void *h) {
  Backend *b = self_recording(h);
  if (!b->ctx_iteration || b->ctx_group) throw std::runtime_error("litnice_b200: exec context iteration not open");
  b->ctx_iteration = 0;
}
void api_start_group(void *h) {
  Backend *b = self_recording(h);
  if (!b->ctx_iteration || b->ctx_group) throw std::runtime_error("litnice_b200: exec context group misuse");
  b->ctx_group = 1;
}
void api_finish_group(void *h) {
  Backend *b = self_recording(h);
  if (!b->ctx_group) throw std::runtime_error("litnice_b200: exec context group not open");
  b->ctx_group = 0;
}
void require_group(void *h, const char *who) {
  if (!self_recording(h)->ctx_group) throw std::runtime_error(std::string(who) + ": no exec context group is open");
}
void api_gemm_batched_ctx(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  require_group(h, "litnice_b200::gemm_batched_exec_context");
  api_gemm_batched(h, a, bb, out);
}
void api_gemm_batched_rhs_t_ctx(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  require_group(h, "litnice_b200::gemm_batched_rhs_t_exec_context");
  api_gemm_batched_rhs_t(h, a, bb, out);
}
void api_causal_softmax_ctx(void *h, LitniceView scores, float scale, LitniceView out) {
  require_group(h, "litnice_b200::scaled_causal_softmax_rows_exec_context");
  api_causal_softmax(h, scores, scale, out);
}

// ---- training entries ------------------------------------------------------------------
// What `litnicelm train` calls beyond the inference entries. Kernels in training.cu.

void *scratch_for(Backend *b, long long rows, long long cols) {
  const size_t need = training_scratch_bytes(rows, cols);
  if (need > b->scratch_bytes) {
    LB_CUDA(cudaStreamSynchronize(b->st));
    if (b->scratch) cudaFree(b->scratch);
    b->scratch = nullptr;
    b->scratch_bytes = 0;
    const size_t grown = need + need / 2;
    if (cudaMalloc(&b->scratch, grown) != cudaSuccess) {
      (void)cudaGetLastError();
      throw std::runtime_error("litnice_b200: device allocation of " + std::to_string(grown) + " bytes of scratch failed");
    }
    b->scratch_bytes = grown;
  }
  return b->scratch;
}

void require_index(LitniceView t, const char *who) {
  if (t == nullptr) throw std::invalid_argument(std::string(who) + ": null view");
  if (t->device != 1u) throw std::runtime_error(std::string(who) + " requires a GPU tensor");
  if (t->dtype > 1u) throw std::runtime_error(std::string(who) + ": unsupported index dtype");
}

// device_backend.cpp:966-976: double accumulation, synchronous float result.
float api_sum_squares(void *h, LitniceView x) {
  Backend *b = self_reader(h);
  require_gpu_f32(x, "litnice_b200::sum_squares_f32");
  if (!view_is_contiguous(x)) throw std::runtime_error("litnice_b200::sum_squares_f32 requires a contiguous tensor");
  bind(b);
  const long long n = view_numel(x);
  char *scr = static_cast<char *>(scratch_for(b, 1, 1));
  double *result = reinterpret_cast<double *>(scr + 148 * 8 * sizeof(double));
  launch_sum_squares(static_cast<const float *>(x->data), n, scr, result, b->st);
  b->launches += 2;
  double v = 0.0;
  LB_CUDA(cudaMemcpyAsync(&v, result, sizeof(double), cudaMemcpyDeviceToHost, b->st));
  sync_and_check(b);
  return static_cast<float>(v);
}

// device_backend.cpp:1003-1060
void relu_backward_op(void *h, LitniceView preact, LitniceView dout, LitniceView dx, const char *who) {
  Backend *b = self(h);
  require_gpu_f32(preact, who);
  require_gpu_f32(dout, who);
  require_gpu_f32(dx, who);
  bind(b);
  if (view_numel(preact) != view_numel(dout) || view_numel(preact) != view_numel(dx))
    throw std::runtime_error(std::string(who) + ": numel mismatch");
  if (view_is_contiguous(preact) && view_is_contiguous(dout) && view_is_contiguous(dx)) {
    RowView fb = flat_view(dout);
    launch_rowwise(EW_RELU_BWD, flat_view(preact), &fb, 0, 0.f, flat_view(dx), b->st);
  } else {
    RowView rp = make_row_view(preact, who), rd = make_row_view(dout, who), rx = make_row_view(dx, who);
    if (rp.cols != rd.cols || rp.cols != rx.cols || rp.rows != rd.rows || rp.rows != rx.rows)
      throw std::runtime_error(std::string(who) + ": shape mismatch");
    launch_rowwise(EW_RELU_BWD, rp, &rd, 0, 0.f, rx, b->st);
  }
  ++b->launches;
}
void api_relu_backward(void *h, LitniceView preact, LitniceView dout, LitniceView dx) {
  relu_backward_op(h, preact, dout, dx, "litnice_b200::relu_backward");
}
void api_relu_backward_inplace(void *h, LitniceView preact, LitniceView dout_dx) {
  relu_backward_op(h, preact, dout_dx, dout_dx, "litnice_b200::relu_backward_inplace");
}

// device_backend.cpp:1062-1094: out[c] = sum over every row of x[.., c].
void api_row_sum(void *h, LitniceView x, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(x, "litnice_b200::row_sum(x)");
  require_gpu_f32(out, "litnice_b200::row_sum(out)");
  bind(b);
  RowView rx = make_row_view(x, "row_sum(x)");
  if (view_numel(out) != rx.cols) throw std::runtime_error("litnice_b200::row_sum: semantic shape mismatch");
  launch_column_sum(rx, static_cast<char *>(out->data), out->strides_bytes[out->rank - 1],
                    scratch_for(b, rx.rows, rx.cols), b->st);
  b->launches += 2;
}

// device_backend.cpp:1133-1152: out[p, r, c] = sum_k a[p, r, k] * b[c, k]
void api_gemm_ranked_matrix_rhs_t(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(a, "litnice_b200::gemm_ranked_matrix_rhs_t(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_ranked_matrix_rhs_t(b)");
  require_gpu_f32(out, "litnice_b200::gemm_ranked_matrix_rhs_t(out)");
  run_gemm(b, make_mat_view(a, "gemm_ranked_matrix_rhs_t(a)"),
           transposed(shared_matrix(bb, "gemm_ranked_matrix_rhs_t(b)")),
           make_mat_view(out, "gemm_ranked_matrix_rhs_t(out)"), "litnice_b200::gemm_ranked_matrix_rhs_t");
}

// device_backend.cpp:1154-1173: out[r, c] = sum over p and k of a[p, k, r] * b[p, k, c] (weight
// gradients). One product per leading index, each added to the sum of those before it.
void api_gemm_ranked_reduce_lhs_t(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(a, "litnice_b200::gemm_ranked_reduce_lhs_t(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_ranked_reduce_lhs_t(b)");
  require_gpu_f32(out, "litnice_b200::gemm_ranked_reduce_lhs_t(out)");
  MatView av = make_mat_view(a, "gemm_ranked_reduce_lhs_t(a)"), bv = make_mat_view(bb, "gemm_ranked_reduce_lhs_t(b)");
  MatView ov = make_mat_view(out, "gemm_ranked_reduce_lhs_t(out)");
  if (av.batch != bv.batch || av.rows != bv.rows || ov.batch != 1 || ov.rows != av.cols || ov.cols != bv.cols)
    throw std::runtime_error("litnice_b200::gemm_ranked_reduce_lhs_t: shape mismatch");
  bind(b);
  for (long long p = 0; p < av.batch; ++p) {
    MatView ap = av, bp = bv;
    ap.data = av.data + batch_offset(av, p);
    bp.data = bv.data + batch_offset(bv, p);
    ap.nb = bp.nb = 0;
    ap.batch = bp.batch = 1;
    GemmEpilogue ep;
    if (p > 0) ep.residual = reinterpret_cast<const float *>(ov.data);  // in place: every element by one thread
    launch_gemm_simt(transposed(ap), bp, ov, ov.rows, ov.cols, av.rows, ep, b->st);
    ++b->launches;
  }
}

// device_backend.cpp:1195-1214: out[p] = a[p]^T * b[p]
void api_gemm_batched_lhs_t(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  Backend *b = self(h);
  require_gpu_f32(a, "litnice_b200::gemm_batched_lhs_t(a)");
  require_gpu_f32(bb, "litnice_b200::gemm_batched_lhs_t(b)");
  require_gpu_f32(out, "litnice_b200::gemm_batched_lhs_t(out)");
  run_gemm(b, transposed(make_mat_view(a, "gemm_batched_lhs_t(a)")), make_mat_view(bb, "gemm_batched_lhs_t(b)"),
           make_mat_view(out, "gemm_batched_lhs_t(out)"), "litnice_b200::gemm_batched_lhs_t");
}
void api_gemm_batched_lhs_t_ctx(void *h, LitniceView a, LitniceView bb, LitniceView out) {
  require_group(h, "litnice_b200::gemm_batched_lhs_t_exec_context");
  api_gemm_batched_lhs_t(h, a, bb, out);
}

// device_backend.cpp:1281-1343
void api_layernorm_backward(void *h, LitniceView x, LitniceView gamma, LitniceView dout, LitniceView dx,
                            LitniceView dgamma, LitniceView dbeta) {
  Backend *b = self(h);
  const char *who = "litnice_b200::layernorm_backward";
  for (LitniceView t : {x, gamma, dout, dx, dgamma, dbeta}) require_gpu_f32(t, who);
  bind(b);
  RowView rx = make_row_view(x, who), rd = make_row_view(dout, who), ro = make_row_view(dx, who);
  if (rd.rows != rx.rows || rd.cols != rx.cols || ro.rows != rx.rows || ro.cols != rx.cols ||
      view_numel(gamma) != rx.cols || view_numel(dgamma) != rx.cols || view_numel(dbeta) != rx.cols)
    throw std::runtime_error(std::string(who) + ": shape mismatch");
  launch_layernorm_backward(rx, static_cast<const char *>(gamma->data), gamma->strides_bytes[gamma->rank - 1], rd, ro,
                            static_cast<char *>(dgamma->data), dgamma->strides_bytes[dgamma->rank - 1],
                            static_cast<char *>(dbeta->data), dbeta->strides_bytes[dbeta->rank - 1],
                            scratch_for(b, rx.rows, rx.cols), b->st);
  b->launches += 3;
}

// device_backend.cpp:1368-1389
void api_accumulate_embedding_grads(void *h, LitniceView ids, LitniceView d_cur, LitniceView d_tok, LitniceView d_pos) {
  Backend *b = self(h);
  const char *who = "litnice_b200::accumulate_embedding_grads";
  require_index(ids, who);
  require_gpu_f32(d_cur, who);
  require_gpu_f32(d_tok, who);
  require_gpu_f32(d_pos, who);
  if (d_tok->rank != 2 || d_pos->rank != 2) throw std::runtime_error(std::string(who) + ": tables must be rank 2");
  bind(b);
  RowView iv = make_row_view(ids, who), rc = make_row_view(d_cur, who);
  auto table = [](LitniceView t) {  // keep the (row, column) axes apart
    RowView v{};
    v.data = static_cast<char *>(t->data);
    v.np = 1;
    v.pd[0] = t->dims[0];
    v.ps[0] = t->strides_bytes[0];
    v.rows = t->dims[0];
    v.cols = t->dims[1];
    v.cs = t->strides_bytes[1];
    return v;
  };
  RowView rt = table(d_tok), rp = table(d_pos);
  const long long tokens = iv.rows * iv.cols, seq = ids->dims[ids->rank - 1];
  if (rc.rows != tokens || rt.cols != rc.cols || rp.cols != rc.cols || rp.rows < seq)
    throw std::runtime_error(std::string(who) + ": shape mismatch");
  launch_embedding_grads(static_cast<const char *>(ids->data), ids->dtype == 0u ? 1 : 0, iv, rc, rt, rp, seq,
                         b->err_dev, b->st);
  b->launches += 2;
}

// device_backend.cpp:1391-1464
void cross_entropy_op(void *h, LitniceView logits, LitniceView targets, LitniceView out_loss, bool loss, bool backward,
                      const char *who) {
  Backend *b = self(h);
  require_gpu_f32(logits, who);
  require_index(targets, who);
  if (loss) require_gpu_f32(out_loss, who);
  bind(b);
  RowView rl = make_row_view(logits, who), rt = make_row_view(targets, who);
  const long long tokens = rt.rows * rt.cols;
  if (rl.rows != tokens) throw std::runtime_error(std::string(who) + ": logits rows and target count differ");
  launch_cross_entropy(rl, static_cast<const char *>(targets->data), targets->dtype == 0u ? 1 : 0, rt, loss, backward,
                       loss ? static_cast<float *>(out_loss->data) : nullptr, scratch_for(b, tokens, 1), b->err_dev,
                       b->st);
  b->launches += loss ? 2 : 1;
}
void api_cross_entropy_mean(void *h, LitniceView logits, LitniceView targets, LitniceView out_loss) {
  cross_entropy_op(h, logits, targets, out_loss, true, false, "litnice_b200::cross_entropy_mean");
}
void api_cross_entropy_mean_backward_inplace(void *h, LitniceView logits, LitniceView targets, LitniceView out_loss) {
  cross_entropy_op(h, logits, targets, out_loss, true, true, "litnice_b200::cross_entropy_mean_backward_inplace");
}
void api_backward_from_logits_targets(void *h, LitniceView logits, LitniceView targets) {
  cross_entropy_op(h, logits, targets, nullptr, false, true, "litnice_b200::backward_from_logits_targets");
}

// device_backend.cpp:1519-1552, :1649-1673
void softmax_backward_op(void *h, LitniceView sm, LitniceView dout, LitniceView dx, bool causal, const char *who) {
  Backend *b = self(h);
  require_gpu_f32(sm, who);
  require_gpu_f32(dout, who);
  require_gpu_f32(dx, who);
  bind(b);
  RowView rs = make_row_view(sm, who), rd = make_row_view(dout, who), rx = make_row_view(dx, who);
  if (rs.rows != rd.rows || rs.cols != rd.cols || rs.rows != rx.rows || rs.cols != rx.cols)
    throw std::runtime_error(std::string(who) + ": shape mismatch");
  launch_softmax_backward(rs, rd, rx, causal, b->st);
  ++b->launches;
}
void api_softmax_backward_rows(void *h, LitniceView sm, LitniceView dout, LitniceView dx) {
  softmax_backward_op(h, sm, dout, dx, false, "litnice_b200::softmax_backward_rows");
}
void api_softmax_backward_causal_rows(void *h, LitniceView sm, LitniceView dout, LitniceView dx) {
  softmax_backward_op(h, sm, dout, dx, true, "litnice_b200::softmax_backward_causal_rows");
}
void api_softmax_backward_causal_rows_ctx(void *h, LitniceView sm, LitniceView dout, LitniceView dx) {
  require_group(h, "litnice_b200::softmax_backward_causal_rows_exec_context");
  softmax_backward_op(h, sm, dout, dx, true, "litnice_b200::softmax_backward_causal_rows_exec_context");
}

// device_backend.cpp:1699-1750
void api_adamw_step(void *h, LitniceView params, LitniceView grads, LitniceView m, LitniceView v, uint64_t step,
                    float learning_rate, float beta1, float beta2, float weight_decay, uint32_t apply_weight_decay) {
  Backend *b = self(h);
  const char *who = "litnice_b200::adamw_step";
  for (LitniceView t : {params, grads, m, v}) {
    require_gpu_f32(t, who);
    if (!view_is_contiguous(t)) throw std::runtime_error(std::string(who) + " requires contiguous tensors");
    if (t->rank < 2 || t->dims[0] != params->dims[0] || t->dims[1] != params->dims[1])
      throw std::runtime_error(std::string(who) + ": params/grads/m/v shape mismatch");
  }
  if (step < 1) throw std::runtime_error(std::string(who) + ": step must be >= 1");
  if (!(learning_rate > 0.0f)) throw std::runtime_error(std::string(who) + ": learning_rate must be > 0");
  if (!(beta1 >= 0.0f && beta1 < 1.0f)) throw std::runtime_error(std::string(who) + ": beta1 must be in [0,1)");
  if (!(beta2 >= 0.0f && beta2 < 1.0f)) throw std::runtime_error(std::string(who) + ": beta2 must be in [0,1)");
  const double t = static_cast<double>(step);
  const float b1_corr = 1.0f - static_cast<float>(std::pow(static_cast<double>(beta1), t));
  const float b2_corr = 1.0f - static_cast<float>(std::pow(static_cast<double>(beta2), t));
  if (!(b1_corr > 0.0f && b2_corr > 0.0f)) throw std::runtime_error(std::string(who) + ": invalid bias correction");
  bind(b);
  launch_adamw(static_cast<float *>(params->data), static_cast<const float *>(grads->data),
               static_cast<float *>(m->data), static_cast<float *>(v->data), params->dims[0] * params->dims[1],
               learning_rate, beta1, beta2, b1_corr, b2_corr, weight_decay, apply_weight_decay ? 1 : 0, b->st);
  ++b->launches;
}

// device_backend.cpp:1426-1428: synchronous scalar read.
float api_read_scalar(void *h, LitniceView x) {
  Backend *b = self_reader(h);
  require_gpu_f32(x, "litnice_b200::read_scalar_f32");
  bind(b);
  float v = 0.f;
  LB_CUDA(cudaMemcpyAsync(&v, x->data, sizeof(float), cudaMemcpyDeviceToHost, b->st));
  sync_and_check(b);
  return v;
}

// device_backend.cpp:1752-1775. No caller exists in the host code. The range goes to the device
// in pieces through pinned memory, file reads overlapping the copies.
uint32_t api_file2device_supported(void *h) {
  self(h);
  return 1u;
}
void api_read_file2device(void *h, const char *path, void *dst, uint64_t size, uint64_t file_offset) {
  Backend *b = self(h);
  if (size == 0) return;
  if (dst == nullptr || path == nullptr)
    throw std::invalid_argument("litnice_b200::read_file2device: null argument");
  bind(b);
  try {
    file_to_device(path, file_offset, size, dst, b->st, false);
  } catch (const CudaError &) {
    throw;
  } catch (const std::exception &e) {
    throw std::runtime_error(std::string("litnice_b200::read_file2device: ") + e.what());
  }
}

const BackendApiV1 kApi = {
    LITNICE_BACKEND_ABI_VERSION,
    api_create,
    api_destroy,
    api_device,
    api_alloc,
    api_free,
    api_h2d,
    api_d2h,
    api_copy,
    api_fill,
    api_add,
    api_add_inplace,
    api_add_bias,
    api_add_bias_relu,
    api_add_bias_relu_inplace,
    api_mul_scalar,
    api_sum_squares,
    api_relu,
    api_relu_backward,
    api_relu_backward_inplace,
    api_row_sum,
    api_gemm,
    api_gemm_ranked_matrix_rhs,
    api_gemm_ranked_matrix_rhs_t,
    api_gemm_ranked_reduce_lhs_t,
    api_gemm_batched,
    api_gemm_batched_lhs_t,
    api_gemm_batched_rhs_t,
    api_transpose,
    api_layernorm,
    api_layernorm_backward,
    api_embedding,
    api_accumulate_embedding_grads,
    api_cross_entropy_mean,
    api_cross_entropy_mean_backward_inplace,
    api_read_scalar,
    api_backward_from_logits_targets,
    api_softmax_rows,
    api_softmax_backward_rows,
    api_causal_softmax,
    api_supports_ctx,
    api_start_iter,
    api_finish_iter,
    api_start_group,
    api_finish_group,
    api_gemm_batched_ctx,
    api_gemm_batched_lhs_t_ctx,
    api_gemm_batched_rhs_t_ctx,
    api_causal_softmax_ctx,
    api_softmax_backward_causal_rows_ctx,
    api_softmax_backward_causal_rows,
    api_causal_mask,
    api_adamw_step,
    api_file2device_supported,
    api_read_file2device,
    api_memory_info,
};

}  // namespace
}  // namespace lb

extern "C" const BackendApiV1 *litnice_backend_get_api(void) { return &lb::kApi; }
