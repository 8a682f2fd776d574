// Row-wise elementwise kernels of the plugin contract: copy, fill, add (with
// the position-embedding broadcast), bias (+ReLU), ReLU, scalar multiply,
// causal mask, embedding gather, transpose. They follow DefaultCpuBackend in
// litnicelm's src/model/backend/device_backend.cpp (lines cited per kernel) and
// accept the byte-strided views the host builds.
#include "common.cuh"

namespace lb {

namespace {

template <int OP>
__device__ __forceinline__ float ew_apply(float a, float b, float s) {
  if (OP == EW_COPY) return a;
  if (OP == EW_ADD || OP == EW_ADD_BIAS) return a + b;
  if (OP == EW_ADD_BIAS_RELU) {
    const float v = a + b;
    return v > 0.0f ? v : 0.0f;
  }
  if (OP == EW_RELU) return a > 0.0f ? a : 0.0f;
  if (OP == EW_MUL_SCALAR) return a * s;
  if (OP == EW_RELU_BWD) return a > 0.0f ? b : 0.0f;  // device_backend.cpp:1003-1060
  return s;  // EW_FILL
}

// One thread per VEC consecutive columns of one row. HAS_A / HAS_B say which
// inputs the operation reads.
// device_backend.cpp:715-732 (copy), :734-750 (fill), :752-813 (add),
// :840-940 (bias variants), :942-964 (mul_scalar), :978-1001 (relu).
template <int OP, int VEC>
__global__ void rowwise_kernel(RowView a, RowView b, long long b_mod_rows, float scalar,
                               RowView out, long long chunks_per_row, long long total_chunks) {
  constexpr bool HAS_A = OP != EW_FILL;
  constexpr bool HAS_B = OP == EW_ADD || OP == EW_ADD_BIAS || OP == EW_ADD_BIAS_RELU || OP == EW_RELU_BWD;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_chunks;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / chunks_per_row;
    const long long c0 = (idx - row * chunks_per_row) * VEC;
    char *op = out.data + row_offset(out, row) + c0 * out.cs;
    const char *ap = HAS_A ? a.data + row_offset(a, row) + c0 * a.cs : nullptr;
    const char *bp = nullptr;
    if (HAS_B) {
      const long long br = b_mod_rows > 0 ? row % b_mod_rows : row;
      bp = b.data + row_offset(b, br) + c0 * b.cs;
    }
    if (VEC == 4) {
      float4 av = HAS_A ? *reinterpret_cast<const float4 *>(ap) : make_float4(0, 0, 0, 0);
      float4 bv = HAS_B ? *reinterpret_cast<const float4 *>(bp) : make_float4(0, 0, 0, 0);
      float4 r;
      r.x = ew_apply<OP>(av.x, bv.x, scalar);
      r.y = ew_apply<OP>(av.y, bv.y, scalar);
      r.z = ew_apply<OP>(av.z, bv.z, scalar);
      r.w = ew_apply<OP>(av.w, bv.w, scalar);
      *reinterpret_cast<float4 *>(op) = r;
    } else {
      const float av = HAS_A ? *reinterpret_cast<const float *>(ap) : 0.0f;
      const float bv = HAS_B ? *reinterpret_cast<const float *>(bp) : 0.0f;
      *reinterpret_cast<float *>(op) = ew_apply<OP>(av, bv, scalar);
    }
  }
}

bool vec4_ok(const RowView &v) {
  if (v.cs != 4 || (v.cols & 3) != 0) return false;
  if ((reinterpret_cast<uintptr_t>(v.data) & 15) != 0) return false;
  for (int i = 0; i < v.np; ++i)
    if ((v.ps[i] & 15) != 0) return false;
  return true;
}

template <int OP>
void launch_rowwise_op(const RowView &a, const RowView *b, long long b_mod_rows, float scalar,
                       const RowView &out, cudaStream_t st) {
  constexpr bool HAS_A = OP != EW_FILL;
  constexpr bool HAS_B = OP == EW_ADD || OP == EW_ADD_BIAS || OP == EW_ADD_BIAS_RELU || OP == EW_RELU_BWD;
  bool vec = vec4_ok(out);
  if (HAS_A) vec = vec && vec4_ok(a);
  if (HAS_B) vec = vec && vec4_ok(*b);
  const long long rows = out.rows, cols = out.cols;
  if (rows <= 0 || cols <= 0) return;
  RowView bb = HAS_B ? *b : out;
  RowView aa = HAS_A ? a : out;
  const int threads = 256;
  if (vec) {
    const long long cpr = cols / 4, total = rows * cpr;
    const long long blocks = (total + threads - 1) / threads;
    rowwise_kernel<OP, 4><<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), threads, 0, st>>>(
        aa, bb, b_mod_rows, scalar, out, cpr, total);
  } else {
    const long long total = rows * cols;
    const long long blocks = (total + threads - 1) / threads;
    rowwise_kernel<OP, 1><<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), threads, 0, st>>>(
        aa, bb, b_mod_rows, scalar, out, cols, total);
  }
  LB_LAUNCH_CHECK();
}

// device_backend.cpp:1675-1697: scores[.., i, j] = neg_inf for j > i.
__global__ void causal_mask_kernel(MatView sc, float neg_inf, long long total) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long per = sc.rows * sc.cols;
    const long long b = idx / per;
    const long long rem = idx - b * per;
    const long long i = rem / sc.cols, j = rem - i * sc.cols;
    if (j > i)
      *reinterpret_cast<float *>(sc.data + batch_offset(sc, b) + i * sc.rs + j * sc.cs) = neg_inf;
  }
}

// device_backend.cpp:1345-1366: out[t, :] = table[ids[t], :]. The CPU backend
// throws on an id outside [0, vocab); here the row is zero-filled and the error
// word is set, and the host raises at its next synchronisation.
__global__ void embedding_kernel(RowView table, const char *ids_data, int ids_is_f32,
                                 RowView ids_rows, RowView out, long long vocab, DevErr *err) {
  const long long t = blockIdx.x;
  const long long ir = t / ids_rows.cols, ic = t - ir * ids_rows.cols;
  const char *ip = ids_data + row_offset(ids_rows, ir) + ic * ids_rows.cs;
  long long id = ids_is_f32 ? (long long)(*reinterpret_cast<const float *>(ip))
                            : (long long)(*reinterpret_cast<const int *>(ip));
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) {
    err->code = DEVERR_BAD_TOKEN_ID;
    err->detail = (int)id;
  }
  char *op = out.data + row_offset(out, t);
  const char *tp = table.data + (bad ? 0 : id) * table.ps[0];
  for (long long c = threadIdx.x; c < out.cols; c += blockDim.x) {
    const float v = bad ? 0.0f : *reinterpret_cast<const float *>(tp + c * table.cs);
    *reinterpret_cast<float *>(op + c * out.cs) = v;
  }
}

// device_backend.cpp:1237-1245.
__global__ void transpose_kernel(MatView x, MatView out, long long total) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / x.cols, c = idx - r * x.cols;
    *reinterpret_cast<float *>(out.data + c * out.rs + r * out.cs) =
        *reinterpret_cast<const float *>(x.data + r * x.rs + c * x.cs);
  }
}

}  // namespace

void launch_rowwise(EwOp op, const RowView &a, const RowView *b, long long b_mod_rows,
                    float scalar, const RowView &out, cudaStream_t st) {
  switch (op) {
    case EW_COPY: launch_rowwise_op<EW_COPY>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_ADD: launch_rowwise_op<EW_ADD>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_ADD_BIAS: launch_rowwise_op<EW_ADD_BIAS>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_ADD_BIAS_RELU: launch_rowwise_op<EW_ADD_BIAS_RELU>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_RELU: launch_rowwise_op<EW_RELU>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_MUL_SCALAR: launch_rowwise_op<EW_MUL_SCALAR>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_FILL: launch_rowwise_op<EW_FILL>(a, b, b_mod_rows, scalar, out, st); break;
    case EW_RELU_BWD: launch_rowwise_op<EW_RELU_BWD>(a, b, b_mod_rows, scalar, out, st); break;
  }
}

void launch_causal_mask(const MatView &scores, float neg_inf, cudaStream_t st) {
  const long long total = scores.batch * scores.rows * scores.cols;
  if (total <= 0) return;
  const long long blocks = (total + 255) / 256;
  causal_mask_kernel<<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), 256, 0, st>>>(
      scores, neg_inf, total);
  LB_LAUNCH_CHECK();
}

void launch_embedding(const RowView &table, const char *ids_data, int ids_is_f32,
                      const RowView &ids_rows, const RowView &out, DevErr *err, cudaStream_t st) {
  const long long tokens = ids_rows.rows * ids_rows.cols;
  if (tokens <= 0) return;
  // The table must keep its (vocab, d) axes apart: rebuild an unmerged view.
  embedding_kernel<<<(unsigned)tokens, 128, 0, st>>>(table, ids_data, ids_is_f32, ids_rows, out,
                                                     table.pd[0], err);
  LB_LAUNCH_CHECK();
}

void launch_transpose(const MatView &x, const MatView &out, cudaStream_t st) {
  const long long total = x.rows * x.cols;
  if (total <= 0) return;
  const long long blocks = (total + 255) / 256;
  transpose_kernel<<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), 256, 0, st>>>(x, out, total);
  LB_LAUNCH_CHECK();
}

}  // namespace lb
