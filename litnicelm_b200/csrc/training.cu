// Training entries of the plugin table on CUDA: the backward and optimiser
// operators that `litnicelm train` calls through BackendApiV1. Semantics follow
// DefaultCpuBackend (litnicelm src/model/backend/device_backend.cpp, lines
// cited per kernel): the same widths (double where the CPU code sums in
// double, float where it sums in float), the same formulas. Reductions that
// the CPU code runs as one sequential loop are cut over threads here and
// joined in a fixed order, so results are reproducible from run to run and
// agree with the CPU backend to rounding; the optimiser step and the
// embedding-gradient scatter keep the CPU order exactly and are bit-identical.
#include "common.cuh"

namespace lb {

namespace {

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float ld(const RowView &v, long long row_off, long long c) {
  return *reinterpret_cast<const float *>(v.data + row_off + c * v.cs);
}
__device__ __forceinline__ void st(const RowView &v, long long row_off, long long c, float x) {
  *reinterpret_cast<float *>(v.data + row_off + c * v.cs) = x;
}

// Block-wide sums in a fixed order: warps reduce by shuffles, warp 0 adds the warp results in
// warp order. `red` holds one slot per warp.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T *red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  T total = red[0];
  for (int i = 1; i < nw; ++i) total += red[i];
  return total;
}
__device__ __forceinline__ float block_max(float v, float *red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float total = red[0];
  for (int i = 1; i < nw; ++i) total = fmaxf(total, red[i]);
  return total;
}

// ---- sum of squares (device_backend.cpp:966-976): double accumulation -------------------

__global__ void sum_squares_kernel(const float *__restrict__ x, long long n, double *__restrict__ partial) {
  __shared__ double red[8];
  double acc = 0.0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const double v = (double)x[i];
    acc += v * v;
  }
  const double total = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

__global__ void ordered_sum_kernel(const double *__restrict__ partial, int count, double scale, double *out_f64,
                                   float *out_f32) {
  // One warp: the lanes bring 256 consecutive terms at a time into shared memory (eight loads in
  // flight per lane), lane 0 adds them in index order from there (a chain of dependent adds, four
  // clocks each, instead of a shuffle per term), which keeps the sum identical to a sequential loop.
  __shared__ double terms[256];
  double acc = 0.0;
  for (int i0 = 0; i0 < count; i0 += 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * 32 + (int)threadIdx.x;
      terms[j * 32 + threadIdx.x] = i < count ? partial[i] : 0.0;
    }
    __syncwarp();
    if (threadIdx.x == 0) {
      const int n = min(256, count - i0);
      for (int j = 0; j < n; ++j) acc += terms[j];
    }
    __syncwarp();
  }
  if (threadIdx.x != 0) return;
  acc *= scale;
  if (out_f64) *out_f64 = acc;
  if (out_f32) *out_f32 = (float)acc;
}

// ---- column sums over rows (row_sum, device_backend.cpp:1062-1094) --------------------------
// A CTA owns 32 columns and one chunk of rows; its 8 warps take interleaved rows of the chunk and
// are joined in warp order, the chunks in chunk order by the second kernel.

constexpr int CS_COLS = 32, CS_LANES = 8;

__global__ void column_sum_kernel(RowView x, long long rows_per_chunk, float *__restrict__ partial) {
  __shared__ float red[CS_LANES][CS_COLS];
  const int cx = threadIdx.x % CS_COLS, ry = threadIdx.x / CS_COLS;
  const long long c = blockIdx.x * (long long)CS_COLS + cx;
  const long long r0 = blockIdx.y * rows_per_chunk;
  const long long r1 = r0 + rows_per_chunk < x.rows ? r0 + rows_per_chunk : x.rows;
  float acc = 0.f;
  if (c < x.cols)
    for (long long r = r0 + ry; r < r1; r += CS_LANES) acc += ld(x, row_offset(x, r), c);
  red[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && c < x.cols) {
    float t = red[0][cx];
    for (int i = 1; i < CS_LANES; ++i) t += red[i][cx];
    partial[blockIdx.y * x.cols + c] = t;
  }
}

__global__ void column_join_kernel(const float *__restrict__ partial, int chunks, long long cols, char *out,
                                   long long out_cs) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.f;
  for (int i = 0; i < chunks; ++i) t += partial[i * cols + c];
  *reinterpret_cast<float *>(out + c * out_cs) = t;
}

// ---- LayerNorm backward (device_backend.cpp:1281-1343) -------------------------------------------
// Rows: one warp per row, statistics and the two row sums in double as the CPU code has them.
// Columns: dgamma[c] = sum_rows float(dy * xhat), dbeta[c] = sum_rows dy, float sums, by the
// chunked column reduction above with xhat rebuilt from the saved row statistics.

__global__ void ln_bwd_rows_kernel(RowView x, const char *gamma, long long gamma_cs, RowView dout, RowView dx,
                                   double2 *__restrict__ row_stats) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= x.rows) return;
  const int lane = threadIdx.x & 31;
  const long long xo = row_offset(x, row), go = row_offset(dout, row), dxo = row_offset(dx, row);
  const long long d = x.cols;
  double s = 0.0;
  for (long long c = lane; c < d; c += 32) s += (double)ld(x, xo, c);
  const double mean = warp_sum(s) / (double)d;
  double v = 0.0;
  for (long long c = lane; c < d; c += 32) {
    const double t = (double)ld(x, xo, c) - mean;
    v += t * t;
  }
  const double var = warp_sum(v) / (double)d;
  const double inv_std = 1.0 / sqrt(var + (double)1e-5f);
  double s1 = 0.0, s2 = 0.0;
  for (long long c = lane; c < d; c += 32) {
    const double xhat = ((double)ld(x, xo, c) - mean) * inv_std;
    const double g = (double)*reinterpret_cast<const float *>(gamma + c * gamma_cs);
    const double dxhat = (double)ld(dout, go, c) * g;
    s1 += dxhat;
    s2 += dxhat * xhat;
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  const double n = (double)d;
  for (long long c = lane; c < d; c += 32) {
    const double xhat = ((double)ld(x, xo, c) - mean) * inv_std;
    const double g = (double)*reinterpret_cast<const float *>(gamma + c * gamma_cs);
    const double dxhat = (double)ld(dout, go, c) * g;
    st(dx, dxo, c, (float)((inv_std / n) * (n * dxhat - s1 - xhat * s2)));
  }
  if (lane == 0) row_stats[row] = make_double2(mean, inv_std);
}

__global__ void ln_bwd_columns_kernel(RowView x, RowView dout, const double2 *__restrict__ row_stats,
                                      long long rows_per_chunk, float *__restrict__ partial) {
  __shared__ float red_g[CS_LANES][CS_COLS], red_b[CS_LANES][CS_COLS];
  const int cx = threadIdx.x % CS_COLS, ry = threadIdx.x / CS_COLS;
  const long long c = blockIdx.x * (long long)CS_COLS + cx;
  const long long r0 = blockIdx.y * rows_per_chunk;
  const long long r1 = r0 + rows_per_chunk < x.rows ? r0 + rows_per_chunk : x.rows;
  float ag = 0.f, ab = 0.f;
  if (c < x.cols)
    for (long long r = r0 + ry; r < r1; r += CS_LANES) {
      const double2 ms = row_stats[r];
      const double xhat = ((double)ld(x, row_offset(x, r), c) - ms.x) * ms.y;
      const double dy = (double)ld(dout, row_offset(dout, r), c);
      ag += (float)(dy * xhat);
      ab += (float)dy;
    }
  red_g[ry][cx] = ag;
  red_b[ry][cx] = ab;
  __syncthreads();
  if (ry == 0 && c < x.cols) {
    float tg = red_g[0][cx], tb = red_b[0][cx];
    for (int i = 1; i < CS_LANES; ++i) {
      tg += red_g[i][cx];
      tb += red_b[i][cx];
    }
    partial[(2 * blockIdx.y) * x.cols + c] = tg;
    partial[(2 * blockIdx.y + 1) * x.cols + c] = tb;
  }
}

__global__ void ln_bwd_join_kernel(const float *__restrict__ partial, int chunks, long long cols, char *dgamma,
                                   long long dgamma_cs, char *dbeta, long long dbeta_cs) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float tg = 0.f, tb = 0.f;
  for (int i = 0; i < chunks; ++i) {
    tg += partial[(2 * i) * cols + c];
    tb += partial[(2 * i + 1) * cols + c];
  }
  *reinterpret_cast<float *>(dgamma + c * dgamma_cs) = tg;
  *reinterpret_cast<float *>(dbeta + c * dbeta_cs) = tb;
}

// ---- embedding gradients (device_backend.cpp:1368-1389) ----------------------------------------------
// d_pos[t % seq, :] += d_cur[t, :] and d_tok[ids[t], :] += d_cur[t, :] for t = 0, 1, ... in that
// order. Positions: one thread per (position, column) walks the batch in order. Tokens: a CTA owns
// 128 columns and the ids of one residue class, and walks every token in order, so each table row
// receives its rows of d_cur in the CPU order.

__device__ __forceinline__ long long load_index(const char *ids, int is_f32, const RowView &iv, long long t) {
  const long long r = t / iv.cols, c = t - r * iv.cols;
  const char *p = ids + row_offset(iv, r) + c * iv.cs;
  return is_f32 ? (long long)*reinterpret_cast<const float *>(p) : (long long)*reinterpret_cast<const int *>(p);
}

__global__ void embedding_grad_pos_kernel(RowView d_cur, long long tokens, long long seq, RowView d_pos) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long d = d_cur.cols;
  if (idx >= seq * d) return;
  const long long pos = idx / d, c = idx - pos * d;
  const long long po = row_offset(d_pos, pos);
  float acc = ld(d_pos, po, c);
  for (long long t = pos; t < tokens; t += seq) acc += ld(d_cur, row_offset(d_cur, t), c);
  st(d_pos, po, c, acc);
}

__global__ void embedding_grad_tok_kernel(const char *ids, int ids_is_f32, RowView iv, RowView d_cur, long long tokens,
                                          RowView d_tok, long long vocab, DevErr *err) {
  // Thread = one column of the embedding rows whose id falls into this CTA's class (id mod classes):
  // it walks the tokens in order, so every element of d_tok receives its additions in token order as
  // the CPU loop does. The ids come through shared memory in pieces (one coalesced load per token
  // instead of a dependent global load per token and thread); -1 marks an id out of range or of
  // another class.
  constexpr int PIECE = 1024;
  __shared__ int sid[PIECE];
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int klass = blockIdx.y, classes = gridDim.y;
  for (long long t0 = 0; t0 < tokens; t0 += PIECE) {
    const int n = (int)(tokens - t0 < PIECE ? tokens - t0 : PIECE);
    __syncthreads();
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      const long long id = load_index(ids, ids_is_f32, iv, t0 + j);
      const bool bad = id < 0 || id >= vocab;
      if (bad && klass == 0 && blockIdx.x == 0) {
        err->code = DEVERR_BAD_TOKEN_ID;
        err->detail = (int)id;
      }
      sid[j] = (bad || (int)(id % classes) != klass) ? -1 : (int)id;  // only this CTA's class is kept
    }
    __syncthreads();
    if (c >= d_cur.cols) continue;
    for (int j = 0; j < n; ++j) {
      const int id = sid[j];
      if (id < 0) continue;
      const long long to = row_offset(d_tok, id);
      st(d_tok, to, c, ld(d_tok, to, c) + ld(d_cur, row_offset(d_cur, t0 + j), c));
    }
  }
}

// ---- cross entropy (device_backend.cpp:1391-1464) -------------------------------------------------------
// One CTA per token row: float maximum, double sum of exponentials. LOSS: the row's
// log-sum-exp minus its target logit goes to row_loss[t] (double), summed in row order by
// ordered_sum_kernel. BACKWARD: logits[t, c] <- (softmax - onehot) / tokens, in place.

template <bool LOSS, bool BACKWARD>
__global__ void cross_entropy_kernel(RowView logits, const char *targets, int targets_is_f32, RowView tv,
                                     double *__restrict__ row_loss, float inv_rows, DevErr *err) {
  __shared__ float red_f[8];
  __shared__ double red_d[8];
  const long long t = blockIdx.x;
  const long long v = logits.cols;
  const long long lo = row_offset(logits, t);
  const long long target = load_index(targets, targets_is_f32, tv, t);
  if (target < 0 || target >= v) {
    if (threadIdx.x == 0) {
      err->code = DEVERR_BAD_TARGET;
      err->detail = (int)target;
      if (LOSS) row_loss[t] = 0.0;
    }
    return;
  }
  float m = -INFINITY;
  for (long long c = threadIdx.x; c < v; c += blockDim.x) m = fmaxf(m, ld(logits, lo, c));
  m = block_max(m, red_f);
  double s = 0.0;
  for (long long c = threadIdx.x; c < v; c += blockDim.x) s += exp((double)(ld(logits, lo, c) - m));
  s = block_sum(s, red_d);
  if (LOSS && threadIdx.x == 0) row_loss[t] = ((double)m + log(s)) - (double)ld(logits, lo, target);
  if (BACKWARD) {
    __syncthreads();
    for (long long c = threadIdx.x; c < v; c += blockDim.x) {
      float p = (float)(exp((double)(ld(logits, lo, c) - m)) / s);
      if (c == target) p -= 1.0f;
      st(logits, lo, c, p * inv_rows);
    }
  }
}

// ---- softmax backward (device_backend.cpp:1519-1552, :1649-1673) ----------------------------------------
// dx = s * (dout - dot), dot = sum_c s * dout in float; causal: only columns c <= row % cols take
// part and the others receive zero. One warp per row.

template <bool CAUSAL>
__global__ void softmax_bwd_kernel(RowView sm, RowView dout, RowView dx) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= sm.rows) return;
  const int lane = threadIdx.x & 31;
  const long long so = row_offset(sm, row), go = row_offset(dout, row), xo = row_offset(dx, row);
  const long long cols = sm.cols;
  const long long live = CAUSAL ? (row % cols) + 1 : cols;
  float dot = 0.f;
  for (long long c = lane; c < live; c += 32) dot += ld(sm, so, c) * ld(dout, go, c);
  dot = warp_sum(dot);
  for (long long c = lane; c < cols; c += 32) {
    float g = 0.f;
    if (c < live) g = ld(sm, so, c) * (ld(dout, go, c) - dot);
    st(dx, xo, c, g);
  }
}

// ---- AdamW (device_backend.cpp:1699-1750) ----------------------------------------------------------------
// Every operation rounded separately, in the CPU code's order (no fused multiply-add), so the
// update is bit-identical to the CPU backend's.

__global__ void adamw_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m1,
                             float *__restrict__ m2, long long n, float lr, float beta1, float beta2,
                             float b1_corr, float b2_corr, float weight_decay, int apply_decay) {
  const float one_minus_b1 = __fsub_rn(1.0f, beta1), one_minus_b2 = __fsub_rn(1.0f, beta2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float grad = g[i];
    const float m = __fadd_rn(__fmul_rn(beta1, m1[i]), __fmul_rn(one_minus_b1, grad));
    const float v = __fadd_rn(__fmul_rn(beta2, m2[i]), __fmul_rn(__fmul_rn(one_minus_b2, grad), grad));
    m1[i] = m;
    m2[i] = v;
    const float mhat = __fdiv_rn(m, b1_corr);
    const float vhat = __fdiv_rn(v, b2_corr);
    const float adam = __fdiv_rn(mhat, __fadd_rn(__fsqrt_rn(vhat), 1e-8f));
    const float decay = apply_decay ? __fmul_rn(weight_decay, p[i]) : 0.0f;
    p[i] = __fsub_rn(p[i], __fmul_rn(lr, __fadd_rn(adam, decay)));
  }
}

int chunk_count(long long rows) {
  // enough chunks to fill the GPU with 32-column CTAs, at least 64 rows each
  long long chunks = (rows + 63) / 64;
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  return (int)chunks;
}

}  // namespace

size_t training_scratch_bytes(long long rows, long long cols) {
  // the largest user: LayerNorm backward (row statistics + two partial rows per chunk)
  const size_t stats = (size_t)rows * sizeof(double2);
  const size_t partial = (size_t)2 * 64 * (size_t)cols * sizeof(float);
  const size_t blocks = (size_t)148 * 8 * sizeof(double) + 64;
  const size_t losses = (size_t)rows * sizeof(double);
  size_t need = stats + partial;
  if (blocks > need) need = blocks;
  if (losses > need) need = losses;
  return need + 256;
}

void launch_sum_squares(const float *x, long long n, void *scratch, double *result_dev, cudaStream_t st) {
  double *partial = static_cast<double *>(scratch);
  long long blocks = (n + 4095) / 4096;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  sum_squares_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, n, partial);
  LB_LAUNCH_CHECK();
  ordered_sum_kernel<<<1, 32, 0, st>>>(partial, (int)blocks, 1.0, result_dev, nullptr);
  LB_LAUNCH_CHECK();
}

void launch_column_sum(const RowView &x, char *out, long long out_cs, void *scratch, cudaStream_t st) {
  if (x.cols <= 0) return;
  const int chunks = chunk_count(x.rows);
  const long long rpc = (x.rows + chunks - 1) / chunks;
  float *partial = static_cast<float *>(scratch);
  dim3 grid((unsigned)((x.cols + CS_COLS - 1) / CS_COLS), (unsigned)chunks);
  column_sum_kernel<<<grid, CS_COLS * CS_LANES, 0, st>>>(x, rpc > 0 ? rpc : 1, partial);
  LB_LAUNCH_CHECK();
  column_join_kernel<<<(unsigned)((x.cols + 255) / 256), 256, 0, st>>>(partial, chunks, x.cols, out, out_cs);
  LB_LAUNCH_CHECK();
}

void launch_layernorm_backward(const RowView &x, const char *gamma, long long gamma_cs, const RowView &dout,
                               const RowView &dx, char *dgamma, long long dgamma_cs, char *dbeta, long long dbeta_cs,
                               void *scratch, cudaStream_t st) {
  if (x.rows <= 0 || x.cols <= 0) return;
  double2 *stats = static_cast<double2 *>(scratch);
  float *partial = reinterpret_cast<float *>(stats + x.rows);
  ln_bwd_rows_kernel<<<(unsigned)((x.rows + 7) / 8), 256, 0, st>>>(x, gamma, gamma_cs, dout, dx, stats);
  LB_LAUNCH_CHECK();
  const int chunks = chunk_count(x.rows);
  const long long rpc = (x.rows + chunks - 1) / chunks;
  dim3 grid((unsigned)((x.cols + CS_COLS - 1) / CS_COLS), (unsigned)chunks);
  ln_bwd_columns_kernel<<<grid, CS_COLS * CS_LANES, 0, st>>>(x, dout, stats, rpc, partial);
  LB_LAUNCH_CHECK();
  ln_bwd_join_kernel<<<(unsigned)((x.cols + 255) / 256), 256, 0, st>>>(partial, chunks, x.cols, dgamma, dgamma_cs, dbeta,
                                                                      dbeta_cs);
  LB_LAUNCH_CHECK();
}

void launch_embedding_grads(const char *ids, int ids_is_f32, const RowView &ids_rows, const RowView &d_cur,
                            const RowView &d_tok, const RowView &d_pos, long long seq, DevErr *err, cudaStream_t st) {
  const long long tokens = ids_rows.rows * ids_rows.cols;
  if (tokens <= 0 || d_cur.cols <= 0) return;
  const long long total = seq * d_cur.cols;
  embedding_grad_pos_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_cur, tokens, seq, d_pos);
  LB_LAUNCH_CHECK();
  long long classes = d_tok.rows < 64 ? d_tok.rows : 64;
  if (classes < 1) classes = 1;
  dim3 grid((unsigned)((d_cur.cols + 127) / 128), (unsigned)classes);
  embedding_grad_tok_kernel<<<grid, 128, 0, st>>>(ids, ids_is_f32, ids_rows, d_cur, tokens, d_tok, d_tok.rows, err);
  LB_LAUNCH_CHECK();
}

void launch_cross_entropy(const RowView &logits, const char *targets, int targets_is_f32, const RowView &targets_rows,
                          bool want_loss, bool want_backward, float *loss_out, void *scratch, DevErr *err,
                          cudaStream_t st) {
  const long long tokens = targets_rows.rows * targets_rows.cols;
  if (tokens <= 0) return;
  double *row_loss = static_cast<double *>(scratch);
  const float inv_rows = 1.0f / (float)tokens;
  const unsigned grid = (unsigned)tokens;
  if (want_loss && want_backward)
    cross_entropy_kernel<true, true><<<grid, 256, 0, st>>>(logits, targets, targets_is_f32, targets_rows, row_loss,
                                                           inv_rows, err);
  else if (want_loss)
    cross_entropy_kernel<true, false><<<grid, 256, 0, st>>>(logits, targets, targets_is_f32, targets_rows, row_loss,
                                                            inv_rows, err);
  else
    cross_entropy_kernel<false, true><<<grid, 256, 0, st>>>(logits, targets, targets_is_f32, targets_rows, row_loss,
                                                            inv_rows, err);
  LB_LAUNCH_CHECK();
  if (want_loss) {
    ordered_sum_kernel<<<1, 32, 0, st>>>(row_loss, (int)tokens, 1.0 / (double)tokens, nullptr, loss_out);
    LB_LAUNCH_CHECK();
  }
}

void launch_softmax_backward(const RowView &sm, const RowView &dout, const RowView &dx, bool causal, cudaStream_t st) {
  if (sm.rows <= 0 || sm.cols <= 0) return;
  const unsigned grid = (unsigned)((sm.rows + 7) / 8);
  if (causal) softmax_bwd_kernel<true><<<grid, 256, 0, st>>>(sm, dout, dx);
  else softmax_bwd_kernel<false><<<grid, 256, 0, st>>>(sm, dout, dx);
  LB_LAUNCH_CHECK();
}

void launch_adamw(float *params, const float *grads, float *m, float *v, long long n, float lr, float beta1,
                  float beta2, float b1_corr, float b2_corr, float weight_decay, int apply_decay, cudaStream_t st) {
  if (n <= 0) return;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_kernel<<<(unsigned)blocks, 256, 0, st>>>(params, grads, m, v, n, lr, beta1, beta2, b1_corr, b2_corr,
                                                 weight_decay, apply_decay);
  LB_LAUNCH_CHECK();
}

}  // namespace lb
