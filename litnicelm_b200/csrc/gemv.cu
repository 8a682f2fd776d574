// Few-row matrix-vector products: out[m, n] = sum_k x[m, k] * W[k, n] for
// m <= 8 dense rows and row-major W [k, n] (the `[in, out]` weight layout of
// litnicelm's parameter arena, named_layout.cpp:52-160). This is the M=1
// regime of gemm_ranked_matrix_rhs (device_backend.cpp:1112-1131), used for
// the output head on the last row of each stream. The kernel is bound by HBM
// bandwidth: every weight byte is read exactly once with 16-byte coalesced
// loads, 4*k*n bytes per call.
//
// A CTA owns 128 consecutive output columns (32 lanes x float4) and a slice of
// k; its 8 warps take interleaved rows of that slice and combine through shared
// memory. When n/128 CTAs cannot fill the GPU, k is also split across CTAs:
// partial sums go to scratch [split][m][n] and a second kernel adds them in a
// fixed order, so results do not depend on scheduling.
#include "common.cuh"

namespace lb {

namespace {

constexpr int GV_COLS = 128;   // columns per CTA
constexpr int GV_WARPS = 8;
constexpr int GV_XCHUNK = 256; // k rows of x staged in shared memory at a time

template <int M, bool VEC>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_kernel(const float *__restrict__ x, const float *__restrict__ w, int k, int n,
            int k_per_split, const float *__restrict__ bias, float *__restrict__ out,
            float *__restrict__ partial) {
  __shared__ __align__(16) float xs[M][GV_XCHUNK];
  __shared__ __align__(16) float red[GV_WARPS][M][GV_COLS];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int n0 = blockIdx.x * GV_COLS + lane * 4;
  const int kb = blockIdx.y * k_per_split;
  const int ke = min(k, kb + k_per_split);

  float acc[M][4];
#pragma unroll
  for (int i = 0; i < M; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int kc = kb; kc < ke; kc += GV_XCHUNK) {
    const int kn = min(GV_XCHUNK, ke - kc);
    __syncthreads();
    for (int i = threadIdx.x; i < M * GV_XCHUNK; i += blockDim.x) {
      const int mi = i / GV_XCHUNK, kk = i - mi * GV_XCHUNK;
      xs[mi][kk] = kk < kn ? x[(long long)mi * k + kc + kk] : 0.f;
    }
    __syncthreads();
    if (n0 < n) {
#pragma unroll 4
      for (int kk = wid; kk < kn; kk += GV_WARPS) {
        const float *wp = w + (long long)(kc + kk) * n + n0;
        float4 wv;
        if (VEC) {
          wv = __ldg(reinterpret_cast<const float4 *>(wp));
        } else {
          wv.x = wp[0];
          wv.y = n0 + 1 < n ? wp[1] : 0.f;
          wv.z = n0 + 2 < n ? wp[2] : 0.f;
          wv.w = n0 + 3 < n ? wp[3] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < M; ++i) {
          const float xv = xs[i][kk];
          acc[i][0] = fmaf(xv, wv.x, acc[i][0]);
          acc[i][1] = fmaf(xv, wv.y, acc[i][1]);
          acc[i][2] = fmaf(xv, wv.z, acc[i][2]);
          acc[i][3] = fmaf(xv, wv.w, acc[i][3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < M; ++i)
    *reinterpret_cast<float4 *>(&red[wid][i][lane * 4]) =
        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  __syncthreads();
  // 256 threads fold the 8 warp rows: thread -> (row i, column c) pairs.
  for (int e = threadIdx.x; e < M * GV_COLS; e += blockDim.x) {
    const int i = e / GV_COLS, c = e - i * GV_COLS;
    const int col = blockIdx.x * GV_COLS + c;
    if (col >= n) continue;
    float v = red[0][i][c];
#pragma unroll
    for (int q = 1; q < GV_WARPS; ++q) v += red[q][i][c];
    if (partial) {
      partial[((long long)blockIdx.y * M + i) * n + col] = v;
    } else {
      if (bias) v += bias[col];
      out[(long long)i * n + col] = v;
    }
  }
}

__global__ void gemv_reduce_kernel(const float *__restrict__ partial, int splits, int m, int n,
                                   const float *__restrict__ bias, float *__restrict__ out) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)m * n) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[(long long)s * m * n + idx];
  if (bias) v += bias[idx % n];
  out[idx] = v;
}

int choose_splits(int n, int k) {
  const int col_blocks = (n + GV_COLS - 1) / GV_COLS;
  if (col_blocks >= 148) return 1;
  int splits = (2 * 148 + col_blocks - 1) / col_blocks;
  const int max_splits = (k + 63) / 64;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  return splits;
}

template <int M>
void launch_m(const float *x, const float *w, int k, int n, const float *bias, float *out,
              float *scratch, cudaStream_t st) {
  const int splits = scratch ? choose_splits(n, k) : 1;
  const int k_per_split = (k + splits - 1) / splits;
  dim3 grid((n + GV_COLS - 1) / GV_COLS, splits);
  float *partial = splits > 1 ? scratch : nullptr;
  const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
  if (vec)
    gemv_kernel<M, true><<<grid, GV_WARPS * 32, 0, st>>>(x, w, k, n, k_per_split, bias, out, partial);
  else
    gemv_kernel<M, false><<<grid, GV_WARPS * 32, 0, st>>>(x, w, k, n, k_per_split, bias, out, partial);
  LB_LAUNCH_CHECK();
  if (splits > 1) {
    const long long total = (long long)M * n;
    gemv_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(partial, splits, M, n, bias, out);
    LB_LAUNCH_CHECK();
  }
}

}  // namespace

size_t gemv_scratch_floats(int m, int n, int k) {
  const int splits = choose_splits(n, k);
  const int mm = m <= 1 ? 1 : (m <= 2 ? 2 : (m <= 4 ? 4 : 8));
  return splits > 1 ? (size_t)splits * mm * n : 0;
}

void launch_gemv(const float *x, int m, const float *w, int k, int n, const float *bias,
                 float *out, float *scratch, cudaStream_t st) {
  // Rows beyond m up to the template width read as zeros inside the kernel only
  // if x holds them; callers pass buffers padded to 8 rows.
  if (m <= 1) launch_m<1>(x, w, k, n, bias, out, scratch, st);
  else if (m <= 2) launch_m<2>(x, w, k, n, bias, out, scratch, st);
  else if (m <= 4) launch_m<4>(x, w, k, n, bias, out, scratch, st);
  else if (m <= 8) launch_m<8>(x, w, k, n, bias, out, scratch, st);
  else throw std::invalid_argument("launch_gemv: m must be <= 8");
}

}  // namespace lb
