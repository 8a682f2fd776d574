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

#include <cstdio>
#include <mutex>

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
  pdl_launch_dependents();
  pdl_wait();
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
  pdl_launch_dependents();
  pdl_wait();
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
    launch_pdl(gemv_kernel<M, true>, grid, dim3(GV_WARPS * 32), 0, st, g_pdl_enabled, x, w, k, n, k_per_split, bias, out,
               partial);
  else
    launch_pdl(gemv_kernel<M, false>, grid, dim3(GV_WARPS * 32), 0, st, g_pdl_enabled, x, w, k, n, k_per_split, bias, out,
               partial);
  if (splits > 1) {
    const long long total = (long long)M * n;
    launch_pdl(gemv_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, g_pdl_enabled,
               (const float *)partial, splits, M, n, bias, out);
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

// ---------------------------------------------------------------------------
// Few-row product for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc once they are running: a
// host that sized its own arenas from memory_info at start-up and has handed
// every remaining byte to them (litnicelm's memory managers do exactly that),
// or a serving loop in which an allocation would stall the whole device. For
// them the split-k partial sums of the kernel above live in a fixed array that
// is part of the library image instead of a buffer from cudaMalloc. Every GPU
// that loads the library holds these 1.5 MiB until the process exits.
// ---------------------------------------------------------------------------

namespace {

constexpr size_t NOALLOC_MAX_FLOATS = 384 * 1024;  // 1.5 MiB of partial sums
static __device__ __align__(256) float g_noalloc_partials[NOALLOC_MAX_FLOATS];

// In host code g_noalloc_partials is only a handle; the address kernels may
// use is looked up once per device, with that device current.
float *noalloc_partials_for_current_device(cudaError_t *err) {
  static float *ptr[64] = {};
  static std::mutex mu;
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptr[dev] == nullptr) {
    void *p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_noalloc_partials);
    if (*err != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<float *>(p);
  }
  return ptr[dev];
}

}  // namespace
}  // namespace lb

extern "C" int litnice_b200_gemv_noalloc(const float *x, int32_t m, const float *w, int32_t k, int32_t n,
                                         const float *bias, float *out, void *stream) {
  using namespace lb;
  if (x == nullptr || w == nullptr || out == nullptr || k <= 0 || n <= 0) {
    std::fprintf(stderr, "litnice_b200_gemv_noalloc: null pointer or non-positive size\n");
    return LITNICE_B200_EINVAL;
  }
  if (m != 1 && m != 2 && m != 4 && m != 8) {
    std::fprintf(stderr, "litnice_b200_gemv_noalloc: m must be 1, 2, 4 or 8 (got %d)\n", m);
    return LITNICE_B200_EINVAL;
  }
  const size_t need = gemv_scratch_floats(m, n, k);
  if (need > NOALLOC_MAX_FLOATS) {
    std::fprintf(stderr,
                 "litnice_b200_gemv_noalloc: m=%d k=%d n=%d needs %zu floats of partial sums, the built-in "
                 "array holds %zu\n", m, k, n, need, (size_t)NOALLOC_MAX_FLOATS);
    return LITNICE_B200_ETOOBIG;
  }
  cudaError_t e = cudaSuccess;
  float *partials = noalloc_partials_for_current_device(&e);
  if (partials == nullptr) {
    std::fprintf(stderr, "litnice_b200_gemv_noalloc: scratch set-up failed: %s\n", cudaGetErrorString(e));
    return LITNICE_B200_ECUDA;
  }
  try {
    // Every partial sum the reduction reads is written by the first kernel of
    // the same call, so nothing left over from an earlier call is ever used.
    launch_gemv(x, m, w, k, n, bias, out, partials, static_cast<cudaStream_t>(stream));
  } catch (const std::exception &ex) {
    std::fprintf(stderr, "litnice_b200_gemv_noalloc: %s\n", ex.what());
    return LITNICE_B200_ECUDA;
  }
  return LITNICE_B200_OK;
}
