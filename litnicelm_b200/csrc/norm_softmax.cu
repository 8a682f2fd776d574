// LayerNorm and row softmax kernels. Numerics follow DefaultCpuBackend in
// litnicelm's src/model/backend/device_backend.cpp: LayerNorm accumulates mean
// and biased variance in double and forms inv_std = 1/sqrt(float(var)+1e-5f)
// in float (:1247-1279); softmax takes an fp32 maximum, exp in fp32, the sum in
// double and scales by float(1/sum) (:1466-1494, causal form :1554-1592).
#include "common.cuh"
#include "gemm_tc.cuh"

namespace lb {

namespace {

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row, any strides.
__global__ void layernorm_kernel(RowView x, const char *gamma, long long gcs, const char *beta,
                                 long long bcs, RowView out) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= x.rows) return;
  const int lane = threadIdx.x & 31;
  const char *xp = x.data + row_offset(x, row);
  char *op = out.data + row_offset(out, row);
  const long long n = x.cols;
  double sum = 0.0;
  for (long long c = lane; c < n; c += 32) sum += (double)*reinterpret_cast<const float *>(xp + c * x.cs);
  const double mean = warp_sum(sum) / (double)n;
  double var = 0.0;
  for (long long c = lane; c < n; c += 32) {
    const double d = (double)*reinterpret_cast<const float *>(xp + c * x.cs) - mean;
    var += d * d;
  }
  var = warp_sum(var) / (double)n;
  const float inv_std = 1.0f / sqrtf((float)var + 1e-5f);
  const float fmean = (float)mean;
  for (long long c = lane; c < n; c += 32) {
    const float xv = *reinterpret_cast<const float *>(xp + c * x.cs);
    const float g = *reinterpret_cast<const float *>(gamma + c * gcs);
    const float b = *reinterpret_cast<const float *>(beta + c * bcs);
    const float xn = (xv - fmean) * inv_std;
    *reinterpret_cast<float *>(op + c * out.cs) = __fadd_rn(__fmul_rn(xn, g), b);
  }
}

// Dense rows of d floats (d % 4 == 0), one warp per row, float4 traffic.
__global__ void layernorm_dense_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                       const float *__restrict__ beta, long long rows, int d,
                                       float *__restrict__ out, float *__restrict__ out_lo,
                                       const LoopState *state, int n_streams) {
  pdl_launch_dependents();
  pdl_wait();
  if (state) rows = (long long)n_streams * state->s;  // launch sized for an upper bound
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float4 *xp = reinterpret_cast<const float4 *>(x + row * d);
  const int n4 = d >> 2;
  double sum = 0.0;
  for (int c = lane; c < n4; c += 32) {
    const float4 v = xp[c];
    sum += (double)v.x + (double)v.y + (double)v.z + (double)v.w;
  }
  const double mean = warp_sum(sum) / (double)d;
  double var = 0.0;
  for (int c = lane; c < n4; c += 32) {
    const float4 v = xp[c];
    const double a = v.x - mean, b = v.y - mean, cc = v.z - mean, e = v.w - mean;
    var += a * a + b * b + cc * cc + e * e;
  }
  var = warp_sum(var) / (double)d;
  const float inv_std = 1.0f / sqrtf((float)var + 1e-5f);
  const float fmean = (float)mean;
  float4 *op = reinterpret_cast<float4 *>(out + row * d);
  const float4 *gp = reinterpret_cast<const float4 *>(gamma);
  const float4 *bp = reinterpret_cast<const float4 *>(beta);
  for (int c = lane; c < n4; c += 32) {
    const float4 v = xp[c], g = gp[c], b = bp[c];
    float4 r;
    r.x = __fadd_rn(__fmul_rn((v.x - fmean) * inv_std, g.x), b.x);
    r.y = __fadd_rn(__fmul_rn((v.y - fmean) * inv_std, g.y), b.y);
    r.z = __fadd_rn(__fmul_rn((v.z - fmean) * inv_std, g.z), b.z);
    r.w = __fadd_rn(__fmul_rn((v.w - fmean) * inv_std, g.w), b.w);
    if (out_lo == nullptr) {
      op[c] = r;
    } else {  // TF32 hi/lo split for the tensor-core projection that follows
      float4 h, l;
      split_tf32(r.x, h.x, l.x);
      split_tf32(r.y, h.y, l.y);
      split_tf32(r.z, h.z, l.z);
      split_tf32(r.w, h.w, l.w);
      op[c] = h;
      reinterpret_cast<float4 *>(out_lo + row * d)[c] = l;
    }
  }
}

// One block per row. causal != 0: row r keeps columns c <= r % cols, scores are
// multiplied by `scale` first, and the other columns receive 0.
__global__ void softmax_rows_kernel(RowView x, RowView out, int causal, float scale) {
  __shared__ float s_max[32];
  __shared__ double s_sum[32];
  const long long row = blockIdx.x;
  const long long n = x.cols;
  const long long last = causal ? (row % n) : (n - 1);
  const char *xp = x.data + row_offset(x, row);
  char *op = out.data + row_offset(out, row);
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;

  float mx = -3.402823466e+38f;
  for (long long c = tid; c <= last; c += blockDim.x) {
    float v = *reinterpret_cast<const float *>(xp + c * x.cs);
    if (causal) v = __fmul_rn(v, scale);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[wid] = mx;
  __syncthreads();
  mx = s_max[0];
  for (int w = 1; w < nw; ++w) mx = fmaxf(mx, s_max[w]);

  double sum = 0.0;
  for (long long c = tid; c < n; c += blockDim.x) {
    float e = 0.0f;
    if (c <= last) {
      float v = *reinterpret_cast<const float *>(xp + c * x.cs);
      if (causal) v = __fmul_rn(v, scale);
      e = expf(__fsub_rn(v, mx));
      sum += (double)e;
    }
    *reinterpret_cast<float *>(op + c * out.cs) = e;
  }
  sum = warp_sum(sum);
  if (lane == 0) s_sum[wid] = sum;
  __syncthreads();
  double tot = 0.0;
  for (int w = 0; w < nw; ++w) tot += s_sum[w];
  const float inv = (float)(1.0 / tot);
  for (long long c = tid; c <= last; c += blockDim.x) {
    float *p = reinterpret_cast<float *>(op + c * out.cs);
    *p = *p * inv;
  }
}

}  // namespace

void launch_layernorm(const RowView &x, const float *gamma, long long gamma_cs, const float *beta,
                      long long beta_cs, const RowView &out, cudaStream_t st) {
  if (x.rows <= 0) return;
  const int warps = 4;
  const long long blocks = (x.rows + warps - 1) / warps;
  layernorm_kernel<<<(unsigned)blocks, warps * 32, 0, st>>>(
      x, reinterpret_cast<const char *>(gamma), gamma_cs, reinterpret_cast<const char *>(beta),
      beta_cs, out);
  LB_LAUNCH_CHECK();
}

void launch_layernorm_dense(const float *x, const float *gamma, const float *beta, long long rows,
                            int d, float *out, float *out_lo, const LoopState *state, int n_streams,
                            cudaStream_t st) {
  if (rows <= 0) return;
  const int warps = 4;
  const long long blocks = (rows + warps - 1) / warps;
  launch_pdl(layernorm_dense_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, st, g_pdl_enabled, x, gamma, beta, rows,
             d, out, out_lo, state, n_streams);
}

void launch_softmax_rows(const RowView &x, const RowView &out, int causal, float scale,
                         cudaStream_t st) {
  if (x.rows <= 0) return;
  const int threads = x.cols >= 512 ? 256 : (x.cols >= 128 ? 128 : 32);
  softmax_rows_kernel<<<(unsigned)x.rows, threads, 0, st>>>(x, out, causal, scale);
  LB_LAUNCH_CHECK();
}

}  // namespace lb
