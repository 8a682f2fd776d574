// The tail of a greedy token step as one launch, for small vocabularies and a
// handful of streams: the final LayerNorm of each stream's last row
// (output_head.cpp:58-70 restricted to the row the loop reads), the output-head
// product with the row-major [d, vocab] weight, the first-max selection
// (inference.cpp:109-115 with a greedy config: a strict '>' scan from index 0),
// the append of the token to the stream's ids, and the advance of the
// device-side loop state. Five launches of a few microseconds each otherwise
// (norm, matrix-vector product, its split reduce, selector, advance), which at
// a vocabulary of 96 is launch latency and nothing else.
//
// One CTA per stream. The weight (d * vocab * 4 bytes, 196 KB at d 512 and
// vocabulary 96) is read by every CTA and is L2-resident after the first.
// The CTA that finishes last (a counter next to the loop state) advances the
// state, so no CTA reads a length another has already moved.
#include "common.cuh"

namespace lb {

namespace {

constexpr int HG_THREADS = 1024;  // the head product is a few L2 latencies deep only with this many loads in flight
constexpr int HG_BATCH = 8;       // weight loads a thread issues before it uses the first
constexpr int HG_WARPS = HG_THREADS / 32;

__device__ __forceinline__ double hg_block_sum(double v, double *s_red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // s_red may still be read from the previous call
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = s_red[0];
#pragma unroll
  for (int w = 1; w < HG_WARPS; ++w) t += s_red[w];
  return t;
}

__global__ void __launch_bounds__(HG_THREADS, 1)
head_greedy_kernel(const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                   const float *__restrict__ w, int d, int vocab, int s_cap, const LoopState *dstate,
                   LoopState *state, unsigned *done, int *ids, int ids_ld, int *out_tokens, int out_ld,
                   float *__restrict__ logits_out) {
  extern __shared__ __align__(16) float hg_smem[];
  __shared__ double s_red[HG_WARPS];
  __shared__ float s_val[HG_WARPS];
  __shared__ int s_idx[HG_WARPS];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int b = blockIdx.x;
  const int s = dstate ? dstate->s : s_cap;
  const int write_pos = state->s, write_step = state->step;
  float *xl = hg_smem;          // [d]
  float *red = hg_smem + d;     // [groups][vocab], then the logits [vocab]

  // final LayerNorm of row s-1, sums in double as the host code does
  const float *xp = x + ((long long)b * s + (s - 1)) * d;
  double sum = 0.0;
  for (int c = tid; c < d; c += HG_THREADS) {
    const float v = xp[c];
    xl[c] = v;
    sum += (double)v;
  }
  const double mean = hg_block_sum(sum, s_red) / (double)d;
  double var = 0.0;
  for (int c = tid; c < d; c += HG_THREADS) {
    const double dd = (double)xl[c] - mean;
    var += dd * dd;
  }
  var = hg_block_sum(var, s_red) / (double)d;
  const float inv_std = 1.0f / sqrtf((float)var + 1e-5f);
  const float fmean = (float)mean;
  for (int c = tid; c < d; c += HG_THREADS)
    xl[c] = __fadd_rn(__fmul_rn((xl[c] - fmean) * inv_std, gamma[c]), beta[c]);
  __syncthreads();

  // logits: a thread owns four consecutive columns and every groups-th k row
  const int nvec = vocab >> 2;
  const int groups = HG_THREADS / nvec;
  const int g = tid / nvec, cv = tid - g * nvec;
  float *lg = red + groups * vocab;
  if (g < groups) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 *wp = reinterpret_cast<const float4 *>(w) + cv;
    for (int k0 = g; k0 < d; k0 += groups * HG_BATCH) {
      float4 wv[HG_BATCH];
#pragma unroll
      for (int j = 0; j < HG_BATCH; ++j) {
        const int k = k0 + j * groups;
        wv[j] = k < d ? __ldg(wp + (long long)k * nvec) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < HG_BATCH; ++j) {
        const int k = k0 + j * groups;
        const float xv = k < d ? xl[k] : 0.f;
        acc.x = fmaf(xv, wv[j].x, acc.x);
        acc.y = fmaf(xv, wv[j].y, acc.y);
        acc.z = fmaf(xv, wv[j].z, acc.z);
        acc.w = fmaf(xv, wv[j].w, acc.w);
      }
    }
    *reinterpret_cast<float4 *>(red + g * vocab + cv * 4) = acc;
  }
  __syncthreads();
  for (int c = tid; c < vocab; c += HG_THREADS) {
    float v = red[c];
    for (int q = 1; q < groups; ++q) v += red[q * vocab + c];
    lg[c] = v;
    logits_out[(long long)b * vocab + c] = v;
  }
  __syncthreads();

  // lowest index holding the maximum
  float best = -3.402823466e+38f;
  int bi = 0x7fffffff;
  for (int i = tid; i < vocab; i += HG_THREADS) {
    const float v = lg[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
    }
  }
  if ((tid & 31) == 0) {
    s_val[tid >> 5] = best;
    s_idx[tid >> 5] = bi;
  }
  __syncthreads();
  if (tid == 0) {
    for (int q = 1; q < HG_WARPS; ++q)
      if (s_val[q] > best || (s_val[q] == best && s_idx[q] < bi)) {
        best = s_val[q];
        bi = s_idx[q];
      }
    if (bi == 0x7fffffff) bi = 0;  // every entry NaN or below the sentinel
    out_tokens[(long long)b * out_ld + write_step] = bi;
    ids[(long long)b * ids_ld + write_pos] = bi;
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      state->s = write_pos + 1;
      state->step = write_step + 1;
      *done = 0u;
    }
  }
}

}  // namespace

bool head_greedy_supports(int n_streams, int d, int vocab) {
  if (n_streams < 1 || n_streams > 8) return false;
  if (vocab < 4 || vocab % 4 != 0 || vocab > 1024) return false;
  return d >= 4 && d % 4 == 0 && d <= 4096;
}

void launch_head_greedy(const float *x, const float *gamma, const float *beta, const float *w, int d, int vocab,
                        int n_streams, int s_host, const LoopState *dstate, LoopState *state, unsigned *done,
                        int *ids, int ids_ld, int *out_tokens, int out_ld, float *logits, cudaStream_t st) {
  const int groups = HG_THREADS / (vocab >> 2);
  const size_t smem = ((size_t)d + (size_t)(groups + 1) * vocab) * sizeof(float);
  launch_pdl(head_greedy_kernel, dim3((unsigned)n_streams), dim3(HG_THREADS), smem, st, g_pdl_enabled, x, gamma, beta,
             w, d, vocab, s_host, dstate, state, done, ids, ids_ld, out_tokens, out_ld, logits);
}

}  // namespace lb
