// Native-loop kernels around the dense activations: token + position
// embedding, and the final LayerNorm applied to the last row of every stream.
// Activations of a step are packed as rows r = stream * s + t of a dense
// [n_streams * s, d] matrix; s is read from the device-resident LoopState so a
// launch sized for an upper bound `s_cap` serves every shorter context.
#include "common.cuh"
#include "gemm_tc.cuh"

namespace lb {

namespace {

// Transformer::forward, litnicelm src/model/algo/transformer.cpp:91-94:
// X = tok_emb[ids] + pos_emb[0:s].
__global__ void embed_pos_kernel(const float *__restrict__ tok_emb,
                                 const float *__restrict__ pos_emb, const int *__restrict__ ids,
                                 int ids_ld, const LoopState *state, int n_streams, int s_cap, int d,
                                 int vocab, float *__restrict__ x, float *__restrict__ x_hi,
                                 float *__restrict__ x_lo, double2 *__restrict__ stats, TcPairF16 x_f16,
                                 DevErr *err) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = state ? state->s : s_cap;
  const long long r = blockIdx.x;
  if (r >= (long long)n_streams * s) return;
  const int b = (int)(r / s), t = (int)(r - (long long)b * s);
  int id = ids[(long long)b * ids_ld + t];
  const bool bad = id < 0 || id >= vocab;
  if (bad) {
    if (threadIdx.x == 0) {
      err->code = DEVERR_BAD_TOKEN_ID;
      err->detail = id;
    }
    id = 0;
  }
  const float4 *tp = reinterpret_cast<const float4 *>(tok_emb + (long long)id * d);
  const float4 *pp = reinterpret_cast<const float4 *>(pos_emb + (long long)t * d);
  float4 *xp = reinterpret_cast<float4 *>(x + r * d);
  const int n4 = d >> 2;
  // Uniform trip count: with `stats` the 16 lanes that share a 64-column slot
  // reduce their sums by shuffles, so every lane of a warp takes part.
  for (int c0 = 0; c0 < n4; c0 += blockDim.x) {
    const int c = c0 + threadIdx.x;
    const bool valid = c < n4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      const float4 a = tp[c], p = pp[c];
      v = make_float4(a.x + p.x, a.y + p.y, a.z + p.z, a.w + p.w);
      xp[c] = v;
      if (x_hi != nullptr) {  // TF32 pair for a tensor-core projection that reads x itself
        float4 hh, ll;
        split_tf32(v.x, hh.x, ll.x);
        split_tf32(v.y, hh.y, ll.y);
        split_tf32(v.z, hh.z, ll.z);
        split_tf32(v.w, hh.w, ll.w);
        reinterpret_cast<float4 *>(x_hi + r * d)[c] = hh;
        reinterpret_cast<float4 *>(x_lo + r * d)[c] = ll;
      }
    }
    if (x_f16.hi != nullptr)  // or the fp16 pair, one scale per block of 64 columns
      f16_store_block(v, valid, x_f16.hi + r * d + c * 4, x_f16.lo + r * d + c * 4,
                      x_f16.inv_scale + r * (d / TC_F16_SLOT) + (c >> 4));
    if (stats != nullptr) {  // (sum x, sum x^2) per slot of 64 columns, for a LayerNorm folded into that projection
      double sx = ((double)v.x + (double)v.y) + ((double)v.z + (double)v.w);
      double sxx = ((double)v.x * v.x + (double)v.y * v.y) + ((double)v.z * v.z + (double)v.w * v.w);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        sx += __shfl_xor_sync(0xffffffffu, sx, o);
        sxx += __shfl_xor_sync(0xffffffffu, sxx, o);
      }
      if (valid && (c & 15) == 0) stats[r * TC_STAT_SLOTS + (c >> 4)] = make_double2(sx, sxx);
    }
  }
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// OutputHead::forward (output_head.cpp:58-70) applies LN_f to every row, but
// the token loop reads only row s-1 of each stream (inference.cpp:109-115), so
// the final norm runs on those rows alone: out[b, :] = LN_f(x[b*s + s-1, :]).
__global__ void gather_last_ln_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                      const float *__restrict__ beta, const LoopState *state,
                                      int n_streams, int s_cap, int d, float *__restrict__ out,
                                      float *__restrict__ out_lo) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = state ? state->s : s_cap;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= n_streams) return;
  const int lane = threadIdx.x & 31;
  const float *xp = x + ((long long)b * s + (s - 1)) * d;
  double sum = 0.0;
  for (int c = lane; c < d; c += 32) sum += (double)xp[c];
  const double mean = warp_sum_d(sum) / (double)d;
  double var = 0.0;
  for (int c = lane; c < d; c += 32) {
    const double dd = (double)xp[c] - mean;
    var += dd * dd;
  }
  var = warp_sum_d(var) / (double)d;
  const float inv_std = 1.0f / sqrtf((float)var + 1e-5f);
  const float fmean = (float)mean;
  for (int c = lane; c < d; c += 32) {
    const float v = __fadd_rn(__fmul_rn((xp[c] - fmean) * inv_std, gamma[c]), beta[c]);
    if (out_lo == nullptr) {
      out[(long long)b * d + c] = v;
    } else {
      float h, l;
      split_tf32(v, h, l);
      out[(long long)b * d + c] = h;
      out_lo[(long long)b * d + c] = l;
    }
  }
}

__global__ void advance_state_kernel(LoopState *state) {
  pdl_launch_dependents();
  pdl_wait();
  state->s += 1;
  state->step += 1;
}

}  // namespace

void launch_embed_pos(const float *tok_emb, const float *pos_emb, const int *ids, int ids_ld,
                      const LoopState *state, int n_streams, int s_host, int d, int vocab,
                      float *x, DevErr *err, cudaStream_t st, float *x_hi, float *x_lo, double2 *stats,
                      const TcPairF16 *x_f16) {
  const long long rows = (long long)n_streams * s_host;
  if (rows <= 0) return;
  launch_pdl(embed_pos_kernel, dim3((unsigned)rows), dim3(d >= 512 ? 128 : 32), 0, st, g_pdl_enabled, tok_emb, pos_emb,
             ids, ids_ld, state, n_streams, s_host, d, vocab, x, x_hi, x_lo, stats, x_f16 ? *x_f16 : TcPairF16{}, err);
}

void launch_gather_last_ln(const float *x, const float *gamma, const float *beta,
                           const LoopState *state, int n_streams, int s_host, int d, float *out,
                           float *out_lo, cudaStream_t st) {
  const int warps = 4;
  launch_pdl(gather_last_ln_kernel, dim3((n_streams + warps - 1) / warps), dim3(warps * 32), 0, st, g_pdl_enabled, x,
             gamma, beta, state, n_streams, s_host, d, out, out_lo);
}

void launch_advance_state(LoopState *state, cudaStream_t st) {
  launch_pdl(advance_state_kernel, dim3(1), dim3(1), 0, st, g_pdl_enabled, state);
}

}  // namespace lb
