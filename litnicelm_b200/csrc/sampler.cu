// Fused token selector: logit scaling, top-k, top-p, seeded draw and token
// write in one kernel, one CTA per stream, so no logits return to the host.
//
// Restates select_next_token_greedy / select_next_token_sampled of litnicelm's
// src/model/inference.cpp:188-263:
//   * temp <= 0 or top_k == 1: first index of the maximum (strict '>').
//   * otherwise: candidates ordered by double(logit)/temp descending, the first
//     top_k kept (when 0 < top_k < V), then the shortest prefix whose cumulative
//     probability reaches top_p (inclusive, at least one) when top_p < 1, then
//     one draw from std::discrete_distribution over exp(x - max) in double.
// The draw follows libstdc++ (GCC 13): weights divided by their sequential sum,
// running sums with the last forced to 1.0, a canonical double made of two
// 32-bit outputs of std::mt19937 (low word first), and lower_bound. With fewer
// than two candidates nothing is drawn. Sums that the host code evaluates
// sequentially are evaluated sequentially here (one thread), because their
// rounding decides the top-p cut. Candidates with exactly equal logits are
// ordered by ascending id (std::sort leaves that order unspecified).
#include "common.cuh"

namespace lb {

namespace {

constexpr int SM_CAP = 2048;     // candidates sorted in shared memory
constexpr int SM_THREADS = 256;
constexpr int MT_N = 624;

__device__ __forceinline__ unsigned order_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending with the float
}
__device__ __forceinline__ float key_to_float(unsigned k) {
  const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}
// Smaller composite = better candidate: larger logit first, then smaller id.
__device__ __forceinline__ unsigned long long composite(float x, int id) {
  return ((unsigned long long)(~order_key(x)) << 32) | (unsigned)id;
}

struct MtState {
  unsigned mt[MT_N];
  int idx;
};

__device__ unsigned mt_next(MtState *g) {
  if (g->idx >= MT_N) {
    for (int i = 0; i < MT_N; ++i) {
      const unsigned y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % MT_N] & 0x7fffffffu);
      g->mt[i] = g->mt[(i + 397) % MT_N] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    g->idx = 0;
  }
  unsigned y = g->mt[g->idx++];
  y ^= y >> 11;
  y ^= (y << 7) & 0x9d2c5680u;
  y ^= (y << 15) & 0xefc60000u;
  y ^= y >> 18;
  return y;
}

// Ascending bitonic sort of n (power of two) 64-bit keys by the whole block.
__device__ void bitonic_sort(unsigned long long *a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int p = i ^ j;
        if (p > i) {
          const bool up = (i & k) == 0;
          const unsigned long long x = a[i], y = a[p];
          if ((x > y) == up) {
            a[i] = y;
            a[p] = x;
          }
        }
      }
    }
  }
  __syncthreads();
}

__device__ int block_argmax_first(const float *row, int v, float *s_val, int *s_idx) {
  float best = -3.402823466e+38f;
  int bi = 0x7fffffff;
  // The host loop starts from row[0] and moves only on a strict '>', i.e. it
  // returns the lowest index holding the maximum.
  for (int i = threadIdx.x; i < v; i += blockDim.x) {
    const float x = row[i];
    if (x > best || (x == best && i < bi)) {
      best = x;
      bi = i;
    }
  }
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    s_val[wid] = best;
    s_idx[wid] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < bi)) {
        best = s_val[w];
        bi = s_idx[w];
      }
    if (bi == 0x7fffffff) bi = 0;  // every entry NaN or -inf below the sentinel
    s_idx[0] = bi;
  }
  __syncthreads();
  return s_idx[0];
}

// Selects the `want` smallest composites of a row into dst (any order) by an
// 8-pass radix select over 64-bit keys; composites are distinct (ids differ).
__device__ void select_smallest(const float *row, int v, int want, unsigned long long *dst,
                                unsigned *hist, unsigned long long *s_prefix, int *s_count) {
  unsigned long long prefix = 0, mask = 0;
  int remaining = want;
  for (int pass = 7; pass >= 0; --pass) {
    const int shift = pass * 8;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < v; i += blockDim.x) {
      const unsigned long long c = composite(row[i], i);
      if ((c & mask) == prefix) atomicAdd(&hist[(unsigned)(c >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, bin = 0;
      for (; bin < 256; ++bin) {
        if (acc + (int)hist[bin] >= remaining) break;
        acc += (int)hist[bin];
      }
      *s_prefix = prefix | ((unsigned long long)bin << shift);
      *s_count = remaining - acc;
    }
    __syncthreads();
    prefix = *s_prefix;
    remaining = *s_count;
    mask |= 255ull << shift;
    __syncthreads();
  }
  // prefix is now the want-th smallest composite.
  if (threadIdx.x == 0) *s_count = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < v; i += blockDim.x) {
    const unsigned long long c = composite(row[i], i);
    if (c <= prefix) {
      const int pos = atomicAdd(s_count, 1);
      if (pos < want) dst[pos] = c;
    }
  }
  __syncthreads();
}

// One CTA per row. mode_loop != 0: the token-loop form (writes the token into
// ids[row][s] and out_tokens[row][step]); otherwise `draws` draws per row into
// out[row][0..draws).
__global__ void __launch_bounds__(SM_THREADS)
sampler_kernel(const float *__restrict__ logits, int vocab, SamplerParams sp,
               unsigned *__restrict__ mt_state, int draws, int *ids, int ids_ld, int *out,
               int out_ld, const LoopState *state, unsigned long long *scratch_keys,
               double *scratch_w, int scratch_pow2) {
  __shared__ unsigned long long s_keys[SM_CAP];
  __shared__ double s_w[SM_CAP];
  __shared__ MtState s_mt;
  __shared__ unsigned s_hist[256];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned long long s_prefix;
  __shared__ int s_count, s_keep, s_token;
  pdl_launch_dependents();
  pdl_wait();

  const int row = blockIdx.x;
  const float *lr = logits + (long long)row * vocab;
  const bool greedy = sp.temp <= 0.0f || sp.top_k == 1u;

  int out_col0 = 0;
  if (state) out_col0 = state->step;

  if (greedy) {
    const int tok = block_argmax_first(lr, vocab, s_val, s_idx);
    if (threadIdx.x == 0) {
      for (int d = 0; d < draws; ++d) out[(long long)row * out_ld + out_col0 + d] = tok;
      if (state) ids[(long long)row * ids_ld + state->s] = tok;
    }
    return;
  }

  // candidate set, sorted: keys[0..n_c)
  const int n_c = (sp.top_k > 0u && sp.top_k < (unsigned)vocab) ? (int)sp.top_k : vocab;
  unsigned long long *keys;
  double *w;
  if (vocab <= SM_CAP) {
    int p2 = 1;
    while (p2 < vocab) p2 <<= 1;
    for (int i = threadIdx.x; i < p2; i += blockDim.x)
      s_keys[i] = i < vocab ? composite(lr[i], i) : ~0ull;
    bitonic_sort(s_keys, p2);
    keys = s_keys;
    w = s_w;
  } else if (n_c <= SM_CAP) {
    select_smallest(lr, vocab, n_c, s_keys, s_hist, &s_prefix, &s_count);
    int p2 = 1;
    while (p2 < n_c) p2 <<= 1;
    for (int i = n_c + threadIdx.x; i < p2; i += blockDim.x) s_keys[i] = ~0ull;
    bitonic_sort(s_keys, p2);
    keys = s_keys;
    w = s_w;
  } else {
    keys = scratch_keys + (long long)row * scratch_pow2;
    w = scratch_w + (long long)row * scratch_pow2;
    for (int i = threadIdx.x; i < scratch_pow2; i += blockDim.x)
      keys[i] = i < vocab ? composite(lr[i], i) : ~0ull;
    bitonic_sort(keys, scratch_pow2);
  }

  // generator state of this row
  unsigned *gm = mt_state + (long long)row * (MT_N + 1);
  for (int i = threadIdx.x; i < MT_N; i += blockDim.x) s_mt.mt[i] = gm[i];
  if (threadIdx.x == 0) s_mt.idx = (int)gm[MT_N];

  const double inv_temp = 1.0 / (double)sp.temp;
  const double mx = (double)key_to_float(~(unsigned)(keys[0] >> 32)) * inv_temp;
  for (int i = threadIdx.x; i < n_c; i += blockDim.x) {
    const double x = (double)key_to_float(~(unsigned)(keys[i] >> 32)) * inv_temp;
    w[i] = exp(x - mx);
  }
  __syncthreads();

  if (threadIdx.x == 0) {
    int keep = n_c;
    if (sp.top_p < 1.0f) {
      double sum = 0.0;
      for (int i = 0; i < n_c; ++i) sum += w[i];
      double cum = 0.0;
      int kp = 0;
      for (; kp < n_c; ++kp) {
        cum += w[kp] / sum;
        if (cum >= (double)sp.top_p) {
          ++kp;
          break;
        }
      }
      keep = kp < 1 ? 1 : kp;
    }
    s_keep = keep;
    // discrete_distribution over w[0..keep): normalise, running sums, last = 1
    if (keep >= 2) {
      double sum = 0.0;
      for (int i = 0; i < keep; ++i) sum += w[i];
      double run = 0.0;
      for (int i = 0; i < keep; ++i) {
        run += w[i] / sum;
        w[i] = run;
      }
      w[keep - 1] = 1.0;
    }
    for (int d = 0; d < draws; ++d) {
      int pick = 0;
      if (keep >= 2) {
        const double lo = (double)mt_next(&s_mt);
        const double hi = (double)mt_next(&s_mt);
        double p = (lo + hi * 4294967296.0) / 18446744073709551616.0;
        if (p >= 1.0) p = 0.99999999999999988897769753748;  // nextafter(1.0, 0.0)
        int a = 0, b = keep;
        while (a < b) {
          const int m = a + ((b - a) >> 1);
          if (w[m] < p) a = m + 1; else b = m;
        }
        pick = a;
      }
      const int tok = (int)(unsigned)(keys[pick] & 0xffffffffull);
      out[(long long)row * out_ld + out_col0 + d] = tok;
      s_token = tok;
    }
    if (state) ids[(long long)row * ids_ld + state->s] = s_token;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < MT_N; i += blockDim.x) gm[i] = s_mt.mt[i];
  if (threadIdx.x == 0) gm[MT_N] = (unsigned)s_mt.idx;
}

// std::mersenne_twister_engine::seed(value) for std::mt19937.
__global__ void mt_seed_kernel(unsigned *mt_state, const unsigned *seeds, int n) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  unsigned *g = mt_state + (long long)r * (MT_N + 1);
  unsigned prev = seeds ? seeds[r] : 12345u;
  g[0] = prev;
  for (int i = 1; i < MT_N; ++i) {
    prev = 1812433253u * (prev ^ (prev >> 30)) + (unsigned)i;
    g[i] = prev;
  }
  g[MT_N] = MT_N;
}

// inspect_distribution (inference.cpp:305-322): probabilities of one row with
// exp and the sum in double.
__global__ void softmax_probs_f64_kernel(const float *__restrict__ logits, int vocab,
                                         float *__restrict__ probs) {
  __shared__ float s_max[32];
  __shared__ double s_sum[32];
  const float *lr = logits + (long long)blockIdx.x * vocab;
  float *pr = probs + (long long)blockIdx.x * vocab;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float mx = -3.402823466e+38f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, lr[i]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[wid] = mx;
  __syncthreads();
  mx = s_max[0];
  for (int q = 1; q < nw; ++q) mx = fmaxf(mx, s_max[q]);
  double sum = 0.0;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += exp((double)(lr[i] - mx));
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) s_sum[wid] = sum;
  __syncthreads();
  double tot = 0.0;
  for (int q = 0; q < nw; ++q) tot += s_sum[q];
  for (int i = threadIdx.x; i < vocab; i += blockDim.x)
    pr[i] = (float)(exp((double)(lr[i] - mx)) / tot);
}

int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

// Bytes of global scratch per row for the path that sorts the whole vocabulary
// (top_k == 0 or top_k > 2048 with a vocabulary above 2048).
size_t sampler_scratch_bytes(int vocab) {
  if (vocab <= SM_CAP) return 0;
  return (size_t)pow2_at_least(vocab) * (sizeof(unsigned long long) + sizeof(double));
}

static void run_sampler(const float *logits, int vocab, int n_rows, const SamplerParams &sp,
                        unsigned *mt_state, int draws, int *ids, int ids_ld, int *out, int out_ld,
                        const LoopState *state, void *scratch, cudaStream_t st) {
  if (n_rows <= 0) return;
  const bool greedy = sp.temp <= 0.0f || sp.top_k == 1u;
  const int n_c = (sp.top_k > 0u && sp.top_k < (unsigned)vocab) ? (int)sp.top_k : vocab;
  const int p2 = pow2_at_least(vocab);
  unsigned long long *sk = nullptr;
  double *sw = nullptr;
  if (!greedy && vocab > SM_CAP && n_c > SM_CAP) {
    if (scratch == nullptr)
      throw std::invalid_argument("litnice_b200 sampler: scratch required for a full-vocabulary sort");
    sk = static_cast<unsigned long long *>(scratch);
    sw = reinterpret_cast<double *>(sk + (size_t)n_rows * p2);
  }
  launch_pdl(sampler_kernel, dim3(n_rows), dim3(SM_THREADS), 0, st, g_pdl_enabled, logits, vocab, sp, mt_state, draws, ids,
             ids_ld, out, out_ld, state, sk, sw, p2);
}

void launch_sampler(const float *logits, int vocab, int n_streams, const SamplerParams &sp,
                    unsigned *mt_state, int *ids, int ids_ld, int *out_tokens, int out_ld,
                    LoopState *state, void *scratch, cudaStream_t st) {
  run_sampler(logits, vocab, n_streams, sp, mt_state, 1, ids, ids_ld, out_tokens, out_ld, state,
              scratch, st);
}

void launch_sampler_rows(const float *logits, int vocab, int n_rows, const SamplerParams &sp,
                         unsigned *mt_state, int draws, int *out, void *scratch, cudaStream_t st) {
  run_sampler(logits, vocab, n_rows, sp, mt_state, draws, nullptr, 0, out, draws, nullptr, scratch, st);
}

void launch_mt_seed(unsigned *mt_state, const unsigned *seeds, int n, cudaStream_t st) {
  if (n <= 0) return;
  mt_seed_kernel<<<(n + 63) / 64, 64, 0, st>>>(mt_state, seeds, n);
  LB_LAUNCH_CHECK();
}

void launch_softmax_probs_f64(const float *logits, int vocab, int n_rows, float *probs,
                              cudaStream_t st) {
  if (n_rows <= 0) return;
  softmax_probs_f64_kernel<<<n_rows, 256, 0, st>>>(logits, vocab, probs);
  LB_LAUNCH_CHECK();
}

}  // namespace lb
