// Kernels of the opt-in cached mode (LITNICE_B200_KV_CACHE=1): one new row per
// stream and step. The reference keeps no key/value cache (inference.cpp:278-284
// runs Transformer::forward over the whole context for every token), so this mode
// is an extension: the same arithmetic per row (transformer_layer.cpp:50-92,
// self_attention_fused_inplace.cpp:82-97), with the keys and values of earlier
// positions read back from HBM instead of being recomputed.
//
// Layout: kcache, vcache [n_layers][n_streams][cap][d_model] fp32, a position's
// row as the QKV projection produced it (heads side by side). The step's rows
// live in [n_streams, ...] buffers: x (residual stream), ln, qkv [.., 3 d_model],
// ctx, h [.., d_ff].
#include "common.cuh"

namespace lb {

namespace {

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// x[b, :] = tok_emb[ids[b, s-1]] + pos_emb[s-1] (transformer.cpp:91-94 for the newest row) and
// ln[b, :] = LayerNorm(x[b, :]) with the first layer's gamma / beta (device_backend.cpp:1247-1279:
// mean and biased variance in double, inv_std = 1/sqrt(float(var) + 1e-5f)). One warp per stream.
__global__ void embed_last_ln_kernel(const float *__restrict__ tok_emb, const float *__restrict__ pos_emb,
                                     const int *__restrict__ ids, int ids_ld, const LoopState *state, int s_host,
                                     int n_streams, int d, int vocab, const float *__restrict__ gamma,
                                     const float *__restrict__ beta, float *__restrict__ x, float *__restrict__ ln,
                                     DevErr *err) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = state ? state->s : s_host;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= n_streams) return;
  const int lane = threadIdx.x & 31, t = s - 1;
  int id = ids[(long long)b * ids_ld + t];
  if (id < 0 || id >= vocab) {
    if (lane == 0) {
      err->code = DEVERR_BAD_TOKEN_ID;
      err->detail = id;
    }
    id = 0;
  }
  const float *tp = tok_emb + (long long)id * d, *pp = pos_emb + (long long)t * d;
  float *xp = x + (long long)b * d;
  double sum = 0.0;
  for (int c = lane; c < d; c += 32) {
    const float v = tp[c] + pp[c];
    xp[c] = v;
    sum += (double)v;
  }
  if (ln == nullptr) return;  // the consumer normalises the row itself
  const double mean = warp_sum_d(sum) / (double)d;
  double var = 0.0;
  for (int c = lane; c < d; c += 32) {  // each lane re-reads the elements it wrote itself
    const double dd = (double)xp[c] - mean;
    var += dd * dd;
  }
  var = warp_sum_d(var) / (double)d;
  const float inv_std = 1.0f / sqrtf((float)var + 1e-5f);
  const float fmean = (float)mean;
  for (int c = lane; c < d; c += 32)
    ln[(long long)b * d + c] = __fadd_rn(__fmul_rn((xp[c] - fmean) * inv_std, gamma[c]), beta[c]);
}

// Prefill: the K and V thirds of the QKV rows of a whole-context pass, rows r = b * s + t of
// qkv [rows, 3 d], to the caches at position t of stream b.
__global__ void kv_store_kernel(const float *__restrict__ qkv, const LoopState *state, int s_host, int n_streams,
                                int d, int cap, float *__restrict__ kc, float *__restrict__ vc) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = state ? state->s : s_host;
  const long long r = blockIdx.x;
  if (r >= (long long)n_streams * s) return;
  const int b = (int)(r / s), t = (int)(r - (long long)b * s);
  const float4 *src = reinterpret_cast<const float4 *>(qkv + r * 3 * d);
  float4 *kd = reinterpret_cast<float4 *>(kc + ((long long)b * cap + t) * d);
  float4 *vd = reinterpret_cast<float4 *>(vc + ((long long)b * cap + t) * d);
  const int n4 = d >> 2;
  for (int c = threadIdx.x; c < n4; c += blockDim.x) {
    kd[c] = src[n4 + c];
    vd[c] = src[2 * n4 + c];
  }
}

// Attention of the newest row of stream b, head h, over the keys of one chunk of positions:
// scores q.k / sqrt(dh) in fp32, their maximum, e = expf(score - max), the sum of e in double
// (scaled_causal_softmax_rows, device_backend.cpp:1554-1592, restricted to one row) and
// o = sum e_j v_j. The CTA whose chunk holds the newest position first appends that position's K
// and V (this step's QKV row) to the caches. With one chunk the normalised context row is
// written directly; otherwise (o, max, sum) go to `part` and the chunk that finishes last joins them.
template <int DH>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const float *__restrict__ qkv, float *__restrict__ kc, float *__restrict__ vc, int cap,
                   int d_model, const LoopState *state, int s_host, int keys_per_chunk, float scale,
                   float *__restrict__ part, float *__restrict__ ctx, int *__restrict__ counters) {
  constexpr int LPK = DH / 8;      // lanes that share one key: 8 floats of the head each
  constexpr int KPI = 128 / LPK;   // keys per trip of the CTA
  constexpr int PARTS = 128 / DH;  // threads per output column in the second product
  extern __shared__ float sc[];    // scores, then e, of the chunk's keys
  __shared__ float red_f[4];
  __shared__ double red_d[4];
  __shared__ float o_part[128];
  __shared__ int is_last;
  pdl_launch_dependents();
  pdl_wait();
  const int s = state ? state->s : s_host;  // context length including the newest token
  const int p = s - 1;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, chunks = gridDim.x;
  const int c0 = c * keys_per_chunk, c1 = min(s, c0 + keys_per_chunk);
  float *out = part ? part + (((long long)b * gridDim.y + h) * chunks + c) * (DH + 2) : nullptr;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (c0 >= s) {  // a launch sized for a longer context: nothing in this chunk
    if (out == nullptr) return;
    if (tid == 0) {
      out[DH] = -INFINITY;
      out[DH + 1] = 0.f;
    }
  } else {
  const float *row = qkv + (long long)b * 3 * d_model;
  if (p >= c0 && p < c1 && tid < DH / 4) {
    const float4 k4 = *reinterpret_cast<const float4 *>(row + d_model + h * DH + tid * 4);
    const float4 v4 = *reinterpret_cast<const float4 *>(row + 2 * d_model + h * DH + tid * 4);
    *reinterpret_cast<float4 *>(kc + ((long long)b * cap + p) * d_model + h * DH + tid * 4) = k4;
    *reinterpret_cast<float4 *>(vc + ((long long)b * cap + p) * d_model + h * DH + tid * 4) = v4;
  }
  __syncthreads();
  const int sub = tid % LPK;
  const float4 q0 = *reinterpret_cast<const float4 *>(row + h * DH + sub * 8);
  const float4 q1 = *reinterpret_cast<const float4 *>(row + h * DH + sub * 8 + 4);
  for (int base = c0; base < c1; base += KPI) {  // uniform trip count: the shuffles need whole warps
    const int j = base + tid / LPK;
    float dot = 0.f;
    if (j < c1) {
      const float *kp = kc + ((long long)b * cap + j) * d_model + h * DH + sub * 8;
      const float4 k0 = *reinterpret_cast<const float4 *>(kp), k1 = *reinterpret_cast<const float4 *>(kp + 4);
      dot = q0.x * k0.x;
      dot = fmaf(q0.y, k0.y, dot);
      dot = fmaf(q0.z, k0.z, dot);
      dot = fmaf(q0.w, k0.w, dot);
      dot = fmaf(q1.x, k1.x, dot);
      dot = fmaf(q1.y, k1.y, dot);
      dot = fmaf(q1.z, k1.z, dot);
      dot = fmaf(q1.w, k1.w, dot);
    }
#pragma unroll
    for (int o = LPK >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (j < c1 && sub == 0) sc[j - c0] = dot * scale;
  }
  __syncthreads();
  const int nk = c1 - c0;
  float m = -INFINITY;
  for (int i = tid; i < nk; i += 128) m = fmaxf(m, sc[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red_f[wid] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red_f[0], red_f[1]), fmaxf(red_f[2], red_f[3]));
  double l = 0.0;
  for (int i = tid; i < nk; i += 128) {
    const float e = expf(sc[i] - m);
    sc[i] = e;
    l += (double)e;
  }
  l = warp_sum_d(l);
  if (lane == 0) red_d[wid] = l;
  __syncthreads();
  l = ((red_d[0] + red_d[1]) + red_d[2]) + red_d[3];
  // second product: thread -> (column d of the head, every PARTS-th key)
  const int d = tid % DH, pt = tid / DH;
  float o = 0.f;
  const float *vp = vc + ((long long)b * cap + c0) * d_model + h * DH + d;
  for (int i = pt; i < nk; i += PARTS) o = fmaf(sc[i], vp[(long long)i * d_model], o);
  o_part[tid] = o;
  __syncthreads();
  if (tid < DH) {
    float t = o_part[tid];
#pragma unroll
    for (int q = 1; q < PARTS; ++q) t += o_part[q * DH + tid];
    if (out == nullptr) {
      ctx[(long long)b * d_model + h * DH + tid] = t * (float)(1.0 / l);
    } else {
      out[tid] = t;
      if (tid == 0) {
        out[DH] = m;
        out[DH + 1] = (float)l;
      }
    }
  }
  }  // chunk with keys
  if (out == nullptr) return;
  // The chunk that finishes last joins all chunks of its (stream, head) in chunk order: the common
  // maximum, every chunk's sums rescaled to it, the context row normalised by the total. The
  // counter rests at zero between launches.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    is_last = atomicAdd(&counters[b * gridDim.y + h], 1) == chunks - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid < DH) {
    const float *pp = part + ((long long)b * gridDim.y + h) * chunks * (DH + 2);
    float mm = -INFINITY;
    for (int q = 0; q < chunks; ++q) mm = fmaxf(mm, __ldcg(&pp[q * (DH + 2) + DH]));
    double ll = 0.0;
    float oo = 0.f;
    for (int q = 0; q < chunks; ++q) {
      const float mc = __ldcg(&pp[q * (DH + 2) + DH]);
      if (mc == -INFINITY) continue;  // an empty chunk of a launch sized for a longer context
      const float w = expf(mc - mm);
      ll += (double)__ldcg(&pp[q * (DH + 2) + DH + 1]) * (double)w;
      oo = fmaf(__ldcg(&pp[q * (DH + 2) + tid]), w, oo);
    }
    ctx[(long long)b * d_model + h * DH + tid] = oo * (float)(1.0 / ll);
    if (tid == 0) counters[b * gridDim.y + h] = 0;
  }
}

}  // namespace

void launch_embed_last_ln(const float *tok_emb, const float *pos_emb, const int *ids, int ids_ld,
                          const LoopState *state, int s_host, int n_streams, int d, int vocab, const float *gamma,
                          const float *beta, float *x, float *ln, DevErr *err, cudaStream_t st) {
  const int warps = 4;
  launch_pdl(embed_last_ln_kernel, dim3((n_streams + warps - 1) / warps), dim3(warps * 32), 0, st, g_pdl_enabled,
             tok_emb, pos_emb, ids, ids_ld, state, s_host, n_streams, d, vocab, gamma, beta, x, ln, err);
}

void launch_kv_store(const float *qkv, const LoopState *state, int s_host, int n_streams, int d, int cap, float *kc,
                     float *vc, cudaStream_t st) {
  const long long rows = (long long)n_streams * s_host;
  if (rows <= 0) return;
  launch_pdl(kv_store_kernel, dim3((unsigned)rows), dim3(128), 0, st, g_pdl_enabled, qkv, state, s_host, n_streams, d,
             cap, kc, vc);
}

DecodeAttnPlan attn_decode_plan(int n_streams, int s, int n_heads, int dh) {
  DecodeAttnPlan p{};
  const long long heads = (long long)n_streams * n_heads;
  // about two CTAs per SM, chunks of 32..1024 keys
  long long want = (2 * 148 + heads - 1) / heads;
  if (want < 1) want = 1;
  int keys = (int)((s + want - 1) / want);
  keys = (keys + 31) / 32 * 32;
  if (keys < 32) keys = 32;
  if (keys > 1024) keys = 1024;
  p.keys_per_chunk = keys;
  p.chunks = (s + keys - 1) / keys;
  p.scratch_floats = p.chunks > 1 ? (size_t)heads * p.chunks * (dh + 2) : 0;
  return p;
}

template <int DH>
static void launch_attn_decode_dh(const float *qkv, float *kc, float *vc, int cap, int d_model, int n_heads,
                                  int n_streams, const LoopState *state, int s_host, const DecodeAttnPlan &plan,
                                  float *part, int *counters, float *ctx, cudaStream_t st) {
  const float scale = 1.0f / sqrtf((float)DH);
  dim3 grid((unsigned)plan.chunks, (unsigned)n_heads, (unsigned)n_streams);
  float *pp = plan.chunks > 1 ? part : nullptr;
  launch_pdl(attn_decode_kernel<DH>, grid, dim3(128), (size_t)plan.keys_per_chunk * sizeof(float), st, g_pdl_enabled,
             qkv, kc, vc, cap, d_model, state, s_host, plan.keys_per_chunk, scale, pp, ctx, counters);
}

int launch_attn_decode(const float *qkv, float *kc, float *vc, int cap, int d_model, int n_heads, int n_streams,
                       const LoopState *state, int s_host, float *part, int *counters, float *ctx, cudaStream_t st) {
  const int dh = d_model / n_heads;
  const DecodeAttnPlan plan = attn_decode_plan(n_streams, s_host, n_heads, dh);
  if (plan.chunks > 1 && (part == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: decode attention needs scratch");
  switch (dh) {
    case 16: launch_attn_decode_dh<16>(qkv, kc, vc, cap, d_model, n_heads, n_streams, state, s_host, plan, part, counters, ctx, st); break;
    case 32: launch_attn_decode_dh<32>(qkv, kc, vc, cap, d_model, n_heads, n_streams, state, s_host, plan, part, counters, ctx, st); break;
    case 64: launch_attn_decode_dh<64>(qkv, kc, vc, cap, d_model, n_heads, n_streams, state, s_host, plan, part, counters, ctx, st); break;
    case 128: launch_attn_decode_dh<128>(qkv, kc, vc, cap, d_model, n_heads, n_streams, state, s_host, plan, part, counters, ctx, st); break;
    default: throw std::invalid_argument("litnice_b200: decode attention supports head dimensions 16, 32, 64, 128");
  }
  return 1;
}

}  // namespace lb
