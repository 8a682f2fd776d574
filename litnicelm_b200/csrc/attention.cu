// Fused causal self-attention for the native token loop (fp32 SIMT version).
//
// Computes, per stream b and head h, ctx = softmax(mask(Q K^T / sqrt(dh))) V
// without materialising the [s, s] score matrix: the maths of litnicelm's
// src/model/algo/self_attention_fused_inplace.cpp:82-94 (gemm_batched_rhs_t,
// scaled_causal_softmax_rows, gemm_batched) restated as one pass with a
// running maximum and running sum per query row. Scores are multiplied by the
// scale in fp32 before the maximum is taken, as device_backend.cpp:1561-1577.
//
// Layout: qkv is the dense [n_streams*s, 3*d] output of the QKV projection
// (columns [0,d) Q, [d,2d) K, [2d,3d) V; head h owns columns h*dh..), ctx is
// dense [n_streams*s, d]. One CTA of 256 threads handles 64 query rows of one
// (stream, head).
//
// Causal work is triangular: query tile t needs key tiles 0..t. When streams x
// heads x tiles alone cannot fill the GPU (one short stream), a query tile's
// key range is cut into chunks of `kc` tiles handled by separate CTAs. Each CTA
// leaves its unnormalised partial output with its running maximum and sum in
// scratch; the CTA that finishes last for a query tile (atomic counter) merges
// the partials in chunk order, so the result does not depend on scheduling.
#include "common.cuh"
#include "gemm_tc.cuh"

namespace lb {

namespace {

constexpr int AT_BQ = 64;    // query rows per CTA
constexpr int AT_BK = 64;    // keys per tile
constexpr int AT_PLD = 68;   // row pitch of the probability tile (floats)
constexpr float AT_NEG = -3.402823466e+38f;

__host__ __device__ inline int chunks_of(int qt, int kc) { return (qt + kc) / kc; }  // ceil((qt+1)/kc)

template <int DH>
__global__ void __launch_bounds__(256)
attention_kernel(const float *__restrict__ qkv, float *__restrict__ ctx, float *__restrict__ ctx_lo, int s_cap,
                 int d_model, float scale, int kc, float *__restrict__ part, int *__restrict__ counters,
                 const LoopState *state) {
  constexpr int CPT = DH / 16;  // output columns per thread
  constexpr int PART = AT_BQ * (DH + 2);  // floats of one partial: o[64][DH], m[64], l[64]
  extern __shared__ __align__(16) float smem[];
  float (*Qt)[AT_BQ] = reinterpret_cast<float (*)[AT_BQ]>(smem);                 // [DH][64]
  float (*Kt)[AT_BK] = reinterpret_cast<float (*)[AT_BK]>(smem + DH * AT_BQ);    // [DH][64]
  float (*Vs)[DH] = reinterpret_cast<float (*)[DH]>(smem + 2 * DH * AT_BQ);      // [64][DH]
  float (*Ps)[AT_PLD] = reinterpret_cast<float (*)[AT_PLD]>(smem + 3 * DH * AT_BQ);  // [64][68]
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();

  // The grid is laid out for s_cap; the actual length shares its tile count.
  const int s = state ? state->s : s_cap;
  // blockIdx.x enumerates (query tile, chunk) pairs, longest query tiles first.
  const int tiles = (s_cap + AT_BQ - 1) / AT_BQ;
  int idx = blockIdx.x, qt = tiles - 1;
  for (; qt > 0; --qt) {
    const int nc = chunks_of(qt, kc);
    if (idx < nc) break;
    idx -= nc;
  }
  const int chunk = idx, nchunks = chunks_of(qt, kc);
  const int kt_begin = chunk * kc, kt_end = min(qt + 1, kt_begin + kc);
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * AT_BQ;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long ld = 3LL * d_model;
  const float *base = qkv + (long long)b * s * ld + (long long)h * DH;

  // Q tile -> Qt[d][row] (transposed so that the score loop reads float4s).
  for (int f = tid; f < AT_BQ * DH / 4; f += 256) {
    const int row = f % AT_BQ, dq = f / AT_BQ;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + row < s) v = *reinterpret_cast<const float4 *>(base + (long long)(q0 + row) * ld + dq * 4);
    Qt[dq * 4 + 0][row] = v.x;
    Qt[dq * 4 + 1][row] = v.y;
    Qt[dq * 4 + 2][row] = v.z;
    Qt[dq * 4 + 3][row] = v.w;
  }

  float o[4][CPT];
  float m_run[4], l_run[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = AT_NEG;
    l_run[i] = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) o[i][c] = 0.f;
  }

  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int k0 = kt * AT_BK;
    __syncthreads();  // previous tile fully consumed (and Qt written, first time)
    for (int f = tid; f < AT_BK * DH / 4; f += 256) {
      const int row = f % AT_BK, dq = f / AT_BK;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k0 + row < s)
        v = *reinterpret_cast<const float4 *>(base + d_model + (long long)(k0 + row) * ld + dq * 4);
      Kt[dq * 4 + 0][row] = v.x;
      Kt[dq * 4 + 1][row] = v.y;
      Kt[dq * 4 + 2][row] = v.z;
      Kt[dq * 4 + 3][row] = v.w;
    }
    for (int f = tid; f < AT_BK * DH / 4; f += 256) {
      const int row = f / (DH / 4), dq = f % (DH / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k0 + row < s)
        v = *reinterpret_cast<const float4 *>(base + 2 * d_model + (long long)(k0 + row) * ld + dq * 4);
      *reinterpret_cast<float4 *>(&Vs[row][dq * 4]) = v;
    }
    __syncthreads();

    // scores for rows ty*4+i, keys tx*4+j
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll 8
    for (int d = 0; d < DH; ++d) {
      const float4 q4 = *reinterpret_cast<const float4 *>(&Qt[d][ty * 4]);
      const float4 k4 = *reinterpret_cast<const float4 *>(&Kt[d][tx * 4]);
      const float qa[4] = {q4.x, q4.y, q4.z, q4.w};
      const float ka[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[i][j] = fmaf(qa[i], ka[j], sc[i][j]);
    }

    // running softmax per query row; the 16 threads sharing ty hold one row
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = q0 + ty * 4 + i;
      float mx = AT_NEG;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = k0 + tx * 4 + j;
        sc[i][j] = __fmul_rn(sc[i][j], scale);
        if (kj <= qi) mx = fmaxf(mx, sc[i][j]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[i], mx);
      float psum = 0.f;
      float p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = k0 + tx * 4 + j;
        p[j] = kj <= qi ? expf(sc[i][j] - m_new) : 0.f;
        psum += p[j];
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
      const float alpha = expf(m_run[i] - m_new);
      l_run[i] = l_run[i] * alpha + psum;
      m_run[i] = m_new;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[i][c] *= alpha;
      *reinterpret_cast<float4 *>(&Ps[ty * 4 + i][tx * 4]) = make_float4(p[0], p[1], p[2], p[3]);
    }
    __syncthreads();

    // o[row][tx*CPT + c] += sum_j P[row][j] * V[j][tx*CPT + c]
#pragma unroll 4
    for (int j4 = 0; j4 < AT_BK / 4; ++j4) {
      float pr[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 t = *reinterpret_cast<const float4 *>(&Ps[ty * 4 + i][j4 * 4]);
        pr[i][0] = t.x; pr[i][1] = t.y; pr[i][2] = t.z; pr[i][3] = t.w;
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float vv[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) vv[c] = Vs[j4 * 4 + jj][tx * CPT + c];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < CPT; ++c) o[i][c] = fmaf(pr[i][jj], vv[c], o[i][c]);
      }
    }
  }

  if (nchunks > 1) {
    // Leave this chunk's partial in scratch; the last CTA of the query tile merges.
    const long long bh = (long long)b * gridDim.y + h;
    const long long first_item = bh * gridDim.x + (blockIdx.x - chunk);
    float *mine = part + (first_item + chunk) * PART;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
#pragma unroll
      for (int c = 0; c < CPT; ++c) mine[r * DH + tx * CPT + c] = o[i][c];
      if (tx == 0) {
        mine[AT_BQ * DH + r] = m_run[i];
        mine[AT_BQ * DH + AT_BQ + r] = l_run[i];
      }
    }
    __threadfence();
    __syncthreads();
    int *counter = counters + bh * tiles + qt;
    if (tid == 0) {
      const int prev = atomicAdd(counter, 1);
      s_last = (prev == nchunks - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *counter = 0;  // ready for the next launch
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
      float mm = AT_NEG;
      for (int j = 0; j < nchunks; ++j)
        mm = fmaxf(mm, __ldcg(part + (first_item + j) * PART + AT_BQ * DH + r));
      float ll = 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[i][c] = 0.f;
      for (int j = 0; j < nchunks; ++j) {
        const float *pj = part + (first_item + j) * PART;
        const float w = expf(__ldcg(pj + AT_BQ * DH + r) - mm);
        ll += __ldcg(pj + AT_BQ * DH + AT_BQ + r) * w;
#pragma unroll
        for (int c = 0; c < CPT; ++c) o[i][c] = fmaf(__ldcg(pj + r * DH + tx * CPT + c), w, o[i][c]);
      }
      l_run[i] = ll;
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= s) continue;
    const float inv = 1.0f / l_run[i];
    const long long off = ((long long)b * s + qi) * d_model + h * DH + tx * CPT;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const float v = o[i][c] * inv;
      if (ctx_lo == nullptr) {
        ctx[off + c] = v;
      } else {
        float hh, ll;
        split_tf32(v, hh, ll);
        ctx[off + c] = hh;
        ctx_lo[off + c] = ll;
      }
    }
  }
}

template <int DH>
void launch_dh(const float *qkv, float *ctx, float *ctx_lo, int n_streams, int s, int n_heads, int d_model,
               const AttentionPlan &plan, float *scratch, int *counters, const LoopState *state, cudaStream_t st) {
  const size_t smem = (size_t)(3 * DH * AT_BQ + AT_BQ * AT_PLD) * sizeof(float);
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    LB_CUDA(cudaFuncSetAttribute(attention_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    configured[dev] = true;
  }
  dim3 grid(plan.ctas_per_head, n_heads, n_streams);
  const float scale = 1.0f / sqrtf((float)DH);
  launch_pdl(attention_kernel<DH>, grid, dim3(256), smem, st, g_pdl_enabled, qkv, ctx, ctx_lo, s, d_model, scale, plan.kc,
             scratch, counters, state);
}

}  // namespace

AttentionPlan attention_plan(int n_streams, int s, int n_heads, int dh) {
  AttentionPlan p{};
  const int tiles = (s + AT_BQ - 1) / AT_BQ;
  const long long bh = (long long)n_streams * n_heads;
  const long long units = bh * tiles * (tiles + 1) / 2;  // (query tile, key tile) pairs
  // No split when the unsplit grid already gives every SM two CTAs; otherwise
  // aim at about two CTAs per SM of equal length.
  int kc = tiles;
  if (bh * tiles < 2 * 148) {
    long long per_cta = (units + 2 * 148 - 1) / (2 * 148);
    if (per_cta < 1) per_cta = 1;
    if (per_cta < tiles) kc = (int)per_cta;
  }
  p.kc = kc;
  int ctas = 0;
  bool split = false;
  for (int qt = 0; qt < tiles; ++qt) {
    ctas += chunks_of(qt, kc);
    split = split || chunks_of(qt, kc) > 1;
  }
  p.ctas_per_head = ctas;
  p.scratch_floats = split ? (size_t)bh * ctas * AT_BQ * (dh + 2) : 0;
  p.counters = split ? (size_t)bh * tiles : 0;
  return p;
}

void launch_attention(const float *qkv, float *ctx, float *ctx_lo, int n_streams, int s, int n_heads, int d_model,
                      float *scratch, int *counters, const LoopState *state, cudaStream_t st) {
  const int dh = d_model / n_heads;
  const AttentionPlan plan = attention_plan(n_streams, s, n_heads, dh);
  if (plan.scratch_floats > 0 && (scratch == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: attention needs scratch for this shape");
  switch (dh) {
    case 16: launch_dh<16>(qkv, ctx, ctx_lo, n_streams, s, n_heads, d_model, plan, scratch, counters, state, st); break;
    case 32: launch_dh<32>(qkv, ctx, ctx_lo, n_streams, s, n_heads, d_model, plan, scratch, counters, state, st); break;
    case 64: launch_dh<64>(qkv, ctx, ctx_lo, n_streams, s, n_heads, d_model, plan, scratch, counters, state, st); break;
    case 128: launch_dh<128>(qkv, ctx, ctx_lo, n_streams, s, n_heads, d_model, plan, scratch, counters, state, st); break;
    default:
      throw std::invalid_argument("litnice_b200: fused attention supports head_dim 16, 32, 64, 128");
  }
}

}  // namespace lb
