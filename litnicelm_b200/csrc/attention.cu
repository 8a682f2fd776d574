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
// (stream, head) and walks the key tiles up to the diagonal.
#include "common.cuh"
#include "gemm_tc.cuh"

namespace lb {

namespace {

constexpr int AT_BQ = 64;    // query rows per CTA
constexpr int AT_BK = 64;    // keys per tile
constexpr int AT_PLD = 68;   // row pitch of the probability tile (floats)

template <int DH>
__global__ void __launch_bounds__(256)
attention_kernel(const float *__restrict__ qkv, float *__restrict__ ctx, float *__restrict__ ctx_lo,
                 const LoopState *state, int s_cap, int d_model, float scale) {
  constexpr int CPT = DH / 16;  // output columns per thread
  extern __shared__ __align__(16) float smem[];
  float (*Qt)[AT_BQ] = reinterpret_cast<float (*)[AT_BQ]>(smem);                 // [DH][64]
  float (*Kt)[AT_BK] = reinterpret_cast<float (*)[AT_BK]>(smem + DH * AT_BQ);    // [DH][64]
  float (*Vs)[DH] = reinterpret_cast<float (*)[DH]>(smem + 2 * DH * AT_BQ);      // [64][DH]
  float (*Ps)[AT_PLD] = reinterpret_cast<float (*)[AT_PLD]>(smem + 3 * DH * AT_BQ);  // [64][68]

  const int s = state ? state->s : s_cap;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * AT_BQ;
  if (q0 >= s) return;
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
    m_run[i] = -3.402823466e+38f;
    l_run[i] = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) o[i][c] = 0.f;
  }

  for (int kt = 0; kt <= qt; ++kt) {
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
      float mx = -3.402823466e+38f;
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
void launch_dh(const float *qkv, float *ctx, float *ctx_lo, const LoopState *state, int n_streams, int s_cap,
               int n_heads, int d_model, cudaStream_t st) {
  const size_t smem = (size_t)(3 * DH * AT_BQ + AT_BQ * AT_PLD) * sizeof(float);
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    LB_CUDA(cudaFuncSetAttribute(attention_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    configured[dev] = true;
  }
  dim3 grid((s_cap + AT_BQ - 1) / AT_BQ, n_heads, n_streams);
  const float scale = 1.0f / sqrtf((float)DH);
  attention_kernel<DH><<<grid, 256, smem, st>>>(qkv, ctx, ctx_lo, state, s_cap, d_model, scale);
  LB_LAUNCH_CHECK();
}

}  // namespace

void launch_attention(const float *qkv, float *ctx, float *ctx_lo, const LoopState *state, int n_streams,
                      int s_host, int n_heads, int d_model, cudaStream_t st) {
  const int dh = d_model / n_heads;
  switch (dh) {
    case 16: launch_dh<16>(qkv, ctx, ctx_lo, state, n_streams, s_host, n_heads, d_model, st); break;
    case 32: launch_dh<32>(qkv, ctx, ctx_lo, state, n_streams, s_host, n_heads, d_model, st); break;
    case 64: launch_dh<64>(qkv, ctx, ctx_lo, state, n_streams, s_host, n_heads, d_model, st); break;
    case 128: launch_dh<128>(qkv, ctx, ctx_lo, state, n_streams, s_host, n_heads, d_model, st); break;
    default:
      throw std::invalid_argument("litnice_b200: fused attention supports head_dim 16, 32, 64, 128");
  }
}

}  // namespace lb
