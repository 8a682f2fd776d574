// fp32 SIMT matrix product for every GEMM shape of the plugin contract:
// gemm, gemm_ranked_matrix_rhs(_t), gemm_ranked_reduce_lhs_t, gemm_batched,
// gemm_batched_lhs_t, gemm_batched_rhs_t (litnicelm
// src/model/backend/device_backend.cpp:1096-1235). All of them are
// C[b] = A[b] * B[b] once transposition is expressed as strides, so one kernel
// takes byte-strided operands; vectorised loaders are picked when an operand is
// unit-stride along k or along its outer axis and 16-byte aligned.
//
// Tiling: BM x BN x 16 tiles in shared memory (double buffered through
// registers), 256 threads, TM x TN accumulators per thread, fp32 FMA.
#include "common.cuh"

namespace lb {

namespace {

constexpr int BK = 16;

enum LoadMode : int { LM_GENERIC = 0, LM_KVEC = 1, LM_OUTERVEC = 2 };

struct GemmArgs {
  const float *a;
  const float *b;
  float *c;
  const float *residual;
  const float *bias;
  long long a_rs, a_cs, b_rs, b_cs, c_rs, c_cs;  // element strides of logical (row, col)
  int m, n, k;
  int relu;
  int c_vec;  // C (and residual) rows are unit-stride and 16-byte aligned
  MatView av, bv, cv;  // batch axes only
};

// Tile of a logical [outer, k] operand (outer = m for A, n for B) stored in
// shared memory as dst[kk][outer]. For B the logical element (kk, col) lives at
// kk*b_rs + col*b_cs, so its "outer stride" is b_cs and its "k stride" is b_rs.
template <int BO, int NT, int MODE>
struct TileLoader {
  static constexpr int VEC_COUNT = (BO * BK / 4 + NT - 1) / NT;
  static constexpr int SCALAR_COUNT = (BO * BK + NT - 1) / NT;
  float4 v[MODE == LM_GENERIC ? 1 : VEC_COUNT];
  float s[MODE == LM_GENERIC ? SCALAR_COUNT : 1];

  __device__ __forceinline__ void load(const float *base, long long outer_stride,
                                       long long k_stride, int o0, int k0, int outer_n, int k_n,
                                       int tid) {
    if (MODE == LM_KVEC) {
#pragma unroll
      for (int i = 0; i < VEC_COUNT; ++i) {
        const int f = tid + i * NT;
        const int o = f % BO, kq = f / BO;
        float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kq < BK / 4 && o0 + o < outer_n) {
          const float *p = base + (long long)(o0 + o) * outer_stride + (k0 + kq * 4);
          const int left = k_n - (k0 + kq * 4);
          if (left >= 4) {
            r = *reinterpret_cast<const float4 *>(p);
          } else {
            if (left > 0) r.x = p[0];
            if (left > 1) r.y = p[1];
            if (left > 2) r.z = p[2];
          }
        }
        v[i] = r;
      }
    } else if (MODE == LM_OUTERVEC) {
#pragma unroll
      for (int i = 0; i < VEC_COUNT; ++i) {
        const int f = tid + i * NT;
        const int kk = f / (BO / 4), oq = f % (BO / 4);
        float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kk < BK && k0 + kk < k_n) {
          const float *p = base + (long long)(k0 + kk) * k_stride + (o0 + oq * 4);
          const int left = outer_n - (o0 + oq * 4);
          if (left >= 4) {
            r = *reinterpret_cast<const float4 *>(p);
          } else {
            if (left > 0) r.x = p[0];
            if (left > 1) r.y = p[1];
            if (left > 2) r.z = p[2];
          }
        }
        v[i] = r;
      }
    } else {
#pragma unroll
      for (int i = 0; i < SCALAR_COUNT; ++i) {
        const int e = tid + i * NT;
        const int o = e % BO, kk = e / BO;
        float r = 0.f;
        if (kk < BK && o0 + o < outer_n && k0 + kk < k_n)
          r = base[(long long)(o0 + o) * outer_stride + (long long)(k0 + kk) * k_stride];
        s[i] = r;
      }
    }
  }

  __device__ __forceinline__ void store(float (*dst)[BO], int tid) const {
    if (MODE == LM_KVEC) {
#pragma unroll
      for (int i = 0; i < VEC_COUNT; ++i) {
        const int f = tid + i * NT;
        const int o = f % BO, kq = f / BO;
        if (kq < BK / 4) {
          dst[kq * 4 + 0][o] = v[i].x;
          dst[kq * 4 + 1][o] = v[i].y;
          dst[kq * 4 + 2][o] = v[i].z;
          dst[kq * 4 + 3][o] = v[i].w;
        }
      }
    } else if (MODE == LM_OUTERVEC) {
#pragma unroll
      for (int i = 0; i < VEC_COUNT; ++i) {
        const int f = tid + i * NT;
        const int kk = f / (BO / 4), oq = f % (BO / 4);
        if (kk < BK) *reinterpret_cast<float4 *>(&dst[kk][oq * 4]) = v[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < SCALAR_COUNT; ++i) {
        const int e = tid + i * NT;
        const int o = e % BO, kk = e / BO;
        if (kk < BK) dst[kk][o] = s[i];
      }
    }
  }
};

template <int BM, int BN, int TM, int TN, int AMODE, int BMODE>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(GemmArgs g) {
  constexpr int NT = (BM / TM) * (BN / TN);
  __shared__ __align__(16) float As[2][BK][BM];
  __shared__ __align__(16) float Bs[2][BK][BN];
  pdl_launch_dependents();
  pdl_wait();

  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const long long bz = blockIdx.z;
  const float *A = reinterpret_cast<const float *>(reinterpret_cast<const char *>(g.a) +
                                                   batch_offset(g.av, bz));
  const float *B = reinterpret_cast<const float *>(reinterpret_cast<const char *>(g.b) +
                                                   batch_offset(g.bv, bz));
  const long long c_boff = batch_offset(g.cv, bz);
  float *C = reinterpret_cast<float *>(reinterpret_cast<char *>(g.c) + c_boff);
  const float *R = g.residual ? reinterpret_cast<const float *>(
                                    reinterpret_cast<const char *>(g.residual) + c_boff)
                              : nullptr;

  TileLoader<BM, NT, AMODE> la;
  TileLoader<BN, NT, BMODE> lb_;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int ktiles = (g.k + BK - 1) / BK;
  // For A the k axis is the column axis (stride a_cs); for B it is the row axis.
  la.load(A, g.a_rs, g.a_cs, m0, 0, g.m, g.k, tid);
  lb_.load(B, g.b_cs, g.b_rs, n0, 0, g.n, g.k, tid);
  la.store(As[0], tid);
  lb_.store(Bs[0], tid);
  __syncthreads();

  for (int kt = 0; kt < ktiles; ++kt) {
    const int cur = kt & 1;
    if (kt + 1 < ktiles) {
      la.load(A, g.a_rs, g.a_cs, m0, (kt + 1) * BK, g.m, g.k, tid);
      lb_.load(B, g.b_cs, g.b_rs, n0, (kt + 1) * BK, g.n, g.k, tid);
    }
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float af[TM], bf[TN];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        const int r = (TM == 8 ? (i / 4) * (BM / 2) : 0) + ty * 4;
        const float4 t = *reinterpret_cast<const float4 *>(&As[cur][kk][r]);
        af[i] = t.x; af[i + 1] = t.y; af[i + 2] = t.z; af[i + 3] = t.w;
      }
#pragma unroll
      for (int j = 0; j < TN; j += 4) {
        const int c = (TN == 8 ? (j / 4) * (BN / 2) : 0) + tx * 4;
        const float4 t = *reinterpret_cast<const float4 *>(&Bs[cur][kk][c]);
        bf[j] = t.x; bf[j + 1] = t.y; bf[j + 2] = t.z; bf[j + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(af[i], bf[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) {
      la.store(As[cur ^ 1], tid);
      lb_.store(Bs[cur ^ 1], tid);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int row = m0 + (TM == 8 ? (i / 4) * (BM / 2) : 0) + ty * 4 + (i & 3);
    if (row >= g.m) continue;
#pragma unroll
    for (int jq = 0; jq < TN; jq += 4) {
      const int col = n0 + (TN == 8 ? (jq / 4) * (BN / 2) : 0) + tx * 4;
      if (col >= g.n) continue;
      float v[4] = {acc[i][jq], acc[i][jq + 1], acc[i][jq + 2], acc[i][jq + 3]};
      if (g.c_vec && col + 3 < g.n) {
        const long long off = (long long)row * g.c_rs + col;
        if (g.bias) {
          const float4 bb = *reinterpret_cast<const float4 *>(g.bias + col);
          v[0] += bb.x; v[1] += bb.y; v[2] += bb.z; v[3] += bb.w;
        }
        if (R) {
          const float4 rr = *reinterpret_cast<const float4 *>(R + off);
          v[0] += rr.x; v[1] += rr.y; v[2] += rr.z; v[3] += rr.w;
        }
        if (g.relu) {
#pragma unroll
          for (int q = 0; q < 4; ++q) v[q] = v[q] > 0.f ? v[q] : 0.f;
        }
        *reinterpret_cast<float4 *>(C + off) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col + q >= g.n) break;
          const long long off = (long long)row * g.c_rs + (long long)(col + q) * g.c_cs;
          float o = v[q];
          if (g.bias) o += g.bias[col + q];
          if (R) o += R[off];
          if (g.relu) o = o > 0.f ? o : 0.f;
          C[off] = o;
        }
      }
    }
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool batch_aligned16(const MatView &v) {
  for (int i = 0; i < v.nb; ++i)
    if ((v.bs[i] & 15) != 0) return false;
  return true;
}

template <int BM, int BN, int TM, int TN, int AMODE, int BMODE>
void launch_cfg(const GemmArgs &g, long long batch, cudaStream_t st) {
  dim3 grid((g.n + BN - 1) / BN, (g.m + BM - 1) / BM, (unsigned)batch);
  launch_pdl(gemm_simt_kernel<BM, BN, TM, TN, AMODE, BMODE>, grid, dim3((BM / TM) * (BN / TN)), 0, st, g_pdl_enabled, g);
}

template <int AMODE, int BMODE>
void launch_tiles(const GemmArgs &g, long long batch, cudaStream_t st) {
  // Large tiles only when they still give every SM work; the 64x64 tile keeps
  // small-M (short context) products spread over the 148 SMs.
  const long long big = (long long)((g.m + 127) / 128) * ((g.n + 127) / 128) * batch;
  if (big >= 148 * 2)
    launch_cfg<128, 128, 8, 8, AMODE, BMODE>(g, batch, st);
  else
    launch_cfg<64, 64, 4, 4, AMODE, BMODE>(g, batch, st);
}

template <int AMODE>
void launch_bmode(int bmode, const GemmArgs &g, long long batch, cudaStream_t st) {
  if (bmode == LM_KVEC) launch_tiles<AMODE, LM_KVEC>(g, batch, st);
  else if (bmode == LM_OUTERVEC) launch_tiles<AMODE, LM_OUTERVEC>(g, batch, st);
  else launch_tiles<AMODE, LM_GENERIC>(g, batch, st);
}

}  // namespace

void launch_gemm_simt(const MatView &a, const MatView &bmat, const MatView &c, long long m,
                      long long n, long long k, const GemmEpilogue &ep, cudaStream_t st) {
  if (m <= 0 || n <= 0) return;
  GemmArgs g{};
  g.a = reinterpret_cast<const float *>(a.data);
  g.b = reinterpret_cast<const float *>(bmat.data);
  g.c = reinterpret_cast<float *>(c.data);
  g.residual = ep.residual;
  g.bias = ep.bias;
  g.relu = ep.relu;
  g.a_rs = a.rs / 4; g.a_cs = a.cs / 4;
  g.b_rs = bmat.rs / 4; g.b_cs = bmat.cs / 4;
  g.c_rs = c.rs / 4; g.c_cs = c.cs / 4;
  g.m = (int)m; g.n = (int)n; g.k = (int)k;
  g.av = a; g.bv = bmat; g.cv = c;
  const long long batch = c.batch;

  // A: logical [m, k]. k-vector loads need unit stride along k; outer-vector
  // loads need unit stride along m (transposed left operand).
  int amode = LM_GENERIC;
  if (g.a_cs == 1 && (g.a_rs & 3) == 0 && aligned16(a.data) && batch_aligned16(a)) amode = LM_KVEC;
  else if (g.a_rs == 1 && (g.a_cs & 3) == 0 && aligned16(a.data) && batch_aligned16(a)) amode = LM_OUTERVEC;
  // B: logical [k, n]. Unit stride along n (row-major weights) -> outer-vector;
  // unit stride along k (transposed right operand) -> k-vector.
  int bmode = LM_GENERIC;
  if (g.b_cs == 1 && (g.b_rs & 3) == 0 && aligned16(bmat.data) && batch_aligned16(bmat)) bmode = LM_OUTERVEC;
  else if (g.b_rs == 1 && (g.b_cs & 3) == 0 && aligned16(bmat.data) && batch_aligned16(bmat)) bmode = LM_KVEC;
  g.c_vec = (g.c_cs == 1 && (g.c_rs & 3) == 0 && aligned16(c.data) && batch_aligned16(c) &&
             (!ep.residual || aligned16(ep.residual)) && (!ep.bias || aligned16(ep.bias)))
                ? 1 : 0;

  if (amode == LM_KVEC) launch_bmode<LM_KVEC>(bmode, g, batch, st);
  else if (amode == LM_OUTERVEC) launch_bmode<LM_OUTERVEC>(bmode, g, batch, st);
  else launch_bmode<LM_GENERIC>(bmode, g, batch, st);
}

}  // namespace lb
