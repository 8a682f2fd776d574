// Shared tail of the tensor-core projection kernels: what the drain warps do
// once a thread holds CW accumulated columns of one row of the 128 x BN tile.
#pragma once

#include "gemm_tc.cuh"

namespace lb {

// acc: this thread's columns [col0, col0 + CW) of tile row rl. finish: false when
// the pipeline gave up (nothing is stored then, barriers are still joined).
// t2: index of the thread among the DRAIN_THREADS epilogue threads, which share
// named barrier 1; leader: the one thread that counts split-k arrivals. stage:
// shared memory for a 128 x (BN + 4) float tile that nothing else uses any more.
// ln_st: (mean, 1/std) of this thread's row when ep.ln_u is set; row_stats: 128
// float2 of shared memory through which the store phase learns them.
template <int BN, int CW, int DRAIN_THREADS>
__device__ __forceinline__ void tc_finish_tile(float (&acc)[CW], bool finish, const TcEpilogue &ep, int m, int n, int m0,
                                               int n0, int col0, int rl, int t2, bool leader, int splits,
                                               float *__restrict__ part, int *__restrict__ counters,
                                               volatile int *last_flag, float *stage, float2 ln_st,
                                               float2 *row_stats) {
  const int row = m0 + rl;
  finish = __all_sync(0xffffffffu, finish);  // whole warps store or skip together (the stores shuffle)
  if (splits > 1) {
    // Split-k: leave the partial tile in scratch; the CTA that arrives last at
    // the tile's counter adds all partials in split order and stores C.
    // Partial tiles are laid out [column / 4][row][4] so that the 32 rows of a
    // warp are contiguous (a row-major tile would cost 32 lines per access).
    const long long tile = (long long)blockIdx.y * gridDim.x + blockIdx.x;
    float4 *mine = reinterpret_cast<float4 *>(part + (tile * splits + blockIdx.z) * TC_BM * BN) +
                   (col0 / 4) * TC_BM + rl;
#pragma unroll
    for (int j = 0; j < CW; j += 4) mine[(j / 4) * TC_BM] = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(DRAIN_THREADS) : "memory");
    if (leader) {
      const int prev = atomicAdd(counters + tile, 1);
      const int last = (prev == splits - 1) ? 1 : 0;
      if (last) counters[tile] = 0;  // ready for the next launch
      *last_flag = last;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DRAIN_THREADS) : "memory");
    finish = finish && (*last_flag != 0);
    if (finish) {
      __threadfence();
#pragma unroll
      for (int j = 0; j < CW; ++j) acc[j] = 0.f;
      // Two partials per step (narrow tiles) with every load issued before the first add (the
      // reduction is a chain of L2 round trips otherwise); added in split order.
      constexpr int ZU = BN == 64 ? 2 : 1;  // wider tiles have no registers to spare
      for (int z = 0; z < splits; z += ZU) {
        const float4 *p0 = reinterpret_cast<const float4 *>(part + (tile * splits + z) * TC_BM * BN) +
                           (col0 / 4) * TC_BM + rl;
        const bool two = ZU == 2 && z + 1 < splits;
        const float4 *p1 = two ? p0 + TC_BM * BN / 4 : p0;
#pragma unroll
        for (int j0 = 0; j0 < CW; j0 += 64) {
          float4 t0[16], t1[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            t0[j] = __ldcg(p0 + (j0 / 4 + j) * TC_BM);
            if (ZU == 2) t1[j] = __ldcg(p1 + (j0 / 4 + j) * TC_BM);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[j0 + 4 * j] += t0[j].x; acc[j0 + 4 * j + 1] += t0[j].y;
            acc[j0 + 4 * j + 2] += t0[j].z; acc[j0 + 4 * j + 3] += t0[j].w;
            if (ZU == 2 && two) {
              acc[j0 + 4 * j] += t1[j].x; acc[j0 + 4 * j + 1] += t1[j].y;
              acc[j0 + 4 * j + 2] += t1[j].z; acc[j0 + 4 * j + 3] += t1[j].w;
            }
          }
        }
      }
    }
  }

  // Stores. A thread holds CW columns of one row; written directly, every
  // instruction of a warp would touch 32 different lines. The V^T columns of a
  // QKV projection are the exception (lanes = consecutive positions of one
  // column): they go out from the registers. Everything else is transposed
  // through the pipeline's shared memory (idle by now: every load has landed
  // and every MMA has completed) and stored row by row, where bias, residual,
  // ReLU and the TF32 split are applied on coalesced float4s.
  const bool vt_on = ep.vt_hi != nullptr;
  if (finish && vt_on && row < m && n0 + col0 + CW > ep.vt_col0) {
    const int sl = ep.state ? ep.state->s : ep.vt_s;
    const int v_stream = row / sl, v_tok = row - v_stream * sl;
    if (v_stream < ep.vt_streams) {
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        const int col = n0 + col0 + j;
        if (col >= ep.vt_col0) {
          float val = acc[j];
          if (ep.ln_u != nullptr) val = __fmul_rn(ln_st.y, __fmaf_rn(-ln_st.x, ep.ln_u[col], val));
          float hh, ll;
          split_tf32(val + (ep.bias ? ep.bias[col] : 0.f), hh, ll);
          const long long at = ((long long)v_stream * ep.vt_rows + (col - ep.vt_col0)) * ep.vt_pitch + v_tok;
          ep.vt_hi[at] = hh;
          ep.vt_lo[at] = ll;
        }
      }
    }
  }
  constexpr int LDS = BN + 4;  // staging pitch: 16-byte accesses of 8 consecutive rows hit all banks once
  if (finish) {
#pragma unroll
    for (int j = 0; j < CW; j += 4)
      *reinterpret_cast<float4 *>(stage + rl * LDS + col0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    if (ep.ln_u != nullptr && col0 == 0) row_stats[rl] = ln_st;
  }
  const bool tstamp = ep.timeline != nullptr && leader && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  if (tstamp) ep.timeline[12] = clock64();
  asm volatile("bar.sync 1, %0;" ::"n"(DRAIN_THREADS) : "memory");
  if (tstamp) ep.timeline[13] = clock64();
  if (finish) {
    constexpr int PER_ROW = BN / 4;
    constexpr int UNITS = TC_BM * PER_ROW / DRAIN_THREADS;  // float4s per thread: 16 or 32
    constexpr int BATCH = 16;
    static_assert(UNITS % BATCH == 0, "whole batches");
    for (int i0 = 0; i0 < UNITS; i0 += BATCH) {
    // The residual rows come from L2 / HBM: all loads of a batch are issued before
    // the first is used (a few in flight per thread would leave the SM at a
    // fraction of its bandwidth, and the epilogue is a quarter of a short k loop).
    float4 res[BATCH];
    if (ep.residual) {
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int u = t2 + (i0 + b) * DRAIN_THREADS;
        const int rr = u / PER_ROW, c4 = u % PER_ROW;
        res[b] = (m0 + rr < m) ? __ldg(reinterpret_cast<const float4 *>(ep.residual + (long long)(m0 + rr) * n + n0 + c4 * 4))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int i = i0 + b;
      const int u = t2 + i * DRAIN_THREADS;
      const int rr = u / PER_ROW, c4 = u % PER_ROW;
      const int col = n0 + c4 * 4;
      // (no early exit: with an fp16-pair result the 16 lanes of a 64-column block shuffle together)
      const bool active = m0 + rr < m && !(vt_on && col >= ep.vt_col0);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const long long off = (long long)(m0 + rr) * n + col;
      if (active) {
      v = *reinterpret_cast<const float4 *>(stage + rr * LDS + c4 * 4);
      if (ep.ln_u != nullptr) {  // inv_std * (x W' - mean * u); v comes in as the bias
        const float2 st = row_stats[rr];
        const float4 uu = *reinterpret_cast<const float4 *>(ep.ln_u + col);
        v.x = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.x, v.x));
        v.y = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.y, v.y));
        v.z = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.z, v.z));
        v.w = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.w, v.w));
      }
      if (ep.bias) {
        const float4 bb = *reinterpret_cast<const float4 *>(ep.bias + col);
        v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
      }
      if (ep.residual) {
        const float4 rs = res[b];
        v.x += rs.x; v.y += rs.y; v.z += rs.z; v.w += rs.w;
      }
      if (ep.relu) {
        v.x = v.x > 0.f ? v.x : 0.f; v.y = v.y > 0.f ? v.y : 0.f;
        v.z = v.z > 0.f ? v.z : 0.f; v.w = v.w > 0.f ? v.w : 0.f;
      }
      if (ep.c) *reinterpret_cast<float4 *>(ep.c + off) = v;
      if (ep.c_hi) {
        float4 hh, ll;
        split_tf32(v.x, hh.x, ll.x);
        split_tf32(v.y, hh.y, ll.y);
        split_tf32(v.z, hh.z, ll.z);
        split_tf32(v.w, hh.w, ll.w);
        *reinterpret_cast<float4 *>(ep.c_hi + off) = hh;
        *reinterpret_cast<float4 *>(ep.c_lo + off) = ll;
      }
      if (ep.stats_out != nullptr) *reinterpret_cast<float4 *>(stage + rr * LDS + c4 * 4) = v;  // final values
      }
      if (ep.c_f16.hi != nullptr)
        f16_store_block(v, active, ep.c_f16.hi + off, ep.c_f16.lo + off,
                        ep.c_f16.inv_scale + (long long)(m0 + rr) * (n / TC_F16_SLOT) + col / TC_F16_SLOT);
    }
    }
  }
  if (tstamp) ep.timeline[14] = clock64();
  if (ep.stats_out != nullptr) {
    // Row statistics for a LayerNorm folded into the next product: thread = row
    // again, sums of its stored values over slots of 64 columns, in column order.
    asm volatile("bar.sync 1, %0;" ::"n"(DRAIN_THREADS) : "memory");
    if (finish && row < m) {
#pragma unroll
      for (int j0 = 0; j0 < CW; j0 += 64) {
        double sx = 0.0, sxx = 0.0;
#pragma unroll 4
        for (int j = 0; j < 64; j += 4) {
          const float4 t = *reinterpret_cast<const float4 *>(stage + rl * LDS + col0 + j0 + j);
          sx += (double)t.x; sxx += (double)t.x * (double)t.x;
          sx += (double)t.y; sxx += (double)t.y * (double)t.y;
          sx += (double)t.z; sxx += (double)t.z * (double)t.z;
          sx += (double)t.w; sxx += (double)t.w * (double)t.w;
        }
        ep.stats_out[(long long)row * TC_STAT_SLOTS + (n0 + col0 + j0) / 64] = make_double2(sx, sxx);
      }
    }
  }
}

}  // namespace lb
