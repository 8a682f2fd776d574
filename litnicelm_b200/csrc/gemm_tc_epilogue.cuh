// Shared tail of the tensor-core projection kernels: what the drain warps do
// once a thread holds CW accumulated columns of one row of the 128 x BN tile.
#pragma once

#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace lb {

// What the store phase reads from global memory before its first arithmetic: the per-column
// terms (bias, folded-LayerNorm u) and the residual rows of the first step. Loaded ahead of
// it (before the wait for the cluster's partial tiles), because the store loop would
// otherwise start with an L2 round trip. Same thread-to-element mapping as tc_store_rows.
// Rows a thread of the store phase has in flight per trip. Measured: one for tiles up to 128 columns
// (the single-stream shapes: 2696 against 2650 tokens/s at config 2 with two), two for the 256-column
// tiles of the many-row shapes (config 4: 80.6 against 82.3 ms with one); four is slower everywhere.
__host__ __device__ constexpr int tc_store_g(int bn) { return bn > 128 ? 2 : 1; }
constexpr int TC_STORE_G_MAX = 2;

struct TcStoreFirst {
  float4 res[TC_STORE_G_MAX];
  float4 uu, bb;
};
template <int BN, int NT>
__device__ __forceinline__ void tc_store_first(const TcEpilogue &ep, int m, int n, int m0, int n0, int tid,
                                               int row_begin, int row_end, TcStoreFirst &out) {
  constexpr int PER_ROW = BN / 4;
  constexpr int RPT = NT / PER_ROW;
  const int c4 = tid % PER_ROW, r0 = tid / PER_ROW;
  const int col = n0 + c4 * 4;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  out.uu = ep.ln_u != nullptr ? __ldg(reinterpret_cast<const float4 *>(ep.ln_u + col)) : zero4;
  out.bb = ep.bias != nullptr ? __ldg(reinterpret_cast<const float4 *>(ep.bias + col)) : zero4;
#pragma unroll
  for (int g = 0; g < tc_store_g(BN); ++g) {
    const int rg = row_begin + r0 + g * RPT;
    out.res[g] = (ep.residual != nullptr && rg < row_end && m0 + rg < m)
                     ? __ldg(reinterpret_cast<const float4 *>(ep.residual + (long long)(m0 + rg) * n + col))
                     : zero4;
  }
}

// The store phase: NT threads (whole warps, thread index tid) walk the staged
// 128 x BN fp32 tile row by row, a float4 each, apply the epilogue terms and
// write the results in every requested format. A thread keeps its column for the
// whole walk (NT is a multiple of the float4s per row), so the per-column terms
// (bias, folded-LayerNorm u) are loaded once; two rows per trip of a loop that is
// deliberately not unrolled (this code runs once per CTA: as straight-line code
// it ran at the speed of instruction fetch), with the residual rows of the next
// trip requested before this trip's arithmetic.
// csplits > 1 (split-k over a cluster): this CTA stores rows [row_begin, row_end) of the tile;
// every rank has pushed its partial sums of those rows into this CTA's staging area, rank z
// at rows [z * rows_each, z * rows_each + row_end - row_begin), and they are added in rank
// order. Otherwise the area holds the tile itself (row_begin 0).
// The loop runs out of the instruction cache of a scheduler only when its body is small: with every
// epilogue term and output format behind run-time tests the body is several hundred instructions and
// each trip is fetched again (two rows per trip measured faster than four, one faster than two). F
// names the terms at compile time (TC_EP_* bits) for the forms the token loop uses; TC_EP_GENERIC
// keeps the run-time tests for every other caller.
constexpr unsigned TC_EP_FOLD = 1u, TC_EP_RELU = 2u, TC_EP_RESIDUAL = 4u, TC_EP_C = 8u, TC_EP_SPLIT = 16u,
                   TC_EP_QK16 = 32u, TC_EP_F16 = 64u, TC_EP_STATS = 128u, TC_EP_BIAS = 256u, TC_EP_GENERIC = 1u << 31;
// the three forms of the fp16-pair token loop
constexpr unsigned TC_EP_FORM_QKV = TC_EP_FOLD | TC_EP_BIAS | TC_EP_QK16;
constexpr unsigned TC_EP_FORM_W1 = TC_EP_FOLD | TC_EP_BIAS | TC_EP_RELU | TC_EP_F16;
constexpr unsigned TC_EP_FORM_RES = TC_EP_BIAS | TC_EP_RESIDUAL | TC_EP_C | TC_EP_F16 | TC_EP_STATS;
__device__ __forceinline__ unsigned tc_ep_form(const TcEpilogue &ep) {
  return (ep.ln_u != nullptr ? TC_EP_FOLD : 0u) | (ep.relu ? TC_EP_RELU : 0u) | (ep.residual != nullptr ? TC_EP_RESIDUAL : 0u) |
         (ep.c != nullptr ? TC_EP_C : 0u) | (ep.c_hi != nullptr ? TC_EP_SPLIT : 0u) | (ep.qk16_hi != nullptr ? TC_EP_QK16 : 0u) |
         (ep.c_f16.hi != nullptr ? TC_EP_F16 : 0u) | (ep.stats_out != nullptr ? TC_EP_STATS : 0u) |
         (ep.bias != nullptr ? TC_EP_BIAS : 0u);
}

template <int BN, int NT, unsigned F = TC_EP_GENERIC>
__device__ __forceinline__ void tc_store_rows(const TcEpilogue &ep, int m, int n, int m0, int n0, int tid,
                                              float *stage, const float2 *row_stats, int csplits, int rows_each,
                                              int row_begin, int row_end, const TcStoreFirst &first) {
  constexpr bool GEN = (F & TC_EP_GENERIC) != 0;
  const bool has_relu = GEN ? ep.relu != 0 : (F & TC_EP_RELU) != 0;
  const bool has_res = GEN ? ep.residual != nullptr : (F & TC_EP_RESIDUAL) != 0;
  const bool out_c = GEN ? ep.c != nullptr : (F & TC_EP_C) != 0;
  const bool out_split = GEN ? ep.c_hi != nullptr : (F & TC_EP_SPLIT) != 0;
  const bool out_qk16 = GEN ? ep.qk16_hi != nullptr : (F & TC_EP_QK16) != 0;
  const bool out_f16 = GEN ? ep.c_f16.hi != nullptr : (F & TC_EP_F16) != 0;
  const bool out_stats = GEN ? ep.stats_out != nullptr : (F & TC_EP_STATS) != 0;
  constexpr int LDS = BN + 4;
  constexpr int PER_ROW = BN / 4;
  static_assert(NT % PER_ROW == 0 && NT % 32 == 0, "a thread keeps its column; whole warps");
  constexpr int RPT = NT / PER_ROW;  // rows covered by the threads at once
  constexpr int G = tc_store_g(BN);
  const int c4 = tid % PER_ROW, r0 = tid / PER_ROW;
  const int col = n0 + c4 * 4;
  const bool col_active = !(ep.has_vt() && col >= ep.vt_col0);  // V columns leave transposed, elsewhere
  const float cs16 = out_qk16 ? __ldg(ep.col_scale + col / 64) : 1.f;
  const bool fold = GEN ? ep.ln_u != nullptr : (F & TC_EP_FOLD) != 0;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 uu = first.uu, bb = first.bb;
  const float *res_col = has_res ? ep.residual + (long long)m0 * n + col : nullptr;
  auto residual_row = [&](int rg) {
    return (res_col != nullptr && rg < row_end && m0 + rg < m) ? __ldg(reinterpret_cast<const float4 *>(res_col + (long long)rg * n))
                                                               : zero4;
  };
  float4 res_next[G];
#pragma unroll
  for (int g = 0; g < G; ++g) res_next[g] = first.res[g];
#pragma unroll 1
  for (int rr = row_begin + r0; rr < row_end; rr += G * RPT) {
    float4 v[G], res[G];
    bool act[G], valid[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      res[g] = res_next[g];
      res_next[g] = residual_row(rr + (G + g) * RPT);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int rg = rr + g * RPT;
      valid[g] = rg < row_end;  // the same for all lanes of a warp (a warp covers whole rows or a part of one)
      act[g] = valid[g] && m0 + rg < m && col_active;
      const int rc = valid[g] ? rg : row_begin;
      const float *sp = stage + (rc - row_begin) * LDS + c4 * 4;
      v[g] = *reinterpret_cast<const float4 *>(sp);
      for (int z = 1; z < csplits; ++z) {
        const float4 t = *reinterpret_cast<const float4 *>(sp + z * rows_each * LDS);
        v[g].x += t.x; v[g].y += t.y; v[g].z += t.z; v[g].w += t.w;
      }
      if (fold) {  // inv_std * (x W' - mean * u); v comes in as the bias
        const float2 st = row_stats[rc];
        v[g].x = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.x, v[g].x));
        v[g].y = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.y, v[g].y));
        v[g].z = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.z, v[g].z));
        v[g].w = __fmul_rn(st.y, __fmaf_rn(-st.x, uu.w, v[g].w));
      }
      v[g].x += bb.x + res[g].x;
      v[g].y += bb.y + res[g].y;
      v[g].z += bb.z + res[g].z;
      v[g].w += bb.w + res[g].w;
      if (has_relu) {
        v[g].x = fmaxf(v[g].x, 0.f); v[g].y = fmaxf(v[g].y, 0.f);
        v[g].z = fmaxf(v[g].z, 0.f); v[g].w = fmaxf(v[g].w, 0.f);
      }
      if (!act[g]) v[g] = zero4;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!act[g]) continue;
      const int rg = rr + g * RPT;
      const long long off = (long long)(m0 + rg) * n + col;
      if (out_c) *reinterpret_cast<float4 *>(ep.c + off) = v[g];
      if (out_split) {
        float4 hh, ll;
        split_tf32(v[g].x, hh.x, ll.x);
        split_tf32(v[g].y, hh.y, ll.y);
        split_tf32(v[g].z, hh.z, ll.z);
        split_tf32(v[g].w, hh.w, ll.w);
        *reinterpret_cast<float4 *>(ep.c_hi + off) = hh;
        *reinterpret_cast<float4 *>(ep.c_lo + off) = ll;
      }
      if (out_qk16) {  // fp16 pair under the head's fixed scale
        uint2 hi, lo;
        f16_pair4(v[g], cs16, hi, lo);
        *reinterpret_cast<uint2 *>(ep.qk16_hi + off) = hi;
        *reinterpret_cast<uint2 *>(ep.qk16_lo + off) = lo;
      }
      if (out_stats)  // final values, over the thread's own rank-0 partial
        *reinterpret_cast<float4 *>(stage + (rg - row_begin) * LDS + c4 * 4) = v[g];
    }
    if (out_f16) {
      // fp16 pair: the 16 lanes of a 64-column block of a row agree on its scale
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (!valid[g]) continue;  // whole warps
        float am = fmaxf(fmaxf(fabsf(v[g].x), fabsf(v[g].y)), fmaxf(fabsf(v[g].z), fabsf(v[g].w)));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        float inv;
        const float scale = f16_block_scale(am, &inv);
        if (act[g]) {
          const int rg = rr + g * RPT;
          const long long off = (long long)(m0 + rg) * n + col;
          uint2 hi, lo;
          f16_pair4(v[g], scale, hi, lo);
          *reinterpret_cast<uint2 *>(ep.c_f16.hi + off) = hi;
          *reinterpret_cast<uint2 *>(ep.c_f16.lo + off) = lo;
          if ((c4 & 15) == 0) ep.c_f16.inv_scale[(long long)(m0 + rg) * (n / TC_F16_SLOT) + col / TC_F16_SLOT] = inv;
        }
      }
    }
  }
}

// What the drain warps do once a thread holds CW accumulated columns of tile
// row rl: with split-k, leave the partial tile in scratch and let the CTA that
// arrives last add all partials in split order; then stage the tile in shared
// memory (row pitch BN + 4: 16-byte accesses of 8 consecutive rows hit all banks
// once) for the store phase. finish: false when the pipeline gave up. t2 / leader:
// index among the DRAIN_THREADS threads (named barrier 1) and the one that counts
// arrivals. Returns whether this CTA stores the tile; the leader also leaves that
// in *store_flag for the warps that were not draining.
template <int BN, int CW, int DRAIN_THREADS>
__device__ __forceinline__ bool tc_stage_tile(float (&acc)[CW], bool finish, const TcEpilogue &ep, int col0, int rl,
                                              bool leader, int splits, float *__restrict__ part,
                                              int *__restrict__ counters, volatile int *last_flag,
                                              volatile int *store_flag, float *stage, float2 ln_st,
                                              float2 *row_stats, bool defer_stage) {
  finish = __all_sync(0xffffffffu, finish);
  if (splits > 1) {
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
  constexpr int LDS = BN + 4;
  if (finish) {
    if (!defer_stage) {
#pragma unroll
      for (int j = 0; j < CW; j += 4)
        *reinterpret_cast<float4 *>(stage + rl * LDS + col0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    }
    if (ep.ln_u != nullptr && col0 == 0) row_stats[rl] = ln_st;
  }
  if (leader) *store_flag = finish ? 1 : 0;
  return finish;
}

// Split-k over a cluster: a drain thread sends its CW partial sums of tile row rl to the CTA
// that stores that row (rank rl / rows_each), into the slot of this CTA's rank, with remote
// shared-memory stores: nothing waits for them but the cluster barrier that follows, whereas
// the owner pulling the rows cost a remote round trip of over a microsecond at the start of
// its store phase. Only after a cluster barrier that says every CTA's operand tiles are dead
// (the staging area overlays them).
template <int BN, int CW>
__device__ __forceinline__ void tc_push_tile(const float (&acc)[CW], const float *stage, int col0, int rl,
                                             int rows_each) {
  constexpr int LDS = BN + 4;
  const int owner = rl / rows_each, local = rl - owner * rows_each;
  const unsigned at = cluster_map(smem_u32(stage) + (unsigned)(((int)blockIdx.z * rows_each + local) * LDS + col0) * 4u,
                                  (unsigned)owner);
#pragma unroll
  for (int j = 0; j < CW; j += 4)
    st_cluster_f4(at + (unsigned)j * 4u, make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]));
}

// The same exchange for tiles up to 128 columns, by all NT threads from a copy of the tile the
// drain threads staged in this CTA's own shared memory (at `local`, behind the exchange area):
// the lanes of a warp run along a row, so a warp's remote store is one or two whole rows (256 or
// 512 contiguous bytes). With a thread per row (tc_push_tile) every lane's 16 bytes go to a line
// of their own; the exchange of six 128 x 128 partial tiles took 3.7 us that way and 2.9 us this
// way (remote shared-memory stores move about 25 GB/s per SM when every SM sends at once).
template <int BN, int NT>
__device__ __forceinline__ void tc_push_rows(const float *local, const float *stage, int tid, int rows_each) {
  constexpr int LDS = BN + 4;
  constexpr int PER_ROW = BN / 4;
  constexpr int RPT = NT / PER_ROW;
  const int c4 = tid % PER_ROW, r0 = tid / PER_ROW;
  const unsigned slot0 = smem_u32(stage) + (unsigned)(((int)blockIdx.z * rows_each) * LDS + c4 * 4) * 4u;
#pragma unroll 4
  for (int r = r0; r < TC_BM; r += RPT) {
    const int owner = r / rows_each, at = r - owner * rows_each;
    const float4 v = *reinterpret_cast<const float4 *>(local + r * LDS + c4 * 4);
    st_cluster_f4(cluster_map(slot0 + (unsigned)(at * LDS) * 4u, (unsigned)owner), v);
  }
}

// After the staged tile is visible to every warp (a barrier): the V^T columns of a QKV
// projection leave transposed, element (row r = stream * s + t, column vt_col0 + c) to
// vt[(stream * vt_rows + c) * vt_pitch + t]. All NT threads take part: a warp handles units
// of 32 consecutive rows x 4 columns (lane = row, so the 32 lanes write consecutive positions
// of one V^T row: whole 128-byte lines), a float4 of the staged tile per lane. vt_col0 is a
// multiple of 64, so a unit is all V or not V.
template <int BN, int NT>
__device__ __forceinline__ void tc_store_vt(const TcEpilogue &ep, int m, int m0, int n0, int tid, const float *stage,
                                            const float2 *row_stats, int csplits, int rows_each, int row_begin,
                                            int row_end) {
  constexpr int LDS = BN + 4;
  if (n0 + BN <= ep.vt_col0) return;
  // the rows this CTA stores (all of the tile without a cluster), and the partial sums of every rank as tc_store_rows
  const int rows = row_end - row_begin, rgroups = (rows + 31) / 32;
  const int units = (BN / 4) * rgroups;
  const int warp = tid >> 5, lane = tid & 31;
  const int sl = ep.state ? ep.state->s : ep.vt_s;
  const bool fold = ep.ln_u != nullptr;
#pragma unroll 1
  for (int u = warp; u < units; u += NT / 32) {
    const int cg = u / rgroups, rg = u - cg * rgroups;
    const int col = n0 + cg * 4;
    if (col < ep.vt_col0) continue;  // uniform over the warp
    const int local = rg * 32 + lane;
    const bool valid = local < rows;
    const int rl = row_begin + (valid ? local : 0), row = m0 + rl;
    const int v_stream = row / sl, v_tok = row - v_stream * sl;
    const bool act = valid && row < m && v_stream < ep.vt_streams;
    const float *sp = stage + (rl - row_begin) * LDS + cg * 4;
    float4 t = *reinterpret_cast<const float4 *>(sp);
    for (int z = 1; z < csplits; ++z) {
      const float4 tz = *reinterpret_cast<const float4 *>(sp + z * rows_each * LDS);
      t.x += tz.x; t.y += tz.y; t.z += tz.z; t.w += tz.w;
    }
    const float4 u4 = fold ? __ldg(reinterpret_cast<const float4 *>(ep.ln_u + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 b4 = ep.bias ? __ldg(reinterpret_cast<const float4 *>(ep.bias + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float2 st = fold ? row_stats[rl] : make_float2(0.f, 1.f);
    if (!act) continue;
    const float vals[4] = {t.x, t.y, t.z, t.w}, us[4] = {u4.x, u4.y, u4.z, u4.w}, bs[4] = {b4.x, b4.y, b4.z, b4.w};
    const long long at0 = ((long long)v_stream * ep.vt_rows + (col - ep.vt_col0)) * ep.vt_pitch + v_tok;
    if (ep.vt16_hi != nullptr) {  // fp16 pair under the head's fixed scale (the four columns share a head)
      const float cs = __ldg(ep.col_scale + col / 64);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float val = fold ? __fmul_rn(st.y, __fmaf_rn(-st.x, us[e], vals[e])) : vals[e];
        const float a = (val + bs[e]) * cs;
        const __half hh = __float2half_rn(a);
        ep.vt16_hi[at0 + (long long)e * ep.vt_pitch] = hh;
        ep.vt16_lo[at0 + (long long)e * ep.vt_pitch] = __float2half_rn(a - __half2float(hh));
      }
      continue;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float val = fold ? __fmul_rn(st.y, __fmaf_rn(-st.x, us[e], vals[e])) : vals[e];
      float hh, ll;
      split_tf32(val + bs[e], hh, ll);
      ep.vt_hi[at0 + (long long)e * ep.vt_pitch] = hh;
      ep.vt_lo[at0 + (long long)e * ep.vt_pitch] = ll;
    }
  }
}

// After the store phase has put the final values back into the staged tile (a
// barrier): row statistics for a LayerNorm folded into the next product, (sum x,
// sum x^2) in double per row and slot of 64 columns. By all NT threads: four
// consecutive lanes share a (row, slot), each sums 16 columns in column order and
// the first adds the four partial sums in order (a fixed order, so the statistics
// do not depend on the tile plan).
template <int BN, int NT>
__device__ __forceinline__ void tc_store_row_stats(const TcEpilogue &ep, int m, int m0, int n0, int tid,
                                                   const float *stage, int row_begin, int row_end) {
  constexpr int LDS = BN + 4;
  constexpr int SLOTS = BN / 64;
  const int total = (row_end - row_begin) * SLOTS;
  const int q = tid & 3;
#pragma unroll 1
  for (int u0 = (tid >> 5) * 8; u0 < total; u0 += NT / 4) {  // the warp's first unit: the trip count is per warp
    const int u = u0 + ((tid & 31) >> 2);
    const bool valid = u < total;
    const int rl = row_begin + (valid ? u / SLOTS : 0), slot = valid ? u % SLOTS : 0;
    const float *sp = stage + (rl - row_begin) * LDS + slot * 64 + q * 16;
    double sx = 0.0, sxx = 0.0;
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
      const float4 t = *reinterpret_cast<const float4 *>(sp + j);
      sx += (double)t.x; sxx += (double)t.x * (double)t.x;
      sx += (double)t.y; sxx += (double)t.y * (double)t.y;
      sx += (double)t.z; sxx += (double)t.z * (double)t.z;
      sx += (double)t.w; sxx += (double)t.w * (double)t.w;
    }
    double tx = sx, txx = sxx;
#pragma unroll
    for (int d = 1; d < 4; ++d) {
      tx += __shfl_down_sync(0xffffffffu, sx, d);
      txx += __shfl_down_sync(0xffffffffu, sxx, d);
    }
    const int row = m0 + rl;
    if (valid && q == 0 && row < m)
      ep.stats_out[(long long)row * TC_STAT_SLOTS + (n0 + slot * 64) / 64] = make_double2(tx, txx);
  }
}

}  // namespace lb
