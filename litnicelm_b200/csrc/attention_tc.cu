// Fused causal self-attention on the sm_100a tensor cores (tcgen05 + TMEM + TMA),
// head dimension 64, fp32 accuracy by the three-product TF32 split.
//
// Same maths as attention.cu (litnicelm's
// src/model/algo/self_attention_fused_inplace.cpp:82-94: gemm_batched_rhs_t,
// scaled_causal_softmax_rows, gemm_batched; scores scaled in fp32 before the
// maximum, device_backend.cpp:1561-1577) as one pass with a running maximum and
// sum per query row, but both contractions run as tcgen05.mma:
//
//   S = Q K^T   A = Q tile (128 queries x 64) and B = K tile (128 keys x 64),
//               both K-major TF32 hi/lo pairs brought by TMA from the split
//               output of the QKV projection; one accumulation chain in tensor
//               memory (24 instructions).
//   P           eight warps read S from tensor memory (thread = one query row
//               and 64 of the 128 keys), scale, mask, and exponentiate against
//               the maximum of their own 64 keys (no exchange between threads:
//               the 64 keys of a thread are exactly one accumulation chain of
//               the next product), and store P as a TF32 hi/lo pair in tensor
//               memory. 2^x with scores pre-multiplied by log2(e), ex2.approx.
//   O += P V    A = P read from tensor memory, B = V^T tile (64 x 128 keys,
//               K-major; the QKV projection stores V transposed for this), two
//               chains (keys 0-63, 64-127) which the same threads rescale to the
//               row's running maximum and add into fp32 registers.
//
// Tensor-core accumulation truncates, so chains are kept to 24 instructions and
// summed in registers with round-to-nearest. The MMA warp issues S of tile t+1
// before P V of tile t: the softmax of tile t+1 overlaps the tensor work of
// tile t. Warp 0 issues TMA, warp 1 owns tensor memory and issues the MMAs,
// warps 2-9 do the softmax and the output. Causal work is triangular; with few
// (stream, head) pairs a query tile's key range is cut into chunks for separate
// CTAs whose partial results the last CTA to finish merges in chunk order (as
// attention.cu). Every mbarrier wait is bounded; no cluster launch and no
// multicast.
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace lb {

namespace {

constexpr int TA_BQ = 128;   // query rows per CTA (one UMMA M = 128 tile)
constexpr int TA_BK = 128;   // keys per tile
constexpr int TA_DH = 64;    // head dimension
constexpr int TA_THREADS = 320;
constexpr int TA_SOFTMAX_THREADS = 256;
constexpr float TA_NEG = -3.402823466e+38f;
constexpr int TA_STAGE_LD = TA_DH + 4;  // row pitch of the output staging tile: conflict-free 16-byte accesses
constexpr int TA_MAX_CHUNKS = 16;  // chunks one query tile's keys are cut into, at most
constexpr int TA_PART = TA_BQ * TA_DH + 2 * TA_BQ;  // floats of one partial: o[128][64], m[128], l[128]
constexpr int TA_O_BYTES = TA_BQ * TA_DH * 4;       // the o part of a partial
constexpr int TA_MERGE_SLOTS = 6;  // partial outputs the merging CTA holds in shared memory at a time (the Q, K and V^T tiles)

// shared memory (after 1024-byte alignment)
constexpr int TA_SLAB = TA_BQ * 128;                    // one 32-wide k-block of a 128-row tile
constexpr int TA_Q_BYTES = 2 * (TA_DH / 32) * TA_SLAB;  // hi + lo
constexpr int TA_K_BYTES = TA_Q_BYTES;
constexpr int TA_VSLAB = TA_DH * 128;                   // 32 keys of the 64-row V^T tile
constexpr int TA_V_BYTES = 2 * (TA_BK / 32) * TA_VSLAB;
constexpr int TA_Q_OFF = 0;
constexpr int TA_K_OFF = TA_Q_OFF + TA_Q_BYTES;
constexpr int TA_V_OFF = TA_K_OFF + TA_K_BYTES;
constexpr int TA_BAR_OFF = TA_V_OFF + TA_V_BYTES;       // 7 barriers + holders
constexpr int TA_XCH_OFF = TA_BAR_OFF + 128;            // [2 parities][max half 0, max half 1, sum half 0, sum half 1][128]
constexpr int TA_AMAX_OFF = TA_XCH_OFF + 8 * TA_BQ * 4;  // [2 halves][128 rows]: largest magnitudes of the output rows
constexpr int TA_SMEM = TA_AMAX_OFF + 2 * TA_BQ * 4 + 1024;
constexpr int TA_STAGE16_LD = TA_DH * 2 + 16;  // bytes per row of a staged fp16 tile: conflict-free 16-byte accesses

// tensor-memory columns
constexpr unsigned TA_S_COL = 0;      // S: 128 columns (keys)
constexpr unsigned TA_PHI_COL = 128;  // P high parts: 128 columns (keys)
constexpr unsigned TA_PLO_COL = 256;  // P low parts
constexpr unsigned TA_O_COL = 384;    // O chains: 2 x 64 columns (keys 0-63, keys 64-127)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__host__ __device__ inline int ta_chunks_of(int qt, int kc) { return (qt + kc) / kc; }  // ceil((qt+1)/kc)

__global__ void __launch_bounds__(TA_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_qk_hi, const __grid_constant__ CUtensorMap map_qk_lo,
                    const __grid_constant__ CUtensorMap map_vt_hi, const __grid_constant__ CUtensorMap map_vt_lo,
                    float *__restrict__ ctx_hi, float *__restrict__ ctx_lo, int s_cap, int d_model, float scale_log2e,
                    int kc, float *__restrict__ part, int *__restrict__ counters, const LoopState *state,
                    DevErr *err, unsigned long long *timeline, TcPairF16 ctx_f16) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bar_base = base + TA_BAR_OFF;
  const unsigned q_full = bar_base, k_full = bar_base + 8, v_full = bar_base + 16, s_full = bar_base + 24,
                 p_ready = bar_base + 32, o_full = bar_base + 40, s_read = bar_base + 48, m_full = bar_base + 56;
  volatile unsigned *tmem_holder = reinterpret_cast<volatile unsigned *>(base_ptr + TA_BAR_OFF + 64);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + TA_BAR_OFF + 68);
  volatile int *last_flag = reinterpret_cast<volatile int *>(base_ptr + TA_BAR_OFF + 72);
  // per tile parity: maximum [half][row] and sum [half][row] of each thread's 64 keys
  float *xch = reinterpret_cast<float *>(base_ptr + TA_XCH_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The grid is laid out for s_cap; the actual length shares its tile count.
  const int s = state ? state->s : s_cap;
  const int tiles = (s_cap + TA_BQ - 1) / TA_BQ;
  int idx = blockIdx.x, qt = tiles - 1;
  for (; qt > 0; --qt) {  // (query tile, chunk) pairs, longest query tiles first
    const int nc = ta_chunks_of(qt, kc);
    if (idx < nc) break;
    idx -= nc;
  }
  const int chunk = idx, nchunks = ta_chunks_of(qt, kc);
  const int kt_begin = chunk * kc, kt_end = min(qt + 1, kt_begin + kc);
  const int ntiles = kt_end - kt_begin;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * TA_BQ;
  const int row0 = b * s;  // first row of this stream in the packed activations

  pdl_launch_dependents();
  // Measurement aid: the CTA of head 0, stream 0 that takes the diagonal tile of the last query tile (it usually
  // ends last and merges) stamps its milestones in timeline[0..7]; every
  // CTA contributes to the earliest start [8], the latest end [9] and the latest start [10].
  const bool stamp = timeline != nullptr && (int)blockIdx.x == ta_chunks_of(tiles - 1, kc) - 1 && blockIdx.y == 0 && blockIdx.z == 0;
  if (timeline != nullptr && threadIdx.x == 0) {
    const unsigned long long t = global_timer();
    atomicMin(timeline + 8, t);
    atomicMax(timeline + 10, t);
    if (stamp) timeline[0] = t;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, TA_SOFTMAX_THREADS / 32);  // one arrival per softmax warp
    mbar_init(o_full, 1);
    mbar_init(s_read, TA_SOFTMAX_THREADS / 32);
    mbar_init(m_full, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_holder)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_holder;
  if (stamp && threadIdx.x == 0) timeline[1] = global_timer();

  if (warp == 0) {
    // ---- TMA producer: Q once, then K and V^T of each key tile as their buffers free up ----
    if (lane == 0) {
      tma_prefetch_map(&map_qk_hi);
      tma_prefetch_map(&map_qk_lo);
      tma_prefetch_map(&map_vt_hi);
      tma_prefetch_map(&map_vt_lo);
    }
    pdl_wait();
    if (lane == 0) {
      if (timeline != nullptr) atomicMin(timeline + 16, global_timer());  // the predecessor has completed
      mbar_expect_tx(q_full, (unsigned)TA_Q_BYTES);
      for (int kb = 0; kb < TA_DH / 32; ++kb) {
        tma_load_2d(base + TA_Q_OFF + kb * TA_SLAB, &map_qk_hi, h * TA_DH + kb * 32, row0 + q0, q_full);
        tma_load_2d(base + TA_Q_OFF + (TA_DH / 32 + kb) * TA_SLAB, &map_qk_lo, h * TA_DH + kb * 32, row0 + q0, q_full);
      }
    }
    __syncwarp();
    // K(t) may be overwritten once S(t-1) has completed, V^T(t) once P V(t-1) has. The MMA warp issues
    // S(t+1) ahead of P V(t), so in time order: S(0), S(1), PV(0), S(2), PV(1), ... and the loads follow
    // that order: K runs one tile further ahead than V^T.
    int k_issued = 0, v_issued = 0;
    auto load_k = [&](int it) {
      if (lane == 0) {
        const int k0 = (kt_begin + it) * TA_BK;
        mbar_expect_tx(k_full, (unsigned)TA_K_BYTES);
        for (int kb = 0; kb < TA_DH / 32; ++kb) {
          tma_load_2d(base + TA_K_OFF + kb * TA_SLAB, &map_qk_hi, d_model + h * TA_DH + kb * 32, row0 + k0, k_full);
          tma_load_2d(base + TA_K_OFF + (TA_DH / 32 + kb) * TA_SLAB, &map_qk_lo, d_model + h * TA_DH + kb * 32,
                      row0 + k0, k_full);
        }
      }
      __syncwarp();
      ++k_issued;
    };
    auto load_v = [&](int it) {
      if (lane == 0) {
        const int k0 = (kt_begin + it) * TA_BK;
        mbar_expect_tx(v_full, (unsigned)TA_V_BYTES);
        for (int kb = 0; kb < TA_BK / 32; ++kb) {
          tma_load_2d(base + TA_V_OFF + kb * TA_VSLAB, &map_vt_hi, k0 + kb * 32, b * d_model + h * TA_DH, v_full);
          tma_load_2d(base + TA_V_OFF + (TA_BK / 32 + kb) * TA_VSLAB, &map_vt_lo, k0 + kb * 32,
                      b * d_model + h * TA_DH, v_full);
        }
      }
      __syncwarp();
      ++v_issued;
    };
    load_k(0);
    load_v(0);
    bool ok = true;
    if (ntiles > 1) {
      ok = mbar_wait_warp(s_full, 0u, abort_flag, err, 11);
      if (ok) load_k(1);
    }
    for (int it = 0; it + 1 < ntiles && ok; ++it) {
      if (it + 2 < ntiles) {  // S(it+1) has read K
        ok = mbar_wait_warp(s_full, (unsigned)(it + 1) & 1u, abort_flag, err, 11);
        if (!ok) break;
        load_k(it + 2);
      }
      ok = mbar_wait_warp(o_full, (unsigned)it & 1u, abort_flag, err, 12);  // P V(it) has read V^T
      if (!ok) break;
      load_v(it + 1);
    }
    if (*abort_flag) {
      // let copies already in flight land before the CTA's shared memory goes away
      const unsigned long long t0 = global_timer();
      while (!mbar_try_wait(q_full, 0u))
        if (global_timer() - t0 > WAIT_LIMIT_NS) break;
      if (k_issued > 0)
        while (!mbar_try_wait(k_full, (unsigned)(k_issued - 1) & 1u))
          if (global_timer() - t0 > 2 * WAIT_LIMIT_NS) break;
      if (v_issued > 0)
        while (!mbar_try_wait(v_full, (unsigned)(v_issued - 1) & 1u))
          if (global_timer() - t0 > 3 * WAIT_LIMIT_NS) break;
    }
  } else if (warp == 1) {
    // ---- MMA issuer: S(0), then per tile S(it+1) ahead of PV(it) so that the softmax of tile it+1
    //      runs while the tensor pipe works on PV(it) ----
    const unsigned idesc_s = umma_idesc_tf32(TA_BK);   // N = 128 keys
    const unsigned idesc_o = umma_idesc_tf32(TA_DH);   // N = 64 output columns
    auto issue_s = [&]() {  // one chain: S = Q K^T over both 32-wide k-blocks
      const unsigned tmem_d = tmem_base + TA_S_COL;
#pragma unroll
      for (int kb = 0; kb < TA_DH / 32; ++kb) {
        const unsigned long long a_hi = umma_desc_k128(base + TA_Q_OFF + kb * TA_SLAB);
        const unsigned long long a_lo = umma_desc_k128(base + TA_Q_OFF + (TA_DH / 32 + kb) * TA_SLAB);
        const unsigned long long b_hi = umma_desc_k128(base + TA_K_OFF + kb * TA_SLAB);
        const unsigned long long b_lo = umma_desc_k128(base + TA_K_OFF + (TA_DH / 32 + kb) * TA_SLAB);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
          tc_mma_tf32(tmem_d, a_lo + adv, b_hi + adv, idesc_s, (kb == 0 && ks == 0) ? 0u : 1u);
          tc_mma_tf32(tmem_d, a_hi + adv, b_lo + adv, idesc_s, 1u);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
          tc_mma_tf32(tmem_d, a_hi + adv, b_hi + adv, idesc_s, 1u);
        }
      }
      tc_commit(s_full);  // S complete; K may be overwritten
    };
    bool ok = mbar_wait_warp(q_full, 0u, abort_flag, err, 13);
    if (ok) ok = mbar_wait_warp(k_full, 0u, abort_flag, err, 14);
    if (ok) {
      if (stamp && lane == 0) timeline[2] = global_timer();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) issue_s();
      __syncwarp();
    }
    int pv_commits = 0;
    for (int it = 0; it < ntiles && ok; ++it) {
      const unsigned ph = (unsigned)it & 1u;
      if (it + 1 < ntiles) {
        // S(it+1) overwrites S(it): every softmax warp must have read it
        ok = mbar_wait_warp(s_read, ph, abort_flag, err, 21);
        if (ok) ok = mbar_wait_warp(k_full, ph ^ 1u, abort_flag, err, 14);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) issue_s();
        __syncwarp();
      }
      ok = mbar_wait_warp(p_ready, ph, abort_flag, err, 15);  // P(it) stored, O(it-1) drained
      if (ok) ok = mbar_wait_warp(v_full, ph, abort_flag, err, 16);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const unsigned p_hi = tmem_base + TA_PHI_COL, p_lo = tmem_base + TA_PLO_COL;
#pragma unroll
        for (int kb = 0; kb < TA_BK / 32; ++kb) {
          // chain kb/2 covers 64 keys: the keys one softmax thread scales by its own maximum
          const unsigned tmem_d = tmem_base + TA_O_COL + (unsigned)((kb >> 1) * TA_DH);
          const unsigned long long b_hi = umma_desc_k128(base + TA_V_OFF + kb * TA_VSLAB);
          const unsigned long long b_lo = umma_desc_k128(base + TA_V_OFF + (TA_BK / 32 + kb) * TA_VSLAB);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
            const unsigned ac = (unsigned)(kb * 32 + ks * 8);
            tc_mma_tf32_ts(tmem_d, p_lo + ac, b_hi + adv, idesc_o, ((kb & 1) == 0 && ks == 0) ? 0u : 1u);
            tc_mma_tf32_ts(tmem_d, p_hi + ac, b_lo + adv, idesc_o, 1u);
          }
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
            const unsigned ac = (unsigned)(kb * 32 + ks * 8);
            tc_mma_tf32_ts(tmem_d, p_hi + ac, b_hi + adv, idesc_o, 1u);
          }
        }
        tc_commit(o_full);  // O chains complete; P and V^T may be overwritten
      }
      __syncwarp();
      ++pv_commits;
    }
    if (!ok) {  // give the tensor pipe a bounded chance to finish before TMEM is freed
      if (lane == 0) tc_commit(o_full);
      __syncwarp();
      const unsigned long long t0 = global_timer();
      while (!mbar_try_wait(o_full, (unsigned)pv_commits & 1u))
        if (global_timer() - t0 > WAIT_LIMIT_NS) break;
    }
    __syncwarp();
  } else {
    // ---- softmax + output: thread = query row `r`, key half `g` (64 of the 128 keys = one O chain;
    //      32 of the 64 output columns) ----
    pdl_wait();  // scratch and ctx writes must follow the predecessor
    const int q = warp & 3;          // TMEM lane quarter this warp may touch
    const int g = (warp - 2) >> 2;   // 0: warps 2-5, 1: warps 6-9
    const int r = q * 32 + lane;
    const int qi = q0 + r;
    const unsigned lane_base = tmem_base + ((unsigned)(q * 32) << 16);
    float o[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = 0.f;
    // Running maximum (of scores times log2 e) and sum of the whole row; both
    // threads of a row keep identical copies.
    float m_run = TA_NEG, l_run = 0.f;
    bool ok = true;

    // O(t) = chain 0 * 2^(m0 - M) + chain 1 * 2^(m1 - M): each chain was scaled by the maximum of its own 64 keys
    auto drain = [&](int t) {
      const float *x = xch + (t & 1) * 4 * TA_BQ;
      const float m0 = x[r], m1 = x[TA_BQ + r], ps0 = x[2 * TA_BQ + r], ps1 = x[3 * TA_BQ + r];
      const float m_new = fmaxf(m_run, fmaxf(m0, m1));
      const float a = fast_exp2(m_run - m_new), w0 = fast_exp2(m0 - m_new), w1 = fast_exp2(m1 - m_new);
      unsigned c0[32], c1[32];
      tc_ld32(lane_base + TA_O_COL + (unsigned)(g * 32), c0);
      tc_ld32(lane_base + TA_O_COL + (unsigned)(TA_DH + g * 32), c1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j)
        o[j] = fmaf(o[j], a, fmaf(__uint_as_float(c0[j]), w0, __fmul_rn(__uint_as_float(c1[j]), w1)));
      l_run = fmaf(l_run, a, fmaf(ps0, w0, __fmul_rn(ps1, w1)));
      m_run = m_new;
    };

    for (int it = 0; it < ntiles && ok; ++it) {
      const unsigned ph = (unsigned)it & 1u;
      const int kbase = (kt_begin + it) * TA_BK + g * 64;
      ok = mbar_wait_warp(s_full, ph, abort_flag, err, 18);
      if (!ok) break;
      if (stamp && it == 0 && warp == 2 && lane == 0) timeline[3] = global_timer();
      if (stamp && nchunks == 1 && it >= 1 && it <= 4 && warp == 2 && lane == 0) timeline[11 + it] = global_timer();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float p[64];
      {
        unsigned t0[32], t1[32];
        tc_ld32(lane_base + TA_S_COL + (unsigned)(g * 64), t0);
        tc_ld32(lane_base + TA_S_COL + (unsigned)(g * 64 + 32), t1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(s_read);  // S may be overwritten by the next tile's product
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          p[j] = __uint_as_float(t0[j]);
          p[32 + j] = __uint_as_float(t1[j]);
        }
      }
      // Raw scores: the maximum commutes with the positive scale, and the scale joins the
      // subtraction in one fused multiply-add: p = 2^(s * c - max(s) * c). Only the tile on the
      // diagonal has keys past a query; the others skip the mask.
      float mx = TA_NEG, psum = 0.f;
      if (kt_begin + it == qt) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (kbase + j <= qi) mx = fmaxf(mx, p[j]);
        mx = __fmul_rn(mx, scale_log2e);
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          p[j] = (kbase + j <= qi) ? fast_exp2(__fmaf_rn(p[j], scale_log2e, -mx)) : 0.f;
          psum += p[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) mx = fmaxf(mx, p[j]);
        mx = __fmul_rn(mx, scale_log2e);
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          p[j] = fast_exp2(__fmaf_rn(p[j], scale_log2e, -mx));
          psum += p[j];
        }
      }
      if (it > 0) {  // PV(it-1) complete: P may be overwritten, O(it-1) can be read
        ok = mbar_wait_warp(o_full, ph ^ 1u, abort_flag, err, 19);
        if (!ok) break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      {
        float *x = xch + (it & 1) * 4 * TA_BQ;
        x[g * TA_BQ + r] = mx;
        x[(2 + g) * TA_BQ + r] = psum;
      }
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        unsigned hi[32], lo[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          unsigned hbits;
          asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hbits) : "f"(p[c0 + j]));
          hi[j] = hbits;
          // exact remainder; the tensor core reads its leading 11 bits
          lo[j] = __float_as_uint(p[c0 + j] - __uint_as_float(hbits));
        }
        tc_st32(lane_base + TA_PHI_COL + (unsigned)(g * 64 + c0), hi);
        tc_st32(lane_base + TA_PLO_COL + (unsigned)(g * 64 + c0), lo);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      if (stamp && it == 0 && warp == 2 && lane == 0) timeline[4] = global_timer();
      if (it > 0) drain(it - 1);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok) ok = mbar_wait_warp(o_full, (unsigned)(ntiles - 1) & 1u, abort_flag, err, 19);
    if (ok) {
      if (stamp && warp == 2 && lane == 0) timeline[5] = global_timer();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      drain(ntiles - 1);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    bool finish = ok && !*abort_flag;
    bool cta_out = true;  // uniform over the CTA: false for a chunk's CTA that does not merge
    float l_tot = l_run;

    if (nchunks > 1) {
      // Leave this chunk's partial in scratch; the last CTA of the query tile merges.
      const long long bh = (long long)b * gridDim.y + h;
      const long long first_item = bh * gridDim.x + (blockIdx.x - chunk);
      float *mine = part + (first_item + chunk) * TA_PART;
      // partial outputs as [column / 4][row][4]: the 32 rows of a warp are contiguous
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        reinterpret_cast<float4 *>(mine)[(g * 8 + j / 4) * TA_BQ + r] = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
      if (g == 0) {
        mine[TA_BQ * TA_DH + r] = m_run;
        mine[TA_BQ * TA_DH + TA_BQ + r] = l_tot;
      }
      if (stamp && warp == 2 && lane == 0) timeline[12] = global_timer();
      // The partial outputs come into the merging CTA's shared memory (the operand tiles are dead
      // by then) as bulk copies that are all in flight together, so that the merge costs one L2
      // round trip and not one per chunk; the maxima and sums are read directly meanwhile.
      auto fetch = [&](int first) {
        const int n = min(TA_MERGE_SLOTS, nchunks - first);
        const bool own = chunk >= first && chunk < first + n;  // this CTA's chunk is still in its registers
        asm volatile("fence.proxy.async;" ::: "memory");
        mbar_expect_tx(m_full, (unsigned)((n - (own ? 1 : 0)) * TA_O_BYTES));
        for (int j = 0; j < n; ++j)
          if (first + j != chunk)
            bulk_load(base + (unsigned)(j * TA_O_BYTES), part + (first_item + first + j) * TA_PART,
                      (unsigned)TA_O_BYTES, m_full);
      };
      asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");  // every thread's stores are issued
      if (stamp && warp == 2 && lane == 0) timeline[13] = global_timer();
      int *counter = counters + bh * tiles + qt;
      if (warp == 2 && lane == 0) {
        __threadfence();  // cumulative over the stores ordered before it by the barrier
        const int prev = atomicAdd(counter, 1);
        const int last = (prev == nchunks - 1) ? 1 : 0;
        if (last) {
          *counter = 0;  // ready for the next launch
          __threadfence();
          fetch(0);
        }
        *last_flag = last;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");
      const bool merging = *last_flag != 0;  // uniform over the CTA
      finish = finish && merging;
      cta_out = merging;
      if (stamp && warp == 2 && lane == 0) timeline[14] = global_timer();
      if (merging) {
        float wv[TA_MAX_CHUNKS], lv[TA_MAX_CHUNKS];
#pragma unroll
        for (int j = 0; j < TA_MAX_CHUNKS; ++j) {
          const float *pj = part + (first_item + min(j, nchunks - 1)) * TA_PART + TA_BQ * TA_DH;
          wv[j] = __ldcg(pj + r);
          lv[j] = __ldcg(pj + TA_BQ + r);
        }
        float mm = TA_NEG;
#pragma unroll
        for (int j = 0; j < TA_MAX_CHUNKS; ++j)
          if (j < nchunks) mm = fmaxf(mm, wv[j]);
        float ll = 0.f;
#pragma unroll
        for (int j = 0; j < TA_MAX_CHUNKS; ++j) {
          wv[j] = j < nchunks ? fast_exp2(wv[j] - mm) : 0.f;
          ll = fmaf(lv[j], wv[j], ll);
        }
        float acc[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) acc[c] = 0.f;
        // Chunks are combined in chunk order.
#pragma unroll 1
        for (int first = 0, batch = 0; first < nchunks; first += TA_MERGE_SLOTS, ++batch) {
          if (batch > 0) {
            asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");  // the slots have been read
            if (warp == 2 && lane == 0) fetch(first);
          }
          const bool got = mbar_wait_warp(m_full, (unsigned)batch & 1u, abort_flag, err, 20);
          finish = finish && got;
          if (stamp && batch == 0 && warp == 2 && lane == 0) timeline[15] = global_timer();
          const int n = got ? min(TA_MERGE_SLOTS, nchunks - first) : 0;
#pragma unroll 1
          for (int j = 0; j < n; ++j) {
            const float4 *ps = reinterpret_cast<const float4 *>(base_ptr + j * TA_O_BYTES) + g * 8 * TA_BQ + r;
            const float w = wv[first + j];
            if (first + j == chunk) {  // uniform over the CTA
#pragma unroll
              for (int c = 0; c < 32; ++c) acc[c] = fmaf(o[c], w, acc[c]);
            } else {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const float4 t = ps[c * TA_BQ];
                acc[4 * c] = fmaf(t.x, w, acc[4 * c]);
                acc[4 * c + 1] = fmaf(t.y, w, acc[4 * c + 1]);
                acc[4 * c + 2] = fmaf(t.z, w, acc[4 * c + 2]);
                acc[4 * c + 3] = fmaf(t.w, w, acc[4 * c + 3]);
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = acc[c];
        asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");  // before the output is staged over the slots
        l_tot = ll;
      }
    }

    if (stamp && warp == 2 && lane == 0) timeline[6] = global_timer();
    // Output: a thread holds 32 columns of one row, so direct stores would touch 32
    // different lines per instruction. Normalise, transpose through the (now idle) Q
    // tile in shared memory, and store whole rows.
    if (!cta_out) {
      // nothing to store: another CTA merges this chunk
    } else if (ctx_f16.hi != nullptr) {
      // fp16 pair with one scale per row of this head's 64 columns. The two threads of a row
      // exchange their largest magnitudes and convert before staging, so the store loop only copies.
      float *amx = reinterpret_cast<float *>(base_ptr + TA_AMAX_OFF);  // [2][128]
      unsigned char *st_hi = base_ptr + TA_Q_OFF;                      // [128][TA_STAGE16_LD] bytes
      unsigned char *st_lo = st_hi + TA_BQ * TA_STAGE16_LD;
      const float inv = finish ? 1.0f / l_tot : 0.f;
      float am = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        o[j] *= inv;
        am = fmaxf(am, fabsf(o[j]));
      }
      amx[g * TA_BQ + r] = am;
      asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");
      am = fmaxf(amx[r], amx[TA_BQ + r]);
      float sinv;
      const float scale = f16_block_scale(am, &sinv);
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint2 h0, l0, h1, l1;
        f16_pair4(make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]), scale, h0, l0);
        f16_pair4(make_float4(o[j + 4], o[j + 5], o[j + 6], o[j + 7]), scale, h1, l1);
        *reinterpret_cast<uint4 *>(st_hi + r * TA_STAGE16_LD + g * 64 + j * 2) = make_uint4(h0.x, h0.y, h1.x, h1.y);
        *reinterpret_cast<uint4 *>(st_lo + r * TA_STAGE16_LD + g * 64 + j * 2) = make_uint4(l0.x, l0.y, l1.x, l1.y);
      }
      if (finish && g == 0 && q0 + r < s)
        ctx_f16.inv_scale[((long long)row0 + q0 + r) * (d_model / TC_F16_SLOT) + h] = sinv;
      asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");
      if (finish) {
        const int t2 = threadIdx.x - 64;
#pragma unroll
        for (int i = 0; i < TA_BQ * 8 / TA_SOFTMAX_THREADS; ++i) {  // 8 lanes x 16 bytes = one row of 64 halves
          const int u = t2 + i * TA_SOFTMAX_THREADS;
          const int row = u >> 3, seg = u & 7;
          if (q0 + row < s) {
            const long long off = ((long long)row0 + q0 + row) * d_model + h * TA_DH + seg * 8;
            *reinterpret_cast<uint4 *>(ctx_f16.hi + off) =
                *reinterpret_cast<const uint4 *>(st_hi + row * TA_STAGE16_LD + seg * 16);
            *reinterpret_cast<uint4 *>(ctx_f16.lo + off) =
                *reinterpret_cast<const uint4 *>(st_lo + row * TA_STAGE16_LD + seg * 16);
          }
        }
      }
    } else {
      float *stage = reinterpret_cast<float *>(base_ptr + TA_Q_OFF);  // [128][TA_STAGE_LD]
      if (finish) {
        const float inv = 1.0f / l_tot;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(stage + r * TA_STAGE_LD + g * 32 + j) =
              make_float4(o[j] * inv, o[j + 1] * inv, o[j + 2] * inv, o[j + 3] * inv);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(TA_SOFTMAX_THREADS) : "memory");
      if (finish) {
        const int t2 = threadIdx.x - 64;
#pragma unroll 1  // runs once per CTA: a short loop is fetched once, eight copies of it eight times
        for (int i = 0; i < TA_BQ * TA_DH / 4 / TA_SOFTMAX_THREADS; ++i) {
          const int u = t2 + i * TA_SOFTMAX_THREADS;
          const int row = u >> 4, c4 = u & 15;
          if (q0 + row < s) {
            const float4 v = *reinterpret_cast<const float4 *>(stage + row * TA_STAGE_LD + c4 * 4);
            float4 hh, ll;
            split_tf32(v.x, hh.x, ll.x);
            split_tf32(v.y, hh.y, ll.y);
            split_tf32(v.z, hh.z, ll.z);
            split_tf32(v.w, hh.w, ll.w);
            const long long off = ((long long)row0 + q0 + row) * d_model + h * TA_DH + c4 * 4;
            *reinterpret_cast<float4 *>(ctx_hi + off) = hh;
            *reinterpret_cast<float4 *>(ctx_lo + off) = ll;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (timeline != nullptr && threadIdx.x == 0) {
    const unsigned long long t = global_timer();
    atomicMax(timeline + 9, t);
    // which CTA ended last: time in the high bits, blockIdx.x and the merge flag in the low 12
    atomicMax(timeline + 11, (t << 12) | (unsigned long long)((blockIdx.x & 0x3ff) << 1) | (unsigned long long)(*last_flag & 1));
    if (stamp) timeline[7] = t;
  }
}

}  // namespace

bool attention_tc_supports(int n_heads, int d_model) {
  return n_heads > 0 && d_model == n_heads * TA_DH;
}

AttentionPlan attention_tc_plan(int n_streams, int s, int n_heads) {
  AttentionPlan p{};
  const int tiles = (s + TA_BQ - 1) / TA_BQ;
  const long long bh = (long long)n_streams * n_heads;
  const long long units = bh * tiles * (tiles + 1) / 2;  // (query tile, key tile) pairs
  // One CTA per SM (all of tensor memory, 192 KB of tiles). Without a split the
  // longest CTA walks `tiles` key tiles; split when that leaves SMs idle.
  int kc = tiles;
  // Two key tiles a CTA walks itself: one more tile (2 us) costs less than the publish / fetch /
  // merge round trip of a split (5 us); from three tiles on the split is as fast or faster.
  if (bh * tiles < 148 && tiles > 2) {
    long long per_cta = (units + 147) / 148;
    if (per_cta < 1) per_cta = 1;
    if (per_cta < tiles) kc = (int)per_cta;
  }
  // The rounding of the chunk counts can still leave more CTAs than SMs (8 heads x 8 tiles at 2 key
  // tiles per CTA: 160): a second wave costs more than a longer walk.
  auto ctas_at = [&](int c) {
    long long n = 0;
    for (int qt = 0; qt < tiles; ++qt) n += ta_chunks_of(qt, c);
    return n * bh;
  };
  if (kc < tiles)
    while (kc < tiles && ctas_at(kc) > 148) ++kc;
  while (ta_chunks_of(tiles - 1, kc) > TA_MAX_CHUNKS) ++kc;
  p.kc = kc;
  int ctas = 0;
  bool split = false;
  for (int qt = 0; qt < tiles; ++qt) {
    ctas += ta_chunks_of(qt, kc);
    split = split || ta_chunks_of(qt, kc) > 1;
  }
  p.ctas_per_head = ctas;
  p.scratch_floats = split ? (size_t)bh * ctas * TA_PART : 0;
  p.counters = split ? (size_t)bh * tiles : 0;
  return p;
}

void launch_attention_tc(const TcMatrix &qk, const TcMatrix &vt, float *ctx_hi, float *ctx_lo, int n_streams, int s,
                         int n_heads, int d_model, float *scratch, int *counters, const LoopState *state,
                         DevErr *err, cudaStream_t st, unsigned long long *timeline, const TcPairF16 *ctx_f16) {
  if (!attention_tc_supports(n_heads, d_model))
    throw std::invalid_argument("litnice_b200: tensor-core attention needs head_dim 64");
  const AttentionPlan plan = attention_tc_plan(n_streams, s, n_heads);
  if (plan.scratch_floats > 0 && (scratch == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: attention needs scratch for this shape");
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    LB_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM));
    configured[dev] = true;
  }
  dim3 grid(plan.ctas_per_head, n_heads, n_streams);
  launch_pdl(attention_tc_kernel, grid, dim3(TA_THREADS), (size_t)TA_SMEM, st, g_pdl_enabled, qk.hi, qk.lo, vt.hi,
             vt.lo, ctx_hi, ctx_lo, s, d_model, (float)(1.4426950408889634 / sqrt((double)TA_DH)), plan.kc, scratch, counters, state, err,
             timeline, ctx_f16 ? *ctx_f16 : TcPairF16{});
}

}  // namespace lb
