// Fused causal self-attention on the sm_100a tensor cores with fp16-pair operands
// (tcgen05 + TMEM + TMA), head dimension 64, fp32-grade accuracy by three products.
//
// Same maths and the same schedule as attention_tc.cu (litnicelm
// src/model/algo/self_attention_fused_inplace.cpp:82-94: gemm_batched_rhs_t,
// scaled_causal_softmax_rows, gemm_batched; device_backend.cpp:1561-1577), but Q, K
// and V^T arrive as fp16 pairs (x * scale = hi + lo) under scales that are fixed when the
// weights are loaded: every row of LayerNorm(x) has a bounded length, so |q|, |k|, |v| of a
// head are bounded by a quantity of the weights alone, and one power of two per head and
// operand keeps every value inside fp16's range with 22 significant bits at the usual
// magnitudes. No per-row scales: the three scalars of a head leave in the exponent's
// factor (Q, K) and in the final normalisation (V). An fp16 instruction covers 16 of k
// at the rate a TF32 instruction covers 8, and the tiles are half the bytes, which makes
// room for two stages of K and V^T tiles: the loads of tile t+1 are in flight while tile
// t is multiplied (with one stage they sat between two products of the dependent chain).
//
//   S = Q K^T   A = Q tile (128 queries x 64), B = K tile (128 keys x 64), K-major fp16
//               pairs; one chain of 12 instructions (N = 128) in tensor memory.
//   P           eight warps read S (thread = one query row and 64 of the 128 keys),
//               scale, mask and exponentiate against the maximum of their own 64 keys,
//               and store P * 2^12 as an fp16 pair over their own columns of S (two keys
//               per column: the pair takes exactly the columns the scores had).
//   O += P V    A = P from tensor memory, B = V^T tile (64 x 128 keys, K-major), two
//               chains (64 keys each) of 12 instructions (N = 64), rescaled to the row's
//               running maximum and added into fp32 registers by the same threads (each
//               32 of the 64 output columns).
// Tensor memory holds two S/P buffers and two O buffers (tile t uses buffers t mod 2), so
// no product waits for the softmax threads to finish with the previous tile's buffers
// (with single buffers every tile paid the chain P stored -> P V -> accumulators read back
// -> next P stored). Measured on the config-4 batch, attention launches of one forward:
// 23.4 ms on TF32 pairs with one stage of K and V^T; 17.8 ms on fp16 pairs with two stages
// and single tensor-memory buffers, two or four threads per row alike (19.0 ms); 17.3 ms
// with these buffers; four threads per row with two S/P buffers and one set of four O
// chains: 19.2 ms. The steps of a tile (24 + 12 instructions of 64 and 128 columns, about
// 1.4 us; the softmax threads' loop; the hand-overs between them) are of similar length.
//
// Warp 0 issues TMA, warp 1 owns tensor memory and issues the MMAs (S of tile t+2 behind
// P V of tile t), warps 2-9 do the softmax and the output. Key ranges of a
// query tile may be cut into chunks for separate CTAs whose partial results the last
// CTA to finish merges in chunk order. Every mbarrier wait is bounded; no cluster
// launch and no multicast.
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

#include <mutex>

namespace lb {

namespace {

constexpr int TB_BQ = 128;   // query rows per CTA (one UMMA M = 128 tile)
constexpr int TB_BK = 128;   // keys per tile
constexpr int TB_DH = 64;    // head dimension
#ifndef LB_ATTN16_GROUPS
#define LB_ATTN16_GROUPS 2
#endif
constexpr int TB_G = LB_ATTN16_GROUPS;  // threads per query row = accumulation chains of P V per key tile
constexpr int TB_KPT = TB_BK / TB_G;    // keys per thread and tile
constexpr int TB_OC = TB_DH / TB_G;     // output columns per thread
static_assert(TB_G == 2, "two S/P and two O buffers of G chains each fill the 512 columns at G = 2");
constexpr int TB_SOFTMAX_THREADS = 128 * TB_G;
constexpr int TB_THREADS = 64 + TB_SOFTMAX_THREADS;
constexpr float TB_NEG = -3.402823466e+38f;
constexpr int TB_MAX_CHUNKS = 16;                   // as attention_tc_plan cuts them
constexpr int TB_PART = TB_BQ * TB_DH + 2 * TB_BQ;  // floats of one partial: o[128][64], m[128], l[128]
constexpr int TB_O_BYTES = TB_BQ * TB_DH * 4;       // the o part of a partial
constexpr int TB_MERGE_SLOTS = 5;  // partial outputs the merging CTA holds in shared memory at a time (over the tiles)
constexpr float TB_P_SCALE = 4096.f;  // probabilities are stored times 2^12: 22 bits down to p = 2^-15
constexpr float TB_P_INV = 1.f / 4096.f;

// shared memory (after 1024-byte alignment)
constexpr int TB_SLAB = TB_BQ * 128;         // 128 rows x 64 halves: the hi or the lo part of a Q or K tile
constexpr int TB_Q_BYTES = 2 * TB_SLAB;
constexpr int TB_K_BYTES = 2 * TB_SLAB;      // per stage
constexpr int TB_VSLAB = TB_DH * 128;        // 64 rows of V^T x 64 keys: one chain's hi or lo part
constexpr int TB_V_BYTES = 4 * TB_VSLAB;     // per stage: hi chain 0, hi chain 1, lo chain 0, lo chain 1
constexpr int TB_STAGES = 2;
constexpr int TB_Q_OFF = 0;
constexpr int TB_K_OFF = TB_Q_OFF + TB_Q_BYTES;
constexpr int TB_V_OFF = TB_K_OFF + TB_STAGES * TB_K_BYTES;
constexpr int TB_BAR_OFF = TB_V_OFF + TB_STAGES * TB_V_BYTES;  // 14 barriers + holders
constexpr int TB_XCH_SLOTS = 4;  // a warp may be one tile ahead of another that still reads the slot of two tiles ago
constexpr int TB_XCH_OFF = TB_BAR_OFF + 256;  // [slot = tile mod 4][maxima of the G key groups, their sums][128]
constexpr int TB_AMAX_OFF = TB_XCH_OFF + TB_XCH_SLOTS * 2 * TB_G * TB_BQ * 4;  // [G][128 rows]: largest magnitudes of the output rows
constexpr int TB_SMEM = TB_AMAX_OFF + TB_G * TB_BQ * 4 + 1024;
constexpr int TB_STAGE16_LD = TB_DH * 2 + 16;  // bytes per row of the staged fp16 output tile: conflict-free 16-byte accesses
static_assert(TB_MERGE_SLOTS * TB_O_BYTES <= TB_BAR_OFF, "merge slots overlay the operand tiles only");
static_assert(2 * TB_BQ * TB_STAGE16_LD <= TB_BAR_OFF, "output staging overlays the operand tiles only");

// tensor-memory columns: buffer b of S/P at 128 b (S: one column per key; the P pair of key group g
// over that group's own columns: high parts at g * KPT, low parts at g * KPT + KPT / 2, two keys per
// column), buffer b of O at 256 + 128 b (G chains of 64 columns)
__device__ __forceinline__ constexpr unsigned tb_s_col(int b) { return (unsigned)(b * TB_BK); }
__device__ __forceinline__ constexpr unsigned tb_phi_col(int b, int g) { return (unsigned)(b * TB_BK + g * TB_KPT); }
__device__ __forceinline__ constexpr unsigned tb_plo_col(int b, int g) { return (unsigned)(b * TB_BK + g * TB_KPT + TB_KPT / 2); }
__device__ __forceinline__ constexpr unsigned tb_o_col(int b) { return (unsigned)(2 * TB_BK + b * TB_G * TB_DH); }
static_assert(2 * TB_BK + 2 * TB_G * TB_DH <= 512, "tensor memory");

__device__ __forceinline__ float fast_exp2_16(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__host__ __device__ inline int tb_chunks_of(int qt, int kc) { return (qt + kc) / kc; }  // ceil((qt+1)/kc)

__global__ void __launch_bounds__(TB_THREADS, 1)
attention_tc16_kernel(const __grid_constant__ CUtensorMap map_qk_hi, const __grid_constant__ CUtensorMap map_qk_lo,
                      const __grid_constant__ CUtensorMap map_vt_hi, const __grid_constant__ CUtensorMap map_vt_lo,
                      const float *__restrict__ head_inv_scale, int s_cap, int d_model, float scale_log2e, int kc,
                      float *__restrict__ part, int *__restrict__ counters, const LoopState *state, DevErr *err,
                      unsigned long long *timeline, TcPairF16 ctx_f16) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bar_base = base + TB_BAR_OFF;
  // Per buffer b = tile mod 2 (use j = tile / 2 of a buffer completes phase j of its barriers; no barrier
  // can complete two phases before its waiter has seen the first: every arrival of use j + 1 depends,
  // through the other barriers, on the waiter having passed use j):
  //   s_full[b]   S complete (tcgen05.commit)            -> softmax threads
  //   p_ready[b]  P stored over S (every softmax warp)   -> MMA warp
  //   o_full[b]   P V complete (commit)                  -> softmax threads (read O), MMA warp (S/P buffer free)
  //   o_free[b]   O read back (every softmax warp)       -> MMA warp
  const unsigned q_full = bar_base, m_full = bar_base + 8;
  auto k_full = [&](int st) { return bar_base + 16u + 8u * st; };
  auto v_full = [&](int st) { return bar_base + 32u + 8u * st; };
  auto k_free = [&](int st) { return bar_base + 48u + 8u * st; };
  auto v_free = [&](int st) { return bar_base + 64u + 8u * st; };
  auto s_full = [&](int b) { return bar_base + 80u + 8u * b; };
  auto p_ready = [&](int b) { return bar_base + 96u + 8u * b; };
  auto o_full = [&](int b) { return bar_base + 112u + 8u * b; };
  auto o_free = [&](int b) { return bar_base + 128u + 8u * b; };
  volatile unsigned *tmem_holder = reinterpret_cast<volatile unsigned *>(base_ptr + TB_BAR_OFF + 160);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + TB_BAR_OFF + 164);
  volatile int *last_flag = reinterpret_cast<volatile int *>(base_ptr + TB_BAR_OFF + 168);
  // per tile (slot = tile mod 4): maximum [group][row] and sum [group][row] of each thread's keys
  float *xch = reinterpret_cast<float *>(base_ptr + TB_XCH_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The grid is laid out for s_cap; the actual length shares its tile count.
  const int s = state ? state->s : s_cap;
  const int tiles = (s_cap + TB_BQ - 1) / TB_BQ;
  int idx = blockIdx.x, qt = tiles - 1;
  for (; qt > 0; --qt) {  // (query tile, chunk) pairs, longest query tiles first
    const int nc = tb_chunks_of(qt, kc);
    if (idx < nc) break;
    idx -= nc;
  }
  const int chunk = idx, nchunks = tb_chunks_of(qt, kc);
  const int kt_begin = chunk * kc, kt_end = min(qt + 1, kt_begin + kc);
  const int ntiles = kt_end - kt_begin;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * TB_BQ;
  const int row0 = b * s;  // first row of this stream in the packed activations

  pdl_launch_dependents();
  // Measurement aid (as attention_tc.cu): the CTA of head 0, stream 0 that takes the diagonal tile of the
  // last query tile stamps its milestones in timeline[0..7]; every CTA contributes to the earliest start
  // [8], the latest end [9], the latest start [10] and the earliest return of the dependency wait [16].
  const bool stamp = timeline != nullptr && (int)blockIdx.x == tb_chunks_of(tiles - 1, kc) - 1 && blockIdx.y == 0 && blockIdx.z == 0;
  if (timeline != nullptr && threadIdx.x == 0) {
    const unsigned long long t = global_timer();
    atomicMin(timeline + 8, t);
    atomicMax(timeline + 10, t);
    if (stamp) timeline[0] = t;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(m_full, 1);
    for (int st = 0; st < TB_STAGES; ++st) {
      mbar_init(k_full(st), 1);
      mbar_init(v_full(st), 1);
      mbar_init(k_free(st), 1);
      mbar_init(v_free(st), 1);
      mbar_init(s_full(st), 1);
      mbar_init(p_ready(st), TB_SOFTMAX_THREADS / 32);  // one arrival per softmax warp
      mbar_init(o_full(st), 1);
      mbar_init(o_free(st), TB_SOFTMAX_THREADS / 32);
    }
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
    // ---- TMA producer: Q once, then K and V^T of each key tile, two stages each ----
    if (lane == 0) {
      tma_prefetch_map(&map_qk_hi);
      tma_prefetch_map(&map_qk_lo);
      tma_prefetch_map(&map_vt_hi);
      tma_prefetch_map(&map_vt_lo);
    }
    pdl_wait();
    if (lane == 0) {
      if (timeline != nullptr) atomicMin(timeline + 16, global_timer());  // the predecessor has completed
      mbar_expect_tx(q_full, (unsigned)TB_Q_BYTES);
      tma_load_2d(base + TB_Q_OFF, &map_qk_hi, h * TB_DH, row0 + q0, q_full);
      tma_load_2d(base + TB_Q_OFF + TB_SLAB, &map_qk_lo, h * TB_DH, row0 + q0, q_full);
    }
    __syncwarp();
    int k_issued = 0, v_issued = 0;
    auto load_k = [&](int it) {
      if (lane == 0) {
        const int st = it & 1, k0 = (kt_begin + it) * TB_BK;
        const unsigned dst = base + TB_K_OFF + (unsigned)st * TB_K_BYTES;
        mbar_expect_tx(k_full(st), (unsigned)TB_K_BYTES);
        tma_load_2d(dst, &map_qk_hi, d_model + h * TB_DH, row0 + k0, k_full(st));
        tma_load_2d(dst + TB_SLAB, &map_qk_lo, d_model + h * TB_DH, row0 + k0, k_full(st));
      }
      __syncwarp();
      ++k_issued;
    };
    auto load_v = [&](int it) {
      if (lane == 0) {
        const int st = it & 1, k0 = (kt_begin + it) * TB_BK;
        const unsigned dst = base + TB_V_OFF + (unsigned)st * TB_V_BYTES;
        mbar_expect_tx(v_full(st), (unsigned)TB_V_BYTES);
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(dst + c * TB_VSLAB, &map_vt_hi, k0 + c * 64, b * d_model + h * TB_DH, v_full(st));
          tma_load_2d(dst + (2 + c) * TB_VSLAB, &map_vt_lo, k0 + c * 64, b * d_model + h * TB_DH, v_full(st));
        }
      }
      __syncwarp();
      ++v_issued;
    };
    load_k(0);
    load_v(0);
    if (ntiles > 1) {
      load_k(1);
      load_v(1);
    }
    // In the tensor pipe's order ... S(t-2), P V(t-2), S(t-1) ...: the stage of K(t) is free once S(t-2)
    // has completed, the stage of V^T(t) once P V(t-2) has.
    bool ok = true;
    for (int it = 2; it < ntiles && ok; ++it) {
      const unsigned ph = (unsigned)((it >> 1) - 1) & 1u;
      ok = mbar_wait_warp(k_free(it & 1), ph, abort_flag, err, 11);
      if (!ok) break;
      load_k(it);
      ok = mbar_wait_warp(v_free(it & 1), ph, abort_flag, err, 12);
      if (!ok) break;
      load_v(it);
    }
    if (*abort_flag) {
      // let copies already in flight land before the CTA's shared memory goes away
      const unsigned long long t0 = global_timer();
      while (!mbar_try_wait(q_full, 0u))
        if (global_timer() - t0 > WAIT_LIMIT_NS) break;
      for (int j = max(0, k_issued - TB_STAGES); j < k_issued; ++j)
        while (!mbar_try_wait(k_full(j & 1), (unsigned)(j >> 1) & 1u))
          if (global_timer() - t0 > 2 * WAIT_LIMIT_NS) break;
      for (int j = max(0, v_issued - TB_STAGES); j < v_issued; ++j)
        while (!mbar_try_wait(v_full(j & 1), (unsigned)(j >> 1) & 1u))
          if (global_timer() - t0 > 3 * WAIT_LIMIT_NS) break;
    }
  } else if (warp == 1) {
    // ---- MMA issuer: S(0), S(1), then per tile P V(it) and, once it has completed (P of tile it lies
    //      over S of tile it), S(it+2) into the same buffer ----
    const unsigned idesc_s = umma_idesc_f16(TB_BK);   // N = 128 keys
    const unsigned idesc_o = umma_idesc_f16(TB_DH);   // N = 64 output columns
    auto issue_s = [&](int it) {  // one chain: S = Q K^T over the 64 head dimensions, 16 per instruction
      const int st = it & 1;
      const unsigned tmem_d = tmem_base + tb_s_col(st);
      const unsigned kb = base + TB_K_OFF + (unsigned)st * TB_K_BYTES;
      const unsigned long long a_hi = umma_desc_k128(base + TB_Q_OFF);
      const unsigned long long a_lo = umma_desc_k128(base + TB_Q_OFF + TB_SLAB);
      const unsigned long long b_hi = umma_desc_k128(kb);
      const unsigned long long b_lo = umma_desc_k128(kb + TB_SLAB);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
        tc_mma_f16(tmem_d, a_lo + adv, b_hi + adv, idesc_s, ks == 0 ? 0u : 1u);
        tc_mma_f16(tmem_d, a_hi + adv, b_lo + adv, idesc_s, 1u);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
        tc_mma_f16(tmem_d, a_hi + adv, b_hi + adv, idesc_s, 1u);
      }
      tc_commit(s_full(st));   // S complete
      tc_commit(k_free(st));   // and this stage of K may be overwritten
    };
    bool ok = mbar_wait_warp(q_full, 0u, abort_flag, err, 13);
    for (int it = 0; it < min(2, ntiles) && ok; ++it) {
      ok = mbar_wait_warp(k_full(it), 0u, abort_flag, err, 14);
      if (!ok) break;
      if (stamp && it == 0 && lane == 0) timeline[2] = global_timer();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) issue_s(it);
      __syncwarp();
    }
    int pv_commits = 0;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int b = it & 1;
      const unsigned ph = (unsigned)(it >> 1) & 1u;
      ok = mbar_wait_warp(p_ready(b), ph, abort_flag, err, 15);  // P(it) stored
      if (ok) ok = mbar_wait_warp(v_full(b), ph, abort_flag, err, 16);
      if (ok && it >= 2) ok = mbar_wait_warp(o_free(b), ph ^ 1u, abort_flag, err, 21);  // O(it-2) read back
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const unsigned vb = base + TB_V_OFF + (unsigned)b * TB_V_BYTES;
#pragma unroll
        for (int c = 0; c < TB_G; ++c) {
          // chain c covers the keys one softmax thread scales by its own maximum
          const unsigned tmem_d = tmem_base + tb_o_col(b) + (unsigned)(c * TB_DH);
          const unsigned p_hi = tmem_base + tb_phi_col(b, c), p_lo = tmem_base + tb_plo_col(b, c);
          const int key0 = c * TB_KPT, slab = key0 / 64;  // a slab of the stage holds 64 keys (128-byte rows)
          const unsigned long long b_hi = umma_desc_k128(vb + slab * TB_VSLAB);
          const unsigned long long b_lo = umma_desc_k128(vb + (2 + slab) * TB_VSLAB);
#pragma unroll
          for (int ks = 0; ks < TB_KPT / 16; ++ks) {
            const unsigned long long adv = (unsigned long long)(((key0 % 64) + ks * 16) * 2 >> 4);
            const unsigned ac = (unsigned)(ks * 8);  // 16 keys = 8 columns
            tc_mma_f16_ts(tmem_d, p_lo + ac, b_hi + adv, idesc_o, ks == 0 ? 0u : 1u);
            tc_mma_f16_ts(tmem_d, p_hi + ac, b_lo + adv, idesc_o, 1u);
          }
#pragma unroll
          for (int ks = 0; ks < TB_KPT / 16; ++ks) {
            const unsigned long long adv = (unsigned long long)(((key0 % 64) + ks * 16) * 2 >> 4);
            const unsigned ac = (unsigned)(ks * 8);
            tc_mma_f16_ts(tmem_d, p_hi + ac, b_hi + adv, idesc_o, 1u);
          }
        }
        tc_commit(o_full(b));   // O chains complete; the S/P buffer may be overwritten
        tc_commit(v_free(b));   // and this stage of V^T
      }
      __syncwarp();
      ++pv_commits;
      if (it + 2 < ntiles) {
        // S(it+2) goes where P(it) lies: after P V(it) has completed (long before its softmax is due)
        ok = mbar_wait_warp(o_full(b), ph, abort_flag, err, 22);
        if (ok) ok = mbar_wait_warp(k_full(b), ph ^ 1u, abort_flag, err, 14);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) issue_s(it + 2);
        __syncwarp();
      }
    }
    if (!ok) {  // give the tensor pipe a bounded chance to finish before TMEM is freed
      const int b = pv_commits & 1;
      if (lane == 0) tc_commit(o_full(b));
      __syncwarp();
      const unsigned long long t0 = global_timer();
      while (!mbar_try_wait(o_full(b), (unsigned)(pv_commits >> 1) & 1u))
        if (global_timer() - t0 > WAIT_LIMIT_NS) break;
    }
    __syncwarp();
  } else {
    // ---- softmax + output: thread = query row `r`, key group `g` (TB_KPT of the 128 keys = one O chain;
    //      TB_OC of the 64 output columns) ----
    // The head's three fixed scales (immutable since the weights were loaded): Q and K in the
    // exponent's factor, V (and the 2^12 of P) in the final normalisation.
    const int n_blocks = d_model / TB_DH;
    const float qk_factor = scale_log2e * head_inv_scale[h] * head_inv_scale[n_blocks + h];
    const float out_factor = head_inv_scale[2 * n_blocks + h] * TB_P_INV;
    pdl_wait();  // scratch and ctx writes must follow the predecessor
    const int q = warp & 3;          // TMEM lane quarter this warp may touch
    const int g = (warp - 2) >> 2;   // warps 2-5: group 0, warps 6-9: group 1, ...
    const int r = q * 32 + lane;
    const int qi = q0 + r;
    const unsigned lane_base = tmem_base + ((unsigned)(q * 32) << 16);
    float o[TB_OC];
#pragma unroll
    for (int j = 0; j < TB_OC; ++j) o[j] = 0.f;
    // Running maximum (of scores times log2 e) and sum of the whole row; all
    // threads of a row keep identical copies.
    float m_run = TB_NEG, l_run = 0.f;
    bool ok = true;

    // O(t) = sum over chains c of chain c * 2^(m_c - M): each chain was scaled by the maximum of its own keys
    auto drain = [&](int t) {
      const float *x = xch + (t & (TB_XCH_SLOTS - 1)) * 2 * TB_G * TB_BQ;
      float mc[TB_G], pc[TB_G];
      float m_new = m_run;
#pragma unroll
      for (int c = 0; c < TB_G; ++c) {
        mc[c] = x[c * TB_BQ + r];
        pc[c] = x[(TB_G + c) * TB_BQ + r];
        m_new = fmaxf(m_new, mc[c]);
      }
      const float a = fast_exp2_16(m_run - m_new);
      unsigned cv[TB_G][16 * (TB_OC / 16)];
#pragma unroll
      for (int c = 0; c < TB_G; ++c)
#pragma unroll
        for (int j0 = 0; j0 < TB_OC; j0 += 16)
          tc_ld16(lane_base + tb_o_col(t & 1) + (unsigned)(c * TB_DH + g * TB_OC + j0),
                  *reinterpret_cast<unsigned(*)[16]>(&cv[c][j0]));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float ls = l_run * a;
#pragma unroll
      for (int j = 0; j < TB_OC; ++j) o[j] *= a;
#pragma unroll
      for (int c = 0; c < TB_G; ++c) {
        const float w = fast_exp2_16(mc[c] - m_new);
        ls = fmaf(pc[c], w, ls);
#pragma unroll
        for (int j = 0; j < TB_OC; ++j) o[j] = fmaf(__uint_as_float(cv[c][j]), w, o[j]);
      }
      l_run = ls;
      m_run = m_new;
    };

    for (int it = 0; it < ntiles && ok; ++it) {
      const int b = it & 1;
      const unsigned ph = (unsigned)(it >> 1) & 1u;
      const int kbase = (kt_begin + it) * TB_BK + g * TB_KPT;
      ok = mbar_wait_warp(s_full(b), ph, abort_flag, err, 18);
      if (!ok) break;
      if (stamp && it == 0 && warp == 2 && lane == 0) timeline[3] = global_timer();
      if (stamp && nchunks == 1 && it >= 1 && it <= 4 && warp == 2 && lane == 0) timeline[11 + it] = global_timer();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float p[TB_KPT];
      {
        unsigned t0[TB_KPT];
#pragma unroll
        for (int j0 = 0; j0 < TB_KPT; j0 += 16)
          tc_ld16(lane_base + tb_s_col(b) + (unsigned)(g * TB_KPT + j0), *reinterpret_cast<unsigned(*)[16]>(&t0[j0]));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");  // all of the thread's scores are in registers: P may go over them
#pragma unroll
        for (int j = 0; j < TB_KPT; ++j) p[j] = __uint_as_float(t0[j]);
      }
      // Raw scores of the scaled operands: the maximum commutes with the positive factor, and the factor
      // joins the subtraction in one fused multiply-add: p = 2^(s * c - max(s) * c). Only the tile on
      // the diagonal has keys past a query; the others skip the mask.
      // (maximum and sum as four interleaved partial chains: a single chain of dependent operations
      // is as long as the thread's keys)
      float mx4[4] = {TB_NEG, TB_NEG, TB_NEG, TB_NEG}, ps4[4] = {0.f, 0.f, 0.f, 0.f};
      float mx;
      if (kt_begin + it == qt) {
#pragma unroll
        for (int j = 0; j < TB_KPT; ++j)
          if (kbase + j <= qi) mx4[j & 3] = fmaxf(mx4[j & 3], p[j]);
        mx = __fmul_rn(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), qk_factor);
#pragma unroll
        for (int j = 0; j < TB_KPT; ++j) {
          p[j] = (kbase + j <= qi) ? fast_exp2_16(__fmaf_rn(p[j], qk_factor, -mx)) : 0.f;
          ps4[j & 3] += p[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < TB_KPT; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], p[j]);
        mx = __fmul_rn(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), qk_factor);
#pragma unroll
        for (int j = 0; j < TB_KPT; ++j) {
          p[j] = fast_exp2_16(__fmaf_rn(p[j], qk_factor, -mx));
          ps4[j & 3] += p[j];
        }
      }
      const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      {
        float *x = xch + (it & (TB_XCH_SLOTS - 1)) * 2 * TB_G * TB_BQ;
        x[g * TB_BQ + r] = mx;
        x[(TB_G + g) * TB_BQ + r] = psum;
      }
#pragma unroll
      for (int j0 = 0; j0 < TB_KPT / 2; j0 += 16) {
        // the thread's keys as columns of packed pairs, times 2^12
        unsigned hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a = p[2 * (j0 + j)] * TB_P_SCALE, c = p[2 * (j0 + j) + 1] * TB_P_SCALE;
          const __half2 h2 = __floats2half2_rn(a, c);
          const float2 f2 = __half22float2(h2);
          const __half2 l2 = __floats2half2_rn(a - f2.x, c - f2.y);
          hi[j] = *reinterpret_cast<const unsigned *>(&h2);
          lo[j] = *reinterpret_cast<const unsigned *>(&l2);
        }
        tc_st16(lane_base + tb_phi_col(b, g) + (unsigned)j0, hi);
        tc_st16(lane_base + tb_plo_col(b, g) + (unsigned)j0, lo);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      if (stamp && it == 0 && warp == 2 && lane == 0) timeline[4] = global_timer();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready(b));
      if (it > 0) {  // P V(it-1) is complete or under way: read its accumulators back and hand the buffer on
        ok = mbar_wait_warp(o_full(b ^ 1), (unsigned)((it - 1) >> 1) & 1u, abort_flag, err, 19);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        drain(it - 1);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free(b ^ 1));
      }
    }
    if (ok) ok = mbar_wait_warp(o_full((ntiles - 1) & 1), (unsigned)((ntiles - 1) >> 1) & 1u, abort_flag, err, 19);
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
      float *mine = part + (first_item + chunk) * TB_PART;
      // partial outputs as [column / 4][row][4]: the 32 rows of a warp are contiguous
#pragma unroll
      for (int j = 0; j < TB_OC; j += 4)
        reinterpret_cast<float4 *>(mine)[(g * (TB_OC / 4) + j / 4) * TB_BQ + r] =
            make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
      if (g == 0) {
        mine[TB_BQ * TB_DH + r] = m_run;
        mine[TB_BQ * TB_DH + TB_BQ + r] = l_tot;
      }
      if (stamp && warp == 2 && lane == 0) timeline[12] = global_timer();
      // The partial outputs come into the merging CTA's shared memory (the operand tiles are dead
      // by then: every tile that was requested has been multiplied) as bulk copies that are all in
      // flight together; the maxima and sums are read directly meanwhile.
      auto fetch = [&](int first) {
        const int n = min(TB_MERGE_SLOTS, nchunks - first);
        const bool own = chunk >= first && chunk < first + n;  // this CTA's chunk is still in its registers
        asm volatile("fence.proxy.async;" ::: "memory");
        mbar_expect_tx(m_full, (unsigned)((n - (own ? 1 : 0)) * TB_O_BYTES));
        for (int j = 0; j < n; ++j)
          if (first + j != chunk)
            bulk_load(base + (unsigned)(j * TB_O_BYTES), part + (first_item + first + j) * TB_PART,
                      (unsigned)TB_O_BYTES, m_full);
      };
      asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");  // every thread's stores are issued
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
      asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");
      const bool merging = *last_flag != 0;  // uniform over the CTA
      finish = finish && merging;
      cta_out = merging;
      if (stamp && warp == 2 && lane == 0) timeline[14] = global_timer();
      if (merging) {
        float wv[TB_MAX_CHUNKS], lv[TB_MAX_CHUNKS];
#pragma unroll
        for (int j = 0; j < TB_MAX_CHUNKS; ++j) {
          const float *pj = part + (first_item + min(j, nchunks - 1)) * TB_PART + TB_BQ * TB_DH;
          wv[j] = __ldcg(pj + r);
          lv[j] = __ldcg(pj + TB_BQ + r);
        }
        float mm = TB_NEG;
#pragma unroll
        for (int j = 0; j < TB_MAX_CHUNKS; ++j)
          if (j < nchunks) mm = fmaxf(mm, wv[j]);
        float ll = 0.f;
#pragma unroll
        for (int j = 0; j < TB_MAX_CHUNKS; ++j) {
          wv[j] = j < nchunks ? fast_exp2_16(wv[j] - mm) : 0.f;
          ll = fmaf(lv[j], wv[j], ll);
        }
        float acc[TB_OC];
#pragma unroll
        for (int c = 0; c < TB_OC; ++c) acc[c] = 0.f;
        // Chunks are combined in chunk order.
#pragma unroll 1
        for (int first = 0, batch = 0; first < nchunks; first += TB_MERGE_SLOTS, ++batch) {
          if (batch > 0) {
            asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");  // the slots have been read
            if (warp == 2 && lane == 0) fetch(first);
          }
          const bool got = mbar_wait_warp(m_full, (unsigned)batch & 1u, abort_flag, err, 20);
          finish = finish && got;
          if (stamp && batch == 0 && warp == 2 && lane == 0) timeline[15] = global_timer();
          const int n = got ? min(TB_MERGE_SLOTS, nchunks - first) : 0;
#pragma unroll 1
          for (int j = 0; j < n; ++j) {
            const float4 *ps = reinterpret_cast<const float4 *>(base_ptr + j * TB_O_BYTES) + g * (TB_OC / 4) * TB_BQ + r;
            const float w = wv[first + j];
            if (first + j == chunk) {  // uniform over the CTA
#pragma unroll
              for (int c = 0; c < TB_OC; ++c) acc[c] = fmaf(o[c], w, acc[c]);
            } else {
#pragma unroll
              for (int c = 0; c < TB_OC / 4; ++c) {
                const float4 t = ps[c * TB_BQ];
                acc[4 * c] = fmaf(t.x, w, acc[4 * c]);
                acc[4 * c + 1] = fmaf(t.y, w, acc[4 * c + 1]);
                acc[4 * c + 2] = fmaf(t.z, w, acc[4 * c + 2]);
                acc[4 * c + 3] = fmaf(t.w, w, acc[4 * c + 3]);
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < TB_OC; ++c) o[c] = acc[c];
        asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");  // before the output is staged over the slots
        l_tot = ll;
      }
    }

    if (stamp && warp == 2 && lane == 0) timeline[6] = global_timer();
    // Output as the fp16 pair the out-projection reads, one scale per row of this head's 64 columns.
    // A thread holds a few columns of one row, so direct stores would touch 32 different lines per
    // instruction: normalise, exchange the row's largest magnitudes, convert, transpose through the
    // (now idle) tiles in shared memory, and store whole rows.
    if (cta_out) {
      float *amx = reinterpret_cast<float *>(base_ptr + TB_AMAX_OFF);  // [G][128]
      unsigned char *st_hi = base_ptr + TB_Q_OFF;                      // [128][TB_STAGE16_LD] bytes
      unsigned char *st_lo = st_hi + TB_BQ * TB_STAGE16_LD;
      const float inv = finish ? out_factor / l_tot : 0.f;
      float am = 0.f;
#pragma unroll
      for (int j = 0; j < TB_OC; ++j) {
        o[j] *= inv;
        am = fmaxf(am, fabsf(o[j]));
      }
      amx[g * TB_BQ + r] = am;
      asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");
#pragma unroll
      for (int c = 0; c < TB_G; ++c) am = fmaxf(am, amx[c * TB_BQ + r]);
      float sinv;
      const float scale = f16_block_scale(am, &sinv);
#pragma unroll
      for (int j = 0; j < TB_OC; j += 8) {
        uint2 h0, l0, h1, l1;
        f16_pair4(make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]), scale, h0, l0);
        f16_pair4(make_float4(o[j + 4], o[j + 5], o[j + 6], o[j + 7]), scale, h1, l1);
        *reinterpret_cast<uint4 *>(st_hi + r * TB_STAGE16_LD + (g * TB_OC + j) * 2) = make_uint4(h0.x, h0.y, h1.x, h1.y);
        *reinterpret_cast<uint4 *>(st_lo + r * TB_STAGE16_LD + (g * TB_OC + j) * 2) = make_uint4(l0.x, l0.y, l1.x, l1.y);
      }
      if (finish && g == 0 && q0 + r < s)
        ctx_f16.inv_scale[((long long)row0 + q0 + r) * (d_model / TC_F16_SLOT) + h] = sinv;
      asm volatile("bar.sync 1, %0;" ::"n"(TB_SOFTMAX_THREADS) : "memory");
      if (finish) {
        const int t2 = threadIdx.x - 64;
#pragma unroll
        for (int i = 0; i < TB_BQ * 8 / TB_SOFTMAX_THREADS; ++i) {  // 8 lanes x 16 bytes = one row of 64 halves
          const int u = t2 + i * TB_SOFTMAX_THREADS;
          const int row = u >> 3, seg = u & 7;
          if (q0 + row < s) {
            const long long off = ((long long)row0 + q0 + row) * d_model + h * TB_DH + seg * 8;
            *reinterpret_cast<uint4 *>(ctx_f16.hi + off) =
                *reinterpret_cast<const uint4 *>(st_hi + row * TB_STAGE16_LD + seg * 16);
            *reinterpret_cast<uint4 *>(ctx_f16.lo + off) =
                *reinterpret_cast<const uint4 *>(st_lo + row * TB_STAGE16_LD + seg * 16);
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

// One block per 64 columns of a projection that follows a LayerNorm: the largest value any of
// them can take, and the power of two that brings it into [2^14, 2^15).
//   LN(x) = gamma * xhat + beta with |xhat|_2 <= sqrt(k)  =>  |LN(x) W[:, c] + b[c]| <=
//   sqrt(k) * |gamma * W[:, c]|_2 + |beta . W[:, c] + b[c]|      (sums in double)
__global__ void head_scale_kernel(const float *__restrict__ w, int k, int n, const float *__restrict__ gamma,
                                  const float *__restrict__ beta, const float *__restrict__ bias,
                                  float *__restrict__ scale, float *__restrict__ inv_scale) {
  __shared__ float bound[64];
  const int col = blockIdx.x * 64 + threadIdx.x;
  double s2 = 0.0, sb = 0.0;
  for (int kk = 0; kk < k; ++kk) {
    const double wv = (double)w[(long long)kk * n + col];
    const double gw = (double)gamma[kk] * wv;
    s2 += gw * gw;
    sb += (double)beta[kk] * wv;
  }
  if (bias != nullptr) sb += (double)bias[col];
  bound[threadIdx.x] = (float)((sqrt((double)k) * sqrt(s2) + fabs(sb)) * 1.001);  // margin for the rounding of the products
  __syncthreads();
  if (threadIdx.x == 0) {
    float am = 0.f;
    for (int j = 0; j < 64; ++j) am = fmaxf(am, bound[j]);
    int eb = (__float_as_int(am) >> 23) & 0xff;  // am = 1.m * 2^(eb - 127)
    if (!(am > 0.f) || eb < 20) eb = 141;        // nothing to scale: 2^0
    if (eb > 250) eb = 250;
    scale[blockIdx.x] = __int_as_float((268 - eb) << 23);      // 2^(141 - eb): am * scale in [2^14, 2^15)
    inv_scale[blockIdx.x] = __int_as_float((eb - 14) << 23);   // 2^(eb - 141)
  }
}

}  // namespace

void launch_head_scales(const float *w, int k, int n, const float *gamma, const float *beta, const float *bias,
                        float *scale, float *inv_scale, cudaStream_t st) {
  if (n % 64 != 0) throw std::invalid_argument("litnice_b200: head scales need n % 64 == 0");
  head_scale_kernel<<<n / 64, 64, 0, st>>>(w, k, n, gamma, beta, bias, scale, inv_scale);
  LB_LAUNCH_CHECK();
}

void launch_attention_tc16(const TcMatrix &qk, const TcMatrix &vt, const float *head_inv_scale, int n_streams, int s,
                           int n_heads, int d_model, float *scratch, int *counters, const LoopState *state,
                           DevErr *err, cudaStream_t st, unsigned long long *timeline, const TcPairF16 &ctx_f16) {
  if (!attention_tc_supports(n_heads, d_model))
    throw std::invalid_argument("litnice_b200: tensor-core attention needs head_dim 64");
  if (ctx_f16.hi == nullptr || head_inv_scale == nullptr)
    throw std::invalid_argument("litnice_b200: the fp16-pair attention needs the head scales and an fp16-pair output");
  const AttentionPlan plan = attention_tc_plan(n_streams, s, n_heads);
  if (plan.scratch_floats > 0 && (scratch == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: attention needs scratch for this shape");
  static std::mutex cfg_mu;         // sessions on several host threads (one per GPU) may launch at once
  static bool configured[64] = {};  // the attribute is per device
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(cfg_mu);
    if (dev >= 64 || !configured[dev]) {
      LB_CUDA(cudaFuncSetAttribute(attention_tc16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TB_SMEM));
      if (dev < 64) configured[dev] = true;
    }
  }
  dim3 grid(plan.ctas_per_head, n_heads, n_streams);
  launch_pdl(attention_tc16_kernel, grid, dim3(TB_THREADS), (size_t)TB_SMEM, st, g_pdl_enabled, qk.hi, qk.lo, vt.hi,
             vt.lo, head_inv_scale, s, d_model, (float)(1.4426950408889634 / sqrt((double)TB_DH)), plan.kc, scratch,
             counters, state, err, timeline, ctx_f16);
}

}  // namespace lb
