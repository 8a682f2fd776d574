// Tensor-core projection GEMM for sm_100a (tcgen05 + TMEM + TMA), fp32 accuracy
// by three products of operand pairs (fp16 pairs with block scales, or TF32
// pairs). Replaces, on the hot path, the sequence gemm_ranked_matrix_rhs +
// add_bias_rowwise (+ReLU) + add of the reference (litnicelm
// src/model/backend/device_backend.cpp:1112-1131, 840-940, 752-813).
//
// One CTA computes a 128 x BN tile of C (or its partial sums over one k range).
// Warp roles:
//   warp 0        one lane issues the TMA loads of the four operand tiles
//                 (A_hi, A_lo, B_hi, B_lo; 128-byte swizzle) into a ring of stages
//   warp 1        allocates tensor memory; one lane issues the tcgen05.mma
//                 instructions (3 products x 4 k-steps per stage) and commits
//   drain warps   tcgen05.ld of each finished accumulation chain (one TMEM lane
//                 quarter each) added into fp32 registers
//   helper warps  nothing until the store phase
// Store phase, by all warps: the tile is staged in shared memory (over the idle
// pipeline stages) and leaves row by row with every epilogue term applied (folded
// LayerNorm, bias, residual, ReLU; fp32 and / or the next product's operand pair;
// row statistics; the V third of a QKV projection transposed).
// Split-k: the CTAs of a tile form a thread-block cluster, each sends its partial
// sums of a row to the CTA that stores the row (remote shared-memory stores between
// two cluster barriers); through global scratch and a last-CTA reduction where a
// cluster cannot be used. No TMA multicast.
// Every wait on an mbarrier is bounded (about one second); a wait that runs out
// sets the error word, lets the pipeline drain and the kernel returns after
// freeing its tensor memory (the cluster barriers are executed unconditionally by
// every thread, so a CTA that gave up cannot leave its peers waiting).
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"
#include "gemm_tc_epilogue.cuh"

#include <cstdlib>
#include <mutex>

namespace lb {

namespace {

// Warps of a CTA: 2 role warps (TMA, MMA), then the drain warps (four per lane quarter set: 64
// accumulator columns per thread for tiles up to 128 columns, 128 for the 256-column tile), then
// helper warps that only take part in the store phase, which is bound by instruction latency and
// wants as many warps as the register file allows.
__host__ __device__ constexpr int tc_drain_warps(int bn) { return bn == 64 ? 4 : 8; }
__host__ __device__ constexpr int tc_threads(int bn) { return bn > 128 ? 384 : 512; }
template <int BN, int STAGES>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 4;  // 16 KiB
  static constexpr int B_BYTES = BN * TC_BK * 4;
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = TILES_BYTES;          // full[S], empty[S], tmem_full
  static constexpr int ROWSTATS_OFFSET = BAR_OFFSET + 256;  // float2 (mean, 1/std) per tile row
  static constexpr int TOTAL = TILES_BYTES + 256 + TC_BM * 8 + 1024;  // + barriers/holders, row statistics, alignment slack
};

// Tensor-core accumulation rounds toward zero: every tcgen05.mma that adds into
// a non-zero accumulator loses up to one ulp of it, always in the same
// direction (measured: ~3e-5 relative at k = 2048 with one long chain). So the
// k loop is cut into chunks of TC_CHUNK k-blocks: each chunk is accumulated in
// one of the TMEM buffers starting from zero, and the epilogue warps add the
// finished chunk into fp32 registers (round to nearest) while the next chunks
// are multiplied into the other buffers. All 512 TMEM columns are used as a
// ring of 512/BN buffers, which hides the MMA -> epilogue -> MMA hand-over
// latency (about a microsecond per round trip). Inside a k-block the two small products
// (a_lo*b_hi, a_hi*b_lo) are issued first, while the accumulator is still
// ~2^-11 of its final size, so only the a_hi*b_hi steps truncate at full scale.
#ifndef LB_TC_CHUNK
#define LB_TC_CHUNK 1
#endif
constexpr int TC_CHUNK = LB_TC_CHUNK;  // k-blocks (of 32) per TMEM accumulation chain


// F16: operands are fp16 pairs with block scales (see TcPairF16) instead of TF32
// pairs: a k-block is 64 elements (still one 128-byte row per tile row), the
// instructions are kind::f16 with K = 16, and the drain multiplies each chain by
// a_inv_scale[row][k-block] * b_inv_scale.
//
// WIDE (fp16 pairs, tiles up to 128 columns): the B_lo tile lies directly behind the
// B_hi tile in a stage, so one instruction of 2*BN columns multiplies a_hi by
// [b_hi | b_lo]: columns 0..BN-1 of the chain's buffer take a_hi*b_hi and columns
// BN..2BN-1 the two small products (a_hi*b_lo from the wide instruction, a_lo*b_hi from
// one of BN columns added there). Two instructions per k-step instead of three, the A_hi
// tile read once instead of twice: (32 + BN) + (32 + BN/2) clocks against 3*(32 + BN/2).
// The drain adds both halves of the buffer into the same registers.
template <int BN, int STAGES, bool F16, bool WIDE>
__global__ void __launch_bounds__(tc_threads(BN), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
               const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
               TcEpilogue ep, int m, int n, int k, int splits, float *__restrict__ part,
               int *__restrict__ counters, DevErr *err, const float *__restrict__ a_inv_scale,
               const float *__restrict__ b_inv_scale, int cluster_splits) {
  constexpr int KBE = F16 ? TC_F16_SLOT : TC_BK;  // k elements per k-block
  using L = TcSmem<BN, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bar_base = base + L::BAR_OFFSET;
  // barriers: full[S], empty[S], tmem_full[NBUF], tmem_empty[NBUF]
  static_assert(!WIDE || (F16 && BN <= 128), "the wide instruction needs fp16 pairs and 2*BN <= 256 columns");
  constexpr int ACCW = WIDE ? 2 * BN : BN;  // tensor-memory columns of one accumulation chain
  constexpr int NBUF = 512 / ACCW;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };
  constexpr int HOLDER_OFFSET = L::BAR_OFFSET + 8 * (2 * STAGES + 2 * NBUF);
  static_assert(HOLDER_OFFSET + 16 <= L::BAR_OFFSET + 256, "barrier area too small");
  volatile unsigned *tmem_holder = reinterpret_cast<volatile unsigned *>(base_ptr + HOLDER_OFFSET);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + HOLDER_OFFSET + 4);
  volatile int *last_flag = reinterpret_cast<volatile int *>(base_ptr + HOLDER_OFFSET + 8);
  volatile int *store_flag = reinterpret_cast<volatile int *>(base_ptr + HOLDER_OFFSET + 12);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * TC_BM;
  // Drain warps (2 and up): warp w may touch TMEM lanes 32*(w%4) .. +31. Tiles wider than 128 columns
  // use two warps per lane quarter, each taking 128 columns, so the accumulators stay in registers.
  constexpr int CW = BN > 128 ? 128 : 64;          // columns per drain warp
  constexpr int DRAIN_WARPS = tc_drain_warps(BN);
  constexpr int DRAIN_THREADS = DRAIN_WARPS * 32;
  static_assert(CW * (DRAIN_WARPS / 4) == BN, "the drain warps cover the tile");
  const int q = warp & 3;
  const bool drains = warp >= 2 && warp < 2 + DRAIN_WARPS;
  const int col0 = drains ? ((warp - 2) >> 2) * CW : 0;     // first column of this warp inside the tile
  const int rl = q * 32 + lane;                             // its row inside the tile
  const int row = m0 + rl;
  float2 ln_st = make_float2(0.f, 1.f);
  float acc[CW];        // the drain warps' accumulated columns (kept past the role code for the cluster's exchange)
  bool pushes = false;  // this thread sends partial sums to the rows' owners
  float *stage = reinterpret_cast<float *>(base_ptr);       // the tile, once the pipeline stages are idle
  constexpr bool LOCAL_COPY = BN <= 128;                    // split-k over a cluster: room for a copy of the own tile
  float *stage_local = stage + (TC_BM + 16) * (BN + 4);     // behind the area the cluster's ranks write into
  float2 *row_stats = reinterpret_cast<float2 *>(base_ptr + L::ROWSTATS_OFFSET);
  // With split-k (gridDim.z CTAs per tile) this CTA owns k-blocks [kb0, kb0 + kblocks).
  const int kb_total = k / KBE;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb0 = blockIdx.z * kb_per;
  const int kblocks = min(kb_per, kb_total - kb0);
  const int nchunks = (kblocks + TC_CHUNK - 1) / TC_CHUNK;

  pdl_launch_dependents();
  const bool stamp = ep.timeline != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  if (ep.timeline != nullptr && threadIdx.x == 0) {
    const unsigned long long t = global_timer();
    atomicMin(ep.timeline + 8, t);   // earliest CTA start
    atomicMax(ep.timeline + 10, t);  // latest CTA start
    if (stamp) ep.timeline[0] = t;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), DRAIN_WARPS);  // one arrival per drain warp
    }
    *abort_flag = 0;
    *store_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // whole warp: allocate all 512 columns (NBUF accumulators of BN columns)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_holder)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_holder;
  if (stamp && threadIdx.x == 0) ep.timeline[1] = global_timer();
  // The store phase starts with the tile's per-column terms (immutable since the weights were
  // loaded): bring their lines into L1 now, so that it does not start with an L2 round trip.
  if (threadIdx.x < BN / 32) {
    if (ep.bias != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(ep.bias + n0 + threadIdx.x * 32));
    if (ep.ln_u != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(ep.ln_u + n0 + threadIdx.x * 32));
  }

  // Whole warps take a role and stay converged (block-wide barriers count
  // warps, so a warp must never reach one in pieces); one lane issues.
  if (warp == 0) {
    // ---- TMA producer ----
    // Weights do not depend on earlier kernels: their tiles of the first
    // stages are requested before waiting for the predecessor to finish.
    const int pre = min(STAGES, kblocks);
    if (lane == 0) {
      tma_prefetch_map(&map_a_hi);
      tma_prefetch_map(&map_a_lo);
      for (int kb = 0; kb < pre; ++kb) {
        const unsigned stage = base + (unsigned)kb * L::STAGE_BYTES;
        const int kx = (kb0 + kb) * KBE;
        mbar_expect_tx(full_bar(kb), (unsigned)L::STAGE_BYTES);
        tma_load_2d(stage + 2 * L::A_BYTES, &map_b_hi, kx, n0, full_bar(kb));
        tma_load_2d(stage + 2 * L::A_BYTES + L::B_BYTES, &map_b_lo, kx, n0, full_bar(kb));
      }
    }
    pdl_wait();
    if (lane == 0) {
      if (ep.timeline != nullptr) atomicMin(ep.timeline + 14, global_timer());  // the predecessor has completed
      for (int kb = 0; kb < pre; ++kb) {
        const unsigned stage = base + (unsigned)kb * L::STAGE_BYTES;
        const int kx = (kb0 + kb) * KBE;
        tma_load_2d(stage, &map_a_hi, kx, m0, full_bar(kb));
        tma_load_2d(stage + L::A_BYTES, &map_a_lo, kx, m0, full_bar(kb));
      }
      if (stamp) ep.timeline[2] = global_timer();
    }
    __syncwarp();
    int issued = pre;
    for (int kb = pre; kb < kblocks; ++kb) {
      const int s = kb % STAGES;
      const unsigned ph = (unsigned)(kb / STAGES) & 1u;
      const bool ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, err, 1);
      __syncwarp();
      if (!ok) break;
      if (lane == 0) {
        const unsigned stage = base + (unsigned)s * L::STAGE_BYTES;
        mbar_expect_tx(full_bar(s), (unsigned)L::STAGE_BYTES);
        const int kx = (kb0 + kb) * KBE;
        tma_load_2d(stage, &map_a_hi, kx, m0, full_bar(s));
        tma_load_2d(stage + L::A_BYTES, &map_a_lo, kx, m0, full_bar(s));
        tma_load_2d(stage + 2 * L::A_BYTES, &map_b_hi, kx, n0, full_bar(s));
        tma_load_2d(stage + 2 * L::A_BYTES + L::B_BYTES, &map_b_lo, kx, n0, full_bar(s));
      }
      __syncwarp();
      ++issued;
    }
    if (*abort_flag) {
      // let copies already in flight land before the CTA's shared memory goes away
      const int first = issued > STAGES ? issued - STAGES : 0;
      for (int j = first; j < issued; ++j) {
        const unsigned long long t0 = global_timer();
        while (!mbar_try_wait(full_bar(j % STAGES), (unsigned)(j / STAGES) & 1u))
          if (global_timer() - t0 > WAIT_LIMIT_NS) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    const unsigned idesc = F16 ? umma_idesc_f16(BN) : umma_idesc_tf32(BN);
    auto mma = [&](unsigned d, unsigned long long a, unsigned long long b, unsigned acc) {
      if (F16) tc_mma_f16(d, a, b, idesc, acc);
      else tc_mma_tf32(d, a, b, idesc, acc);
    };
    bool ok = true;
    int committed = -1;  // last chunk whose completion was committed to a tmem_full barrier
    for (int c = 0; c < nchunks && ok; ++c) {
      const int buf = c % NBUF;
      const unsigned tmem_d = tmem_base + (unsigned)(buf * ACCW);
      // the epilogue must have drained this buffer's previous chunk
      ok = mbar_wait(tmem_empty_bar(buf), ((unsigned)(c / NBUF) & 1u) ^ 1u, abort_flag, err, 4);
      __syncwarp();
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int kb_end = min(kblocks, (c + 1) * TC_CHUNK);
      for (int kb = c * TC_CHUNK; kb < kb_end && ok; ++kb) {
        const int s = kb % STAGES;
        const unsigned ph = (unsigned)(kb / STAGES) & 1u;
        ok = mbar_wait(full_bar(s), ph, abort_flag, err, 2);
        __syncwarp();
        if (!ok) break;
        if (stamp && kb == 0 && lane == 0) ep.timeline[3] = global_timer();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned stage = base + (unsigned)s * L::STAGE_BYTES;
        const unsigned long long a_hi = umma_desc_k128(stage);
        const unsigned long long a_lo = umma_desc_k128(stage + L::A_BYTES);
        const unsigned long long b_hi = umma_desc_k128(stage + 2 * L::A_BYTES);
        const unsigned long long b_lo = umma_desc_k128(stage + 2 * L::A_BYTES + L::B_BYTES);
        if (WIDE) {
          if (lane == 0) {
            const unsigned idesc2 = umma_idesc_f16(2 * BN);
#pragma unroll
            for (int ks = 0; ks < TC_BK / 8; ++ks) {  // a_hi * [b_hi | b_lo]; the first one zeroes both halves
              const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
              tc_mma_f16(tmem_d, a_hi + adv, b_hi + adv, idesc2, (kb == c * TC_CHUNK && ks == 0) ? 0u : 1u);
            }
#pragma unroll
            for (int ks = 0; ks < TC_BK / 8; ++ks) {  // a_lo * b_hi joins the small products
              const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
              tc_mma_f16(tmem_d + (unsigned)BN, a_lo + adv, b_hi + adv, idesc, 1u);
            }
            tc_commit(empty_bar(s));
          }
        } else if (lane == 0) {
#pragma unroll
          for (int ks = 0; ks < TC_BK / 8; ++ks) {
            const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);  // 8 fp32 = 32 bytes along k
            const unsigned first = (kb == c * TC_CHUNK && ks == 0) ? 0u : 1u;   // a chunk starts from zero
            mma(tmem_d, a_lo + adv, b_hi + adv, first);
            mma(tmem_d, a_hi + adv, b_lo + adv, 1u);
          }
#pragma unroll
          for (int ks = 0; ks < TC_BK / 8; ++ks) {
            const unsigned long long adv = (unsigned long long)(ks * 32 >> 4);
            mma(tmem_d, a_hi + adv, b_hi + adv, 1u);
          }
          tc_commit(empty_bar(s));  // the stage is free once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok) {
        if (lane == 0) tc_commit(tmem_full_bar(buf));  // arrives when every MMA of this chunk has completed
        __syncwarp();
        committed = c;
      }
    }
    if (stamp && lane == 0) ep.timeline[4] = global_timer();
    if (!ok) {  // give the tensor pipe a bounded chance to finish before TMEM is freed
      const int buf = (committed + 1) % NBUF;
      if (lane == 0) tc_commit(tmem_full_bar(buf));
      __syncwarp();
      const unsigned long long t0 = global_timer();
      while (!mbar_try_wait(tmem_full_bar(buf), (unsigned)((committed + 1) / NBUF) & 1u))
        if (global_timer() - t0 > WAIT_LIMIT_NS) break;
    }
    __syncwarp();
  } else if (drains) {
    // ---- epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31 ----
    pdl_wait();  // residual reads, C and scratch writes must follow the predecessor
    // LayerNorm folded into this product: the row's statistics from the partial
    // sums its producer left (read while the first tiles are still in flight)
    if (ep.ln_u != nullptr && row < m)
      ln_st = ln_row_stats(ep.ln_stats + (long long)row * TC_STAT_SLOTS, ep.ln_slots, k);
#pragma unroll
    for (int j = 0; j < CW; ++j) acc[j] = 0.f;
    // fp16 pairs: every chain (one 64-wide k-block) carries the product of its operands' block scales
    static_assert(!F16 || TC_CHUNK == 1, "one scale per accumulation chain");
    const float *a_inv_row = F16 ? a_inv_scale + (long long)min(row, m - 1) * kb_total + kb0 : nullptr;
    const float b_inv = F16 ? *b_inv_scale : 1.f;
    float chain_scale = F16 ? a_inv_row[0] * b_inv : 1.f;
    bool ok = true;
    for (int c = 0; c < nchunks && ok; ++c) {
      const int buf = c % NBUF;
      ok = mbar_wait(tmem_full_bar(buf), (unsigned)(c / NBUF) & 1u, abort_flag, err, 3);
      __syncwarp();
      if (!ok) break;
      const float sc = chain_scale;
      if (F16 && c + 1 < nchunks) chain_scale = a_inv_row[c + 1] * b_inv;  // in flight during this chain's adds
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int half = 0; half < (WIDE ? 2 : 1); ++half) {
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 32) {
          unsigned r[32];
          __syncwarp();
          tc_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * ACCW + half * BN + col0 + c0), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j)
            acc[c0 + j] = F16 ? __fmaf_rn(__uint_as_float(r[j]), sc, acc[c0 + j])
                              : __fadd_rn(acc[c0 + j], __uint_as_float(r[j]));
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
    }
    if (stamp && warp == 2 && lane == 0) ep.timeline[5] = global_timer();
    // (a cluster's ranks cover up to 140 rows between them: rows_each is rounded up to even)
    static_assert((TC_BM + 16) * (BN + 4) * 4 <= L::TILES_BYTES, "staging tile must fit in the pipeline stages");
    static_assert(!LOCAL_COPY || (2 * TC_BM + 16) * (BN + 4) * 4 <= L::TILES_BYTES, "exchange area + local copy");
    // With a cluster per tile the partial sums wait for the peers' operand tiles to be dead: as a copy of
    // the tile in this CTA's own shared memory behind the exchange area, or (256-column tiles, which have
    // no room for that) in the registers.
    const bool clustered = cluster_splits > 1;
    pushes = tc_stage_tile<BN, CW, DRAIN_THREADS>(acc, ok && !*abort_flag, ep, col0, rl, warp == 2 && lane == 0,
                                                  clustered ? 1 : splits, part, counters, last_flag, store_flag,
                                                  clustered && LOCAL_COPY ? stage_local : stage, ln_st, row_stats,
                                                  clustered && !LOCAL_COPY) &&
             clustered && !LOCAL_COPY;
  }
  // Store phase, by every warp of the CTA (role and helper warps included: this phase is bound
  // by instruction latency, not bandwidth, and speeds up with the number of warps).
  asm volatile("bar.sync 2, %0;" ::"n"(tc_threads(BN)) : "memory");
  // Split-k over a cluster: the CTAs of a tile (ranks = blockIdx.z) each store a share of its rows.
  // Once every CTA of the cluster is past its k loop (first barrier: the staging area overlays the
  // operand tiles), each sends its partial sums of a row to the CTA that stores the row; after the
  // second barrier every CTA adds what it received, in rank order, from its own shared memory. No
  // scratch, no counters, no remote loads, and the store work is divided as well.
  int row_begin = 0, row_end = TC_BM, rows_each = TC_BM;
  if (stamp && warp == 2 && lane == 0) ep.timeline[10] = global_timer();
  if (cluster_splits > 1) {
    rows_each = ((TC_BM + cluster_splits - 1) / cluster_splits + 1) & ~1;
    row_begin = min(TC_BM, (int)blockIdx.z * rows_each);
    row_end = min(TC_BM, row_begin + rows_each);
  }
  TcStoreFirst first;
  tc_store_first<BN, tc_threads(BN)>(ep, m, n, m0, n0, (int)threadIdx.x, row_begin, row_end, first);
  if (cluster_splits > 1) {
    cluster_arrive_relaxed();
    cluster_wait();
    if (LOCAL_COPY) {
      if (*store_flag != 0) tc_push_rows<BN, tc_threads(BN)>(stage_local, stage, (int)threadIdx.x, rows_each);
    } else if (pushes) {
      tc_push_tile<BN, CW>(acc, stage, col0, rl, rows_each);
    }
    cluster_sync_all();
  }
  const bool go = *store_flag != 0;
  if (stamp && warp == 2 && lane == 0) ep.timeline[11] = global_timer();
  if (go && ep.has_vt())
    tc_store_vt<BN, tc_threads(BN)>(ep, m, m0, n0, (int)threadIdx.x, stage, row_stats, cluster_splits, rows_each, row_begin,
                                    row_end);
  if (go && !(ep.has_vt() && n0 >= ep.vt_col0)) {  // a tile of V columns only has left already
    // the token loop's three forms with their terms fixed at compile time (a loop body that stays in
    // the instruction cache), everything else through the general form
    const unsigned form = tc_ep_form(ep);
    if (F16 && form == TC_EP_FORM_QKV)
      tc_store_rows<BN, tc_threads(BN), TC_EP_FORM_QKV>(ep, m, n, m0, n0, (int)threadIdx.x, stage, row_stats, cluster_splits,
                                                        rows_each, row_begin, row_end, first);
    else if (F16 && form == TC_EP_FORM_W1)
      tc_store_rows<BN, tc_threads(BN), TC_EP_FORM_W1>(ep, m, n, m0, n0, (int)threadIdx.x, stage, row_stats, cluster_splits,
                                                       rows_each, row_begin, row_end, first);
    else if (F16 && form == TC_EP_FORM_RES)
      tc_store_rows<BN, tc_threads(BN), TC_EP_FORM_RES>(ep, m, n, m0, n0, (int)threadIdx.x, stage, row_stats, cluster_splits,
                                                        rows_each, row_begin, row_end, first);
    else
      tc_store_rows<BN, tc_threads(BN)>(ep, m, n, m0, n0, (int)threadIdx.x, stage, row_stats, cluster_splits, rows_each,
                                        row_begin, row_end, first);
  }
  if (stamp && warp == 2 && lane == 0) ep.timeline[12] = global_timer();
  if (ep.stats_out != nullptr) {
    asm volatile("bar.sync 2, %0;" ::"n"(tc_threads(BN)) : "memory");
    if (go) tc_store_row_stats<BN, tc_threads(BN)>(ep, m, m0, n0, (int)threadIdx.x, stage, row_begin, row_end);
  }
  if (stamp && warp == 2 && lane == 0) ep.timeline[13] = global_timer();
  if (stamp && warp == 2 && lane == 0) ep.timeline[6] = global_timer();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (ep.timeline != nullptr && threadIdx.x == 0) {
    const unsigned long long t = global_timer();
    atomicMax(ep.timeline + 9, t);  // latest CTA end
    if (stamp) ep.timeline[7] = t;
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- operand preparation ---------------------------------------------------------

__global__ void split_tf32_kernel(const float *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo,
                                  long long count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    float h, l;
    split_tf32(x[i], h, l);
    hi[i] = h;
    lo[i] = l;
  }
}

// W [k, n] row-major -> wt_hi, wt_lo [n, k] (K-major), 32 x 32 tiles through shared memory.
__global__ void transpose_split_kernel(const float *__restrict__ w, int k, int n, float *__restrict__ wt_hi,
                                       float *__restrict__ wt_lo, const float *__restrict__ row_scale) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int kk = k0 + r, nn = n0 + threadIdx.x;
    float v = (kk < k && nn < n) ? w[(long long)kk * n + nn] : 0.f;
    if (row_scale != nullptr && kk < k) v = __fmul_rn(row_scale[kk], v);
    tile[r][threadIdx.x] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int nn = n0 + r, kk = k0 + threadIdx.x;
    if (nn < n && kk < k) {
      float h, l;
      split_tf32(tile[threadIdx.x][r], h, l);
      wt_hi[(long long)nn * k + kk] = h;
      wt_lo[(long long)nn * k + kk] = l;
    }
  }
}

// One thread per output column: u[n] = sum_k fl(gamma[k] W[k,n]) (the scaled
// weights exactly as transpose_split_kernel stores them, hi + lo), v[n] =
// sum_k beta[k] W[k,n] + bias[n]; sums in double.
__global__ void ln_fold_vectors_kernel(const float *__restrict__ w, int k, int n, const float *__restrict__ gamma,
                                       const float *__restrict__ beta, const float *__restrict__ bias,
                                       float *__restrict__ u, float *__restrict__ v,
                                       const int *__restrict__ f16_amax_bits) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  float inv = 1.f;
  const float scale = f16_amax_bits ? f16_block_scale(__int_as_float(*f16_amax_bits), &inv) : 1.f;
  double su = 0.0, sv = 0.0;
  for (int kk = 0; kk < k; ++kk) {
    const float wv = w[(long long)kk * n + col];
    const float sw = __fmul_rn(gamma[kk], wv);
    if (f16_amax_bits) {  // the fp16 pair transpose_split_f16_kernel stores
      const float a = sw * scale;
      const __half h = __float2half_rn(a);
      su += ((double)__half2float(h) + (double)__half2float(__float2half_rn(a - __half2float(h)))) * (double)inv;
    } else {
      float hh, ll;
      split_tf32(sw, hh, ll);
      su += (double)hh + (double)ll;
    }
    sv += (double)beta[kk] * (double)wv;
  }
  u[col] = (float)su;
  v[col] = (float)(sv + (bias ? (double)bias[col] : 0.0));
}

// ---- host side -----------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// LITNICE_B200_CLUSTER=0: split-k through global scratch instead of clusters.
bool tc_clusters_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("LITNICE_B200_CLUSTER");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <int BN, int STAGES, bool F16, bool WIDE = false>
void launch_cfg(const TcMatrix &a, const TcMatrix &b, int m, int n, int k, const TcEpilogue &ep, int splits,
                float *part, int *counters, DevErr *err, cudaStream_t st, const float *a_inv_scale = nullptr,
                const float *b_inv_scale = nullptr) {
  using L = TcSmem<BN, STAGES>;
  // Sessions on several host threads (one per GPU) may launch at the same time: the per-device
  // set-up below and the occupancy cache are guarded by one mutex per kernel configuration.
  static std::mutex cfg_mu;
  static bool configured[64] = {};
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(cfg_mu);
    if (dev >= 64 || !configured[dev]) {
      LB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, F16, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   L::TOTAL));
      if (dev < 64) configured[dev] = true;
    }
  }
  dim3 grid(n / BN, (m + TC_BM - 1) / TC_BM, splits);
  // The CTAs that share a tile form a cluster and reduce through distributed shared memory when
  // they can (at most 8 per cluster).
  const bool use_clusters = tc_clusters_enabled();
  int cluster_splits = (use_clusters && splits > 1 && splits <= 8) ? splits : 1;
  if (cluster_splits > 1) {
    // A cluster must sit inside one GPC: fewer clusters than SMs / splits may be resident at once. When
    // the grid does not fit in one wave of clusters the scratch path (any SM will do) is the faster one.
    static int max_clusters[9] = {};  // per cluster size; 0 = not asked yet (one device type per process)
    std::lock_guard<std::mutex> lock(cfg_mu);
    if (max_clusters[cluster_splits] == 0) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(tc_threads(BN));
      cfg.dynamicSmemBytes = (size_t)L::TOTAL;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = (unsigned)cluster_splits;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int nc = 0;
      if (cudaOccupancyMaxActiveClusters(&nc, gemm_tc_kernel<BN, STAGES, F16, WIDE>, &cfg) != cudaSuccess || nc <= 0) {
        (void)cudaGetLastError();
        nc = -1;
      }
      max_clusters[cluster_splits] = nc;
    }
    if ((long long)grid.x * grid.y > max_clusters[cluster_splits]) cluster_splits = 1;
  }
  launch_pdl_cluster(gemm_tc_kernel<BN, STAGES, F16, WIDE>, grid, dim3(tc_threads(BN)), (size_t)L::TOTAL, st, g_pdl_enabled,
                     (unsigned)cluster_splits, a.hi, a.lo, b.hi, b.lo, ep, m, n, k, splits, part, counters, err,
                     a_inv_scale, b_inv_scale, cluster_splits);
}

}  // namespace

bool tc_runtime_available() { return encode_tiled_fn() != nullptr; }

void tc_make_map(CUtensorMap *map, const float *base, unsigned long long rows, unsigned long long k,
                 unsigned box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (k * 4) % 16 != 0 || box_rows == 0 || box_rows > 256)
    throw std::invalid_argument("litnice_b200: tensor map operand must be 16-byte aligned with k % 4 == 0");
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k * 4};  // bytes between rows
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

void tc_make_map_f16(CUtensorMap *map, const __half *base, unsigned long long rows, unsigned long long k,
                     unsigned box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || k % TC_F16_SLOT != 0 || box_rows == 0 || box_rows > 256)
    throw std::invalid_argument("litnice_b200: fp16 tensor map operand must be 16-byte aligned with k % 64 == 0");
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k * 2};  // bytes between rows
  const cuuint32_t box[2] = {(cuuint32_t)TC_F16_SLOT, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

void tc_make_map_plain(CUtensorMap *map, const float *base, unsigned long long rows, unsigned long long cols,
                       unsigned box_rows, unsigned box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || cols % 4 != 0 || box_rows == 0 || box_rows > 256 ||
      box_cols == 0 || box_cols > 256 || (box_cols * 4) % 16 != 0)
    throw std::invalid_argument("litnice_b200: tensor map operand must be 16-byte aligned with cols % 4 == 0");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("litnice_b200: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

// How many clusters of 2..8 CTAs of these kernels the device holds at once (a cluster sits inside
// one GPC); -1 where the runtime cannot say. Every configuration runs one CTA per SM, so one of them
// stands for all.
const int *tc_cluster_capacity() {
  static int cap[9] = {};
  static std::once_flag once;
  std::call_once(once, []() {
    using L = TcSmem<128, 3>;
    for (int cs = 2; cs <= 8; ++cs) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(1, 1, (unsigned)cs);
      cfg.blockDim = dim3(tc_threads(128));
      cfg.dynamicSmemBytes = (size_t)L::TOTAL;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = (unsigned)cs;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int nc = 0;
      if (cudaFuncSetAttribute(gemm_tc_kernel<128, 3, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
              cudaSuccess ||
          cudaOccupancyMaxActiveClusters(&nc, gemm_tc_kernel<128, 3, true, false>, &cfg) != cudaSuccess || nc <= 0) {
        (void)cudaGetLastError();
        nc = -1;
      }
      cap[cs] = nc;
    }
  });
  return cap;
}

TcPlan tc_plan(int m, int n, int k, bool has64, bool has128, bool has256, int k_block, bool clusters_ok) {
  TcPlan p{};
  const long long mt = (m + TC_BM - 1) / TC_BM;
  // One thread issues every tcgen05.mma of a CTA, at most one per ~40 ns, and a
  // TF32 instruction covers only 8 of k: the widest tile that still fills the
  // GPU keeps the tensor pipe busy per issue slot; narrow tiles serve short
  // single-stream shapes.
  p.bn = (has128 && (!has64 || mt * (n / 128) >= 74)) ? 128 : 64;
  if (has256 && mt * (n / 256) >= 2 * 148) p.bn = 256;
  const long long ctas = mt * (n / p.bn);
  const int kb = k / k_block;
  // Few tiles (a short single stream): cut k over several CTAs per tile so the
  // serial k loop shortens, keeping one wave and at least 4 k-blocks per CTA.
  int splits = 1;
  if (ctas < 74) {
    splits = (int)(148 / ctas);
    if (splits > kb / 4) splits = kb / 4;
    if (splits < 1) splits = 1;
    const int per = (kb + splits - 1) / splits;
    splits = (kb + per - 1) / per;  // no empty split
    // A long k on few tiles: a 128-column tile halves the tile count, so twice the k ranges fit,
    // and it reads less shared memory per flop; its larger epilogue costs about three k-blocks.
    // Only as clusters (the partial sums of a wide tile through global scratch are too slow).
    // LITNICE_B200_PLAN_WIDE=0 keeps the 64-column tiles (a knob for comparisons).
    static const bool plan_wide = [] {
      const char *e = std::getenv("LITNICE_B200_PLAN_WIDE");
      return !(e && e[0] == '0');
    }();
    if (plan_wide && clusters_ok && tc_clusters_enabled() && p.bn == 64 && has128) {
      const int *cap = tc_cluster_capacity();
      const long long wide = mt * (n / 128);
      int s2 = (int)(148 / wide);
      if (s2 > kb / 4) s2 = kb / 4;
      if (s2 > 8) s2 = 8;
      while (s2 >= 2 && (cap[s2] <= 0 || wide > cap[s2])) --s2;
      if (s2 >= 2) {
        const int per2 = (kb + s2 - 1) / s2;
        s2 = (kb + per2 - 1) / per2;
        if (per2 + 2 <= per && cap[s2] > 0 && wide <= cap[s2]) {
          p.bn = 128;
          p.splits = s2;
          p.scratch_floats = (size_t)wide * s2 * TC_BM * 128;
          p.counters = (size_t)wide;
          return p;
        }
      }
    }
  }
  p.splits = splits;
  p.scratch_floats = splits > 1 ? (size_t)ctas * splits * TC_BM * p.bn : 0;
  p.counters = splits > 1 ? (size_t)ctas : 0;
  return p;
}

void launch_gemm_tc(const TcMatrix &a, const TcMatrix &b, int m, int n, int k, const TcPlan &plan,
                    const TcEpilogue &ep, float *scratch, int *counters, DevErr *err, cudaStream_t st) {
  if (m <= 0) return;
  const int bn = plan.bn;
  if (k < TC_BK || k % TC_BK != 0 || (bn != 64 && bn != 128 && bn != 256) || n % bn != 0)
    throw std::invalid_argument("litnice_b200: tensor-core GEMM needs k % 32 == 0 and n % bn == 0");
  if (plan.splits > 1 && (scratch == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: split-k tensor-core GEMM needs scratch");
  if (bn == 256) launch_cfg<256, 2, false>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st);
  else if (bn == 128) launch_cfg<128, 3, false>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st);
  else launch_cfg<64, 4, false>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st);
}

void launch_gemm_tc_f16(const TcMatrix &a, const float *a_inv_scale, const TcMatrix &b, const float *b_inv_scale,
                        int m, int n, int k, const TcPlan &plan, const TcEpilogue &ep, float *scratch, int *counters,
                        DevErr *err, cudaStream_t st) {
  if (m <= 0) return;
  const int bn = plan.bn;
  if (k < TC_F16_SLOT || k % TC_F16_SLOT != 0 || (bn != 64 && bn != 128 && bn != 256) || n % bn != 0)
    throw std::invalid_argument("litnice_b200: fp16-pair tensor-core GEMM needs k % 64 == 0 and n % bn == 0");
  if (a_inv_scale == nullptr || b_inv_scale == nullptr)
    throw std::invalid_argument("litnice_b200: fp16-pair tensor-core GEMM needs the operands' scales");
  if (plan.splits > 1 && (scratch == nullptr || counters == nullptr))
    throw std::invalid_argument("litnice_b200: split-k tensor-core GEMM needs scratch");
  // LITNICE_B200_TC_WIDE: 0 = three instructions per k-step everywhere, 1 (default) = the wide
  // instruction for 64-column tiles, 2 = for 128-column tiles too (measured slower there: the wide
  // chain leaves only two tensor-memory buffers, and the drain does not keep up with the k loop).
  static const int wide = [] {
    const char *e = std::getenv("LITNICE_B200_TC_WIDE");
    return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
  }();
  if (bn == 256)
    launch_cfg<256, 2, true>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st, a_inv_scale, b_inv_scale);
  else if (bn == 128 && wide >= 2)
    launch_cfg<128, 3, true, true>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st, a_inv_scale, b_inv_scale);
  else if (bn == 128)
    launch_cfg<128, 3, true>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st, a_inv_scale, b_inv_scale);
  else if (wide >= 1)
    launch_cfg<64, 4, true, true>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st, a_inv_scale, b_inv_scale);
  else
    launch_cfg<64, 4, true>(a, b, m, n, k, ep, plan.splits, scratch, counters, err, st, a_inv_scale, b_inv_scale);
}

// ---- fp16-pair operand preparation --------------------------------------------------

namespace {

// One warp per row: per block of 64 columns the scale and the pair.
__global__ void split_f16_kernel(const float *__restrict__ x, long long rows, int k, __half *__restrict__ hi,
                                 __half *__restrict__ lo, float *__restrict__ inv_scale) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int n4 = k >> 2;  // k % 64 == 0: whole warps of float4s, two blocks per pass
  for (int c = lane; c < n4; c += 32) {
    const float4 v = reinterpret_cast<const float4 *>(x + row * k)[c];
    f16_store_block(v, true, hi + row * k + c * 4, lo + row * k + c * 4, inv_scale + row * (k / 64) + (c >> 4));
  }
}

// Largest magnitude of W (rows optionally scaled) -> *amax_bits (float bits; non-negative floats order as ints).
__global__ void amax_kernel(const float *__restrict__ w, int k, int n, const float *__restrict__ row_scale,
                            int *__restrict__ amax_bits) {
  float am = 0.f;
  const long long total = (long long)k * n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float v = w[i];
    if (row_scale != nullptr) v = __fmul_rn(row_scale[i / n], v);
    am = fmaxf(am, fabsf(v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_int(am));
}

// W [k, n] row-major -> K-major fp16 pair [n, k] under the matrix's one scale; 32 x 32 tiles through shared memory.
__global__ void transpose_split_f16_kernel(const float *__restrict__ w, int k, int n, __half *__restrict__ wt_hi,
                                           __half *__restrict__ wt_lo, const float *__restrict__ row_scale,
                                           const int *__restrict__ amax_bits, float *__restrict__ inv_scale_out) {
  __shared__ float tile[32][33];
  float inv;
  const float scale = f16_block_scale(__int_as_float(*amax_bits), &inv);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0) *inv_scale_out = inv;
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int kk = k0 + r, nn = n0 + threadIdx.x;
    float v = (kk < k && nn < n) ? w[(long long)kk * n + nn] : 0.f;
    if (row_scale != nullptr && kk < k) v = __fmul_rn(row_scale[kk], v);
    tile[r][threadIdx.x] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int nn = n0 + r, kk = k0 + threadIdx.x;
    if (nn < n && kk < k) {
      const float a = tile[threadIdx.x][r] * scale;
      const __half h = __float2half_rn(a);
      wt_hi[(long long)nn * k + kk] = h;
      wt_lo[(long long)nn * k + kk] = __float2half_rn(a - __half2float(h));
    }
  }
}

}  // namespace

void launch_split_f16(const float *x, long long rows, int k, const TcPairF16 &out, cudaStream_t st) {
  if (rows <= 0) return;
  if (k % TC_F16_SLOT != 0) throw std::invalid_argument("litnice_b200: fp16 pairs need k % 64 == 0");
  split_f16_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(x, rows, k, out.hi, out.lo, out.inv_scale);
  LB_LAUNCH_CHECK();
}

void launch_transpose_split_f16(const float *w, int k, int n, __half *wt_hi, __half *wt_lo, float *inv_scale_dev,
                                cudaStream_t st, const float *row_scale, int *amax_scratch) {
  LB_CUDA(cudaMemsetAsync(amax_scratch, 0, sizeof(int), st));
  amax_kernel<<<296, 256, 0, st>>>(w, k, n, row_scale, amax_scratch);
  LB_LAUNCH_CHECK();
  dim3 grid((n + 31) / 32, (k + 31) / 32), block(32, 8);
  transpose_split_f16_kernel<<<grid, block, 0, st>>>(w, k, n, wt_hi, wt_lo, row_scale, amax_scratch, inv_scale_dev);
  LB_LAUNCH_CHECK();
}

void launch_split_tf32(const float *x, float *hi, float *lo, long long count, cudaStream_t st) {
  if (count <= 0) return;
  const long long blocks = (count + 255) / 256;
  split_tf32_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, st>>>(x, hi, lo, count);
  LB_LAUNCH_CHECK();
}

void launch_transpose_split(const float *w, int k, int n, float *wt_hi, float *wt_lo, cudaStream_t st,
                            const float *row_scale) {
  dim3 grid((n + 31) / 32, (k + 31) / 32), block(32, 8);
  transpose_split_kernel<<<grid, block, 0, st>>>(w, k, n, wt_hi, wt_lo, row_scale);
  LB_LAUNCH_CHECK();
}

void launch_ln_fold_vectors(const float *w, int k, int n, const float *gamma, const float *beta, const float *bias,
                            float *u, float *v, cudaStream_t st, const int *f16_amax_bits) {
  ln_fold_vectors_kernel<<<(n + 127) / 128, 128, 0, st>>>(w, k, n, gamma, beta, bias, u, v, f16_amax_bits);
  LB_LAUNCH_CHECK();
}

}  // namespace lb
