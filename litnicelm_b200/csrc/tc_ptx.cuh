// Inline PTX for the sm_100a tensor-core kernels: mbarriers with bounded waits,
// TMA tile loads, tcgen05 MMA / commit / tensor-memory loads and stores, and the
// shared-memory and instruction descriptors of K-major TF32 operands.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "gemm_tc.cuh"

namespace lb {

constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;

__device__ __forceinline__ unsigned smem_u32(const void *p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)::"memory");
  return t;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: false (and the error word set) if the phase does not complete
// within WAIT_LIMIT_NS or another role has already given up. The spinning part
// is a real function, not inlined at the several dozen wait sites of a kernel:
// these kernels run a few warps per SM and every kilobyte of code they do not
// execute still costs instruction-cache space.
// err may be null (a caller without an error word): the wait still ends and
// the abort flag still tells the other roles.
static __device__ __noinline__ bool mbar_wait_limit(unsigned bar, unsigned parity, volatile int *abort_flag, DevErr *err,
                                                    int where, unsigned long long limit_ns) {
  const unsigned long long t0 = global_timer();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer() - t0 > limit_ns) {
        *abort_flag = 1;
        if (err != nullptr) {
          err->code = DEVERR_WAIT_TIMEOUT;
          err->detail = where;
        }
        return false;
      }
    }
  }
}
static __device__ __forceinline__ bool mbar_wait_slow(unsigned bar, unsigned parity, volatile int *abort_flag,
                                                      DevErr *err, int where) {
  return mbar_wait_limit(bar, parity, abort_flag, err, where, WAIT_LIMIT_NS);
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag, DevErr *err,
                                          int where) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, err, where);
}
// The same for a whole converged warp: every lane learns the common outcome,
// so the warp cannot split on a wait that runs out for some lanes only.
__device__ __forceinline__ bool mbar_wait_warp(unsigned bar, unsigned parity, volatile int *abort_flag, DevErr *err,
                                               int where) {
  const bool ok = mbar_wait(bar, parity, abort_flag, err, where);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap *map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Brings a tensor map into the descriptor cache ahead of its first use (the maps of operands
// an earlier kernel writes are first used right after the wait for that kernel).
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory, completion counted in bytes on an
// mbarrier. Both addresses 16-byte aligned, the size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                            unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp16 operands (K = 16 per instruction), fp32 accumulation.
__device__ __forceinline__ void tc_mma_f16(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                           unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st16(unsigned taddr, const unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (32 fp32) stored with the 128-byte swizzle: groups of 8 rows are 1024 bytes
// apart (stride byte offset), the leading byte offset is unused for this layout,
// descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ unsigned long long umma_desc_k128(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
  d |= 1ull << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor: D fp32, A and B TF32, both K-major, M = 128, N = bn.
// The same with fp16 operands (format code 0).
__host__ __device__ constexpr unsigned umma_idesc_f16(int bn) {
  return (1u << 4) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
}
__host__ __device__ constexpr unsigned umma_idesc_tf32(int bn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Thread-block cluster: barrier over all threads of all CTAs of the cluster (hardware barrier; the
// CTAs of a cluster are co-scheduled), and 16-byte stores into the shared memory of the CTA of a
// given rank.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Split form for a barrier that orders no memory of this CTA ("every CTA of the cluster is past
// its k loop"): a relaxed arrive does not wait for the stores the CTA has in flight.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address in the cluster's shared window of this CTA's shared address in the CTA of the given rank.
__device__ __forceinline__ unsigned cluster_map(unsigned local_smem_addr, unsigned cta_rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta_rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f4(unsigned cluster_addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

__device__ __forceinline__ float4 ld_cluster_f4(unsigned cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// A operand read from tensor memory (lane = row, one column per k element).
__device__ __forceinline__ void tc_mma_tf32_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with fp16 operands: a 32-bit tensor-memory column holds two consecutive k elements
// (the lower k in the low half), so an instruction (16 of k) reads 8 columns of A.
__device__ __forceinline__ void tc_mma_f16_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc,
                                              unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

}  // namespace lb
