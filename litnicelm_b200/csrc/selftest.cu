// Self-test of the bounded waits. Every spin of this library's kernels on an
// mbarrier gives up after a time limit, records DEVERR_WAIT_TIMEOUT in the
// error word the host reads, and lets the kernel return normally, so that a
// lost copy or a missing peer costs one failed call instead of a hung GPU.
// This file holds a one-CTA kernel whose barrier nothing ever completes, so
// that the give-up path can be exercised without touching a production kernel.
#include "common.cuh"
#include "tc_ptx.cuh"

#include <cstdio>

namespace lb {
namespace {

__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns, DevErr *err, unsigned long long *waited_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);  // one arrival expected; none will come
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const unsigned long long t0 = global_timer();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, err, 99, limit_ns);
  if (threadIdx.x == 0) *waited_ns = ok ? 0ull : global_timer() - t0;
  __syncthreads();  // the other threads of a real kernel read abort_flag after such a barrier and leave too
}

}  // namespace
}  // namespace lb

extern "C" int litnice_b200_selftest_wait_timeout(int32_t limit_us, int32_t *code, int32_t *detail, double *waited_us) {
  using namespace lb;
  if (limit_us <= 0 || limit_us > 1000 || code == nullptr || detail == nullptr || waited_us == nullptr)
    return LITNICE_B200_EINVAL;  // the limit of this test is capped at 1 ms
  DevErr *err_host = nullptr, *err_dev = nullptr;
  unsigned long long *waited = nullptr;
  int rc = LITNICE_B200_OK;
  try {
    LB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&err_host), sizeof(DevErr), cudaHostAllocMapped));
    err_host->code = DEVERR_NONE;
    err_host->detail = 0;
    LB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&err_dev), err_host, 0));
    LB_CUDA(cudaMalloc(reinterpret_cast<void **>(&waited), 8));
    LB_CUDA(cudaMemset(waited, 0, 8));
    wait_timeout_selftest_kernel<<<1, 64>>>((unsigned long long)limit_us * 1000ull, err_dev, waited);
    LB_LAUNCH_CHECK();
    LB_CUDA(cudaDeviceSynchronize());
    unsigned long long ns = 0;
    LB_CUDA(cudaMemcpy(&ns, waited, 8, cudaMemcpyDeviceToHost));
    *code = err_host->code;
    *detail = err_host->detail;
    *waited_us = 1e-3 * (double)ns;
  } catch (const std::exception &e) {
    std::fprintf(stderr, "litnice_b200_selftest_wait_timeout: %s\n", e.what());
    rc = LITNICE_B200_ECUDA;
  }
  if (waited) cudaFree(waited);
  if (err_host) cudaFreeHost(err_host);
  return rc;
}
