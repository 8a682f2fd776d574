// Weight ingest: a byte range of a file straight into device memory.
//
// The reference stages a checkpoint through one host buffer of the whole arena
// and one copy_host2device per arena (checkpoint.cpp:207-241, 300-727). Here the
// range moves in 16 MiB pieces through two pinned buffers: while piece i
// crosses PCIe (cudaMemcpyAsync from pinned memory, asynchronous to the host),
// piece i+1 is read from the file and, when asked, checked for non-finite
// floats (the all-finite rule of checkpoint.cpp:176-205) on the host.
#include "common.cuh"

#include <cmath>
#include <cstdio>
#include <cstring>

namespace lb {

namespace {

constexpr size_t INGEST_PIECE = (size_t)16 << 20;

struct PinnedPair {
  char *buf[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  ~PinnedPair() {
    for (int i = 0; i < 2; ++i) {
      if (done[i]) cudaEventDestroy(done[i]);
      if (buf[i]) cudaFreeHost(buf[i]);
    }
  }
};

bool all_finite(const float *p, size_t n) {
  // exponent bits all ones <=> infinity or NaN
  const uint32_t *u = reinterpret_cast<const uint32_t *>(p);
  uint32_t bad = 0;
  for (size_t i = 0; i < n; ++i) bad |= ((u[i] & 0x7f800000u) == 0x7f800000u) ? 1u : 0u;
  return bad == 0;
}

}  // namespace

void file_to_device(const char *path, uint64_t file_offset, uint64_t bytes, void *dst, cudaStream_t st,
                    bool check_finite_f32) {
  if (bytes == 0) return;
  std::FILE *f = std::fopen(path, "rb");
  if (f == nullptr) throw std::runtime_error(std::string("failed to open file ") + path);
  struct Closer {
    std::FILE *f;
    ~Closer() { std::fclose(f); }
  } closer{f};
  if (fseeko(f, (off_t)file_offset, SEEK_SET) != 0) throw std::runtime_error(std::string("failed to seek file ") + path);
  PinnedPair pp;
  const size_t piece = bytes < INGEST_PIECE ? (size_t)((bytes + 15) / 16 * 16) : INGEST_PIECE;
  for (int i = 0; i < 2; ++i) {
    LB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&pp.buf[i]), piece, cudaHostAllocDefault));
    LB_CUDA(cudaEventCreateWithFlags(&pp.done[i], cudaEventDisableTiming));
  }
  uint64_t done = 0;
  int which = 0;
  bool used[2] = {false, false};
  while (done < bytes) {
    const size_t n = (size_t)(bytes - done < piece ? bytes - done : piece);
    if (used[which]) LB_CUDA(cudaEventSynchronize(pp.done[which]));  // the buffer's last copy has left it
    const size_t got = std::fread(pp.buf[which], 1, n, f);
    if (got != n) {
      cudaStreamSynchronize(st);
      throw std::runtime_error(std::string("short read from ") + path);
    }
    if (check_finite_f32 && !all_finite(reinterpret_cast<const float *>(pp.buf[which]), n / 4)) {
      cudaStreamSynchronize(st);
      throw std::domain_error(std::string("non-finite value in ") + path);
    }
    LB_CUDA(cudaMemcpyAsync(static_cast<char *>(dst) + done, pp.buf[which], n, cudaMemcpyHostToDevice, st));
    LB_CUDA(cudaEventRecord(pp.done[which], st));
    used[which] = true;
    which ^= 1;
    done += n;
  }
  LB_CUDA(cudaStreamSynchronize(st));
}

}  // namespace lb
