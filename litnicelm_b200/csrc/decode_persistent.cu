// Cached mode, greedy, up to 8 streams: the whole token loop as ONE resident kernel.
//
// The one-row steps of the cached mode are chains of small dependent operators
// (per layer: LayerNorm + QKV product, attention over the cached keys,
// out-projection, LayerNorm + W1, W2; then the head and the selection,
// transformer_layer.cpp:50-92 / output_head.cpp:58-70 / inference.cpp:188-198
// for one row). As separate launches each costs 4-6 microseconds however little
// it computes. Here one CTA per SM stays resident for all tokens of a run; the
// operators become phases separated by a grid-wide barrier (about a microsecond),
// and since the weights never change, every CTA requests the weights of its next
// unit of work before it waits at the barrier, so their latency hides behind it.
//
// Work split. A product out[B, n] = in[B, k] W[k, n] is cut into units of TN
// columns x one range of k; units go round-robin to the CTAs. A unit's result is
// a partial sum written to scratch [range][stream][n]; nobody adds the ranges in
// a pass of its own: the CTAs that read the row next add them, in range order
// (so results do not depend on scheduling), together with the bias, the residual
// and the ReLU of the reference's wiring. Every CTA keeps the residual rows x
// and y in its own shared memory. Attention units are (stream, head, chunk of
// keys); the CTAs of the out-projection join the chunks of the heads they need.
//
// Every spin is bounded: a barrier that does not complete within a second sets
// the error word and an abort flag that all CTAs poll, and the kernel returns.
#include "common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <mutex>

namespace lb {

namespace {

constexpr int PK_THREADS = 256;
constexpr int PK_WARPS = PK_THREADS / 32;
constexpr int PK_BATCH = 8;  // weight loads a thread has in flight
constexpr int PK_MAX_CHUNKS = 24;  // key chunks per (stream, head): the out-projection joins them from registers

struct PkGemv {   // one product of the step: how it is cut
  int k, n, tn, tiles, ranges, k_per;   // k_per: rows per range (multiple of the rows one CTA trip covers)
};

struct PkParams {
  const char *params;            // parameter arena
  const unsigned long long *off; // [n_layers][12] byte offsets (LayerOff order) then tok_emb, pos_emb, lnf_g, lnf_b, lm_head
  int n_layers, n_heads, d, f, vocab, max_seq, n_streams;
  float *kcache, *vcache;
  int cap;
  unsigned long long layer_stride;  // floats
  int *ids;
  int ids_ld;
  int *out_tokens;
  int out_ld;
  LoopState *state;
  float *part_qkv, *part_wo, *part_w1, *part_w2, *part_head, *part_attn;
  float *logits;       // [B, vocab]: the last step's logits, for callers that read them
  unsigned *barrier;   // [0] arrivals, [1] abort flag
  int s0, step0, steps;
  PkGemv g_qkv, g_wo, g_w1, g_w2, g_head;
  int attn_chunks_max;
  DevErr *err;
  unsigned long long *timeline;  // measurement aid: CTA 0 stamps the phases of its 11th token here (64 entries)
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier on a monotonic arrival counter. Returns false when the run was aborted.
__device__ bool pk_grid_sync(unsigned *bar, unsigned &target, unsigned nctas, DevErr *err, int *s_abort) {
  __syncthreads();
  if (threadIdx.x == 0) {
    target += nctas;
    // arrival without waiting for the old value to come back; the release orders this CTA's writes before it
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
    const unsigned long long t0 = global_timer();
    unsigned spins = 0;
    int aborted = 0;
    while (ld_acquire(bar) < target) {
      if ((++spins & 255u) == 0) {
        if (ld_acquire(bar + 1) != 0u) {
          aborted = 1;
          break;
        }
        if (global_timer() - t0 > WAIT_LIMIT_NS) {
          atomicExch(bar + 1, 1u);
          err->code = DEVERR_WAIT_TIMEOUT;
          err->detail = 77;
          aborted = 1;
          break;
        }
      }
    }
    __threadfence();
    *s_abort = aborted;
  }
  __syncthreads();
  return *s_abort == 0;
}

__device__ __forceinline__ double pk_warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// LayerNorm of B rows held in shared memory (device_backend.cpp:1247-1279: mean and biased
// variance in double, inv_std = 1/sqrt(float(var) + 1e-5f)) by the whole CTA. Sum and sum of squares
// are taken in one pass, in double (var = E[x^2] - mean^2 loses nothing that survives the rounding of
// the variance to float at these magnitudes); warps join by shuffles, the eight warp sums in warp
// order. gamma / beta come from registers the caller filled before the barrier (element c = tid + i*256).
constexpr int PK_LN_REGS = 8;  // rows up to 2048 wide
template <int MB>
__device__ void pk_layernorm(const float *src, float *dst, int d, const float *g_reg, const float *b_reg,
                             double *s_red /* [PK_WARPS][2 * MB] */) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  double sum[MB], sq[MB];
#pragma unroll
  for (int b = 0; b < MB; ++b) sum[b] = sq[b] = 0.0;
  for (int c = threadIdx.x; c < d; c += PK_THREADS)
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      const double v = (double)src[b * d + c];
      sum[b] += v;
      sq[b] += v * v;
    }
#pragma unroll
  for (int b = 0; b < MB; ++b) {
    sum[b] = pk_warp_sum(sum[b]);
    sq[b] = pk_warp_sum(sq[b]);
    if (lane == 0) {
      s_red[w * 2 * MB + 2 * b] = sum[b];
      s_red[w * 2 * MB + 2 * b + 1] = sq[b];
    }
  }
  __syncthreads();
  float inv_std[MB], fmean[MB];
#pragma unroll
  for (int b = 0; b < MB; ++b) {
    double t = s_red[2 * b], q = s_red[2 * b + 1];
    for (int k = 1; k < PK_WARPS; ++k) {
      t += s_red[k * 2 * MB + 2 * b];
      q += s_red[k * 2 * MB + 2 * b + 1];
    }
    const double mean = t / (double)d;
    double var = q / (double)d - mean * mean;
    if (var < 0.0) var = 0.0;
    inv_std[b] = 1.0f / sqrtf((float)var + 1e-5f);
    fmean[b] = (float)mean;
  }
#pragma unroll
  for (int i = 0; i < PK_LN_REGS; ++i) {
    const int c = threadIdx.x + i * PK_THREADS;
    if (c < d) {
#pragma unroll
      for (int b = 0; b < MB; ++b)
        dst[b * d + c] = __fadd_rn(__fmul_rn((src[b * d + c] - fmean[b]) * inv_std[b], g_reg[i]), b_reg[i]);
    }
  }
  __syncthreads();
}
// gamma and beta of the LayerNorm a CTA will apply after the next barrier, requested ahead of it
__device__ __forceinline__ void pk_ln_prefetch(float *g_reg, float *b_reg, const float *gamma, const float *beta, int d) {
#pragma unroll
  for (int i = 0; i < PK_LN_REGS; ++i) {
    const int c = threadIdx.x + i * PK_THREADS;
    g_reg[i] = c < d ? __ldg(gamma + c) : 0.f;
    b_reg[i] = c < d ? __ldg(beta + c) : 0.f;
  }
}

// dst[b, c] (shared, row pitch `pitch`) = sum over ranges of part[r][b][col0 + c] (+ bias) (+ residual) (ReLU).
template <int MB>
__device__ void pk_gather(float *dst, int pitch, const float *part, int ranges, int n_total, int col0, int ncols,
                          const float *bias, const float *residual, int res_pitch, int relu) {
  constexpr int GB = 12;  // loads in flight per element: the ranges are independent reads, only the adds are ordered
  // Every CTA reads the same lines at the same moment; each starts at another column so that the
  // requests of one instant spread over the L2 slices instead of queueing at one.
  const int rot = ncols >= 64 ? (int)((blockIdx.x * 32u) % (unsigned)ncols) : 0;
  for (int e = threadIdx.x; e < MB * ncols; e += PK_THREADS) {
    const int b = e / ncols;
    int c = e - b * ncols + rot;
    if (c >= ncols) c -= ncols;
    const float *src = part + (long long)b * n_total + col0 + c;
    const long long step = (long long)MB * n_total;
    float v = 0.f;
    for (int r0 = 0; r0 < ranges; r0 += GB) {
      float t[GB];
#pragma unroll
      for (int j = 0; j < GB; ++j) t[j] = r0 + j < ranges ? __ldcg(src + (r0 + j) * step) : 0.f;
#pragma unroll
      for (int j = 0; j < GB; ++j) v += t[j];
    }
    if (bias) v += __ldg(bias + col0 + c);
    if (residual) v += residual[b * res_pitch + col0 + c];
    if (relu) v = v > 0.f ? v : 0.f;
    dst[b * pitch + c] = v;
  }
  __syncthreads();
}

// The weights of one unit, requested into registers (first PK_BATCH trips) ahead of the barrier.
struct PkUnit {
  int tile, range, kb, ke, valid;
};
__device__ __forceinline__ PkUnit pk_unit(const PkGemv &g, int u) {
  PkUnit t;
  t.valid = u < g.tiles * g.ranges;
  t.tile = u % g.tiles;
  t.range = u / g.tiles;
  t.kb = t.range * g.k_per;
  t.ke = min(g.k, t.kb + g.k_per);
  return t;
}

template <int MB>
struct PkGemvRun {
  float4 w[PK_BATCH];
  // thread -> (row slot within a trip, 4 columns)
  __device__ __forceinline__ void prefetch(const PkGemv &g, const PkUnit &u, const float *wbase) {
    const int lpr = g.tn >> 2, rows_per_trip = PK_THREADS / lpr;
    const int slot = threadIdx.x / lpr, c4 = threadIdx.x - slot * lpr;
    const int col = u.tile * g.tn + c4 * 4;
#pragma unroll
    for (int j = 0; j < PK_BATCH; ++j) {
      const int row = u.kb + j * rows_per_trip + slot;
      w[j] = (u.valid && row < u.ke && col < g.n)
                 ? __ldg(reinterpret_cast<const float4 *>(wbase + (long long)row * g.n + col))
                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // in: shared rows [MB][in_pitch], indexed by (row - in_row0). red: shared scratch of PK_THREADS * MB float4.
  __device__ void finish(const PkGemv &g, const PkUnit &u, const float *wbase, const float *in, int in_pitch,
                         int in_row0, float *part, float4 *red) {
    float4 *red2 = red + PK_THREADS * MB;  // [4][MB][tn / 4]
    if (!u.valid) return;  // uniform per CTA
    const int lpr = g.tn >> 2, rows_per_trip = PK_THREADS / lpr;
    const int slot = threadIdx.x / lpr, c4 = threadIdx.x - slot * lpr;
    const int col = u.tile * g.tn + c4 * 4;
    float4 acc[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) acc[b] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int trips = (u.ke - u.kb + rows_per_trip - 1) / rows_per_trip;
    for (int t0 = 0; t0 < trips; t0 += PK_BATCH) {
      if (t0 > 0) {
#pragma unroll
        for (int j = 0; j < PK_BATCH; ++j) {
          const int row = u.kb + (t0 + j) * rows_per_trip + slot;
          w[j] = (row < u.ke && col < g.n) ? __ldg(reinterpret_cast<const float4 *>(wbase + (long long)row * g.n + col))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < PK_BATCH; ++j) {
        const int row = u.kb + (t0 + j) * rows_per_trip + slot;
        if (row < u.ke) {
#pragma unroll
          for (int b = 0; b < MB; ++b) {
            const float xv = in[b * in_pitch + row - in_row0];
            acc[b].x = fmaf(xv, w[j].x, acc[b].x);
            acc[b].y = fmaf(xv, w[j].y, acc[b].y);
            acc[b].z = fmaf(xv, w[j].z, acc[b].z);
            acc[b].w = fmaf(xv, w[j].w, acc[b].w);
          }
        }
      }
    }
    // join the row slots of a column group in slot order
#pragma unroll
    for (int b = 0; b < MB; ++b) red[(slot * MB + b) * lpr + c4] = acc[b];
    __syncthreads();
    // slots 0, 4, 8, ... / 1, 5, ... / 2, 6, ... / 3, 7, ... by four threads per column group, then the four
    // sums in order (a fixed order, shorter than one thread walking every slot)
    constexpr int QS = 4;
    for (int e = threadIdx.x; e < MB * lpr * QS; e += PK_THREADS) {
      const int qs = e / (MB * lpr), rem = e - qs * (MB * lpr);
      const int b = rem / lpr, cc = rem - b * lpr;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = qs; q < rows_per_trip; q += QS) {
        const float4 t = red[(q * MB + b) * lpr + cc];
        v.x += t.x;
        v.y += t.y;
        v.z += t.z;
        v.w += t.w;
      }
      red2[e] = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < MB * lpr; e += PK_THREADS) {
      const int b = e / lpr, cc = e - b * lpr;
      float4 v = red2[e];
#pragma unroll
      for (int qs = 1; qs < QS; ++qs) {
        const float4 t = red2[qs * MB * lpr + e];
        v.x += t.x;
        v.y += t.y;
        v.z += t.z;
        v.w += t.w;
      }
      const int cg = u.tile * g.tn + cc * 4;
      if (cg < g.n) *reinterpret_cast<float4 *>(part + ((long long)u.range * MB + b) * g.n + cg) = v;
    }
    __syncthreads();
  }
};

template <int MB, int DH>
__global__ void __launch_bounds__(PK_THREADS, 1) decode_persistent_kernel(PkParams P) {
  extern __shared__ __align__(16) float pk_smem[];
  __shared__ int s_abort;
  __shared__ int s_tok[MB];
  __shared__ float red_f[PK_WARPS];
  __shared__ double red_d[PK_WARPS];
  __shared__ double ln_red[PK_WARPS * 2 * MB];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  const int D = P.d, F = P.f, V = P.vocab, H = P.n_heads, B = P.n_streams;
  // shared layout
  float *xrow = pk_smem;                 // [MB][D] residual stream
  float *yrow = xrow + MB * D;           // [MB][D]
  float *inrow = yrow + MB * D;          // [MB][in_pitch] input of the product at hand (whole row or a slice of k)
  const int in_pitch = max(D, max(P.g_w2.k_per, P.g_wo.k_per));
  const int in_floats = (max(MB * in_pitch, 3 * DH) + 3) / 4 * 4;  // also q, k, v of one head in the attention phase
  float4 *red = reinterpret_cast<float4 *>(inrow + in_floats);       // [PK_THREADS * MB] + [4 * MB * 32]
  float *sc = reinterpret_cast<float *>(red + PK_THREADS * MB + 4 * MB * 32);      // attention scores of a chunk
  unsigned target = 0;
  auto off = [&](int layer, int which) { return reinterpret_cast<const float *>(P.params + P.off[layer * 12 + which]); };
  const unsigned long long *tail = P.off + (long long)P.n_layers * 12;
  const float *tok_emb = reinterpret_cast<const float *>(P.params + tail[0]);
  const float *pos_emb = reinterpret_cast<const float *>(P.params + tail[1]);
  const float *lnf_g = reinterpret_cast<const float *>(P.params + tail[2]);
  const float *lnf_b = reinterpret_cast<const float *>(P.params + tail[3]);
  const float *lm_head = reinterpret_cast<const float *>(P.params + tail[4]);
  // LayerOff order: ln1_g, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_g, ln2_b, w1, b1, w2, b2
  enum { LN1G, LN1B, QKVW, QKVB, OUTW, OUTB, LN2G, LN2B, W1, B1, W2, B2 };
  PkGemvRun<MB> run;
  if (tid < MB) s_tok[tid] = 0;
  if (tid == 0) s_abort = 0;
  __syncthreads();
  run.prefetch(P.g_qkv, pk_unit(P.g_qkv, cta), off(0, QKVW));
  float ln_g[PK_LN_REGS], ln_b[PK_LN_REGS];
  pk_ln_prefetch(ln_g, ln_b, off(0, LN1G), off(0, LN1B), D);

  int stamp_i = 0;
  for (int t = 0; t < P.steps; ++t) {
    const int s = P.s0 + t;   // context length including the newest token
    const int p = s - 1;
    const bool stamping = P.timeline != nullptr && cta == 0 && tid == 0 && t == 10;
#define PK_STAMP() do { if (stamping && stamp_i < 64) P.timeline[stamp_i++] = global_timer(); } while (0)
    PK_STAMP();
    // ---- newest row's embedding (every CTA keeps the residual rows itself) ----
    const int rot = (int)((blockIdx.x * 32u) % (unsigned)D);  // CTAs start at different columns (see pk_gather)
    for (int e0 = tid; e0 < MB * D; e0 += PK_THREADS) {
      const int b = e0 / D;
      int c = e0 - b * D + rot;
      if (c >= D) c -= D;
      const int e = b * D + c;
      float v = 0.f;
      if (b < B) {
        int id = t == 0 ? P.ids[(long long)b * P.ids_ld + p] : s_tok[b];
        if (id < 0 || id >= V) {
          if (cta == 0 && c == 0) {
            P.err->code = DEVERR_BAD_TOKEN_ID;
            P.err->detail = id;
          }
          id = 0;
        }
        v = __ldg(tok_emb + (long long)id * D + c) + __ldg(pos_emb + (long long)p * D + c);
      }
      xrow[e] = v;
    }
    __syncthreads();
    for (int l = 0; l < P.n_layers; ++l) {
      // ---- QKV = LN1(x) W + b ----
      if (l > 0) {
        // x of this layer = W2 partial sums of the previous layer + b2 + y
        pk_gather<MB>(xrow, D, P.part_w2, P.g_w2.ranges, D, 0, D, off(l - 1, B2), yrow, D, 0);
      }
      pk_layernorm<MB>(xrow, inrow, D, ln_g, ln_b, ln_red);
      PK_STAMP();  // gathered + normalised
      // (the first unit's weights were requested before the barrier that ended the previous phase)
      for (int u0 = cta; u0 == cta || u0 < P.g_qkv.tiles * P.g_qkv.ranges; u0 += G) {
        const PkUnit u = pk_unit(P.g_qkv, u0);
        if (u0 != cta) run.prefetch(P.g_qkv, u, off(l, QKVW));
        run.finish(P.g_qkv, u, off(l, QKVW), inrow, D, 0, P.part_qkv, red);
      }
      PK_STAMP();  // QKV units done
      if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
      PK_STAMP();  // barrier
      // ---- attention over the cached keys and the newest one ----
      {
        const int chunks = min(min(P.attn_chunks_max, PK_MAX_CHUNKS), max(1, G / (B * H)));
        const int keys_per_chunk = ((s + chunks - 1) / chunks + 7) / 8 * 8;
        float *kc = P.kcache + (unsigned long long)l * P.layer_stride, *vc = P.vcache + (unsigned long long)l * P.layer_stride;
        for (int u = cta; u < B * H * chunks; u += G) {
          const int c = u % chunks, h = (u / chunks) % H, b = u / (chunks * H);
          const int c0 = c * keys_per_chunk, c1 = min(s, c0 + keys_per_chunk);
          float *out = P.part_attn + (((long long)b * H + h) * P.attn_chunks_max + c) * (DH + 2);
          if (c0 >= s) {
            if (tid == 0) {
              out[DH] = -INFINITY;
              out[DH + 1] = 0.f;
            }
            continue;
          }
          // Keys and values of earlier positions do not depend on this token: the first trip of keys
          // (four per thread group) and the first sixteen values per thread are requested before the
          // partial sums of q are gathered, so that all three reads are in flight together.
          constexpr int LPK = DH / 8, KPI = PK_THREADS / LPK, KU = 4, PARTS = PK_THREADS / DH, VU = 16;
          const int sub = tid % LPK, dcol = tid % DH, pt = tid / DH;
          const int nk = c1 - c0;
          float4 k0[KU], k1[KU];
#pragma unroll
          for (int uu = 0; uu < KU; ++uu) {
            const int j = c0 + uu * KPI + tid / LPK;
            if (j < c1 && j != p) {
              const float *kp = kc + ((long long)b * P.cap + j) * D + h * DH + sub * 8;
              k0[uu] = __ldcg(reinterpret_cast<const float4 *>(kp));
              k1[uu] = __ldcg(reinterpret_cast<const float4 *>(kp + 4));
            } else {
              k0[uu] = k1[uu] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          float vv[VU];
#pragma unroll
          for (int jj = 0; jj < VU; ++jj) {
            const int i = pt + jj * PARTS, j = c0 + i;
            vv[jj] = (i < nk && j != p) ? __ldcg(vc + ((long long)b * P.cap + j) * D + h * DH + dcol) : 0.f;
          }
          // q of this head, and the newest position's k and v when this chunk holds it: QKV partial sums + bias
          float *qs = inrow;              // [DH] q, then [DH] k, [DH] v
          const bool owner = p >= c0 && p < c1;
          for (int e = tid; e < (owner ? 3 : 1) * DH; e += PK_THREADS) {
            const int which = e / DH, cc = e - which * DH;
            const int col = which * D + h * DH + cc;
            float v = 0.f;
            {
              constexpr int GB = 12;
              const float *src = P.part_qkv + (long long)b * (3 * D) + col;
              const long long step = (long long)MB * 3 * D;
              for (int r0 = 0; r0 < P.g_qkv.ranges; r0 += GB) {
                float tt[GB];
#pragma unroll
                for (int j = 0; j < GB; ++j) tt[j] = r0 + j < P.g_qkv.ranges ? __ldcg(src + (r0 + j) * step) : 0.f;
#pragma unroll
                for (int j = 0; j < GB; ++j) v += tt[j];
              }
            }
            v += __ldg(off(l, QKVB) + col);
            qs[e] = v;
            if (which == 1) kc[((long long)b * P.cap + p) * D + h * DH + cc] = v;
            if (which == 2) vc[((long long)b * P.cap + p) * D + h * DH + cc] = v;
          }
          __syncthreads();
          const float4 q0 = *reinterpret_cast<const float4 *>(qs + sub * 8), q1 = *reinterpret_cast<const float4 *>(qs + sub * 8 + 4);
          const float scale = 1.0f / sqrtf((float)DH);
          for (int base = c0; base < c1; base += KPI * KU) {
            if (base > c0) {  // further trips of a long chunk
#pragma unroll
              for (int uu = 0; uu < KU; ++uu) {
                const int j = base + uu * KPI + tid / LPK;
                if (j < c1 && j != p) {
                  const float *kp = kc + ((long long)b * P.cap + j) * D + h * DH + sub * 8;
                  k0[uu] = __ldcg(reinterpret_cast<const float4 *>(kp));
                  k1[uu] = __ldcg(reinterpret_cast<const float4 *>(kp + 4));
                } else {
                  k0[uu] = k1[uu] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
              }
            }
#pragma unroll
            for (int uu = 0; uu < KU; ++uu) {
              const int j = base + uu * KPI + tid / LPK;
              if (j == p) {  // the newest position's key is this step's own
                k0[uu] = *reinterpret_cast<const float4 *>(qs + DH + sub * 8);
                k1[uu] = *reinterpret_cast<const float4 *>(qs + DH + sub * 8 + 4);
              }
              float dot = q0.x * k0[uu].x;
              dot = fmaf(q0.y, k0[uu].y, dot);
              dot = fmaf(q0.z, k0[uu].z, dot);
              dot = fmaf(q0.w, k0[uu].w, dot);
              dot = fmaf(q1.x, k1[uu].x, dot);
              dot = fmaf(q1.y, k1[uu].y, dot);
              dot = fmaf(q1.z, k1[uu].z, dot);
              dot = fmaf(q1.w, k1[uu].w, dot);
#pragma unroll
              for (int o = LPK >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
              if (j < c1 && sub == 0) sc[j - c0] = dot * scale;
            }
          }
          __syncthreads();
          float m = -INFINITY;
          for (int i = tid; i < nk; i += PK_THREADS) m = fmaxf(m, sc[i]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) red_f[wid] = m;
          __syncthreads();
          m = red_f[0];
#pragma unroll
          for (int q = 1; q < PK_WARPS; ++q) m = fmaxf(m, red_f[q]);
          double lsum = 0.0;
          for (int i = tid; i < nk; i += PK_THREADS) {
            const float e = expf(sc[i] - m);
            sc[i] = e;
            lsum += (double)e;
          }
          lsum = pk_warp_sum(lsum);
          if (lane == 0) red_d[wid] = lsum;
          __syncthreads();
          lsum = red_d[0];
#pragma unroll
          for (int q = 1; q < PK_WARPS; ++q) lsum += red_d[q];
          float o = 0.f;
#pragma unroll
          for (int jj = 0; jj < VU; ++jj) {  // the values requested at the start of the unit
            const int i = pt + jj * PARTS;
            if (i < nk) o = fmaf(sc[i], c0 + i == p ? qs[2 * DH + dcol] : vv[jj], o);
          }
          for (int i0 = pt + VU * PARTS; i0 < nk; i0 += 8 * PARTS) {  // the rest of a long chunk
            float vw[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int i = i0 + jj * PARTS, j = c0 + i;
              vw[jj] = i >= nk ? 0.f
                       : j == p ? qs[2 * DH + dcol]
                                : __ldcg(vc + ((long long)b * P.cap + j) * D + h * DH + dcol);
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int i = i0 + jj * PARTS;
              if (i < nk) o = fmaf(sc[i], vw[jj], o);
            }
          }
          float *opart = reinterpret_cast<float *>(red);
          opart[tid] = o;
          __syncthreads();
          if (tid < DH) {
            float tsum = opart[tid];
#pragma unroll
            for (int q = 1; q < PARTS; ++q) tsum += opart[q * DH + tid];
            out[tid] = tsum;
            if (tid == 0) {
              out[DH] = m;
              out[DH + 1] = (float)lsum;
            }
          }
          __syncthreads();
        }
        // the out-projection's weights do not depend on the attention: request them before the barrier
        const PkUnit uw = pk_unit(P.g_wo, cta);
        run.prefetch(P.g_wo, uw, off(l, OUTW));
        PK_STAMP();  // attention units done
        if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
        PK_STAMP();  // barrier
        // ---- y = ctx Wo + bo + x: every CTA joins the attention chunks of the heads its k range covers ----
        for (int u0 = cta; u0 == cta || u0 < P.g_wo.tiles * P.g_wo.ranges; u0 += G) {
          const PkUnit u = pk_unit(P.g_wo, u0);
          if (u0 != cta) run.prefetch(P.g_wo, u, off(l, OUTW));
          if (u.valid) {
            // Join the attention chunks of the heads this range of k covers. Every thread reads, for
            // its element, each chunk's maximum, sum and output in one batch of independent loads and
            // forms the common maximum, the weights exp(max_chunk - max) and the total itself, in chunk
            // order (threads of one head repeat the same few operations; one round trip instead of three).
            const int nrows = u.ke - u.kb;
            for (int e = tid; e < MB * nrows; e += PK_THREADS) {
              const int b = e / nrows, r = e - b * nrows, col = u.kb + r;
              float v = 0.f;
              if (b < B) {
                const int h = col / DH, dd = col - h * DH;
                const float *pp = P.part_attn + ((long long)b * H + h) * P.attn_chunks_max * (DH + 2);
                float mq[PK_MAX_CHUNKS], lq[PK_MAX_CHUNKS], oq[PK_MAX_CHUNKS];
#pragma unroll
                for (int q = 0; q < PK_MAX_CHUNKS; ++q) {
                  const bool live = q < chunks;
                  mq[q] = live ? __ldcg(pp + q * (DH + 2) + DH) : -INFINITY;
                  lq[q] = live ? __ldcg(pp + q * (DH + 2) + DH + 1) : 0.f;
                  oq[q] = live ? __ldcg(pp + q * (DH + 2) + dd) : 0.f;
                }
                float mm = -INFINITY;
#pragma unroll
                for (int q = 0; q < PK_MAX_CHUNKS; ++q) mm = fmaxf(mm, mq[q]);
                double ll = 0.0;
                float oo = 0.f;
#pragma unroll
                for (int q = 0; q < PK_MAX_CHUNKS; ++q) {
                  if (mq[q] != -INFINITY) {  // not an empty chunk
                    const float w = expf(mq[q] - mm);
                    ll += (double)lq[q] * (double)w;
                    oo = fmaf(oq[q], w, oo);
                  }
                }
                v = oo * (float)(1.0 / ll);
              }
              inrow[b * in_pitch + r] = v;
            }
            __syncthreads();
          }
          run.finish(P.g_wo, u, off(l, OUTW), inrow, in_pitch, u.kb, P.part_wo, red);
        }
      }
      {
        const PkUnit uw = pk_unit(P.g_w1, cta);
        run.prefetch(P.g_w1, uw, off(l, W1));
        pk_ln_prefetch(ln_g, ln_b, off(l, LN2G), off(l, LN2B), D);
      }
      PK_STAMP();  // out-projection units done
      if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
      PK_STAMP();  // barrier
      // ---- h = relu(LN2(y) W1 + b1), y = out-projection partial sums + bo + x ----
      pk_gather<MB>(yrow, D, P.part_wo, P.g_wo.ranges, D, 0, D, off(l, OUTB), xrow, D, 0);
      pk_layernorm<MB>(yrow, inrow, D, ln_g, ln_b, ln_red);
      PK_STAMP();  // gathered + normalised
      for (int u0 = cta; u0 == cta || u0 < P.g_w1.tiles * P.g_w1.ranges; u0 += G) {
        const PkUnit u = pk_unit(P.g_w1, u0);
        if (u0 != cta) run.prefetch(P.g_w1, u, off(l, W1));
        run.finish(P.g_w1, u, off(l, W1), inrow, D, 0, P.part_w1, red);
      }
      {
        const PkUnit uw = pk_unit(P.g_w2, cta);
        run.prefetch(P.g_w2, uw, off(l, W2));
      }
      PK_STAMP();  // W1 units done
      if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
      PK_STAMP();  // barrier
      // ---- W2 partial sums of the hidden row: each unit gathers its own slice of h ----
      for (int u0 = cta; u0 == cta || u0 < P.g_w2.tiles * P.g_w2.ranges; u0 += G) {
        const PkUnit u = pk_unit(P.g_w2, u0);
        if (u0 != cta) run.prefetch(P.g_w2, u, off(l, W2));
        if (u.valid)
          pk_gather<MB>(inrow, in_pitch, P.part_w1, P.g_w1.ranges, F, u.kb, u.ke - u.kb, off(l, B1), nullptr, 0, 1);
        run.finish(P.g_w2, u, off(l, W2), inrow, in_pitch, u.kb, P.part_w2, red);
      }
      {
        const bool last = l + 1 == P.n_layers;
        const PkGemv &gn = last ? P.g_head : P.g_qkv;
        const PkUnit uw = pk_unit(gn, cta);
        run.prefetch(gn, uw, last ? lm_head : off(l + 1, QKVW));
        pk_ln_prefetch(ln_g, ln_b, last ? lnf_g : off(l + 1, LN1G), last ? lnf_b : off(l + 1, LN1B), D);
      }
      PK_STAMP();  // W2 units done
      if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
      PK_STAMP();  // barrier
    }
    // ---- head: logits = LN_f(x) W_head, x = last W2 partial sums + b2 + y ----
    pk_gather<MB>(xrow, D, P.part_w2, P.g_w2.ranges, D, 0, D, off(P.n_layers - 1, B2), yrow, D, 0);
    pk_layernorm<MB>(xrow, inrow, D, ln_g, ln_b, ln_red);
    for (int u0 = cta; u0 == cta || u0 < P.g_head.tiles * P.g_head.ranges; u0 += G) {
      const PkUnit u = pk_unit(P.g_head, u0);
      if (u0 != cta) run.prefetch(P.g_head, u, lm_head);
      run.finish(P.g_head, u, lm_head, inrow, D, 0, P.part_head, red);
    }
    if (t + 1 < P.steps) {
      const PkUnit uw = pk_unit(P.g_qkv, cta);
      run.prefetch(P.g_qkv, uw, off(0, QKVW));
      pk_ln_prefetch(ln_g, ln_b, off(0, LN1G), off(0, LN1B), D);
    }
    if (!pk_grid_sync(P.barrier, target, G, P.err, &s_abort)) return;
    // ---- selection: every CTA adds the head's partial sums and finds the first maximum itself
    // (inference.cpp:188-198: strict '>' from index 0), so no further barrier is needed before the
    // next token's embedding; CTA 0 records the token.
    for (int b = 0; b < B; ++b) {
      float best = -3.402823466e+38f;
      int bi = 0x7fffffff;
      for (int c = tid; c < V; c += PK_THREADS) {
        float v = 0.f;
        {
          constexpr int GB = 16;
          const float *src = P.part_head + (long long)b * V + c;
          const long long step = (long long)MB * V;
          for (int r0 = 0; r0 < P.g_head.ranges; r0 += GB) {
            float tt[GB];
#pragma unroll
            for (int j = 0; j < GB; ++j) tt[j] = r0 + j < P.g_head.ranges ? __ldcg(src + (r0 + j) * step) : 0.f;
#pragma unroll
            for (int j = 0; j < GB; ++j) v += tt[j];
          }
        }
        if (cta == 0 && t + 1 == P.steps) P.logits[(long long)b * V + c] = v;
        if (v > best || (v == best && c < bi)) {
          best = v;
          bi = c;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) {
          best = ob;
          bi = oi;
        }
      }
      __syncthreads();
      if (lane == 0) {
        red_f[wid] = best;
        reinterpret_cast<int *>(red_d)[wid] = bi;
      }
      __syncthreads();
      if (tid == 0) {
        for (int q = 1; q < PK_WARPS; ++q) {
          const float ob = red_f[q];
          const int oi = reinterpret_cast<int *>(red_d)[q];
          if (ob > best || (ob == best && oi < bi)) {
            best = ob;
            bi = oi;
          }
        }
        if (bi == 0x7fffffff) bi = 0;
        s_tok[b] = bi;
        if (cta == 0) {
          P.ids[(long long)b * P.ids_ld + s] = bi;
          P.out_tokens[(long long)b * P.out_ld + P.step0 + t] = bi;
        }
      }
      __syncthreads();
    }
  }
  if (cta == 0 && tid == 0) {
    P.state->s = P.s0 + P.steps;
    P.state->step = P.step0 + P.steps;
  }
}

PkGemv pk_plan(int k, int n, int G) {
  PkGemv g{};
  g.k = k;
  g.n = n;
  // column tiles wide enough for whole sectors, narrow enough that about ten k ranges per tile fill the GPU
  g.tn = 128;
  while (g.tn > 32 && ((n + g.tn - 1) / g.tn) * 10 < G) g.tn >>= 1;
  g.tiles = (n + g.tn - 1) / g.tn;
  int ranges = G / g.tiles;
  if (ranges > k / 16) ranges = k / 16;
  if (ranges < 1) ranges = 1;
  g.k_per = (k + ranges - 1) / ranges;
  g.ranges = (k + g.k_per - 1) / g.k_per;
  return g;
}

template <int MB, int DH>
void pk_launch(const PkParams &P, int G, size_t smem, cudaStream_t st) {
  static std::mutex mu;
  static bool configured[64] = {};
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LB_CUDA(cudaFuncSetAttribute(decode_persistent_kernel<MB, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem > 200 * 1024 ? (int)smem : 200 * 1024));
      if (dev < 64) configured[dev] = true;
    }
  }
  PkParams copy = P;
  void *args[] = {&copy};
  LB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(decode_persistent_kernel<MB, DH>), dim3((unsigned)G),
                                      dim3(PK_THREADS), args, smem, st));
}

}  // namespace

bool decode_persistent_supports(int n_streams, int n_heads, int d_model, int d_ff, int vocab) {
  if (n_streams < 1 || n_streams > 8 || d_model % n_heads != 0) return false;
  const int dh = d_model / n_heads;
  if (dh != 32 && dh != 64) return false;
  return d_model % 4 == 0 && d_ff % 4 == 0 && vocab % 4 == 0 && d_model >= 32 && d_model <= 2048;
}

size_t decode_persistent_scratch_floats(int n_streams, int n_heads, int d_model, int d_ff, int vocab, int sm_count) {
  const int mb = n_streams <= 1 ? 1 : n_streams <= 2 ? 2 : n_streams <= 4 ? 4 : 8;
  const int G = sm_count;
  auto part = [&](int k, int n) { return (size_t)pk_plan(k, n, G).ranges * mb * n; };
  const int dh = d_model / n_heads;
  const size_t attn = (size_t)mb * n_heads * (size_t)G * (dh + 2);
  return part(d_model, 3 * d_model) + part(d_model, d_model) + part(d_model, d_ff) + part(d_ff, d_model) +
         part(d_model, vocab) + attn + 64;
}

void launch_decode_persistent(const DecodePersistentArgs &a, cudaStream_t st) {
  const int mb = a.n_streams <= 1 ? 1 : a.n_streams <= 2 ? 2 : a.n_streams <= 4 ? 4 : 8;
  const int G = a.sm_count, dh = a.d_model / a.n_heads;
  PkParams P{};
  P.params = a.params;
  P.off = a.offsets;
  P.n_layers = a.n_layers;
  P.n_heads = a.n_heads;
  P.d = a.d_model;
  P.f = a.d_ff;
  P.vocab = a.vocab;
  P.max_seq = a.max_seq;
  P.n_streams = a.n_streams;
  P.kcache = a.kcache;
  P.vcache = a.vcache;
  P.cap = a.cap;
  P.layer_stride = a.layer_stride;
  P.ids = a.ids;
  P.ids_ld = a.ids_ld;
  P.out_tokens = a.out_tokens;
  P.out_ld = a.out_ld;
  P.state = a.state;
  P.logits = a.logits;
  P.barrier = a.barrier;
  P.s0 = a.s0;
  P.step0 = a.step0;
  P.steps = a.steps;
  P.err = a.err;
  P.timeline = a.timeline;
  P.g_qkv = pk_plan(a.d_model, 3 * a.d_model, G);
  P.g_wo = pk_plan(a.d_model, a.d_model, G);
  P.g_w1 = pk_plan(a.d_model, a.d_ff, G);
  P.g_w2 = pk_plan(a.d_ff, a.d_model, G);
  P.g_head = pk_plan(a.d_model, a.vocab, G);
  P.attn_chunks_max = G;
  float *p = a.scratch;
  P.part_qkv = p;
  p += (size_t)P.g_qkv.ranges * mb * 3 * a.d_model;
  P.part_wo = p;
  p += (size_t)P.g_wo.ranges * mb * a.d_model;
  P.part_w1 = p;
  p += (size_t)P.g_w1.ranges * mb * a.d_ff;
  P.part_w2 = p;
  p += (size_t)P.g_w2.ranges * mb * a.d_model;
  P.part_head = p;
  p += (size_t)P.g_head.ranges * mb * a.vocab;
  P.part_attn = p;
  const int in_pitch = std::max(a.d_model, std::max(P.g_w2.k_per, P.g_wo.k_per));
  const int in_floats = (std::max(mb * in_pitch, 3 * dh) + 3) / 4 * 4;
  // scores of a chunk (up to the whole context) or the chunk weights of the heads a unit joins
  const int sc_floats = std::max(a.max_seq, 4 * G) + 64;
  const size_t smem = ((size_t)2 * mb * a.d_model + in_floats + (size_t)4 * (PK_THREADS * mb + 4 * mb * 32) + sc_floats) * 4;
  LB_CUDA(cudaMemsetAsync(a.barrier, 0, 8, st));
#define PK_CASE(MBV, DHV)                                  \
  if (mb == MBV && dh == DHV) {                            \
    pk_launch<MBV, DHV>(P, G, smem, st);                   \
    return;                                                \
  }
  PK_CASE(1, 64) PK_CASE(2, 64) PK_CASE(4, 64) PK_CASE(8, 64)
  PK_CASE(1, 32) PK_CASE(2, 32) PK_CASE(4, 32) PK_CASE(8, 32)
#undef PK_CASE
  throw std::invalid_argument("litnice_b200: the resident decode kernel does not take this shape");
}

}  // namespace lb
