// Tensor-core projection GEMM for sm_100a: interface.
//
// C[M,N] = A[M,K] * W[K,N] (+ bias, + residual, ReLU) with fp32 accuracy on the
// 5th-generation tensor cores by the three-product TF32 split
//     a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo,   x_hi = tf32(x), x_lo = tf32(x - x_hi)
// accumulated in fp32 in tensor memory. Operands are stored already split:
// activations as two dense [rows, K] arrays written by the producing kernel,
// weights as two K-major [N, K] arrays built once when parameters are loaded.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace lb {

constexpr int TC_BM = 128;  // rows per CTA (one UMMA M=128 tile)
constexpr int TC_BK = 32;   // fp32 elements per k-block = one 128-byte swizzle row
constexpr int TC_STAT_SLOTS = 32;  // row-statistics slots of 64 columns per row (rows up to 2048 wide)

struct TcMatrix {  // one split operand: two tensor maps over K-major arrays (fp32 TF32 pairs or fp16 pairs)
  CUtensorMap hi, lo;
};

// Second operand format: x = (hi + lo) / scale with hi, lo fp16 and scale a power
// of two chosen per block of 64 consecutive k (per row for activations, one for a
// whole weight matrix) so that the block's largest magnitude lands in [2^12, 2^13).
// hi = fp16(x * scale), lo = fp16(x * scale - hi): 22 significant bits like a TF32
// pair, but an fp16 instruction covers 16 of k at twice the TF32 rate and the
// operands take half the bytes. Products are formed on scaled operands; the drain
// multiplies every 64-wide accumulation chain by the two inverse scales.
constexpr int TC_F16_SLOT = 64;  // k elements per scale block = one 128-byte swizzle row of fp16
struct TcPairF16 {  // activations in that format
  __half *hi = nullptr, *lo = nullptr;  // [rows, k]
  float *inv_scale = nullptr;           // [rows, k / 64]
};

struct TcEpilogue {
  const float *bias = nullptr;      // [N]
  const float *residual = nullptr;  // [M, N] dense, added after the bias
  int relu = 0;
  float *c = nullptr;               // [M, N] dense fp32 result (may be null)
  float *c_hi = nullptr;            // optional split result for a following GEMM
  float *c_lo = nullptr;
  TcPairF16 c_f16;                  // optional fp16-pair result (n % 64 == 0) for a following GEMM
  // Optional transposed store of the columns from vt_col0 on (the V third of a
  // QKV projection) for the tensor-core attention, which wants V K-major:
  // element (row r = stream * s + t, column vt_col0 + c) goes, split, to
  // vt_hi/vt_lo[(stream * vt_rows + c) * vt_pitch + t] instead of c / c_hi / c_lo.
  // s is state->s when state is set (graph replay), else vt_s.
  float *vt_hi = nullptr;
  float *vt_lo = nullptr;
  int vt_col0 = 0, vt_rows = 0, vt_pitch = 0, vt_s = 0, vt_streams = 0;
  const LoopState *state = nullptr;
  // The same outputs as fp16 pairs under fixed scales, for the fp16-pair attention kernel: every
  // 64-column block of the result (one head of Q, K or V) is multiplied by col_scale[column / 64],
  // a power of two chosen when the weights were loaded so that no value can leave fp16's range;
  // columns below vt_col0 go row-major to qk16_hi/lo [M, N], the V columns transposed to
  // vt16_hi/lo (laid out as vt_hi/vt_lo).
  __half *qk16_hi = nullptr, *qk16_lo = nullptr;
  __half *vt16_hi = nullptr, *vt16_lo = nullptr;
  const float *col_scale = nullptr;  // [N / 64]
  __host__ __device__ bool has_vt() const { return vt_hi != nullptr || vt16_hi != nullptr; }
  // LayerNorm folded into the product. With W' = diag(gamma) W the reference's
  // LN(x) W + b (layernorm_forward then gemm_ranked_matrix_rhs + add_bias_rowwise)
  // equals inv_std * (x W' - mean * u) + v, u[n] = sum_k W'[k,n],
  // v[n] = sum_k beta[k] W[k,n] + b[n]: the kernel multiplies the raw rows by W'
  // and the epilogue applies the row statistics. ln_u != nullptr turns this on;
  // `bias` then holds v. Statistics come as partial sums (sum x, sum x^2) in
  // double over slots of 64 columns, ln_slots per row, written by the kernel
  // that produced x (stats_out below) and added here in slot order.
  const float *ln_u = nullptr;
  const double2 *ln_stats = nullptr;  // [rows][TC_STAT_SLOTS]
  int ln_slots = 0;
  // Producer side: per row and 64-column slot of the stored result (after bias,
  // residual, ReLU) the sums (x, x^2) in double, at stats_out[row][column / 64].
  double2 *stats_out = nullptr;
  // Measurement aid: when set, CTA (0,0,0) stores %globaltimer stamps of its
  // pipeline milestones here (entries 0-7) and every CTA contributes to the
  // earliest start [8] (preset to all ones), latest end [9] and latest start [10].
  unsigned long long *timeline = nullptr;
};

// True when the driver exposes cuTensorMapEncodeTiled (resolved at run time so
// that the library loads on machines without a GPU driver).
bool tc_runtime_available();

// Tensor map over a dense row-major fp32 array [rows, k] with boxes of
// box_rows x 32 elements and the 128-byte swizzle the UMMA descriptors expect.
void tc_make_map(CUtensorMap *map, const float *base, unsigned long long rows, unsigned long long k,
                 unsigned box_rows);
// The same over an fp16 array, boxes of box_rows x 64 elements (k % 64 == 0).
void tc_make_map_f16(CUtensorMap *map, const __half *base, unsigned long long rows, unsigned long long k,
                     unsigned box_rows);

// Tensor map over a dense row-major fp32 array [rows, cols] with boxes of box_rows x box_cols
// elements stored as they lie (no swizzle); cols % 4 == 0, base 16-byte aligned.
void tc_make_map_plain(CUtensorMap *map, const float *base, unsigned long long rows, unsigned long long cols,
                       unsigned box_rows, unsigned box_cols);

// How one product is tiled: tile width (64, 128 or 256 columns), how many CTAs share
// the k range of a tile, and the scratch that sharing needs (floats of partial
// tiles; int counters that must be zero before the first launch and are left
// at zero by every launch).
struct TcPlan {
  int bn;
  int splits;
  size_t scratch_floats;
  size_t counters;
};
// k_block: k elements per pipeline stage (32 for TF32 pairs, 64 for fp16 pairs).
// clusters_ok: false plans for split-k through global scratch only.
TcPlan tc_plan(int m, int n, int k, bool has64, bool has128, bool has256, int k_block = TC_BK,
               bool clusters_ok = true);

// Requires n % plan.bn == 0, k % 32 == 0; a maps must use box rows 128, b maps
// box rows plan.bn.
void launch_gemm_tc(const TcMatrix &a, const TcMatrix &b, int m, int n, int k, const TcPlan &plan,
                    const TcEpilogue &ep, float *scratch, int *counters, DevErr *err, cudaStream_t st);
// The same product on fp16 pairs: maps over the fp16 arrays (k % 64 == 0), the
// activations' inverse scales [rows, k / 64] and the weight matrix's inverse scale
// (one float in device memory, written when the weights were converted).
void launch_gemm_tc_f16(const TcMatrix &a, const float *a_inv_scale, const TcMatrix &b, const float *b_inv_scale,
                        int m, int n, int k, const TcPlan &plan, const TcEpilogue &ep, float *scratch, int *counters,
                        DevErr *err, cudaStream_t st);
// Row-major W [k, n] (rows optionally scaled) -> K-major fp16 pair [n, k] with one
// scale for the matrix; *inv_scale_dev (device float) receives its inverse.
// amax_scratch: one int of device memory.
void launch_transpose_split_f16(const float *w, int k, int n, __half *wt_hi, __half *wt_lo, float *inv_scale_dev,
                                cudaStream_t st, const float *row_scale, int *amax_scratch);
// Dense rows x [rows, k] -> fp16 pair with per-row scales per 64 columns.
void launch_split_f16(const float *x, long long rows, int k, const TcPairF16 &out, cudaStream_t st);

// Scale of one block from its largest magnitude: a power of two with
// amax * scale in [2^12, 2^13) (1 for a block of zeros or denormals).
__device__ __forceinline__ float f16_block_scale(float amax, float *inv) {
  int eb = (__float_as_int(amax) >> 23) & 0xff;  // amax = 1.m * 2^(eb - 127)
  eb = eb < 20 ? 139 : eb;                        // nothing to scale: 2^0
  eb = eb > 250 ? 250 : eb;
  *inv = __int_as_float((eb - 12) << 23);         // 2^(eb - 139)
  return __int_as_float((266 - eb) << 23);        // 2^(139 - eb)
}
// Four consecutive elements of a block whose scale is known -> the pair, packed for 8-byte stores.
__device__ __forceinline__ void f16_pair4(float4 v, float scale, uint2 &hi, uint2 &lo) {
  const float a = v.x * scale, b = v.y * scale, c = v.z * scale, d = v.w * scale;
  const __half2 h01 = __floats2half2_rn(a, b), h23 = __floats2half2_rn(c, d);  // packed conversions
  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
  const __half2 l01 = __floats2half2_rn(a - f01.x, b - f01.y), l23 = __floats2half2_rn(c - f23.x, d - f23.y);
  hi.x = *reinterpret_cast<const unsigned *>(&h01);
  hi.y = *reinterpret_cast<const unsigned *>(&h23);
  lo.x = *reinterpret_cast<const unsigned *>(&l01);
  lo.y = *reinterpret_cast<const unsigned *>(&l23);
}
// 16 consecutive lanes hold the 64 columns of one block of one row, a float4
// each (all 32 lanes of the warp call this together): scale from the block's
// largest magnitude, the lane's four elements stored, the inverse scale by the
// block's first lane. `active` false: the lane's values are ignored and nothing
// is stored for it.
__device__ __forceinline__ void f16_store_block(float4 v, bool active, __half *hi4, __half *lo4, float *inv_slot) {
  float am = active ? fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))) : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  float inv;
  const float scale = f16_block_scale(am, &inv);
  if (active) {
    uint2 hi, lo;
    f16_pair4(v, scale, hi, lo);
    *reinterpret_cast<uint2 *>(hi4) = hi;
    *reinterpret_cast<uint2 *>(lo4) = lo;
    if ((threadIdx.x & 15) == 0) *inv_slot = inv;
  }
}

// attention_tc.cu: fused causal attention on the tensor cores for head
// dimension 64. qk: maps (box 128 rows x 32) over the split [rows, 3*d_model]
// output of the QKV projection; vt: maps (box 64 rows x 32) over the split V^T
// arrays [n_streams * d_model, pitch] the same projection stores (pitch a
// multiple of 128 that covers s). Writes the context as a TF32 hi/lo pair, or as
// the fp16 pair ctx_f16 (one scale per row and head) when that is given.
// state != nullptr: s is an upper bound with the same number of 128-row tiles
// as the actual context length state->s. Scratch and zero-resting counters as
// attention_tc_plan says. timeline (optional, 12 entries: [8] preset to all ones,
// the rest zero): %globaltimer stamps of CTA (0,0,0) and the kernel's span.
bool attention_tc_supports(int n_heads, int d_model);
AttentionPlan attention_tc_plan(int n_streams, int s, int n_heads);
void launch_attention_tc(const TcMatrix &qk, const TcMatrix &vt, float *ctx_hi, float *ctx_lo, int n_streams, int s,
                         int n_heads, int d_model, float *scratch, int *counters, const LoopState *state,
                         DevErr *err, cudaStream_t st, unsigned long long *timeline = nullptr,
                         const TcPairF16 *ctx_f16 = nullptr);
// attention_tc16.cu: the same on fp16 pairs under fixed per-head scales. qk: fp16 maps (box 128
// rows x 64) over the [rows, 3*d_model] pair the QKV projection stores (TcEpilogue::qk16_*); vt:
// fp16 maps (box 64 rows x 64) over its transposed V pair; head_inv_scale [3 * n_heads]: the
// inverse scales of the heads of Q, K and V (launch_head_scales). Plan, scratch, counters, state
// and timeline as launch_attention_tc; the context leaves as the fp16 pair ctx_f16.
void launch_attention_tc16(const TcMatrix &qk, const TcMatrix &vt, const float *head_inv_scale, int n_streams, int s,
                           int n_heads, int d_model, float *scratch, int *counters, const LoopState *state,
                           DevErr *err, cudaStream_t st, unsigned long long *timeline, const TcPairF16 &ctx_f16);
// scale / inv_scale [n / 64]: per 64 columns of LN(x) W + bias (W [k, n] row-major, the LayerNorm's
// gamma and beta [k]) the power of two that brings the largest value those columns can take for
// any input row into [2^14, 2^15), and its inverse.
void launch_head_scales(const float *w, int k, int n, const float *gamma, const float *beta, const float *bias,
                        float *scale, float *inv_scale, cudaStream_t st);

// x -> (hi, lo) elementwise.
void launch_split_tf32(const float *x, float *hi, float *lo, long long count, cudaStream_t st);
// Row-major W [k, n] -> K-major split copies wt_hi, wt_lo [n, k]; row_scale
// (optional, [k]) multiplies row k first (the LayerNorm scale folded into W).
void launch_transpose_split(const float *w, int k, int n, float *wt_hi, float *wt_lo, cudaStream_t st,
                            const float *row_scale = nullptr);
// u[n] = sum_k gamma[k] W[k,n], v[n] = sum_k beta[k] W[k,n] + bias[n] (sums in double).
// f16_amax_bits (optional): the matrix is stored as an fp16 pair under the scale that
// launch_transpose_split_f16 derived from this maximum; u sums those stored values.
void launch_ln_fold_vectors(const float *w, int k, int n, const float *gamma, const float *beta, const float *bias,
                            float *u, float *v, cudaStream_t st, const int *f16_amax_bits = nullptr);
// Mean and 1/std of one row from its partial sums, as layernorm_forward of the
// reference forms them (biased variance, eps 1e-5 added in float).
__device__ __forceinline__ float2 ln_row_stats(const double2 *slots, int n_slots, int d) {
  double sx = 0.0, sxx = 0.0;
  for (int i = 0; i < n_slots; ++i) {
    const double2 t = slots[i];
    sx += t.x;
    sxx += t.y;
  }
  const double mean = sx / (double)d;
  double var = sxx / (double)d - mean * mean;
  if (var < 0.0) var = 0.0;
  return make_float2((float)mean, 1.0f / sqrtf((float)var + 1e-5f));
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
  unsigned h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  const float rest = x - hi;  // exact: x and hi agree in their leading 11 bits
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
  lo = __uint_as_float(l);
}

}  // namespace lb
