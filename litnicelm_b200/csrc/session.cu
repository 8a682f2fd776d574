// Native token loop (litnice_b200_* entry points). Replaces the host-driven
// loop of litnicelm's src/model/inference.cpp:265-296: per generated token the
// whole context of every stream is recomputed (the reference keeps no KV
// cache: forward_prompt runs Transformer::forward on all ids, :127-143,278-284),
// the next token is chosen on the GPU and appended on the GPU. Only token ids
// cross the host/device boundary.
//
// Data layout in HBM
//   params      the parameter arena image exactly as stored in a checkpoint
//               (named_layout.cpp:40-161); matrices are row-major [in, out].
//   ids         [max_streams, max_seq_len] int32, one row per stream.
//   activations dense row-major, rows r = stream*s + t of the current step:
//               x, y, ln, ctx [R, d]; qkv [R, 3d]; h [R, d_ff].
//   last rows   xl [>=8, d] (final LayerNorm of row s-1 of each stream),
//               logits [>=8, vocab].
// Work elided because nothing can observe it (the loop reads row s-1 only,
// inference.cpp:109-115): LN_f and the output head on rows 0..s-2, the dead
// zero-fill of the attention context, the attention-weights cache.
#include "common.cuh"
#include "gemm_tc.cuh"

#include <array>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

namespace lb {

namespace {

struct LayerOff {
  size_t ln1_g, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_g, ln2_b, w1, b1, w2, b2;
};
struct ParamLayout {
  size_t total = 0, decay = 0, tok_emb = 0, pos_emb = 0, lnf_g = 0, lnf_b = 0, lm_head = 0;
  std::vector<LayerOff> layer;
};

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// named_layout.cpp:40-161: weight-decay parameters (embeddings, matrices) first
// in declaration order, zone padded, then LayerNorm vectors and biases.
ParamLayout build_layout(const litnice_b200_dims &d) {
  ParamLayout L;
  const size_t A = d.alignment_bytes, D = d.d_model, F = d.d_ff, V = d.vocab_size, S = d.max_seq_len;
  L.layer.resize(d.n_layers);
  size_t cur = 0;
  auto put = [&](size_t &field, size_t bytes) {
    cur = align_up(cur, A);
    field = cur;
    cur += bytes;
  };
  put(L.tok_emb, 4 * V * D);
  put(L.pos_emb, 4 * S * D);
  for (auto &o : L.layer) {
    put(o.qkv_w, 4 * D * 3 * D);
    put(o.out_w, 4 * D * D);
    put(o.w1, 4 * D * F);
    put(o.w2, 4 * F * D);
  }
  put(L.lm_head, 4 * D * V);
  L.decay = align_up(cur, A);
  cur = L.decay;
  for (auto &o : L.layer) {
    put(o.ln1_g, 4 * D);
    put(o.ln1_b, 4 * D);
    put(o.qkv_b, 4 * 3 * D);
    put(o.out_b, 4 * D);
    put(o.ln2_g, 4 * D);
    put(o.ln2_b, 4 * D);
    put(o.b1, 4 * F);
    put(o.b2, 4 * D);
  }
  put(L.lnf_g, 4 * D);
  put(L.lnf_b, 4 * D);
  L.total = align_up(cur, A);
  return L;
}

MatView dense(const float *p, long long rows, long long cols) {
  MatView v{};
  v.data = reinterpret_cast<char *>(const_cast<float *>(p));
  v.nb = 0;
  v.batch = 1;
  v.rows = rows;
  v.cols = cols;
  v.rs = cols * 4;
  v.cs = 4;
  return v;
}

// One weight matrix prepared for the tensor-core GEMM: K-major hi/lo copies
// [n, k] and tensor maps for both tile widths.
struct TcWeight {
  float *hi = nullptr, *lo = nullptr;
  int k = 0, n = 0;
  bool has64 = false, has128 = false, has256 = false;
  TcMatrix m64{}, m128{}, m256{};
  // LayerNorm folded into this product (the copies above then hold diag(gamma) W): u[n], v[n] of TcEpilogue
  float *ln_u = nullptr, *ln_v = nullptr;
  // fp16-pair copies (TcPairF16 format with one scale for the matrix) instead of the TF32 pair
  __half *h_hi = nullptr, *h_lo = nullptr;
  float *h_inv_scale = nullptr;  // device float
  TcMatrix f64{}, f128{}, f256{};
  // QKV projection feeding the fp16-pair attention: fixed scale and inverse per 64 output columns (launch_head_scales)
  float *head_scale = nullptr, *head_inv = nullptr;
  bool usable() const { return has64 || has128; }
};

enum AKind { A_LN = 0, A_CTX = 1, A_H = 2, A_XL = 3 };
enum PairKind { PAIR_LN = 0, PAIR_CTX = 1, PAIR_H = 2 };

}  // namespace
}  // namespace lb

using namespace lb;

struct litnice_b200_session {
  litnice_b200_dims dims{};
  int max_streams = 0;
  int device = 0;
  cudaStream_t st = nullptr;
  ParamLayout lay;
  char *params = nullptr;
  bool params_loaded = false;

  long long cap_rows = 0;
  float *x = nullptr, *y = nullptr, *ln = nullptr, *ctx = nullptr, *qkv = nullptr, *h = nullptr;
  float *xl = nullptr, *logits = nullptr, *gemv_scratch = nullptr;
  // tensor-core path: low parts of the split activations (ln/ctx/h/xl hold the high parts)
  bool tc = false;
  bool pdl = true;         // early launch of dependent kernels (LITNICE_B200_PDL=0 disables)
  bool fused_tail = true;  // greedy steps end in one launch: norm, head, selection, advance (LITNICE_B200_FUSED_TAIL=0 disables)
  bool use_graphs = true;  // replay one captured step per 64-token context bucket (LITNICE_B200_GRAPHS=0 disables)
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int streams = 0;
    SamplerParams sp{};
    unsigned long long generation = 0;
    long long launches = 0;  // kernels in one replay
  };
  std::vector<StepGraph> graphs;       // indexed by context bucket (tiles of 64)
  unsigned long long generation = 1;   // bumped whenever a buffer a graph points at is replaced
  float *ln_lo = nullptr, *ctx_lo = nullptr, *h_lo = nullptr, *xl_lo = nullptr;
  long long xl_rows = 0;
  std::vector<std::array<TcWeight, 4>> tcw;  // per layer: qkv, out, w1, w2
  TcWeight tc_head;
  TcMatrix a_map[4]{};
  // tensor-core attention (head dimension 64): the QKV projection stores Q and K
  // split in qkv_hi/qkv_lo [rows, 3D] and V transposed and split in vt_hi/vt_lo
  // [streams * D, vt_pitch] (row = stream * D + column, one entry per position)
  bool tc_attn = false;
  float *qkv_hi = nullptr, *qkv_lo = nullptr, *vt_hi = nullptr, *vt_lo = nullptr;
  long long vt_rows = 0;
  int vt_pitch = 0;
  TcMatrix qk_map{}, vt_map{};
  // the same as fp16 pairs under fixed per-head scales (attention_tc16.cu; LITNICE_B200_ATTN16=0 keeps the TF32 pairs)
  bool attn16 = false;
  __half *qk16_hi = nullptr, *qk16_lo = nullptr, *vt16_hi = nullptr, *vt16_lo = nullptr;
  TcMatrix qk16_map{}, vt16_map{};
  // measurement aid (LITNICE_B200_ATTN_TIMELINE, profile_step only): 10 stamps per profiled attention launch
  unsigned long long *attn_timeline = nullptr;
  int attn_timeline_used = 0;
  unsigned long long *gemm_timeline = nullptr;  // the same for the projections (LITNICE_B200_TC_TIMELINE)
  int gemm_timeline_used = 0;
  static constexpr int kTimelineSlots = 64;
  // LayerNorm folded into the QKV and W1 products: the kernels that produce x and y
  // (embedding, out-projection, W2) also store them as TF32 pairs in (ln, ln_lo) and
  // leave per-row partial sums here, [rows][TC_STAT_SLOTS] (LITNICE_B200_LN_FOLD=0 disables)
  bool ln_fold = false;
  double2 *row_stats = nullptr;
  // fp16-pair operands for the layer projections (LITNICE_B200_F16=0 keeps TF32 pairs): the pairs
  // of x / y (shared, like ln / ln_lo), of the attention context and of the FFN hidden rows
  bool f16 = false;
  TcPairF16 pair_ln, pair_ctx, pair_h;
  TcMatrix pair_map[3]{};  // indexed by PairKind
  int *amax_scratch = nullptr;
  float *tc_scratch = nullptr;   // split-k partial tiles of the tensor-core GEMM
  int *tc_counters = nullptr;
  float *attn_scratch = nullptr;
  int *attn_counters = nullptr;
  size_t attn_scratch_floats = 0, attn_counter_count = 0;
  float *logits_all = nullptr;
  long long logits_all_rows = 0;
  float *probs = nullptr;
  int *ids = nullptr, *out_tokens = nullptr;
  int out_cap = 0;
  unsigned *mt = nullptr;
  LoopState *state = nullptr;
  void *sampler_scratch = nullptr;
  size_t sampler_scratch_bytes_ = 0;
  DevErr *err_host = nullptr, *err_dev = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;

  // Opt-in cached mode (LITNICE_B200_KV_CACHE=1, an extension: the reference keeps no cache). Keys
  // and values of earlier positions stay in HBM, [n_layers][kv_streams][kv_cap][d_model] each, and a
  // step computes one new row per stream (decode.cu). Runs on the fp32 kernels: the whole-context
  // pass over the prompt that fills the caches on the SIMT path, the steps on the few-row products.
  bool kv = false;
  bool kv_fuse = true;  // LayerNorms inside the products, one-launch greedy tail (LITNICE_B200_KV_FUSE=0: kernels of their own)
  float *kcache = nullptr, *vcache = nullptr;
  int kv_cap = 0, kv_streams = 0;
  int kv_len = 0;         // positions of the current streams held in the caches
  bool kv_store = false;  // the whole-context pass under way also fills the caches
  float *dx = nullptr, *dy = nullptr, *dln = nullptr, *dqkv = nullptr, *dctx = nullptr, *dh = nullptr;  // step rows
  float *dec_part = nullptr;  // partial attention sums of the key chunks
  size_t dec_part_floats = 0;
  int *dec_counters = nullptr;  // per (stream, head): chunks finished; rests at zero
  // greedy runs of up to 8 streams: all steps after the first in one resident kernel
  // (decode_persistent.cu; LITNICE_B200_KV_PERSIST=0 keeps one graph replay per token)
  bool kv_persist = true;
  int sm_count = 0;
  unsigned long long *pk_offsets = nullptr;  // device table of parameter offsets
  float *pk_scratch = nullptr;
  size_t pk_scratch_floats = 0;
  unsigned *pk_barrier = nullptr;

  bool keep_logits = false;
  float *step_logits = nullptr;
  long long step_logits_cap = 0, step_logits_count = 0;

  int cur_streams = 0, cur_prompt_len = 0, cur_tokens = 0;
  litnice_b200_stats stats{};
  long long launches = 0;

  // per-class event timing (profile_step only)
  bool profiling = false;
  bool stamping = false;  // device-clock stamps instead of events: launches overlap as in the loop
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> gemm_ev, attn_ev;
  double gemm_flops = 0, stamped_gemm_flops = 0;

  std::string error;
};

namespace {

const float *P(const litnice_b200_session *s, size_t off) {
  return reinterpret_cast<const float *>(s->params + off);
}

void free_activations(litnice_b200_session *s) {
  for (float **p : {&s->x, &s->y, &s->ln, &s->ctx, &s->qkv, &s->h, &s->ln_lo, &s->ctx_lo, &s->h_lo, &s->qkv_hi,
                    &s->qkv_lo}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  if (s->row_stats) cudaFree(s->row_stats);
  s->row_stats = nullptr;
  for (__half **p : {&s->qk16_hi, &s->qk16_lo}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (TcPairF16 *p : {&s->pair_ln, &s->pair_ctx, &s->pair_h}) {
    if (p->hi) cudaFree(p->hi);
    if (p->lo) cudaFree(p->lo);
    if (p->inv_scale) cudaFree(p->inv_scale);
    *p = TcPairF16{};
  }
  s->cap_rows = 0;
}

void make_activation_map(TcMatrix *m, const float *hi, const float *lo, long long rows, int k) {
  tc_make_map(&m->hi, hi, (unsigned long long)rows, (unsigned long long)k, TC_BM);
  tc_make_map(&m->lo, lo, (unsigned long long)rows, (unsigned long long)k, TC_BM);
}

void ensure_rows(litnice_b200_session *s, long long rows) {
  if (s->tc) rows = (rows + TC_BM - 1) / TC_BM * TC_BM;  // whole TMA boxes
  if (rows <= s->cap_rows) return;
  LB_CUDA(cudaStreamSynchronize(s->st));
  free_activations(s);
  const size_t D = s->dims.d_model, F = s->dims.d_ff;
  auto alloc = [&](float **p, size_t floats) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(p), floats * sizeof(float));
    if (e != cudaSuccess) {
      free_activations(s);
      throw std::bad_alloc();
    }
  };
  alloc(&s->x, rows * D);
  alloc(&s->y, rows * D);
  alloc(&s->ln, rows * D);
  // With fp16-pair operands the attention context, the FFN hidden rows and the QKV
  // output exist only in the formats their consumers read (pair_ctx, pair_h,
  // qkv_hi/qkv_lo + vt), not as fp32 arrays.
  if (!s->f16) {
    alloc(&s->ctx, rows * D);
    alloc(&s->qkv, rows * 3 * D);
    alloc(&s->h, rows * F);
  }
  if (s->tc) {
    alloc(&s->ln_lo, rows * D);
    make_activation_map(&s->a_map[A_LN], s->ln, s->ln_lo, rows, (int)D);  // also the final norm before an all-rows head
    if (!s->f16) {
      alloc(&s->ctx_lo, rows * D);
      alloc(&s->h_lo, rows * F);
      make_activation_map(&s->a_map[A_CTX], s->ctx, s->ctx_lo, rows, (int)D);
      make_activation_map(&s->a_map[A_H], s->h, s->h_lo, rows, (int)F);
    }
  }
  if (s->f16) {
    auto alloc_pair = [&](TcPairF16 *p, PairKind kind, size_t cols) {
      const size_t elems = (size_t)rows * cols, slots = (size_t)rows * (cols / TC_F16_SLOT);
      if (cudaMalloc(reinterpret_cast<void **>(&p->hi), elems * 2) != cudaSuccess ||
          cudaMalloc(reinterpret_cast<void **>(&p->lo), elems * 2) != cudaSuccess ||
          cudaMalloc(reinterpret_cast<void **>(&p->inv_scale), slots * 4) != cudaSuccess) {
        free_activations(s);
        throw std::bad_alloc();
      }
      LB_CUDA(cudaMemsetAsync(p->hi, 0, elems * 2, s->st));
      LB_CUDA(cudaMemsetAsync(p->lo, 0, elems * 2, s->st));
      LB_CUDA(cudaMemsetAsync(p->inv_scale, 0, slots * 4, s->st));
      tc_make_map_f16(&s->pair_map[kind].hi, p->hi, (unsigned long long)rows, cols, TC_BM);
      tc_make_map_f16(&s->pair_map[kind].lo, p->lo, (unsigned long long)rows, cols, TC_BM);
    };
    alloc_pair(&s->pair_ln, PAIR_LN, D);
    alloc_pair(&s->pair_ctx, PAIR_CTX, D);
    alloc_pair(&s->pair_h, PAIR_H, F);
  }
  if (s->ln_fold) {
    if (cudaMalloc(reinterpret_cast<void **>(&s->row_stats), (size_t)rows * TC_STAT_SLOTS * sizeof(double2)) !=
        cudaSuccess) {
      free_activations(s);
      throw std::bad_alloc();
    }
    LB_CUDA(cudaMemsetAsync(s->row_stats, 0, (size_t)rows * TC_STAT_SLOTS * sizeof(double2), s->st));
  }
  if (s->attn16) {
    const size_t bytes = (size_t)rows * 3 * D * 2;
    if (cudaMalloc(reinterpret_cast<void **>(&s->qk16_hi), bytes) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void **>(&s->qk16_lo), bytes) != cudaSuccess) {
      free_activations(s);
      throw std::bad_alloc();
    }
    LB_CUDA(cudaMemsetAsync(s->qk16_hi, 0, bytes, s->st));
    LB_CUDA(cudaMemsetAsync(s->qk16_lo, 0, bytes, s->st));
    tc_make_map_f16(&s->qk16_map.hi, s->qk16_hi, (unsigned long long)rows, 3 * D, TC_BM);
    tc_make_map_f16(&s->qk16_map.lo, s->qk16_lo, (unsigned long long)rows, 3 * D, TC_BM);
  } else if (s->tc_attn) {
    alloc(&s->qkv_hi, rows * 3 * D);
    alloc(&s->qkv_lo, rows * 3 * D);
    LB_CUDA(cudaMemsetAsync(s->qkv_hi, 0, rows * 3 * D * 4, s->st));
    LB_CUDA(cudaMemsetAsync(s->qkv_lo, 0, rows * 3 * D * 4, s->st));
    make_activation_map(&s->qk_map, s->qkv_hi, s->qkv_lo, rows, (int)(3 * D));
  }
  s->cap_rows = rows;
  ++s->generation;
}

// Scratch of the attention kernel's key-split mode for contexts s_lo..s_hi.
void ensure_attention_scratch(litnice_b200_session *s, int B, int s_lo, int s_hi) {
  size_t need_f = 0, need_c = 0;
  const int dh = s->dims.d_model / s->dims.n_heads;
  if (s->tc_attn) {
    // V^T: one row per (stream, column), one entry per position, whole key tiles
    const long long rows = (long long)B * s->dims.d_model;
    const int pitch = (s_hi + 127) / 128 * 128;
    if ((rows > s->vt_rows || pitch > s->vt_pitch) && s->attn16) {
      LB_CUDA(cudaStreamSynchronize(s->st));
      const long long new_rows = rows > s->vt_rows ? rows : s->vt_rows;
      const int new_pitch = pitch > s->vt_pitch ? pitch : s->vt_pitch;
      for (__half **p : {&s->vt16_hi, &s->vt16_lo}) {
        if (*p) cudaFree(*p);
        *p = nullptr;
      }
      s->vt_rows = 0;
      s->vt_pitch = 0;
      const size_t bytes = (size_t)new_rows * new_pitch * 2;
      if (cudaMalloc(reinterpret_cast<void **>(&s->vt16_hi), bytes) != cudaSuccess) throw std::bad_alloc();
      if (cudaMalloc(reinterpret_cast<void **>(&s->vt16_lo), bytes) != cudaSuccess) throw std::bad_alloc();
      // positions past a stream's length are multiplied by zero probabilities:
      // they must hold finite values from the start
      LB_CUDA(cudaMemsetAsync(s->vt16_hi, 0, bytes, s->st));
      LB_CUDA(cudaMemsetAsync(s->vt16_lo, 0, bytes, s->st));
      tc_make_map_f16(&s->vt16_map.hi, s->vt16_hi, (unsigned long long)new_rows, (unsigned long long)new_pitch, 64);
      tc_make_map_f16(&s->vt16_map.lo, s->vt16_lo, (unsigned long long)new_rows, (unsigned long long)new_pitch, 64);
      s->vt_rows = new_rows;
      s->vt_pitch = new_pitch;
      ++s->generation;
    } else if (rows > s->vt_rows || pitch > s->vt_pitch) {
      LB_CUDA(cudaStreamSynchronize(s->st));
      const long long new_rows = rows > s->vt_rows ? rows : s->vt_rows;
      const int new_pitch = pitch > s->vt_pitch ? pitch : s->vt_pitch;
      for (float **p : {&s->vt_hi, &s->vt_lo}) {
        if (*p) cudaFree(*p);
        *p = nullptr;
      }
      s->vt_rows = 0;
      s->vt_pitch = 0;
      const size_t bytes = (size_t)new_rows * new_pitch * 4;
      if (cudaMalloc(reinterpret_cast<void **>(&s->vt_hi), bytes) != cudaSuccess) throw std::bad_alloc();
      if (cudaMalloc(reinterpret_cast<void **>(&s->vt_lo), bytes) != cudaSuccess) throw std::bad_alloc();
      // positions past a stream's length are multiplied by zero probabilities:
      // they must hold finite values from the start
      LB_CUDA(cudaMemsetAsync(s->vt_hi, 0, bytes, s->st));
      LB_CUDA(cudaMemsetAsync(s->vt_lo, 0, bytes, s->st));
      tc_make_map(&s->vt_map.hi, s->vt_hi, (unsigned long long)new_rows, (unsigned long long)new_pitch, 64);
      tc_make_map(&s->vt_map.lo, s->vt_lo, (unsigned long long)new_rows, (unsigned long long)new_pitch, 64);
      s->vt_rows = new_rows;
      s->vt_pitch = new_pitch;
      ++s->generation;
    }
  }
  for (int sl = s_lo; sl <= s_hi; ++sl) {
    const AttentionPlan p = s->tc_attn ? attention_tc_plan(B, sl, s->dims.n_heads)
                                       : attention_plan(B, sl, s->dims.n_heads, dh);
    if (p.scratch_floats > need_f) need_f = p.scratch_floats;
    if (p.counters > need_c) need_c = p.counters;
  }
  if (need_f > s->attn_scratch_floats) {
    LB_CUDA(cudaStreamSynchronize(s->st));
    if (s->attn_scratch) cudaFree(s->attn_scratch);
    s->attn_scratch = nullptr;
    s->attn_scratch_floats = 0;
    if (cudaMalloc(reinterpret_cast<void **>(&s->attn_scratch), need_f * 4) != cudaSuccess) throw std::bad_alloc();
    s->attn_scratch_floats = need_f;
    ++s->generation;
  }
  if (need_c > s->attn_counter_count) {
    LB_CUDA(cudaStreamSynchronize(s->st));
    if (s->attn_counters) cudaFree(s->attn_counters);
    s->attn_counters = nullptr;
    s->attn_counter_count = 0;
    if (cudaMalloc(reinterpret_cast<void **>(&s->attn_counters), need_c * 4) != cudaSuccess) throw std::bad_alloc();
    LB_CUDA(cudaMemsetAsync(s->attn_counters, 0, need_c * 4, s->st));  // kernels leave them at zero
    s->attn_counter_count = need_c;
    ++s->generation;
  }
}


struct ClassTimer {
  litnice_b200_session *s;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> *vec;
  cudaEvent_t a = nullptr, b = nullptr;
  ClassTimer(litnice_b200_session *s_, std::vector<std::pair<cudaEvent_t, cudaEvent_t>> *v) : s(s_), vec(v) {
    if (s->profiling) {
      LB_CUDA(cudaEventCreate(&a));
      LB_CUDA(cudaEventCreate(&b));
      LB_CUDA(cudaEventRecord(a, s->st));
    }
  }
  ~ClassTimer() {
    if (s->profiling) {
      cudaEventRecord(b, s->st);
      vec->emplace_back(a, b);
    }
  }
};

// One projection: C[rows, n] = A[rows, k] * W[k, n] + bias (+ residual) (ReLU).
// gemm_ranked_matrix_rhs + add_bias_rowwise(+relu) + add of the reference
// (self_attention.cpp:62-63,96-97; ffn.cpp:56-60; transformer_layer.cpp:81,86)
// in one kernel: on the tensor cores when the weight was prepared for them,
// else the fp32 SIMT kernel. split_out: store the result as a TF32 hi/lo pair
// (c, c_lo) for a tensor-core projection that follows.
void projection(litnice_b200_session *s, AKind ak, long long rows, int k, const float *w, const TcWeight *tw,
                int n, const float *bias, const float *residual, int relu, float *c, float *c_lo,
                const TcEpilogue *extra = nullptr, float *c_plain = nullptr) {
  ClassTimer t(s, &s->gemm_ev);
  if (s->profiling) s->gemm_flops += 2.0 * (double)rows * n * k;
  ++s->launches;
  if (s->tc && tw != nullptr && tw->usable()) {
    TcEpilogue ep;
    if (extra) ep = *extra;  // transposed V store, folded LayerNorm, row statistics
    ep.bias = bias;
    ep.residual = residual;
    ep.relu = relu;
    if (c_lo) {
      ep.c_hi = c;
      ep.c_lo = c_lo;
      ep.c = c_plain;  // optionally the plain fp32 result as well
    } else {
      ep.c = c;
    }
    const TcPlan plan = tc_plan((int)rows, n, k, tw->has64, tw->has128, tw->has256);
    launch_gemm_tc(s->a_map[ak], plan.bn == 256 ? tw->m256 : plan.bn == 128 ? tw->m128 : tw->m64, (int)rows, n, k, plan, ep, s->tc_scratch,
                   s->tc_counters, s->err_dev, s->st);
    return;
  }
  const float *a = ak == A_LN ? s->ln : ak == A_CTX ? s->ctx : ak == A_H ? s->h : s->xl;
  GemmEpilogue ep;
  ep.bias = bias;
  ep.residual = residual;
  ep.relu = relu;
  launch_gemm_simt(dense(a, rows, k), dense(w, k, n), dense(c, rows, n), rows, n, k, ep, s->st);
}

// One projection on fp16-pair operands; the epilogue comes fully prepared.
void projection_f16(litnice_b200_session *s, PairKind pk, long long rows, int k, const TcWeight *tw, int n,
                    const TcEpilogue &ep) {
  ClassTimer t(s, &s->gemm_ev);
  if (s->profiling) s->gemm_flops += 2.0 * (double)rows * n * k;
  ++s->launches;
  const TcPairF16 &a = pk == PAIR_LN ? s->pair_ln : pk == PAIR_CTX ? s->pair_ctx : s->pair_h;
  const TcPlan plan = tc_plan((int)rows, n, k, tw->has64, tw->has128, tw->has256, TC_F16_SLOT);
  TcEpilogue e = ep;
  if (s->stamping && s->gemm_timeline && s->gemm_timeline_used < litnice_b200_session::kTimelineSlots) {
    e.timeline = s->gemm_timeline + 32 * s->gemm_timeline_used++;
    s->stamped_gemm_flops += 2.0 * (double)rows * n * k;
  }
  launch_gemm_tc_f16(s->pair_map[pk], a.inv_scale, plan.bn == 256 ? tw->f256 : plan.bn == 128 ? tw->f128 : tw->f64,
                     tw->h_inv_scale, (int)rows, n, k, plan, e, s->tc_scratch, s->tc_counters, s->err_dev, s->st);
}

// Transformer::forward over all rows up to the last layer's output
// (transformer.cpp:70-114, transformer_layer.cpp:50-92); leaves the final
// hidden state in s->x.
void enqueue_body(litnice_b200_session *s, int B, int sl, const LoopState *dstate = nullptr) {
  const litnice_b200_dims &d = s->dims;
  const long long R = (long long)B * sl;
  const int D = d.d_model, F = d.d_ff;
  // With the LayerNorms folded into the QKV and W1 products, the kernels that
  // produce x and y also store them as TF32 pairs in (ln, ln_lo) with per-row
  // partial sums in row_stats, and no LayerNorm kernel runs in the layers.
  const bool fold = s->ln_fold;
  launch_embed_pos(P(s, s->lay.tok_emb), P(s, s->lay.pos_emb), s->ids, d.max_seq_len, dstate, B, sl, D,
                   d.vocab_size, s->x, s->err_dev, s->st, fold && !s->f16 ? s->ln : nullptr,
                   fold && !s->f16 ? s->ln_lo : nullptr, fold ? s->row_stats : nullptr, s->f16 ? &s->pair_ln : nullptr);
  ++s->launches;
  for (int l = 0; l < d.n_layers; ++l) {
    const LayerOff &o = s->lay.layer[l];
    const std::array<TcWeight, 4> *tw = s->tc ? &s->tcw[l] : nullptr;
    TcEpilogue consume1, consume2, produce;  // extra epilogue terms of the folded form
    if (fold) {
      consume1.ln_u = (*tw)[0].ln_u;
      consume2.ln_u = (*tw)[2].ln_u;
      consume1.ln_stats = consume2.ln_stats = s->row_stats;
      consume1.ln_slots = consume2.ln_slots = D / 64;
      produce.stats_out = s->row_stats;
    } else {
      launch_layernorm_dense(s->x, P(s, o.ln1_g), P(s, o.ln1_b), R, D, s->ln, s->tc ? s->ln_lo : nullptr, dstate, B,
                             s->st);
      ++s->launches;
    }
    const float *qkv_bias = fold ? (*tw)[0].ln_v : P(s, o.qkv_b);
    if (s->f16) {
      // every projection input is an fp16 pair written by the kernel that produced it
      consume1.vt_col0 = 2 * D;
      consume1.vt_rows = D;
      consume1.vt_pitch = s->vt_pitch;
      consume1.vt_s = sl;
      consume1.vt_streams = B;
      consume1.state = dstate;
      consume1.bias = qkv_bias;
      if (s->attn16) {  // Q, K and V^T as fp16 pairs under the heads' fixed scales
        consume1.qk16_hi = s->qk16_hi;
        consume1.qk16_lo = s->qk16_lo;
        consume1.vt16_hi = s->vt16_hi;
        consume1.vt16_lo = s->vt16_lo;
        consume1.col_scale = (*tw)[0].head_scale;
      } else {  // TF32 pairs
        consume1.vt_hi = s->vt_hi;
        consume1.vt_lo = s->vt_lo;
        consume1.c_hi = s->qkv_hi;
        consume1.c_lo = s->qkv_lo;
      }
      projection_f16(s, PAIR_LN, R, D, &(*tw)[0], 3 * D, consume1);
      {
        ClassTimer t(s, &s->attn_ev);
        unsigned long long *tl = (s->stamping && s->attn_timeline &&
                                  s->attn_timeline_used < litnice_b200_session::kTimelineSlots)
                                     ? s->attn_timeline + 32 * s->attn_timeline_used++
                                     : nullptr;
        if (s->attn16)
          launch_attention_tc16(s->qk16_map, s->vt16_map, (*tw)[0].head_inv, B, sl, d.n_heads, D, s->attn_scratch,
                                s->attn_counters, dstate, s->err_dev, s->st, tl, s->pair_ctx);
        else
          launch_attention_tc(s->qk_map, s->vt_map, nullptr, nullptr, B, sl, d.n_heads, D, s->attn_scratch,
                              s->attn_counters, dstate, s->err_dev, s->st, tl, &s->pair_ctx);
        ++s->launches;
      }
      TcEpilogue e_out = produce;
      e_out.bias = P(s, o.out_b);
      e_out.residual = s->x;
      e_out.c = s->y;
      e_out.c_f16 = s->pair_ln;
      projection_f16(s, PAIR_CTX, R, D, &(*tw)[1], D, e_out);
      consume2.bias = (*tw)[2].ln_v;
      consume2.relu = 1;
      consume2.c_f16 = s->pair_h;
      projection_f16(s, PAIR_LN, R, D, &(*tw)[2], F, consume2);
      TcEpilogue e_w2 = produce;
      e_w2.bias = P(s, o.b2);
      e_w2.residual = s->y;
      e_w2.c = s->x;
      e_w2.c_f16 = s->pair_ln;
      projection_f16(s, PAIR_H, R, F, &(*tw)[3], D, e_w2);
      continue;
    }
    if (s->tc_attn) {
      // Q and K as TF32 pairs, V transposed: what the tensor-core attention reads
      consume1.vt_hi = s->vt_hi;
      consume1.vt_lo = s->vt_lo;
      consume1.vt_col0 = 2 * D;
      consume1.vt_rows = D;
      consume1.vt_pitch = s->vt_pitch;
      consume1.vt_s = sl;
      consume1.vt_streams = B;
      consume1.state = dstate;
      projection(s, A_LN, R, D, P(s, o.qkv_w), &(*tw)[0], 3 * D, qkv_bias, nullptr, 0, s->qkv_hi, s->qkv_lo,
                 &consume1);
      ClassTimer t(s, &s->attn_ev);
      launch_attention_tc(s->qk_map, s->vt_map, s->ctx, s->ctx_lo, B, sl, d.n_heads, D, s->attn_scratch,
                          s->attn_counters, dstate, s->err_dev, s->st,
                          (s->stamping && s->attn_timeline &&
                           s->attn_timeline_used < litnice_b200_session::kTimelineSlots)
                              ? s->attn_timeline + 32 * s->attn_timeline_used++
                              : nullptr);
      ++s->launches;
    } else {
      projection(s, A_LN, R, D, P(s, o.qkv_w), tw ? &(*tw)[0] : nullptr, 3 * D, qkv_bias, nullptr, 0, s->qkv,
                 nullptr, fold ? &consume1 : nullptr);
      if (s->kv_store) {  // cached mode, pass over the prompt: this layer's K and V of every position
        const size_t layer = (size_t)s->kv_streams * s->kv_cap * D;
        launch_kv_store(s->qkv, dstate, sl, B, D, s->kv_cap, s->kcache + l * layer, s->vcache + l * layer, s->st);
        ++s->launches;
      }
      ClassTimer t(s, &s->attn_ev);
      launch_attention(s->qkv, s->ctx, s->tc ? s->ctx_lo : nullptr, B, sl, d.n_heads, D, s->attn_scratch,
                       s->attn_counters, dstate, s->st);
      ++s->launches;
    }
    if (fold) {
      projection(s, A_CTX, R, D, P(s, o.out_w), &(*tw)[1], D, P(s, o.out_b), s->x, 0, s->ln, s->ln_lo, &produce, s->y);
      projection(s, A_LN, R, D, P(s, o.w1), &(*tw)[2], F, (*tw)[2].ln_v, nullptr, 1, s->h, s->h_lo, &consume2);
      projection(s, A_H, R, F, P(s, o.w2), &(*tw)[3], D, P(s, o.b2), s->y, 0, s->ln, s->ln_lo, &produce, s->x);
      continue;
    }
    projection(s, A_CTX, R, D, P(s, o.out_w), tw ? &(*tw)[1] : nullptr, D, P(s, o.out_b), s->x, 0, s->y, nullptr);
    launch_layernorm_dense(s->y, P(s, o.ln2_g), P(s, o.ln2_b), R, D, s->ln, s->tc ? s->ln_lo : nullptr, dstate, B,
                           s->st);
    ++s->launches;
    projection(s, A_LN, R, D, P(s, o.w1), tw ? &(*tw)[2] : nullptr, F, P(s, o.b1), nullptr, 1, s->h,
               s->tc ? s->h_lo : nullptr);
    projection(s, A_H, R, F, P(s, o.w2), tw ? &(*tw)[3] : nullptr, D, P(s, o.b2), s->y, 0, s->x, nullptr);
  }
}

// LN_f + output head on the last row of each stream (output_head.cpp:58-70
// restricted to the row the loop reads).
void enqueue_head_last(litnice_b200_session *s, int B, int sl, const LoopState *dstate = nullptr) {
  const litnice_b200_dims &d = s->dims;
  const bool head_tc = s->tc && B > 8 && s->tc_head.usable();
  launch_gather_last_ln(s->x, P(s, s->lay.lnf_g), P(s, s->lay.lnf_b), dstate, B, sl, d.d_model, s->xl,
                        head_tc ? s->xl_lo : nullptr, s->st);
  ++s->launches;
  if (B <= 8) {
    s->launches += launch_gemv(s->xl, B, P(s, s->lay.lm_head), d.d_model, d.vocab_size, nullptr, s->logits,
                               s->gemv_scratch, s->st, s->err_dev);
  } else {
    projection(s, A_XL, B, d.d_model, P(s, s->lay.lm_head), head_tc ? &s->tc_head : nullptr, d.vocab_size,
               nullptr, nullptr, 0, s->logits, nullptr);
  }
}

// Cached mode: one projection of the step's rows, out[B, n] = LN?(a)[B, k] W + bias (+ residual) (ReLU):
// the few-row kernels up to 8 streams (with the LayerNorm in front of the product applied inside the
// kernel where its shape allows), the fp32 tile kernel beyond. ln_g / ln_b: that LayerNorm, or null;
// ln_out: where its rows go when it has to run as a kernel of its own.
void decode_projection(litnice_b200_session *s, const float *a, int B, int k, const float *w, int n, const float *bias,
                       const float *residual, int relu, float *out, const float *ln_g = nullptr,
                       const float *ln_b = nullptr, float *ln_out = nullptr) {
  const bool fuse_ln = ln_g != nullptr && B <= 8 && s->kv_fuse && gemv_fuses_layernorm(n, k);
  if (ln_g != nullptr && !fuse_ln) {
    launch_layernorm_dense(a, ln_g, ln_b, B, k, ln_out, nullptr, nullptr, B, s->st);
    ++s->launches;
    a = ln_out;
  }
  if (B <= 8) {
    s->launches += launch_gemv(a, B, w, k, n, bias, out, s->gemv_scratch, s->st, s->err_dev, residual, relu,
                               fuse_ln ? ln_g : nullptr, fuse_ln ? ln_b : nullptr);
    return;
  }
  GemmEpilogue ep;
  ep.bias = bias;
  ep.residual = residual;
  ep.relu = relu;
  launch_gemm_simt(dense(a, B, k), dense(w, k, n), dense(out, B, n), B, n, k, ep, s->st);
  ++s->launches;
}

// Cached mode: the forward pass of the newest row of every stream at context length sl
// (transformer_layer.cpp:50-92 for one row; attention over the cached positions and the new one).
// with_head: ends with the last-row logits in s->logits; otherwise the final hidden rows stay in
// s->dx for a tail kernel that applies the final norm and the head itself.
void enqueue_decode_step(litnice_b200_session *s, int B, int sl, const LoopState *dstate, bool with_head) {
  const litnice_b200_dims &d = s->dims;
  const int D = d.d_model, F = d.d_ff, V = d.vocab_size;
  const size_t layer = (size_t)s->kv_streams * s->kv_cap * D;
  // the newest row's embedding; its first LayerNorm only when the QKV product cannot apply it itself
  const bool ln_in_qkv = B <= 8 && s->kv_fuse && gemv_fuses_layernorm(3 * D, D);
  launch_embed_last_ln(P(s, s->lay.tok_emb), P(s, s->lay.pos_emb), s->ids, d.max_seq_len, dstate, sl, B, D, V,
                       P(s, s->lay.layer[0].ln1_g), P(s, s->lay.layer[0].ln1_b), s->dx, ln_in_qkv ? nullptr : s->dln,
                       s->err_dev, s->st);
  ++s->launches;
  for (int l = 0; l < d.n_layers; ++l) {
    const LayerOff &o = s->lay.layer[l];
    if (l == 0 && !ln_in_qkv)
      decode_projection(s, s->dln, B, D, P(s, o.qkv_w), 3 * D, P(s, o.qkv_b), nullptr, 0, s->dqkv);
    else
      decode_projection(s, s->dx, B, D, P(s, o.qkv_w), 3 * D, P(s, o.qkv_b), nullptr, 0, s->dqkv, P(s, o.ln1_g),
                        P(s, o.ln1_b), s->dln);
    s->launches += launch_attn_decode(s->dqkv, s->kcache + l * layer, s->vcache + l * layer, s->kv_cap, D, d.n_heads, B,
                                      dstate, sl, s->dec_part, s->dec_counters, s->dctx, s->st);
    decode_projection(s, s->dctx, B, D, P(s, o.out_w), D, P(s, o.out_b), s->dx, 0, s->dy);
    decode_projection(s, s->dy, B, D, P(s, o.w1), F, P(s, o.b1), nullptr, 1, s->dh, P(s, o.ln2_g), P(s, o.ln2_b),
                      s->dln);
    decode_projection(s, s->dh, B, F, P(s, o.w2), D, P(s, o.b2), s->dy, 0, s->dx);
  }
  if (!with_head) return;
  decode_projection(s, s->dx, B, D, P(s, s->lay.lm_head), V, nullptr, nullptr, 0, s->logits, P(s, s->lay.lnf_g),
                    P(s, s->lay.lnf_b), s->xl);
}

// Cached mode: caches for n_streams streams of up to cap positions, and the scratch of the
// attention over key chunks for every context length up to cap.
void ensure_kv(litnice_b200_session *s, int B, int cap) {
  const litnice_b200_dims &d = s->dims;
  if (B > s->kv_streams || cap > s->kv_cap) {
    LB_CUDA(cudaStreamSynchronize(s->st));
    for (float **p : {&s->kcache, &s->vcache}) {
      if (*p) cudaFree(*p);
      *p = nullptr;
    }
    s->kv_streams = s->kv_cap = 0;
    s->kv_len = 0;
    const int nb = B > s->max_streams ? B : s->max_streams;
    const size_t bytes = (size_t)d.n_layers * nb * cap * d.d_model * 4;
    if (cudaMalloc(reinterpret_cast<void **>(&s->kcache), bytes) != cudaSuccess) throw std::bad_alloc();
    if (cudaMalloc(reinterpret_cast<void **>(&s->vcache), bytes) != cudaSuccess) throw std::bad_alloc();
    s->kv_streams = nb;
    s->kv_cap = cap;
    ++s->generation;
  }
  size_t need = 0;
  for (int sl = 64; sl <= (cap + 63) / 64 * 64; sl += 64) {
    const size_t f = attn_decode_plan(B, sl, d.n_heads, d.d_model / d.n_heads).scratch_floats;
    if (f > need) need = f;
  }
  if (s->kv_persist && B <= 8 && decode_persistent_supports(B, d.n_heads, d.d_model, d.d_ff, d.vocab_size)) {
    const size_t need_pk = decode_persistent_scratch_floats(B, d.n_heads, d.d_model, d.d_ff, d.vocab_size, s->sm_count);
    if (need_pk > s->pk_scratch_floats) {
      LB_CUDA(cudaStreamSynchronize(s->st));
      if (s->pk_scratch) cudaFree(s->pk_scratch);
      s->pk_scratch = nullptr;
      s->pk_scratch_floats = 0;
      if (cudaMalloc(reinterpret_cast<void **>(&s->pk_scratch), need_pk * 4) != cudaSuccess) throw std::bad_alloc();
      s->pk_scratch_floats = need_pk;
    }
  }
  if (s->dec_counters == nullptr) {
    const size_t n = (size_t)s->max_streams * d.n_heads;
    if (cudaMalloc(reinterpret_cast<void **>(&s->dec_counters), n * 4) != cudaSuccess) throw std::bad_alloc();
    LB_CUDA(cudaMemsetAsync(s->dec_counters, 0, n * 4, s->st));
  }
  if (need > s->dec_part_floats) {
    LB_CUDA(cudaStreamSynchronize(s->st));
    if (s->dec_part) cudaFree(s->dec_part);
    s->dec_part = nullptr;
    s->dec_part_floats = 0;
    if (cudaMalloc(reinterpret_cast<void **>(&s->dec_part), need * 4) != cudaSuccess) throw std::bad_alloc();
    s->dec_part_floats = need;
    ++s->generation;
  }
}

// Weights are immutable during inference: build, once per load, the K-major
// TF32 hi/lo copies [n, k] the tensor-core GEMM reads, and their tensor maps.
void prepare_one(litnice_b200_session *s, TcWeight *tw, const float *w, int k, int n, const float *ln_gamma = nullptr,
                 const float *ln_beta = nullptr, const float *bias = nullptr, bool as_f16 = false) {
  tw->k = k;
  tw->n = n;
  tw->has64 = (k % TC_BK == 0) && (n % 64 == 0);
  tw->has128 = (k % TC_BK == 0) && (n % 128 == 0);
  tw->has256 = (k % TC_BK == 0) && (n % 256 == 0);
  if (!tw->usable()) return;
  if (as_f16) {
    if (tw->h_hi == nullptr) {
      if (cudaMalloc(reinterpret_cast<void **>(&tw->h_hi), (size_t)k * n * 2) != cudaSuccess ||
          cudaMalloc(reinterpret_cast<void **>(&tw->h_lo), (size_t)k * n * 2) != cudaSuccess ||
          cudaMalloc(reinterpret_cast<void **>(&tw->h_inv_scale), 4) != cudaSuccess)
        throw std::bad_alloc();
    }
    launch_transpose_split_f16(w, k, n, tw->h_hi, tw->h_lo, tw->h_inv_scale, s->st, ln_gamma, s->amax_scratch);
    if (ln_gamma != nullptr) {
      if (tw->ln_u == nullptr) {
        if (cudaMalloc(reinterpret_cast<void **>(&tw->ln_u), (size_t)n * 4) != cudaSuccess) throw std::bad_alloc();
        if (cudaMalloc(reinterpret_cast<void **>(&tw->ln_v), (size_t)n * 4) != cudaSuccess) throw std::bad_alloc();
      }
      launch_ln_fold_vectors(w, k, n, ln_gamma, ln_beta, bias, tw->ln_u, tw->ln_v, s->st, s->amax_scratch);
    }
    for (auto &[map, box] : {std::pair<TcMatrix *, unsigned>{&tw->f64, 64u}, {&tw->f128, 128u}, {&tw->f256, 256u}}) {
      if ((box == 64 && !tw->has64) || (box == 128 && !tw->has128) || (box == 256 && !tw->has256)) continue;
      tc_make_map_f16(&map->hi, tw->h_hi, (unsigned long long)n, (unsigned long long)k, box);
      tc_make_map_f16(&map->lo, tw->h_lo, (unsigned long long)n, (unsigned long long)k, box);
    }
    return;
  }
  const size_t bytes = (size_t)k * n * 4;
  if (tw->hi == nullptr) {
    if (cudaMalloc(reinterpret_cast<void **>(&tw->hi), bytes) != cudaSuccess) throw std::bad_alloc();
    if (cudaMalloc(reinterpret_cast<void **>(&tw->lo), bytes) != cudaSuccess) throw std::bad_alloc();
  }
  launch_transpose_split(w, k, n, tw->hi, tw->lo, s->st, ln_gamma);
  if (ln_gamma != nullptr) {  // the LayerNorm in front of this product is folded into it
    if (tw->ln_u == nullptr) {
      if (cudaMalloc(reinterpret_cast<void **>(&tw->ln_u), (size_t)n * 4) != cudaSuccess) throw std::bad_alloc();
      if (cudaMalloc(reinterpret_cast<void **>(&tw->ln_v), (size_t)n * 4) != cudaSuccess) throw std::bad_alloc();
    }
    launch_ln_fold_vectors(w, k, n, ln_gamma, ln_beta, bias, tw->ln_u, tw->ln_v, s->st);
  }
  if (tw->has64) {
    tc_make_map(&tw->m64.hi, tw->hi, (unsigned long long)n, (unsigned long long)k, 64);
    tc_make_map(&tw->m64.lo, tw->lo, (unsigned long long)n, (unsigned long long)k, 64);
  }
  if (tw->has128) {
    tc_make_map(&tw->m128.hi, tw->hi, (unsigned long long)n, (unsigned long long)k, 128);
    tc_make_map(&tw->m128.lo, tw->lo, (unsigned long long)n, (unsigned long long)k, 128);
  }
  if (tw->has256) {
    tc_make_map(&tw->m256.hi, tw->hi, (unsigned long long)n, (unsigned long long)k, 256);
    tc_make_map(&tw->m256.lo, tw->lo, (unsigned long long)n, (unsigned long long)k, 256);
  }
}

void prepare_tc_weights(litnice_b200_session *s) {
  const litnice_b200_dims &d = s->dims;
  const int D = d.d_model, F = d.d_ff;
  s->tcw.resize(d.n_layers);
  for (int l = 0; l < d.n_layers; ++l) {
    const LayerOff &o = s->lay.layer[l];
    if (s->attn16) {
      TcWeight &q = s->tcw[l][0];
      if (q.head_scale == nullptr) {
        if (cudaMalloc(reinterpret_cast<void **>(&q.head_scale), (size_t)(3 * D / 64) * 4) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void **>(&q.head_inv), (size_t)(3 * D / 64) * 4) != cudaSuccess)
          throw std::bad_alloc();
      }
      launch_head_scales(P(s, o.qkv_w), D, 3 * D, P(s, o.ln1_g), P(s, o.ln1_b), P(s, o.qkv_b), q.head_scale, q.head_inv,
                         s->st);
    }
    if (s->ln_fold) {
      prepare_one(s, &s->tcw[l][0], P(s, o.qkv_w), D, 3 * D, P(s, o.ln1_g), P(s, o.ln1_b), P(s, o.qkv_b), s->f16);
      prepare_one(s, &s->tcw[l][2], P(s, o.w1), D, F, P(s, o.ln2_g), P(s, o.ln2_b), P(s, o.b1), s->f16);
    } else {
      prepare_one(s, &s->tcw[l][0], P(s, o.qkv_w), D, 3 * D);
      prepare_one(s, &s->tcw[l][2], P(s, o.w1), D, F);
    }
    prepare_one(s, &s->tcw[l][1], P(s, o.out_w), D, D, nullptr, nullptr, nullptr, s->f16);
    prepare_one(s, &s->tcw[l][3], P(s, o.w2), F, D, nullptr, nullptr, nullptr, s->f16);
  }
  prepare_one(s, &s->tc_head, P(s, s->lay.lm_head), D, d.vocab_size);
}

void check_device_error(litnice_b200_session *s) {
  if (s->err_host->code == DEVERR_NONE) return;
  const int code = s->err_host->code, detail = s->err_host->detail;
  s->err_host->code = DEVERR_NONE;
  if (code == DEVERR_BAD_TOKEN_ID)
    throw std::runtime_error("embedding id out of range (id=" + std::to_string(detail) + ")");
  if (code == DEVERR_WAIT_TIMEOUT)
    throw std::runtime_error("a bounded wait inside the tensor-core GEMM ran out (role " + std::to_string(detail) +
                             ")");
  throw std::runtime_error("device error code " + std::to_string(code));
}

int fail(litnice_b200_session *s, int code, const std::string &msg) {
  if (s) s->error = msg;
  return code;
}

template <class Fn>
int guarded(litnice_b200_session *s, Fn fn) {
  if (s == nullptr) return LITNICE_B200_EINVAL;
  try {
    LB_CUDA(cudaSetDevice(s->device));
    return fn();
  } catch (const std::bad_alloc &) {
    return fail(s, LITNICE_B200_ENOMEM, "device allocation failed");
  } catch (const CudaError &e) {
    return fail(s, LITNICE_B200_ECUDA, e.what());
  } catch (const std::invalid_argument &e) {
    return fail(s, LITNICE_B200_EINVAL, e.what());
  } catch (const std::exception &e) {
    return fail(s, LITNICE_B200_EDEVICE, e.what());
  }
}

void upload_ids(litnice_b200_session *s, const int32_t *ids, int B, int len) {
  // rows of `ids` are len long on the host and max_seq_len apart on the device
  LB_CUDA(cudaMemcpy2DAsync(s->ids, (size_t)s->dims.max_seq_len * 4, ids, (size_t)len * 4, (size_t)len * 4, B,
                            cudaMemcpyHostToDevice, s->st));
  s->stats.h2d_bytes += (long long)B * len * 4;
}

}  // namespace

extern "C" {

static int session_create_impl(const litnice_b200_dims *dims, int32_t max_streams, int32_t device_or_negative,
                               litnice_b200_session **out);

int litnice_b200_session_create(const litnice_b200_dims *dims, int32_t max_streams,
                                litnice_b200_session **out) {
  return session_create_impl(dims, max_streams, -1, out);
}

int litnice_b200_session_create_on(const litnice_b200_dims *dims, int32_t max_streams, int32_t device,
                                   litnice_b200_session **out) {
  if (device < 0) return LITNICE_B200_EINVAL;
  return session_create_impl(dims, max_streams, device, out);
}

static int session_create_impl(const litnice_b200_dims *dims, int32_t max_streams, int32_t device_or_negative,
                               litnice_b200_session **out) {
  if (out == nullptr) return LITNICE_B200_EINVAL;
  *out = nullptr;
  if (dims == nullptr || max_streams <= 0) return LITNICE_B200_EINVAL;
  const litnice_b200_dims &d = *dims;
  if (d.n_layers <= 0 || d.n_heads <= 0 || d.d_model <= 0 || d.d_ff <= 0 || d.vocab_size <= 0 ||
      d.max_seq_len <= 0 || d.alignment_bytes == 0 || (d.alignment_bytes & 15) != 0 ||
      d.d_model % d.n_heads != 0 || d.d_model % 4 != 0 || d.d_ff % 4 != 0)
    return LITNICE_B200_EINVAL;
  const int dh = d.d_model / d.n_heads;
  if (dh != 16 && dh != 32 && dh != 64 && dh != 128) return LITNICE_B200_EINVAL;

  auto *s = new litnice_b200_session();
  s->dims = d;
  s->max_streams = max_streams;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    delete s;
    return LITNICE_B200_ECUDA;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  if (device_or_negative >= 0) dev = device_or_negative;
  else if (const char *env = std::getenv("LITNICE_B200_DEVICE")) dev = std::atoi(env);
  if (dev < 0 || dev >= count) {
    delete s;
    return LITNICE_B200_EINVAL;
  }
  s->device = dev;
  *out = s;  // handed out even on failure below so the caller can read the error text
  return guarded(s, [&]() {
    cudaDeviceProp prop{};
    LB_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      throw std::invalid_argument("built for sm_100a (B200) only; found sm_" + std::to_string(prop.major) +
                                  std::to_string(prop.minor));
    s->lay = build_layout(d);
    LB_CUDA(cudaStreamCreateWithFlags(&s->st, cudaStreamNonBlocking));
    LB_CUDA(cudaEventCreate(&s->ev0));
    LB_CUDA(cudaEventCreate(&s->ev1));
    LB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&s->err_host), sizeof(DevErr), cudaHostAllocMapped));
    s->err_host->code = DEVERR_NONE;
    s->err_host->detail = 0;
    LB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&s->err_dev), s->err_host, 0));
    auto must = [&](cudaError_t e) { if (e != cudaSuccess) throw std::bad_alloc(); };
    must(cudaMalloc(reinterpret_cast<void **>(&s->params), s->lay.total));
    // Tensor-core projections need k % 32 == 0 and n % 64 == 0 for all four
    // layer matrices; LITNICE_B200_TC=0 forces the fp32 SIMT kernels.
    const char *pdl_env = std::getenv("LITNICE_B200_PDL");
    s->pdl = !(pdl_env && pdl_env[0] == '0');
    const char *graph_env = std::getenv("LITNICE_B200_GRAPHS");
    s->use_graphs = !(graph_env && graph_env[0] == '0');
    const char *tail_env = std::getenv("LITNICE_B200_FUSED_TAIL");
    s->fused_tail = !(tail_env && tail_env[0] == '0');
    const char *kv_env = std::getenv("LITNICE_B200_KV_CACHE");
    s->kv = kv_env && kv_env[0] == '1';
    const char *kvf_env = std::getenv("LITNICE_B200_KV_FUSE");
    s->kv_fuse = !(kvf_env && kvf_env[0] == '0');
    const char *kvp_env = std::getenv("LITNICE_B200_KV_PERSIST");
    s->kv_persist = !(kvp_env && kvp_env[0] == '0') && prop.cooperativeLaunch != 0;
    s->sm_count = prop.multiProcessorCount;
    if (s->kv) {
      std::vector<unsigned long long> offs;
      for (const LayerOff &o : s->lay.layer)
        for (size_t v : {o.ln1_g, o.ln1_b, o.qkv_w, o.qkv_b, o.out_w, o.out_b, o.ln2_g, o.ln2_b, o.w1, o.b1, o.w2, o.b2})
          offs.push_back((unsigned long long)v);
      for (size_t v : {s->lay.tok_emb, s->lay.pos_emb, s->lay.lnf_g, s->lay.lnf_b, s->lay.lm_head})
        offs.push_back((unsigned long long)v);
      must(cudaMalloc(reinterpret_cast<void **>(&s->pk_offsets), offs.size() * 8));
      LB_CUDA(cudaMemcpy(s->pk_offsets, offs.data(), offs.size() * 8, cudaMemcpyHostToDevice));
      must(cudaMalloc(reinterpret_cast<void **>(&s->pk_barrier), 16));
    }
    const char *tc_env = std::getenv("LITNICE_B200_TC");
    s->tc = !s->kv && !(tc_env && tc_env[0] == '0') && tc_runtime_available() && d.d_model % 64 == 0 &&
            d.d_ff % 64 == 0;
    // Attention on the tensor cores needs head dimension 64; LITNICE_B200_TC_ATTN=0
    // keeps the fp32 SIMT attention kernel.
    const char *ta_env = std::getenv("LITNICE_B200_TC_ATTN");
    s->tc_attn = s->tc && !(ta_env && ta_env[0] == '0') && attention_tc_supports(d.n_heads, d.d_model);
    // LayerNorm folded into the projections that follow it: needs the tensor-core
    // path and at most TC_STAT_SLOTS slots of 64 columns per row.
    const char *lf_env = std::getenv("LITNICE_B200_LN_FOLD");
    s->ln_fold = s->tc && !(lf_env && lf_env[0] == '0') && d.d_model / 64 <= TC_STAT_SLOTS;
    // fp16-pair operands in the layer projections: with the tensor-core attention and the folded
    // LayerNorm (every producer of a projection input then writes the pair itself).
    const char *f16_env = std::getenv("LITNICE_B200_F16");
    s->f16 = s->tc_attn && s->ln_fold && !(f16_env && f16_env[0] == '0');
    if (s->f16) must(cudaMalloc(reinterpret_cast<void **>(&s->amax_scratch), sizeof(int)));
    const char *a16_env = std::getenv("LITNICE_B200_ATTN16");
    s->attn16 = s->f16 && !(a16_env && a16_env[0] == '0');
    size_t lr = (size_t)(max_streams < 8 ? 8 : max_streams);
    if (s->tc) lr = (lr + TC_BM - 1) / TC_BM * TC_BM;
    s->xl_rows = (long long)lr;
    must(cudaMalloc(reinterpret_cast<void **>(&s->xl), lr * d.d_model * 4));
    if (s->tc) {
      must(cudaMalloc(reinterpret_cast<void **>(&s->xl_lo), lr * d.d_model * 4));
      LB_CUDA(cudaMemsetAsync(s->xl_lo, 0, lr * d.d_model * 4, s->st));
      make_activation_map(&s->a_map[A_XL], s->xl, s->xl_lo, (long long)lr, d.d_model);
      // A split product never uses more than 148 CTAs of at most 128 x 128 floats.
      must(cudaMalloc(reinterpret_cast<void **>(&s->tc_scratch), (size_t)148 * TC_BM * 128 * 4));
      must(cudaMalloc(reinterpret_cast<void **>(&s->tc_counters), 148 * 4));
      LB_CUDA(cudaMemsetAsync(s->tc_counters, 0, 148 * 4, s->st));
    }
    must(cudaMalloc(reinterpret_cast<void **>(&s->logits), lr * d.vocab_size * 4));
    must(cudaMalloc(reinterpret_cast<void **>(&s->probs), lr * d.vocab_size * 4));
    LB_CUDA(cudaMemsetAsync(s->xl, 0, lr * d.d_model * 4, s->st));
    LB_CUDA(cudaMemsetAsync(s->logits, 0, lr * d.vocab_size * 4, s->st));
    size_t gs = gemv_scratch_floats(8, d.vocab_size, d.d_model);
    if (s->kv) {
      // the step's rows and the few-row products of the layers
      for (size_t f : {gemv_scratch_floats(8, 3 * d.d_model, d.d_model), gemv_scratch_floats(8, d.d_model, d.d_model),
                       gemv_scratch_floats(8, d.d_ff, d.d_model), gemv_scratch_floats(8, d.d_model, d.d_ff)})
        gs = f > gs ? f : gs;
      const size_t rows = (size_t)(max_streams < 8 ? 8 : max_streams);
      for (auto &[p, cols] : {std::pair<float **, size_t>{&s->dx, (size_t)d.d_model}, {&s->dy, (size_t)d.d_model},
                              {&s->dln, (size_t)d.d_model}, {&s->dqkv, (size_t)3 * d.d_model},
                              {&s->dctx, (size_t)d.d_model}, {&s->dh, (size_t)d.d_ff}}) {
        must(cudaMalloc(reinterpret_cast<void **>(p), rows * cols * 4));
        LB_CUDA(cudaMemsetAsync(*p, 0, rows * cols * 4, s->st));
      }
    }
    if (gs) must(cudaMalloc(reinterpret_cast<void **>(&s->gemv_scratch), gs * 4));
    must(cudaMalloc(reinterpret_cast<void **>(&s->ids), (size_t)max_streams * d.max_seq_len * 4));
    LB_CUDA(cudaMemsetAsync(s->ids, 0, (size_t)max_streams * d.max_seq_len * 4, s->st));
    must(cudaMalloc(reinterpret_cast<void **>(&s->mt), (size_t)max_streams * 625 * 4));
    // the loop state, followed by the fused greedy tail's finished-CTA counter
    must(cudaMalloc(reinterpret_cast<void **>(&s->state), sizeof(LoopState) + 16));
    LB_CUDA(cudaMemsetAsync(s->state, 0, sizeof(LoopState) + 16, s->st));
    LB_CUDA(cudaStreamSynchronize(s->st));
    return LITNICE_B200_OK;
  });
}

void litnice_b200_session_destroy(litnice_b200_session *s) {
  if (s == nullptr) return;
  cudaSetDevice(s->device);
  if (s->st) cudaStreamSynchronize(s->st);
  free_activations(s);
  for (void *p : {(void *)s->params, (void *)s->xl, (void *)s->logits, (void *)s->probs, (void *)s->gemv_scratch,
                  (void *)s->logits_all, (void *)s->ids, (void *)s->out_tokens, (void *)s->mt, (void *)s->state,
                  s->sampler_scratch, (void *)s->step_logits})
    if (p) cudaFree(p);
  for (auto &g : s->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  for (float *p : {s->kcache, s->vcache, s->dx, s->dy, s->dln, s->dqkv, s->dctx, s->dh, s->dec_part})
    if (p) cudaFree(p);
  if (s->dec_counters) cudaFree(s->dec_counters);
  if (s->pk_offsets) cudaFree(s->pk_offsets);
  if (s->pk_scratch) cudaFree(s->pk_scratch);
  if (s->pk_barrier) cudaFree(s->pk_barrier);
  if (s->xl_lo) cudaFree(s->xl_lo);
  if (s->tc_scratch) cudaFree(s->tc_scratch);
  if (s->attn_timeline) cudaFree(s->attn_timeline);
  if (s->gemm_timeline) cudaFree(s->gemm_timeline);
  if (s->amax_scratch) cudaFree(s->amax_scratch);
  if (s->vt_hi) cudaFree(s->vt_hi);
  if (s->vt_lo) cudaFree(s->vt_lo);
  if (s->vt16_hi) cudaFree(s->vt16_hi);
  if (s->vt16_lo) cudaFree(s->vt16_lo);
  if (s->tc_counters) cudaFree(s->tc_counters);
  if (s->attn_scratch) cudaFree(s->attn_scratch);
  if (s->attn_counters) cudaFree(s->attn_counters);
  for (auto &layer : s->tcw)
    for (auto &w : layer) {
      if (w.hi) cudaFree(w.hi);
      if (w.lo) cudaFree(w.lo);
      if (w.ln_u) cudaFree(w.ln_u);
      if (w.ln_v) cudaFree(w.ln_v);
      if (w.h_hi) cudaFree(w.h_hi);
      if (w.h_lo) cudaFree(w.h_lo);
      if (w.h_inv_scale) cudaFree(w.h_inv_scale);
      if (w.head_scale) cudaFree(w.head_scale);
      if (w.head_inv) cudaFree(w.head_inv);
    }
  if (s->tc_head.hi) cudaFree(s->tc_head.hi);
  if (s->tc_head.lo) cudaFree(s->tc_head.lo);
  if (s->err_host) cudaFreeHost(s->err_host);
  if (s->ev0) cudaEventDestroy(s->ev0);
  if (s->ev1) cudaEventDestroy(s->ev1);
  if (s->st) cudaStreamDestroy(s->st);
  delete s;
}

const char *litnice_b200_last_error(const litnice_b200_session *s) {
  return s ? s->error.c_str() : "null session";
}

int litnice_b200_load_params(litnice_b200_session *s, const void *host_arena, uint64_t bytes) {
  return guarded(s, [&]() {
    if (host_arena == nullptr || bytes != s->lay.total)
      throw std::invalid_argument("parameter arena must be " + std::to_string(s->lay.total) + " bytes, got " +
                                  std::to_string(bytes));
    LB_CUDA(cudaMemcpyAsync(s->params, host_arena, bytes, cudaMemcpyHostToDevice, s->st));
    if (s->tc) prepare_tc_weights(s);
    LB_CUDA(cudaStreamSynchronize(s->st));
    s->params_loaded = true;
    return LITNICE_B200_OK;
  });
}

int litnice_b200_load_checkpoint(litnice_b200_session *s, const char *path) {
  if (s == nullptr || path == nullptr) return LITNICE_B200_EINVAL;
  // CkptHeaderV6 (checkpoint.cpp:98-116): 136 bytes.
#pragma pack(push, 1)
  struct Header {
    uint32_t magic, version, algo_version;
    char conf_version[32];
    uint32_t n_layers, n_heads, d_model, d_ff, vocab_size, max_seq_len, pad;
    uint64_t alignment_bytes, global_step;
    uint32_t epoch, reserved;
    uint64_t data_bytes, adam_bytes;
    float best_loss, last_epoch_loss;
    uint32_t best_epoch, epochs_without_improvement, flags, stop_reason;
  };
#pragma pack(pop)
  static_assert(sizeof(Header) == 136, "checkpoint v6 header is 136 bytes");
  std::ifstream in(path, std::ios::binary);
  if (!in) return fail(s, LITNICE_B200_EIO, std::string("cannot open checkpoint ") + path);
  Header hd{};
  in.read(reinterpret_cast<char *>(&hd), sizeof(hd));
  if (!in) return fail(s, LITNICE_B200_EIO, "truncated v6 header");
  if (hd.magic != 0x4C474354u || hd.version != 6u)
    return fail(s, LITNICE_B200_EIO, "not a version-6 litnicelm checkpoint");
  const litnice_b200_dims &d = s->dims;
  // the equality checks of checkpoint.cpp:609-628
  if (hd.n_layers != (uint32_t)d.n_layers || hd.n_heads != (uint32_t)d.n_heads ||
      hd.d_model != (uint32_t)d.d_model || hd.d_ff != (uint32_t)d.d_ff ||
      hd.vocab_size != (uint32_t)d.vocab_size || hd.max_seq_len != (uint32_t)d.max_seq_len ||
      hd.alignment_bytes != d.alignment_bytes || hd.data_bytes != s->lay.total ||
      hd.adam_bytes != 2 * s->lay.total)
    return fail(s, LITNICE_B200_EIO, "incompatible checkpoint: model dimensions or arena sizes differ");
  in.close();
  // The file must hold the whole parameter arena behind the header (a short file is refused
  // before anything is copied), then the arena streams to the device in pieces.
  {
    std::ifstream size_probe(path, std::ios::binary | std::ios::ate);
    if (!size_probe || (uint64_t)size_probe.tellg() < sizeof(Header) + (uint64_t)s->lay.total)
      return fail(s, LITNICE_B200_EIO, "could not read parameter arena payload");
  }
  return guarded(s, [&]() {
    s->params_loaded = false;
    try {
      file_to_device(path, sizeof(Header), s->lay.total, s->params, s->st, true);
    } catch (const std::domain_error &) {
      // checkpoint.cpp:176-205 rejects non-finite parameters
      return fail(s, LITNICE_B200_EIO, "parameter arena holds a non-finite value");
    } catch (const CudaError &) {
      throw;
    } catch (const std::runtime_error &e) {
      return fail(s, LITNICE_B200_EIO, std::string("could not read parameter arena payload: ") + e.what());
    }
    if (s->tc) prepare_tc_weights(s);
    LB_CUDA(cudaStreamSynchronize(s->st));
    s->params_loaded = true;
    return LITNICE_B200_OK;
  });
}

int litnice_b200_upload_prompts(litnice_b200_session *s, const int32_t *prompts, int32_t n_streams,
                                int32_t prompt_len, const uint32_t *seeds) {
  return guarded(s, [&]() {
    if (!s->params_loaded) throw std::invalid_argument("no parameters loaded");
    if (prompts == nullptr || n_streams <= 0 || n_streams > s->max_streams || prompt_len <= 0 ||
        prompt_len > s->dims.max_seq_len)
      throw std::invalid_argument("bad prompt batch shape");
    s->stats = litnice_b200_stats{};
    upload_ids(s, prompts, n_streams, prompt_len);
    unsigned *dseeds = nullptr;
    if (seeds) {
      // staged through the (not yet used) logits buffer
      dseeds = reinterpret_cast<unsigned *>(s->probs);
      LB_CUDA(cudaMemcpyAsync(dseeds, seeds, (size_t)n_streams * 4, cudaMemcpyHostToDevice, s->st));
      s->stats.h2d_bytes += (long long)n_streams * 4;
    }
    launch_mt_seed(s->mt, dseeds, n_streams, s->st);
    LoopState ls{prompt_len, 0, n_streams, s->dims.max_seq_len};
    LB_CUDA(cudaMemcpyAsync(s->state, &ls, sizeof(ls), cudaMemcpyHostToDevice, s->st));
    LB_CUDA(cudaStreamSynchronize(s->st));
    s->cur_streams = n_streams;
    s->cur_prompt_len = prompt_len;
    s->cur_tokens = 0;
    s->kv_len = 0;  // cached mode: the caches hold another batch's positions
    return LITNICE_B200_OK;
  });
}

int litnice_b200_run(litnice_b200_session *s, int32_t max_new, const litnice_b200_sampling *sampling,
                     int32_t *out_count) {
  return guarded(s, [&]() {
    PdlScope pdl_scope(s->pdl);
    if (s->cur_streams <= 0) throw std::invalid_argument("no prompts uploaded");
    if (max_new < 0 || sampling == nullptr) throw std::invalid_argument("bad run arguments");
    if (!(sampling->temp <= 0.0f || sampling->top_k == 1u) &&
        !(sampling->top_p > 0.0f && sampling->top_p <= 1.0f))
      throw std::invalid_argument("InferenceConfig.top_p must be in (0,1]");  // inference.cpp:209-211
    const int B = s->cur_streams, V = s->dims.vocab_size;
    const int s0 = s->cur_prompt_len + s->cur_tokens;
    // loop guard of inference.cpp:278
    int steps = s->dims.max_seq_len - s0;
    if (steps > max_new) steps = max_new;
    if (steps < 0) steps = 0;
    const int s_last = s0 + (steps > 0 ? steps - 1 : 0);
    const int s_last_cap = (s_last + 63) / 64 * 64;  // graph replay sizes launches per 64-token bucket
    if (s->kv) {
      // cached mode: whole-context buffers only for the pass over the prompt that fills the caches
      if (steps > 0) {
        ensure_kv(s, B, s_last_cap);
        if (s->kv_len != s0 - 1) {
          ensure_rows(s, (long long)B * s0);
          ensure_attention_scratch(s, B, s0, s0);
        }
      }
    } else {
      ensure_rows(s, (long long)B * s_last_cap);
      if (steps > 0) ensure_attention_scratch(s, B, s0, s_last_cap);
    }
    if (s->out_cap < s->cur_tokens + steps || s->out_tokens == nullptr) {
      LB_CUDA(cudaStreamSynchronize(s->st));
      int *n = nullptr;
      const int cap = s->cur_tokens + steps > 0 ? s->cur_tokens + steps : 1;
      if (cudaMalloc(reinterpret_cast<void **>(&n), (size_t)s->max_streams * cap * 4) != cudaSuccess)
        throw std::bad_alloc();
      if (s->out_tokens) {  // a resumed run keeps the tokens it already produced
        if (s->cur_tokens > 0)
          LB_CUDA(cudaMemcpy2D(n, (size_t)cap * 4, s->out_tokens, (size_t)s->out_cap * 4,
                               (size_t)s->cur_tokens * 4, s->cur_streams, cudaMemcpyDeviceToDevice));
        cudaFree(s->out_tokens);
      }
      s->out_tokens = n;
      ++s->generation;
      s->out_cap = cap;
    }
    SamplerParams sp{sampling->temp, sampling->top_k, sampling->top_p};
    const bool greedy = sp.temp <= 0.0f || sp.top_k == 1u;
    const int n_c = (sp.top_k > 0u && sp.top_k < (unsigned)V) ? (int)sp.top_k : V;
    if (!greedy && V > 2048 && n_c > 2048) {
      const size_t need = sampler_scratch_bytes(V) * (size_t)B;
      if (need > s->sampler_scratch_bytes_) {
        if (s->sampler_scratch) cudaFree(s->sampler_scratch);
        s->sampler_scratch = nullptr;
        if (cudaMalloc(&s->sampler_scratch, need) != cudaSuccess) throw std::bad_alloc();
        s->sampler_scratch_bytes_ = need;
        ++s->generation;
      }
    }
    if (s->keep_logits) {
      const long long need = (long long)(s->cur_tokens + steps) * B * V;
      if (s->cur_tokens == 0) s->step_logits_count = 0;
      if (need > s->step_logits_cap) {
        LB_CUDA(cudaStreamSynchronize(s->st));
        float *n = nullptr;
        if (cudaMalloc(reinterpret_cast<void **>(&n), (size_t)need * 4) != cudaSuccess) throw std::bad_alloc();
        if (s->step_logits) {  // a resumed run keeps the logits of the steps already taken
          const long long have = (long long)s->cur_tokens * B * V;
          if (have > 0 && s->step_logits_count == have)
            LB_CUDA(cudaMemcpy(n, s->step_logits, (size_t)have * 4, cudaMemcpyDeviceToDevice));
          cudaFree(s->step_logits);
        }
        s->step_logits = n;
        s->step_logits_cap = need;
      }
    }

    const long long launches0 = s->launches;
    // One step = whole-context forward + head + selector + state advance. With
    // graph replay the step of a 64-token context bucket is captured once (its
    // launches sized for the bucket's upper bound, the actual length read from
    // the device-side LoopState) and replayed for every step in the bucket, so
    // the host issues one launch per token instead of ~50.
    const bool graphs = s->use_graphs && !s->keep_logits;
    const bool fused_tail =
        greedy && !s->keep_logits && s->fused_tail && !s->kv && head_greedy_supports(B, s->dims.d_model, V);
    // cached mode, greedy, few streams, small vocabulary: the step ends in the one-launch tail too
    const bool decode_tail = s->kv && s->kv_fuse && greedy && !s->keep_logits && s->fused_tail &&
                             head_greedy_supports(B, s->dims.d_model, V);
    auto enqueue_step = [&](int sl_cap, const LoopState *dstate, int step, bool decode) {
      if (decode) {
        enqueue_decode_step(s, B, sl_cap, dstate, !decode_tail);
        if (decode_tail) {  // the step's rows are the last rows: one row per stream
          launch_head_greedy(s->dx, P(s, s->lay.lnf_g), P(s, s->lay.lnf_b), P(s, s->lay.lm_head), s->dims.d_model, V, B,
                             1, nullptr, s->state, reinterpret_cast<unsigned *>(s->state + 1), s->ids,
                             s->dims.max_seq_len, s->out_tokens, s->out_cap, s->logits, s->st);
          ++s->launches;
          return;
        }
      } else {
        s->kv_store = s->kv;
        try {
          enqueue_body(s, B, sl_cap, dstate);
        } catch (...) {
          s->kv_store = false;
          throw;
        }
        s->kv_store = false;
      }
      if (fused_tail) {
        launch_head_greedy(s->x, P(s, s->lay.lnf_g), P(s, s->lay.lnf_b), P(s, s->lay.lm_head), s->dims.d_model, V, B,
                           sl_cap, dstate, s->state, reinterpret_cast<unsigned *>(s->state + 1), s->ids,
                           s->dims.max_seq_len, s->out_tokens, s->out_cap, s->logits, s->st);
        ++s->launches;
        return;
      }
      if (!decode) enqueue_head_last(s, B, sl_cap, dstate);
      if (s->keep_logits) {
        LB_CUDA(cudaMemcpyAsync(s->step_logits + (long long)(s->cur_tokens + step) * B * V, s->logits,
                                (size_t)B * V * 4, cudaMemcpyDeviceToDevice, s->st));
      }
      launch_sampler(s->logits, V, B, sp, s->mt, s->ids, s->dims.max_seq_len, s->out_tokens, s->out_cap,
                     s->state, s->sampler_scratch, s->st);
      launch_advance_state(s->state, s->st);
      s->launches += 2;
    };
    LB_CUDA(cudaEventRecord(s->ev0, s->st));
    for (int step = 0; step < steps; ++step) {
      const int sl = s0 + step;
      // cached mode: a step on one new row per stream when the caches hold every earlier
      // position, else a whole-context pass that also fills them (the first step of a batch)
      const bool decode = s->kv && s->kv_len == sl - 1;
      if (decode && s->kv_persist && greedy && !s->keep_logits && B <= 8 && s->pk_scratch != nullptr &&
          decode_persistent_supports(B, s->dims.n_heads, s->dims.d_model, s->dims.d_ff, V)) {
        // every remaining step in one resident kernel
        DecodePersistentArgs a{};
        a.params = s->params;
        a.offsets = s->pk_offsets;
        a.n_layers = s->dims.n_layers;
        a.n_heads = s->dims.n_heads;
        a.d_model = s->dims.d_model;
        a.d_ff = s->dims.d_ff;
        a.vocab = V;
        a.max_seq = s->dims.max_seq_len;
        a.n_streams = B;
        a.kcache = s->kcache;
        a.vcache = s->vcache;
        a.cap = s->kv_cap;
        a.layer_stride = (unsigned long long)s->kv_streams * s->kv_cap * s->dims.d_model;
        a.ids = s->ids;
        a.ids_ld = s->dims.max_seq_len;
        a.out_tokens = s->out_tokens;
        a.out_ld = s->out_cap;
        a.state = s->state;
        a.logits = s->logits;
        a.scratch = s->pk_scratch;
        a.barrier = s->pk_barrier;
        a.s0 = sl;
        a.step0 = s->cur_tokens + step;
        a.steps = steps - step;
        a.sm_count = s->sm_count;
        a.err = s->err_dev;
        unsigned long long *tl = nullptr;
        if (std::getenv("LITNICE_B200_PK_TIMELINE") != nullptr && steps - step > 11) {
          if (cudaMalloc(reinterpret_cast<void **>(&tl), 64 * 8) != cudaSuccess) throw std::bad_alloc();
          LB_CUDA(cudaMemsetAsync(tl, 0, 64 * 8, s->st));
        }
        a.timeline = tl;
        launch_decode_persistent(a, s->st);
        if (tl != nullptr) {  // measurement aid: the phases of one token of CTA 0, ns from the token's start
          unsigned long long h[64];
          LB_CUDA(cudaMemcpyAsync(h, tl, sizeof(h), cudaMemcpyDeviceToHost, s->st));
          LB_CUDA(cudaStreamSynchronize(s->st));
          cudaFree(tl);
          std::fprintf(stderr, "resident decode kernel, token 11 of CTA 0 (ns):");
          for (int i = 1; i < 64 && h[i] != 0; ++i) std::fprintf(stderr, " %lld", (long long)(h[i] - h[0]));
          std::fprintf(stderr, "\n");
        }
        ++s->launches;
        s->kv_len = s0 + steps - 1;
        break;
      }
      if (s->kv) s->kv_len = sl;
      if (!graphs || (s->kv && !decode)) {
        enqueue_step(sl, nullptr, step, decode);
        continue;
      }
      const int bucket = (sl + 63) / 64;
      if ((int)s->graphs.size() <= bucket) s->graphs.resize(bucket + 1);
      litnice_b200_session::StepGraph &g = s->graphs[bucket];
      const bool valid = g.exec != nullptr && g.streams == B && g.generation == s->generation &&
                         g.sp.temp == sp.temp && g.sp.top_k == sp.top_k && g.sp.top_p == sp.top_p;
      if (!valid) {
        if (g.exec) {
          cudaGraphExecDestroy(g.exec);
          g.exec = nullptr;
        }
        const long long before = s->launches;
        cudaGraph_t graph = nullptr;
        LB_CUDA(cudaStreamBeginCapture(s->st, cudaStreamCaptureModeRelaxed));
        try {
          enqueue_step(bucket * 64, s->state, step, decode);
        } catch (...) {
          cudaStreamEndCapture(s->st, &graph);
          if (graph) cudaGraphDestroy(graph);
          throw;
        }
        LB_CUDA(cudaStreamEndCapture(s->st, &graph));
        const cudaError_t ie = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        LB_CUDA(ie);
        g.streams = B;
        g.sp = sp;
        g.generation = s->generation;
        g.launches = s->launches - before;
        s->launches = before;  // capturing enqueued nothing
      }
      LB_CUDA(cudaGraphLaunch(g.exec, s->st));
      s->launches += g.launches;
    }
    LB_CUDA(cudaEventRecord(s->ev1, s->st));
    LB_CUDA(cudaStreamSynchronize(s->st));
    check_device_error(s);
    float ms = 0.f;
    LB_CUDA(cudaEventElapsedTime(&ms, s->ev0, s->ev1));
    s->stats.device_ms = ms;
    s->stats.kernel_launches = s->launches - launches0;
    s->stats.tokens = (long long)steps * B;
    s->cur_tokens += steps;
    if (s->keep_logits) s->step_logits_count = (long long)s->cur_tokens * B * V;
    if (out_count) *out_count = s->cur_tokens;
    return LITNICE_B200_OK;
  });
}

int litnice_b200_download_tokens(litnice_b200_session *s, int32_t *out_tokens, int32_t max_new) {
  return guarded(s, [&]() {
    if (out_tokens == nullptr || max_new < s->cur_tokens) throw std::invalid_argument("output buffer too small");
    if (s->cur_tokens > 0) {
      LB_CUDA(cudaMemcpy2DAsync(out_tokens, (size_t)max_new * 4, s->out_tokens, (size_t)s->out_cap * 4,
                                (size_t)s->cur_tokens * 4, s->cur_streams, cudaMemcpyDeviceToHost, s->st));
      LB_CUDA(cudaStreamSynchronize(s->st));
      s->stats.d2h_bytes += (long long)s->cur_streams * s->cur_tokens * 4;
    }
    return LITNICE_B200_OK;
  });
}

int litnice_b200_generate(litnice_b200_session *s, const int32_t *prompts, int32_t n_streams,
                          int32_t prompt_len, int32_t max_new, const litnice_b200_sampling *sampling,
                          const uint32_t *seeds, int32_t *out_tokens, int32_t *out_count) {
  int rc = litnice_b200_upload_prompts(s, prompts, n_streams, prompt_len, seeds);
  if (rc != LITNICE_B200_OK) return rc;
  rc = litnice_b200_run(s, max_new, sampling, out_count);
  if (rc != LITNICE_B200_OK) return rc;
  return litnice_b200_download_tokens(s, out_tokens, max_new);
}

int litnice_b200_keep_step_logits(litnice_b200_session *s, int32_t enable) {
  if (s == nullptr) return LITNICE_B200_EINVAL;
  s->keep_logits = enable != 0;
  return LITNICE_B200_OK;
}

int litnice_b200_read_step_logits(litnice_b200_session *s, float *out, int64_t max_floats) {
  return guarded(s, [&]() {
    if (out == nullptr || max_floats < s->step_logits_count) throw std::invalid_argument("output buffer too small");
    if (s->step_logits_count > 0) {
      LB_CUDA(cudaMemcpyAsync(out, s->step_logits, (size_t)s->step_logits_count * 4, cudaMemcpyDeviceToHost, s->st));
      LB_CUDA(cudaStreamSynchronize(s->st));
    }
    return LITNICE_B200_OK;
  });
}

int litnice_b200_forward(litnice_b200_session *s, const int32_t *ids, int32_t n_streams, int32_t seq_len,
                         int32_t all_rows, float *out_logits) {
  return guarded(s, [&]() {
    if (!s->params_loaded) throw std::invalid_argument("no parameters loaded");
    if (ids == nullptr || out_logits == nullptr || n_streams <= 0 || n_streams > s->max_streams || seq_len <= 0 ||
        seq_len > s->dims.max_seq_len)
      throw std::invalid_argument("bad forward shape");
    PdlScope pdl_scope(s->pdl);
    const int B = n_streams, V = s->dims.vocab_size, D = s->dims.d_model;
    const long long R = (long long)B * seq_len;
    s->stats = litnice_b200_stats{};
    s->cur_streams = 0;  // the ids of an uploaded prompt batch are overwritten: run needs a fresh upload
    ensure_rows(s, R);
    ensure_attention_scratch(s, B, seq_len, seq_len);
    upload_ids(s, ids, B, seq_len);
    const long long launches0 = s->launches;
    LB_CUDA(cudaEventRecord(s->ev0, s->st));
    enqueue_body(s, B, seq_len);
    if (all_rows) {
      if (s->logits_all_rows < R) {
        LB_CUDA(cudaStreamSynchronize(s->st));
        if (s->logits_all) cudaFree(s->logits_all);
        s->logits_all = nullptr;
        s->logits_all_rows = 0;
        if (cudaMalloc(reinterpret_cast<void **>(&s->logits_all), (size_t)R * V * 4) != cudaSuccess)
          throw std::bad_alloc();
        s->logits_all_rows = R;
      }
      // OutputHead::forward over every row (output_head.cpp:58-70)
      const bool head_tc = s->tc && s->tc_head.usable();
      launch_layernorm_dense(s->x, P(s, s->lay.lnf_g), P(s, s->lay.lnf_b), R, D, s->ln,
                             head_tc ? s->ln_lo : nullptr, nullptr, B, s->st);
      ++s->launches;
      projection(s, A_LN, R, D, P(s, s->lay.lm_head), head_tc ? &s->tc_head : nullptr, V, nullptr, nullptr, 0,
                 s->logits_all, nullptr);
      LB_CUDA(cudaEventRecord(s->ev1, s->st));
      LB_CUDA(cudaMemcpyAsync(out_logits, s->logits_all, (size_t)R * V * 4, cudaMemcpyDeviceToHost, s->st));
      s->stats.d2h_bytes += R * V * 4;
    } else {
      enqueue_head_last(s, B, seq_len);
      LB_CUDA(cudaEventRecord(s->ev1, s->st));
      LB_CUDA(cudaMemcpyAsync(out_logits, s->logits, (size_t)B * V * 4, cudaMemcpyDeviceToHost, s->st));
      s->stats.d2h_bytes += (long long)B * V * 4;
    }
    LB_CUDA(cudaStreamSynchronize(s->st));
    check_device_error(s);
    float ms = 0.f;
    LB_CUDA(cudaEventElapsedTime(&ms, s->ev0, s->ev1));
    s->stats.device_ms = ms;
    s->stats.kernel_launches = s->launches - launches0;
    return LITNICE_B200_OK;
  });
}

int litnice_b200_inspect(litnice_b200_session *s, const int32_t *ids, int32_t n_streams, int32_t seq_len,
                         float *probs) {
  return guarded(s, [&]() {
    if (!s->params_loaded) throw std::invalid_argument("no parameters loaded");
    if (ids == nullptr || probs == nullptr || n_streams <= 0 || n_streams > s->max_streams || seq_len <= 0 ||
        seq_len > s->dims.max_seq_len)
      throw std::invalid_argument("bad inspect shape");
    PdlScope pdl_scope(s->pdl);
    const int B = n_streams, V = s->dims.vocab_size;
    s->stats = litnice_b200_stats{};
    s->cur_streams = 0;  // as in forward: the uploaded prompt batch is gone
    ensure_rows(s, (long long)B * seq_len);
    ensure_attention_scratch(s, B, seq_len, seq_len);
    upload_ids(s, ids, B, seq_len);
    const long long launches0 = s->launches;
    LB_CUDA(cudaEventRecord(s->ev0, s->st));
    enqueue_body(s, B, seq_len);
    enqueue_head_last(s, B, seq_len);
    launch_softmax_probs_f64(s->logits, V, B, s->probs, s->st);
    ++s->launches;
    LB_CUDA(cudaEventRecord(s->ev1, s->st));
    LB_CUDA(cudaMemcpyAsync(probs, s->probs, (size_t)B * V * 4, cudaMemcpyDeviceToHost, s->st));
    LB_CUDA(cudaStreamSynchronize(s->st));
    check_device_error(s);
    float ms = 0.f;
    LB_CUDA(cudaEventElapsedTime(&ms, s->ev0, s->ev1));
    s->stats.device_ms = ms;
    s->stats.kernel_launches = s->launches - launches0;
    s->stats.d2h_bytes += (long long)B * V * 4;
    s->stats.tokens = 0;
    return LITNICE_B200_OK;
  });
}

int litnice_b200_sample_logits(litnice_b200_session *s, const float *logits, int32_t n_rows,
                               const litnice_b200_sampling *sampling, const uint32_t *seeds, int32_t draws,
                               int32_t *out) {
  return guarded(s, [&]() {
    if (logits == nullptr || sampling == nullptr || out == nullptr || n_rows <= 0 || draws <= 0)
      throw std::invalid_argument("bad sample_logits arguments");
    const int V = s->dims.vocab_size;
    float *dl = nullptr;
    unsigned *dmt = nullptr, *dseeds = nullptr;
    int *dout = nullptr;
    void *scr = nullptr;
    auto cleanup = [&]() {
      for (void *p : {(void *)dl, (void *)dmt, (void *)dseeds, (void *)dout, scr})
        if (p) cudaFree(p);
    };
    try {
      auto must = [&](cudaError_t e) { if (e != cudaSuccess) throw std::bad_alloc(); };
      must(cudaMalloc(reinterpret_cast<void **>(&dl), (size_t)n_rows * V * 4));
      must(cudaMalloc(reinterpret_cast<void **>(&dmt), (size_t)n_rows * 625 * 4));
      must(cudaMalloc(reinterpret_cast<void **>(&dout), (size_t)n_rows * draws * 4));
      if (seeds) {
        must(cudaMalloc(reinterpret_cast<void **>(&dseeds), (size_t)n_rows * 4));
        LB_CUDA(cudaMemcpyAsync(dseeds, seeds, (size_t)n_rows * 4, cudaMemcpyHostToDevice, s->st));
      }
      const size_t sb = sampler_scratch_bytes(V) * (size_t)n_rows;
      if (sb) must(cudaMalloc(&scr, sb));
      LB_CUDA(cudaMemcpyAsync(dl, logits, (size_t)n_rows * V * 4, cudaMemcpyHostToDevice, s->st));
      launch_mt_seed(dmt, dseeds, n_rows, s->st);
      SamplerParams sp{sampling->temp, sampling->top_k, sampling->top_p};
      launch_sampler_rows(dl, V, n_rows, sp, dmt, draws, dout, scr, s->st);
      LB_CUDA(cudaMemcpyAsync(out, dout, (size_t)n_rows * draws * 4, cudaMemcpyDeviceToHost, s->st));
      LB_CUDA(cudaStreamSynchronize(s->st));
    } catch (...) {
      cudaStreamSynchronize(s->st);
      cleanup();
      throw;
    }
    cleanup();
    return LITNICE_B200_OK;
  });
}

int litnice_b200_get_stats(const litnice_b200_session *s, litnice_b200_stats *out) {
  if (s == nullptr || out == nullptr) return LITNICE_B200_EINVAL;
  *out = s->stats;
  return LITNICE_B200_OK;
}

int litnice_b200_profile_step(litnice_b200_session *s, int32_t n_streams, int32_t seq_len, int32_t repeats) {
  return guarded(s, [&]() {
    if (!s->params_loaded) throw std::invalid_argument("no parameters loaded");
    if (n_streams <= 0 || n_streams > s->max_streams || seq_len <= 0 || seq_len > s->dims.max_seq_len ||
        repeats <= 0)
      throw std::invalid_argument("bad profile_step shape");
    PdlScope pdl_scope(s->pdl);
    ensure_rows(s, (long long)n_streams * seq_len);
    ensure_attention_scratch(s, n_streams, seq_len, seq_len);
    s->gemm_ev.clear();
    s->attn_ev.clear();
    s->gemm_flops = 0;
    const bool print_timelines = std::getenv("LITNICE_B200_TC_TIMELINE") != nullptr ||
                                 std::getenv("LITNICE_B200_ATTN_TIMELINE") != nullptr;
    if (s->tc_attn && s->attn_timeline == nullptr)
      if (cudaMalloc(reinterpret_cast<void **>(&s->attn_timeline), litnice_b200_session::kTimelineSlots * 256) !=
          cudaSuccess)
        throw std::bad_alloc();
    if (s->f16 && s->gemm_timeline == nullptr)
      if (cudaMalloc(reinterpret_cast<void **>(&s->gemm_timeline), litnice_b200_session::kTimelineSlots * 256) !=
          cudaSuccess)
        throw std::bad_alloc();
    if (s->gemm_timeline) {
      LB_CUDA(cudaMemsetAsync(s->gemm_timeline, 0, litnice_b200_session::kTimelineSlots * 256, s->st));
      for (int i = 0; i < litnice_b200_session::kTimelineSlots; ++i)
        LB_CUDA(cudaMemsetAsync(s->gemm_timeline + 32 * i + 8, 0xff, 8, s->st));
      for (int i = 0; i < litnice_b200_session::kTimelineSlots; ++i)
        LB_CUDA(cudaMemsetAsync(s->gemm_timeline + 32 * i + 14, 0xff, 8, s->st));  // earliest return of the wait
      s->gemm_timeline_used = 0;
    }
    if (s->attn_timeline) {
      LB_CUDA(cudaMemsetAsync(s->attn_timeline, 0, litnice_b200_session::kTimelineSlots * 256, s->st));
      for (int i = 0; i < litnice_b200_session::kTimelineSlots; ++i)
        LB_CUDA(cudaMemsetAsync(s->attn_timeline + 32 * i + 8, 0xff, 8, s->st));  // earliest start: preset to max
      for (int i = 0; i < litnice_b200_session::kTimelineSlots; ++i)
        LB_CUDA(cudaMemsetAsync(s->attn_timeline + 32 * i + 16, 0xff, 8, s->st));
      s->attn_timeline_used = 0;
    }
    enqueue_body(s, n_streams, seq_len);  // warm-up, untimed
    // One step with device-clock stamps only: the launches overlap through programmatic
    // dependent launch as they do in the token loop (event records between them would
    // serialise them), and every CTA contributes to its launch's earliest start and latest end.
    s->stamped_gemm_flops = 0;
    s->stamping = true;
    try {
      enqueue_body(s, n_streams, seq_len);
    } catch (...) {
      s->stamping = false;
      throw;
    }
    s->stamping = false;
    s->profiling = true;
    try {
      for (int r = 0; r < repeats; ++r) {
        enqueue_body(s, n_streams, seq_len);
        enqueue_head_last(s, n_streams, seq_len);
      }
    } catch (...) {
      s->profiling = false;
      throw;
    }
    s->profiling = false;
    LB_CUDA(cudaStreamSynchronize(s->st));
    if (s->err_host->code == DEVERR_BAD_TOKEN_ID) s->err_host->code = DEVERR_NONE;  // stale ids: timing only
    check_device_error(s);
    auto total = [&](std::vector<std::pair<cudaEvent_t, cudaEvent_t>> &v) {
      double ms = 0;
      for (auto &p : v) {
        float t = 0.f;
        cudaEventElapsedTime(&t, p.first, p.second);
        ms += t;
        cudaEventDestroy(p.first);
        cudaEventDestroy(p.second);
      }
      return ms;
    };
    s->stats.gemm_launches = (long long)s->gemm_ev.size();
    s->stats.attn_launches = (long long)s->attn_ev.size();
    s->stats.gemm_ms = total(s->gemm_ev);
    s->stats.attn_ms = total(s->attn_ev);
    s->stats.gemm_flops = s->gemm_flops;
    s->gemm_ev.clear();
    s->attn_ev.clear();
    s->stats.gemm_span_ms = s->stats.attn_span_ms = s->stats.step_span_ms = 0;
    s->stats.gemm_span_launches = s->stats.attn_span_launches = 0;
    s->stats.gemm_span_flops = s->stamped_gemm_flops;
    unsigned long long first_start = ~0ull, last_end = 0;
    if (s->gemm_timeline) {
      std::vector<unsigned long long> t(32 * (size_t)s->gemm_timeline_used);
      if (!t.empty()) LB_CUDA(cudaMemcpy(t.data(), s->gemm_timeline, t.size() * 8, cudaMemcpyDeviceToHost));
      for (int i = 0; i < s->gemm_timeline_used; ++i) {
        const unsigned long long *u = t.data() + 32 * i;
        // a launch's work runs from the moment its predecessor has completed (the earliest return
        // of its wait; its CTAs are resident and set up before that) to its last CTA's end
        const unsigned long long begin = u[14] != ~0ull && u[14] > u[8] ? u[14] : u[8];
        if (u[9] > begin) {
          s->stats.gemm_span_ms += 1e-6 * (double)(u[9] - begin);
          ++s->stats.gemm_span_launches;
          first_start = begin < first_start ? begin : first_start;
          last_end = u[9] > last_end ? u[9] : last_end;
        }
      }
      for (int i = 0; print_timelines && i < s->gemm_timeline_used; ++i) {
        const unsigned long long *u = t.data() + 32 * i;
        std::fprintf(stderr,
                     "projection launch %d (ns from CTA start): setup %lld, loads issued %lld, first stage %lld, mma "
                     "issued %lld, drained %lld, staged %lld, peers staged %lld, rows stored %lld, statistics %lld, "
                     "stored %lld, end %lld; whole grid %lld\n",
                     i, (long long)(u[1] - u[0]), (long long)(u[2] - u[0]), (long long)(u[3] - u[0]),
                     (long long)(u[4] - u[0]), (long long)(u[5] - u[0]), (long long)(u[10] - u[0]),
                     (long long)(u[11] - u[0]), (long long)(u[12] - u[0]), (long long)(u[13] - u[0]),
                     (long long)(u[6] - u[0]), (long long)(u[7] - u[0]), (long long)(u[9] - u[8]));
      }
    }
    if (s->attn_timeline) {
      // per profiled launch: stamps of CTA (0,0,0) and the span from the first CTA's start to the last CTA's end
      std::vector<unsigned long long> t(32 * (size_t)s->attn_timeline_used);
      if (!t.empty()) LB_CUDA(cudaMemcpy(t.data(), s->attn_timeline, t.size() * 8, cudaMemcpyDeviceToHost));
      for (int i = 0; i < s->attn_timeline_used; ++i) {
        const unsigned long long *u = t.data() + 32 * i;
        const unsigned long long begin = u[16] != ~0ull && u[16] > u[8] ? u[16] : u[8];
        if (u[9] > begin) {
          s->stats.attn_span_ms += 1e-6 * (double)(u[9] - begin);
          ++s->stats.attn_span_launches;
          first_start = begin < first_start ? begin : first_start;
          last_end = u[9] > last_end ? u[9] : last_end;
        }
      }
      if (last_end > first_start) s->stats.step_span_ms = 1e-6 * (double)(last_end - first_start);
      for (int i = 0; print_timelines && i < s->attn_timeline_used; ++i) {
        const unsigned long long *u = t.data() + 32 * i;
        std::fprintf(stderr,
                     "attention launch %d (ns from CTA start): setup %lld, Q+K landed %lld, S ready %lld, P stored %lld, "
                     "O ready %lld, partial merged %lld, end %lld; CTA start after first %lld; last CTA start %lld; whole grid %lld; last to end: blockIdx.x %d merge %d; split path: partial stored %lld, fenced %lld, counted %lld, merge loaded %lld\n",
                     i, (long long)(u[1] - u[0]), (long long)(u[2] - u[0]), (long long)(u[3] - u[0]),
                     (long long)(u[4] - u[0]), (long long)(u[5] - u[0]), (long long)(u[6] - u[0]),
                     (long long)(u[7] - u[0]), (long long)(u[0] - u[8]), (long long)(u[10] - u[8]),
                     (long long)(u[9] - u[8]), (int)((u[11] >> 1) & 0x3ff), (int)(u[11] & 1), (long long)(u[12] - u[0]),
                     (long long)(u[13] - u[0]), (long long)(u[14] - u[0]), (long long)(u[15] - u[0]));
      }
    }
    return LITNICE_B200_OK;
  });
}

static int projection_impl(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                           const float *bias, const float *residual, int32_t relu, float *c, int32_t repeats,
                           double *avg_us);

int litnice_b200_projection_host(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                                 const float *bias, const float *residual, int32_t relu, float *c) {
  return projection_impl(engine, a, m, k, w, n, bias, residual, relu, c, 1, nullptr);
}

int litnice_b200_projection_time(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                                 float *c, int32_t repeats, double *avg_us) {
  if (repeats <= 0 || avg_us == nullptr) return LITNICE_B200_EINVAL;
  return projection_impl(engine, a, m, k, w, n, nullptr, nullptr, 0, c, repeats, avg_us);
}

static int projection_impl(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                           const float *bias, const float *residual, int32_t relu, float *c, int32_t repeats,
                           double *avg_us) {
  if (a == nullptr || w == nullptr || c == nullptr || m <= 0 || k <= 0 || n <= 0 || (engine < 0 || engine > 2)) {
    std::fprintf(stderr, "litnice_b200_projection_host: bad argument\n");
    return LITNICE_B200_EINVAL;
  }
  if (engine >= 1 && (k % (engine == 2 ? TC_F16_SLOT : TC_BK) != 0 || n % 64 != 0 || !tc_runtime_available())) {
    std::fprintf(stderr, "litnice_b200_projection_host: the tensor-core engines need k %% 32 == 0 (fp16 pairs: k %% 64 "
                         "== 0) and n %% 64 == 0\n");
    return LITNICE_B200_EINVAL;
  }
  std::vector<void *> owned;
  DevErr *err_host = nullptr;
  cudaStream_t st = nullptr;
  int rc = LITNICE_B200_OK;
  try {
    auto dev_alloc = [&](size_t bytes) {
      void *p = nullptr;
      if (cudaMalloc(&p, bytes) != cudaSuccess) throw std::bad_alloc();
      owned.push_back(p);
      return static_cast<float *>(p);
    };
    LB_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    LB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&err_host), sizeof(DevErr), cudaHostAllocMapped));
    err_host->code = DEVERR_NONE;
    err_host->detail = 0;
    DevErr *err_dev = nullptr;
    LB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&err_dev), err_host, 0));
    const long long mp = ((long long)m + TC_BM - 1) / TC_BM * TC_BM;
    float *da = dev_alloc((size_t)mp * k * 4), *dw = dev_alloc((size_t)k * n * 4), *dc = dev_alloc((size_t)m * n * 4);
    float *db = bias ? dev_alloc((size_t)n * 4) : nullptr, *dr = residual ? dev_alloc((size_t)m * n * 4) : nullptr;
    LB_CUDA(cudaMemsetAsync(da, 0, (size_t)mp * k * 4, st));
    LB_CUDA(cudaMemcpyAsync(da, a, (size_t)m * k * 4, cudaMemcpyHostToDevice, st));
    LB_CUDA(cudaMemcpyAsync(dw, w, (size_t)k * n * 4, cudaMemcpyHostToDevice, st));
    if (db) LB_CUDA(cudaMemcpyAsync(db, bias, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    if (dr) LB_CUDA(cudaMemcpyAsync(dr, residual, (size_t)m * n * 4, cudaMemcpyHostToDevice, st));
    if (engine == 0) {
      GemmEpilogue ep;
      ep.bias = db;
      ep.residual = dr;
      ep.relu = relu;
      cudaEvent_t e0, e1;
      LB_CUDA(cudaEventCreate(&e0));
      LB_CUDA(cudaEventCreate(&e1));
      launch_gemm_simt(dense(da, m, k), dense(dw, k, n), dense(dc, m, n), m, n, k, ep, st);
      LB_CUDA(cudaEventRecord(e0, st));
      for (int r = 1; r < repeats; ++r)
        launch_gemm_simt(dense(da, m, k), dense(dw, k, n), dense(dc, m, n), m, n, k, ep, st);
      LB_CUDA(cudaEventRecord(e1, st));
      LB_CUDA(cudaStreamSynchronize(st));
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      if (avg_us && repeats > 1) *avg_us = 1e3 * ms / (repeats - 1);
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
    } else {
      // engine 2: the same kernel on fp16 pairs with block scales (k % 64 == 0)
      const bool f16 = engine == 2;
      float *a_hi = dev_alloc((size_t)mp * k * 4), *a_lo = dev_alloc((size_t)mp * k * 4);
      float *w_hi = dev_alloc((size_t)k * n * 4), *w_lo = dev_alloc((size_t)k * n * 4);
      TcPairF16 pa;
      float *w_inv = nullptr;
      if (f16) {
        pa.hi = reinterpret_cast<__half *>(a_hi);
        pa.lo = reinterpret_cast<__half *>(a_lo);
        pa.inv_scale = dev_alloc((size_t)mp * (k / TC_F16_SLOT) * 4);
        LB_CUDA(cudaMemsetAsync(a_hi, 0, (size_t)mp * k * 4, st));
        LB_CUDA(cudaMemsetAsync(a_lo, 0, (size_t)mp * k * 4, st));
        LB_CUDA(cudaMemsetAsync(pa.inv_scale, 0, (size_t)mp * (k / TC_F16_SLOT) * 4, st));
        launch_split_f16(da, m, k, pa, st);
        w_inv = dev_alloc(8);
        launch_transpose_split_f16(dw, k, n, reinterpret_cast<__half *>(w_hi), reinterpret_cast<__half *>(w_lo), w_inv,
                                   st, nullptr, reinterpret_cast<int *>(w_inv + 1));
      } else {
        launch_split_tf32(da, a_hi, a_lo, mp * k, st);
        launch_transpose_split(dw, k, n, w_hi, w_lo, st);
      }
      const TcPlan plan = tc_plan(m, n, k, n % 64 == 0, n % 128 == 0, n % 256 == 0, f16 ? TC_F16_SLOT : TC_BK);
      const int bn = plan.bn;
      float *scr = plan.scratch_floats ? dev_alloc(plan.scratch_floats * 4) : nullptr;
      int *cnt = nullptr;
      if (plan.counters) {
        cnt = reinterpret_cast<int *>(dev_alloc(plan.counters * 4));
        LB_CUDA(cudaMemsetAsync(cnt, 0, plan.counters * 4, st));
      }
      TcMatrix ma{}, mb{};
      if (f16) {
        tc_make_map_f16(&ma.hi, pa.hi, (unsigned long long)mp, (unsigned long long)k, TC_BM);
        tc_make_map_f16(&ma.lo, pa.lo, (unsigned long long)mp, (unsigned long long)k, TC_BM);
        tc_make_map_f16(&mb.hi, reinterpret_cast<__half *>(w_hi), (unsigned long long)n, (unsigned long long)k, (unsigned)bn);
        tc_make_map_f16(&mb.lo, reinterpret_cast<__half *>(w_lo), (unsigned long long)n, (unsigned long long)k, (unsigned)bn);
      } else {
        tc_make_map(&ma.hi, a_hi, (unsigned long long)mp, (unsigned long long)k, TC_BM);
        tc_make_map(&ma.lo, a_lo, (unsigned long long)mp, (unsigned long long)k, TC_BM);
        tc_make_map(&mb.hi, w_hi, (unsigned long long)n, (unsigned long long)k, (unsigned)bn);
        tc_make_map(&mb.lo, w_lo, (unsigned long long)n, (unsigned long long)k, (unsigned)bn);
      }

      TcEpilogue ep;
      ep.bias = db;
      ep.residual = dr;
      ep.relu = relu;
      ep.c = dc;
      const bool want_timeline = std::getenv("LITNICE_B200_TC_TIMELINE") != nullptr;
      if (want_timeline) {
        ep.timeline = reinterpret_cast<unsigned long long *>(dev_alloc(16 * 8));
      }
      auto launch = [&]() {
        if (f16) launch_gemm_tc_f16(ma, pa.inv_scale, mb, w_inv, m, n, k, plan, ep, scr, cnt, err_dev, st);
        else launch_gemm_tc(ma, mb, m, n, k, plan, ep, scr, cnt, err_dev, st);
      };
      cudaEvent_t e0, e1;
      LB_CUDA(cudaEventCreate(&e0));
      LB_CUDA(cudaEventCreate(&e1));
      launch();
      LB_CUDA(cudaEventRecord(e0, st));
      for (int r = 1; r < repeats; ++r) {
        if (want_timeline) {  // stamps of the last launch only
          LB_CUDA(cudaMemsetAsync(ep.timeline, 0, 96, st));
          LB_CUDA(cudaMemsetAsync(ep.timeline + 8, 0xff, 8, st));
        }
        launch();
      }
      LB_CUDA(cudaEventRecord(e1, st));
      LB_CUDA(cudaStreamSynchronize(st));
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      if (avg_us && repeats > 1) *avg_us = 1e3 * ms / (repeats - 1);
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      if (want_timeline) {
        unsigned long long t[16];
        LB_CUDA(cudaMemcpy(t, ep.timeline, 128, cudaMemcpyDeviceToHost));

        std::fprintf(stderr,
                     "tc timeline (ns from start): setup %lld, loads issued %lld, first stage full %lld, mma issued %lld, "
                     "chunks drained %lld, stored %lld, end %lld; last CTA start %lld, whole grid %lld\n",
                     (long long)(t[1] - t[0]), (long long)(t[2] - t[0]), (long long)(t[3] - t[0]),
                     (long long)(t[4] - t[0]), (long long)(t[5] - t[0]), (long long)(t[6] - t[0]),
                     (long long)(t[7] - t[0]), (long long)(t[10] - t[8]), (long long)(t[9] - t[8]));
      }
    }
    LB_CUDA(cudaMemcpyAsync(c, dc, (size_t)m * n * 4, cudaMemcpyDeviceToHost, st));
    LB_CUDA(cudaStreamSynchronize(st));
    if (err_host->code != DEVERR_NONE) {
      std::fprintf(stderr, "litnice_b200_projection_host: device error %d (detail %d)\n", err_host->code,
                   err_host->detail);
      rc = LITNICE_B200_EDEVICE;
    }
  } catch (const std::bad_alloc &) {
    rc = LITNICE_B200_ENOMEM;
  } catch (const std::exception &e) {
    std::fprintf(stderr, "litnice_b200_projection_host: %s\n", e.what());
    rc = LITNICE_B200_ECUDA;
  }
  if (st) {
    cudaStreamSynchronize(st);
    cudaStreamDestroy(st);
  }
  for (void *p : owned) cudaFree(p);
  if (err_host) cudaFreeHost(err_host);
  return rc;
}

}  // extern "C"
