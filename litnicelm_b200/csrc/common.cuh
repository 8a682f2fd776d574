// Shared declarations of the B200 plugin: error handling, strided views as
// the kernels see them, and the launch functions of every kernel family.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/litnice_backend_b200.h"

namespace lb {

// ---- errors ---------------------------------------------------------------

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char *what, const char *file, int line) {
  if (e != cudaSuccess) {
    throw CudaError(std::string("litnice_b200: ") + what + " failed: " + cudaGetErrorString(e) +
                    " (" + file + ":" + std::to_string(line) + ")");
  }
}
#define LB_CUDA(expr) ::lb::cuda_check((expr), #expr, __FILE__, __LINE__)
#define LB_LAUNCH_CHECK() ::lb::cuda_check(cudaGetLastError(), "kernel launch", __FILE__, __LINE__)

// Error word written by kernels into host-mapped memory; the host reads it
// after the next stream synchronisation. Kernels never trap.
enum DevErrCode : int {
  DEVERR_NONE = 0,
  DEVERR_BAD_TOKEN_ID = 1,   // embedding id outside [0, vocab)
  DEVERR_WAIT_TIMEOUT = 2,   // a bounded mbarrier / TMEM wait ran out
  DEVERR_BAD_ARGUMENT = 3,
  DEVERR_BAD_TARGET = 4,     // cross-entropy target outside [0, vocab)
};
struct DevErr {
  int code;
  int detail;
};

// ---- programmatic dependent launch ----------------------------------------------
// Kernels of the native token loop are launched so that a kernel may start
// (set up barriers, allocate tensor memory, prefetch weights) while its
// predecessor on the stream is still draining. pdl_wait() blocks until every
// earlier kernel has completed and its writes are visible; nothing produced or
// consumed by earlier kernels may be touched before it. Launched the ordinary
// way, both calls are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() {
#if defined(__CUDA_ARCH__)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_wait() {
#if defined(__CUDA_ARCH__)
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}

// Whether native-loop launchers on this host thread use the early-launch attribute.
extern thread_local bool g_pdl_enabled;
struct PdlScope {
  bool prev;
  explicit PdlScope(bool on) : prev(g_pdl_enabled) { g_pdl_enabled = on; }
  ~PdlScope() { g_pdl_enabled = prev; }
};

// cluster_z > 1: the CTAs that differ only in blockIdx.z form a thread-block cluster.
template <typename... KArgs, typename... Args>
inline void launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                               unsigned cluster_z, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cuda_check(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), "cudaLaunchKernelEx", __FILE__, __LINE__);
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                       Args... args) {
  launch_pdl_cluster(kernel, grid, block, smem, st, pdl, 1u, args...);
}

// ---- views ----------------------------------------------------------------

// Rows of a tensor: every axis but the last forms the row index ("prefix" in
// the reference, device_backend.cpp:62-125). Axes of extent 1 are dropped and
// axes that are dense with their neighbour are merged on the host, so np is 0
// or 1 for every view the inference path hands over.
struct RowView {
  char *data;
  int np;               // number of prefix axes kept
  long long pd[5];      // prefix extents, outermost first
  long long ps[5];      // prefix strides in bytes
  long long rows;       // product of pd
  long long cols;
  long long cs;         // stride of the last axis in bytes
};

// A batch of matrices: the last two axes are (rows, cols), the rest is batch.
struct MatView {
  char *data;
  int nb;
  long long bd[4];
  long long bs[4];
  long long batch;
  long long rows, cols;
  long long rs, cs;     // bytes
};

__host__ __device__ inline long long row_offset(const RowView &v, long long row) {
  long long off = 0;
  for (int i = v.np - 1; i >= 0; --i) {
    const long long q = row / v.pd[i];
    off += (row - q * v.pd[i]) * v.ps[i];
    row = q;
  }
  return off;
}

__host__ __device__ inline long long batch_offset(const MatView &v, long long b) {
  long long off = 0;
  for (int i = v.nb - 1; i >= 0; --i) {
    const long long q = b / v.bd[i];
    off += (b - q * v.bd[i]) * v.bs[i];
    b = q;
  }
  return off;
}

RowView make_row_view(const BackendTensorView *t, const char *who);
MatView make_mat_view(const BackendTensorView *t, const char *who);
bool view_is_contiguous(const BackendTensorView *t);
long long view_numel(const BackendTensorView *t);

// ---- kernel families (host launchers) ---------------------------------------

// elementwise.cu
enum EwOp : int { EW_COPY = 0, EW_ADD, EW_ADD_BIAS, EW_ADD_BIAS_RELU, EW_RELU, EW_MUL_SCALAR, EW_FILL, EW_RELU_BWD };
// out[row, c] = op(a[row, c], b[...]); b is a full tensor (EW_ADD; EW_RELU_BWD:
// out = a > 0 ? b : 0), a [rows_b, cols] table indexed by row % rows_b (broadcast
// add), or a bias row.
void launch_rowwise(EwOp op, const RowView &a, const RowView *b, long long b_mod_rows,
                    float scalar, const RowView &out, cudaStream_t st);
void launch_causal_mask(const MatView &scores, float neg_inf, cudaStream_t st);
void launch_embedding(const RowView &table, const char *ids_data, int ids_is_f32,
                      const RowView &ids_rows, const RowView &out, DevErr *err, cudaStream_t st);
void launch_transpose(const MatView &x, const MatView &out, cudaStream_t st);

// norm_softmax.cu
void launch_layernorm(const RowView &x, const float *gamma, long long gamma_cs, const float *beta,
                      long long beta_cs, const RowView &out, cudaStream_t st);
void launch_softmax_rows(const RowView &x, const RowView &out, int causal, float scale,
                         cudaStream_t st);

// gemm_simt.cu
struct GemmOperand {
  const char *data;
  long long rs, cs;     // strides in BYTES of the logical (row, col) element
};
struct GemmEpilogue {
  const float *bias = nullptr;      // [n]
  const float *residual = nullptr;  // same layout as C
  int relu = 0;
};
// C[b] (m x n) = A[b] (m x k) * B[b] (k x n), any strides; batch offsets in bytes
// come from the three MatViews' batch axes (b_batch may be null for a shared B).
void launch_gemm_simt(const MatView &a, const MatView &bmat, const MatView &c, long long m,
                      long long n, long long k, const GemmEpilogue &ep, cudaStream_t st);

// ingest.cu: `bytes` of a file from file_offset on into device memory at dst, in pieces through
// pinned buffers so that reading and the host-to-device copies overlap; returns when everything has
// arrived. check_finite_f32: the bytes are floats and a NaN or infinity raises std::domain_error
// (the destination is then partly written). Other failures raise std::runtime_error.
void file_to_device(const char *path, uint64_t file_offset, uint64_t bytes, void *dst, cudaStream_t st,
                    bool check_finite_f32);

// training.cu: backward and optimiser operators of the plugin table. `scratch` is device
// memory of at least training_scratch_bytes(rows, cols) for the operand at hand.
size_t training_scratch_bytes(long long rows, long long cols);
void launch_sum_squares(const float *x, long long n, void *scratch, double *result_dev, cudaStream_t st);
void launch_column_sum(const RowView &x, char *out, long long out_cs, void *scratch, cudaStream_t st);
void launch_layernorm_backward(const RowView &x, const char *gamma, long long gamma_cs, const RowView &dout,
                               const RowView &dx, char *dgamma, long long dgamma_cs, char *dbeta, long long dbeta_cs,
                               void *scratch, cudaStream_t st);
void launch_embedding_grads(const char *ids, int ids_is_f32, const RowView &ids_rows, const RowView &d_cur,
                            const RowView &d_tok, const RowView &d_pos, long long seq, DevErr *err, cudaStream_t st);
void launch_cross_entropy(const RowView &logits, const char *targets, int targets_is_f32, const RowView &targets_rows,
                          bool want_loss, bool want_backward, float *loss_out, void *scratch, DevErr *err,
                          cudaStream_t st);
void launch_softmax_backward(const RowView &sm, const RowView &dout, const RowView &dx, bool causal, cudaStream_t st);
void launch_adamw(float *params, const float *grads, float *m, float *v, long long n, float lr, float beta1,
                  float beta2, float b1_corr, float b2_corr, float weight_decay, int apply_decay, cudaStream_t st);

// native-loop kernels (dense row-major activations) ---------------------------

struct LoopState {
  int s;        // current context length of every stream
  int step;     // tokens generated so far
  int n_streams;
  int max_seq;
};

// embed.cu
void launch_embed_pos(const float *tok_emb, const float *pos_emb, const int *ids, int ids_ld,
                      const LoopState *state, int n_streams, int s_host, int d, int vocab,
                      float *x, DevErr *err, cudaStream_t st, float *x_hi = nullptr, float *x_lo = nullptr,
                      double2 *stats = nullptr, const struct TcPairF16 *x_f16 = nullptr);
// head_greedy.cu: final norm + output head + first-max selection + append +
// state advance in one launch (greedy, few streams, vocabulary up to 1024).
// `done` is a zero-initialised counter the kernel returns to zero.
bool head_greedy_supports(int n_streams, int d, int vocab);
void launch_head_greedy(const float *x, const float *gamma, const float *beta, const float *w, int d, int vocab,
                        int n_streams, int s_host, const LoopState *dstate, LoopState *state, unsigned *done,
                        int *ids, int ids_ld, int *out_tokens, int out_ld, float *logits, cudaStream_t st);
void launch_gather_last_ln(const float *x, const float *gamma, const float *beta,
                           const LoopState *state, int n_streams, int s_host, int d, float *out,
                           float *out_lo, cudaStream_t st);
// out_lo != nullptr: out receives the TF32 high part and out_lo the low part.
// state != nullptr: the launch covers `rows` as an upper bound and the kernel
// takes n_streams * state->s as the actual row count.
void launch_layernorm_dense(const float *x, const float *gamma, const float *beta, long long rows,
                            int d, float *out, float *out_lo, const LoopState *state, int n_streams,
                            cudaStream_t st);

// gemv.cu: out[m, n] = x[m, :] . W[:, n] for m <= 8 rows; W row-major [k, n].
// scratch must hold gemv_scratch_floats(m, n, k) floats when the launcher
// decides to split k across CTAs. x must hold 1, 2, 4 or 8 rows (m rounded up).
// err (optional) receives DEVERR_WAIT_TIMEOUT if a bounded wait of the
// streaming kernel runs out. Returns the number of kernels launched.
size_t gemv_scratch_floats(int m, int n, int k);
// residual ([m, n] dense, added after the bias) and relu finish the product as the layer wiring of
// the reference does (add_bias_rowwise, add, relu).
// ln_gamma / ln_beta ([k], only for shapes gemv_fuses_layernorm accepts): the rows of x pass through
// LayerNorm (layernorm_forward of the reference) on their way into the product.
bool gemv_fuses_layernorm(int n, int k);
int launch_gemv(const float *x, int m, const float *w, int k, int n, const float *bias,
                float *out, float *scratch, cudaStream_t st, DevErr *err = nullptr,
                const float *residual = nullptr, int relu = 0, const float *ln_gamma = nullptr,
                const float *ln_beta = nullptr);

// attention.cu: ctx[r, h*dh + :] for rows r = b*s + t of qkv [rows, 3*d].
// ctx_lo != nullptr: ctx receives the TF32 high part and ctx_lo the low part.
// attention_plan says how the triangular work is cut for a shape and how much
// scratch (floats of partial outputs, zero-initialised int counters) it needs.
struct AttentionPlan {
  int kc;              // key tiles per CTA
  int ctas_per_head;   // grid.x
  size_t scratch_floats;
  size_t counters;
};
AttentionPlan attention_plan(int n_streams, int s, int n_heads, int dh);
// state != nullptr: s is an upper bound with the same number of 64-row tiles
// as the actual context length state->s.
void launch_attention(const float *qkv, float *ctx, float *ctx_lo, int n_streams, int s, int n_heads, int d_model,
                      float *scratch, int *counters, const LoopState *state, cudaStream_t st);

// decode.cu: the one-row-per-stream kernels of the opt-in cached mode. Caches are
// [n_streams][cap][d] per layer; s (state->s when state is set, else s_host) is the context
// length including the newest token, whose K and V the attention kernel appends.
struct DecodeAttnPlan {
  int keys_per_chunk;
  int chunks;
  size_t scratch_floats;
};
DecodeAttnPlan attn_decode_plan(int n_streams, int s, int n_heads, int dh);
void launch_embed_last_ln(const float *tok_emb, const float *pos_emb, const int *ids, int ids_ld,
                          const LoopState *state, int s_host, int n_streams, int d, int vocab, const float *gamma,
                          const float *beta, float *x, float *ln, DevErr *err, cudaStream_t st);
void launch_kv_store(const float *qkv, const LoopState *state, int s_host, int n_streams, int d, int cap, float *kc,
                     float *vc, cudaStream_t st);
// counters: one zero-resting int per (stream, head), needed when the keys are cut into chunks.
// Returns the number of kernels launched.
int launch_attn_decode(const float *qkv, float *kc, float *vc, int cap, int d_model, int n_heads, int n_streams,
                       const LoopState *state, int s_host, float *part, int *counters, float *ctx, cudaStream_t st);

// decode_persistent.cu: cached mode, greedy, up to 8 streams: `steps` tokens in one resident kernel
// (cooperative launch, one CTA per SM, grid-wide barriers between the operators).
struct DecodePersistentArgs {
  const char *params;                 // parameter arena (device)
  const unsigned long long *offsets;  // device: [n_layers][12] byte offsets in LayerOff order, then
                                      // tok_emb, pos_emb, lnf_g, lnf_b, lm_head
  int n_layers, n_heads, d_model, d_ff, vocab, max_seq, n_streams;
  float *kcache, *vcache;
  int cap;
  unsigned long long layer_stride;    // floats between the layers of a cache
  int *ids;
  int ids_ld;
  int *out_tokens;
  int out_ld;
  LoopState *state;
  float *logits;     // [n_streams, vocab] last step's logits
  float *scratch;    // decode_persistent_scratch_floats(...)
  unsigned *barrier; // two words
  int s0, step0, steps;  // context length of the first step (including its new token), tokens made so far
  int sm_count;
  DevErr *err;
  unsigned long long *timeline;  // measurement aid (64 device words) or null
};
bool decode_persistent_supports(int n_streams, int n_heads, int d_model, int d_ff, int vocab);
size_t decode_persistent_scratch_floats(int n_streams, int n_heads, int d_model, int d_ff, int vocab, int sm_count);
void launch_decode_persistent(const DecodePersistentArgs &a, cudaStream_t st);

// sampler.cu
struct SamplerParams {
  float temp;
  unsigned top_k;
  float top_p;
};
size_t sampler_scratch_bytes(int vocab);
void launch_sampler(const float *logits, int vocab, int n_streams, const SamplerParams &sp,
                    unsigned *mt_state, int *ids, int ids_ld, int *out_tokens, int out_ld,
                    LoopState *state, void *scratch, cudaStream_t st);
void launch_sampler_rows(const float *logits, int vocab, int n_rows, const SamplerParams &sp,
                         unsigned *mt_state, int draws, int *out, void *scratch, cudaStream_t st);
void launch_mt_seed(unsigned *mt_state, const unsigned *seeds, int n, cudaStream_t st);
void launch_advance_state(LoopState *state, cudaStream_t st);
void launch_softmax_probs_f64(const float *logits, int vocab, int n_rows, float *probs,
                              cudaStream_t st);

}  // namespace lb
