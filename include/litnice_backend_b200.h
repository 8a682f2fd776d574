/*
 * liblitnice_backend_b200.so — NVIDIA B200 (sm_100a) backend plugin for litnicelm.
 *
 * Two groups of entry points, all plain C ABI:
 *
 *  1. litnice_backend_get_api(): the `backend.library` plugin contract of
 *     litnicelm (src/model/backend/backend_plugin_api.hpp:7-168). The host
 *     resolves this one symbol after dlopen (device_backend.cpp:182-230) and
 *     then calls through the returned table, so the unchanged `infer`,
 *     `inspect` and `inferloop` commands run on the GPU.
 *
 *  2. litnice_b200_*: a native token loop in which nothing but token ids
 *     crosses the host/device boundary per generated token. It replaces the
 *     host-driven loop of src/model/inference.cpp:265-296 and the per-row
 *     logits read-back of host_tensor_stage.hpp:101-125.
 *
 * Group 1 reports failures as C++ exceptions (the contract of the reference
 * loader: no status codes, main.cpp:37-40). Group 2 never throws: functions
 * return 0 on success and a negative LITNICE_B200_E* code otherwise, with
 * text available from litnice_b200_last_error().
 *
 * There is no CPU fallback anywhere: without a CUDA device every compute entry
 * fails loudly.
 */
#ifndef LITNICE_BACKEND_B200_H
#define LITNICE_BACKEND_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* 1. The litnicelm plugin contract (backend_plugin_api.hpp).                 */
/* ------------------------------------------------------------------------ */

#define LITNICE_TENSOR_MAX_RANK 6
#define LITNICE_BACKEND_ABI_VERSION 16u /* backend_plugin_api.hpp:164 */

/* backend_plugin_api.hpp:7-18. Strides are in bytes; rows/cols/stride_r/stride_c
 * repeat dims[0], dims[1] and the strides of the last two axes
 * (device_backend.cpp:154-169). device: 0 CPU, 1 GPU. dtype: 0 f32, 1 i32. */
typedef struct BackendTensorView {
  uint32_t device;
  uint32_t dtype;
  void *data;
  uint32_t rank;
  int64_t rows;
  int64_t cols;
  int64_t stride_r_bytes;
  int64_t stride_c_bytes;
  int64_t dims[LITNICE_TENSOR_MAX_RANK];
  int64_t strides_bytes[LITNICE_TENSOR_MAX_RANK];
} BackendTensorView;

/* backend_plugin_api.hpp:20-24 */
typedef struct BackendMemoryInfo {
  uint32_t available;
  uint64_t free_bytes;
  uint64_t total_bytes;
} BackendMemoryInfo;

typedef const BackendTensorView *LitniceView;

/* backend_plugin_api.hpp:26-162: abi_version followed by 55 entries, in this
 * exact order. Entries marked [inference] are reached by infer / inspect /
 * inferloop; the others belong to training and throw "not implemented" here. */
typedef struct BackendApiV1 {
  uint32_t abi_version;
  void *(*create)(uint32_t device);                                        /* [inference] */
  void (*destroy)(void *backend);                                          /* [inference] */
  uint32_t (*device)(void *backend);                                       /* [inference] */
  void *(*alloc)(void *backend, uint64_t bytes, uint32_t alignment);       /* [inference] */
  void (*free)(void *backend, void *ptr);                                  /* [inference] */
  void (*copy_host2device)(void *backend, void *dst, const void *src, uint64_t bytes); /* [inference] */
  void (*copy_device2host)(void *backend, void *dst, const void *src, uint64_t bytes); /* [inference] */
  void (*copy)(void *backend, LitniceView src, LitniceView dst);           /* [inference] */
  void (*fill)(void *backend, LitniceView t, float v);                     /* [inference] */
  void (*add)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*add_inplace)(void *backend, LitniceView a, LitniceView b);
  void (*add_bias_rowwise)(void *backend, LitniceView x, LitniceView bias_1xC, LitniceView out); /* [inference] */
  void (*add_bias_relu_rowwise)(void *backend, LitniceView x, LitniceView bias_1xC, LitniceView out); /* [inference] */
  void (*add_bias_relu_rowwise_inplace)(void *backend, LitniceView x, LitniceView bias_1xC); /* [inference] */
  void (*mul_scalar)(void *backend, LitniceView x, float s, LitniceView out); /* [inference] */
  float (*sum_squares_f32)(void *backend, LitniceView x);
  void (*relu)(void *backend, LitniceView x, LitniceView out);             /* [inference] */
  void (*relu_backward)(void *backend, LitniceView preact, LitniceView dout, LitniceView dx);
  void (*relu_backward_inplace)(void *backend, LitniceView preact, LitniceView dout_dx);
  void (*row_sum)(void *backend, LitniceView x, LitniceView out_1xC);
  void (*gemm)(void *backend, LitniceView a, LitniceView b, LitniceView out);
  void (*gemm_ranked_matrix_rhs)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*gemm_ranked_matrix_rhs_t)(void *backend, LitniceView a, LitniceView b, LitniceView out);
  void (*gemm_ranked_reduce_lhs_t)(void *backend, LitniceView a, LitniceView b, LitniceView out);
  void (*gemm_batched)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*gemm_batched_lhs_t)(void *backend, LitniceView a, LitniceView b, LitniceView out);
  void (*gemm_batched_rhs_t)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*transpose)(void *backend, LitniceView x, LitniceView out);
  void (*layernorm_forward)(void *backend, LitniceView x, LitniceView gamma_1xC, LitniceView beta_1xC, LitniceView out); /* [inference] */
  void (*layernorm_backward)(void *backend, LitniceView x, LitniceView gamma_1xC, LitniceView dout, LitniceView dx, LitniceView dgamma_1xC, LitniceView dbeta_1xC);
  void (*embedding_lookup)(void *backend, LitniceView table, LitniceView ids, LitniceView out); /* [inference] */
  void (*accumulate_embedding_grads)(void *backend, LitniceView ids, LitniceView d_cur, LitniceView d_tok, LitniceView d_pos);
  void (*cross_entropy_mean)(void *backend, LitniceView logits, LitniceView targets, LitniceView out_loss);
  void (*cross_entropy_mean_backward_inplace)(void *backend, LitniceView logits, LitniceView targets, LitniceView out_loss);
  float (*read_scalar_f32)(void *backend, LitniceView x);
  void (*backward_from_logits_targets)(void *backend, LitniceView logits, LitniceView targets);
  void (*softmax_rows)(void *backend, LitniceView x, LitniceView out);     /* [inference] */
  void (*softmax_backward_rows)(void *backend, LitniceView softmax, LitniceView dout, LitniceView dx);
  void (*scaled_causal_softmax_rows)(void *backend, LitniceView scores, float scale, LitniceView out); /* [inference] */
  uint32_t (*supports_exec_context_iteration)(void *backend);             /* [inference] */
  void (*start_exec_context_iteration)(void *backend);                     /* [inference] */
  void (*finish_exec_context_iteration)(void *backend);                    /* [inference] */
  void (*start_exec_context_group)(void *backend);                         /* [inference] */
  void (*finish_exec_context_group)(void *backend);                        /* [inference] */
  void (*gemm_batched_exec_context)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*gemm_batched_lhs_t_exec_context)(void *backend, LitniceView a, LitniceView b, LitniceView out);
  void (*gemm_batched_rhs_t_exec_context)(void *backend, LitniceView a, LitniceView b, LitniceView out); /* [inference] */
  void (*scaled_causal_softmax_rows_exec_context)(void *backend, LitniceView scores, float scale, LitniceView out); /* [inference] */
  void (*softmax_backward_causal_rows_exec_context)(void *backend, LitniceView softmax, LitniceView dout, LitniceView dx);
  void (*softmax_backward_causal_rows)(void *backend, LitniceView softmax, LitniceView dout, LitniceView dx);
  void (*apply_causal_mask_inplace)(void *backend, LitniceView scores, float neg_inf); /* [inference] */
  void (*adamw_step)(void *backend, LitniceView params, LitniceView grads, LitniceView m, LitniceView v, uint64_t step, float learning_rate, float beta1, float beta2, float weight_decay, uint32_t apply_weight_decay);
  uint32_t (*is_file2device_read_supported)(void *backend);
  void (*read_file2device)(void *backend, const char *path, void *dst, uint64_t size, uint64_t file_offset);
  BackendMemoryInfo (*memory_info)(void *backend);
} BackendApiV1;

/* The symbol the litnicelm loader resolves (device_backend.cpp:191-206;
 * the CPU plugin's counterpart is backend_plugin_cpu.cpp:498-500). The table
 * has static storage and abi_version == 16. The GPU is chosen by
 * CUDA_VISIBLE_DEVICES or the LITNICE_B200_DEVICE environment variable: the
 * contract's create(device) carries the CPU/GPU enum, not an ordinal. */
const BackendApiV1 *litnice_backend_get_api(void);

/* ------------------------------------------------------------------------ */
/* 2. Native token loop.                                                      */
/* ------------------------------------------------------------------------ */

#define LITNICE_B200_OK 0
#define LITNICE_B200_EINVAL (-1)   /* bad argument or shape */
#define LITNICE_B200_ECUDA (-2)    /* CUDA runtime error */
#define LITNICE_B200_ENOMEM (-3)   /* device allocation failed */
#define LITNICE_B200_EIO (-4)      /* checkpoint file unreadable or mismatched */
#define LITNICE_B200_EDEVICE (-5)  /* a kernel reported an error (bad token id, wait ran out) */
#define LITNICE_B200_ETOOBIG (-6)  /* litnice_b200_gemv_noalloc: sizes beyond its built-in scratch */

typedef struct litnice_b200_session litnice_b200_session;

/* model.* and memory.alignment_bytes of the YAML (include/types.hpp:134-146). */
typedef struct litnice_b200_dims {
  int32_t n_layers, n_heads, d_model, d_ff, vocab_size, max_seq_len;
  uint64_t alignment_bytes;
} litnice_b200_dims;

/* inference.temp / top_k / top_p (include/types.hpp:112-119). temp <= 0 or
 * top_k == 1 selects greedy, as in inference.cpp:206-208. */
typedef struct litnice_b200_sampling {
  float temp;
  uint32_t top_k;
  float top_p;
} litnice_b200_sampling;

/* Counters of the most recent generate / run call. */
typedef struct litnice_b200_stats {
  double device_ms;          /* CUDA-event time of the token loop on the session's stream */
  int64_t kernel_launches;   /* kernels of this library launched inside that region */
  int64_t tokens;            /* tokens produced over all streams */
  int64_t h2d_bytes, d2h_bytes;
  double gemm_ms;            /* filled only by litnice_b200_profile_step */
  int64_t gemm_launches;
  double gemm_flops;         /* algorithmic flops of those launches */
  double attn_ms;
  int64_t attn_launches;
  /* litnice_b200_profile_step, one step without events: per launch the span from the
   * earliest CTA start to the latest CTA end on the device clock (launches overlap as in
   * the token loop), summed per kernel class, and the span of the whole step. Filled for
   * the tensor-core kernels only. */
  double gemm_span_ms;
  int64_t gemm_span_launches;
  double gemm_span_flops;
  double attn_span_ms;
  int64_t attn_span_launches;
  double step_span_ms;
} litnice_b200_stats;

/* Builds a session on the current CUDA device (or LITNICE_B200_DEVICE) for up
 * to max_streams independent streams decoded in lockstep. Replaces the runtime
 * object of inference.cpp:49-71 and its three arena allocations
 * (inference_memory_manager.cpp:7-33). */
int litnice_b200_session_create(const litnice_b200_dims *dims, int32_t max_streams,
                                litnice_b200_session **out);
/* The same on an explicit CUDA device ordinal (LITNICE_B200_DEVICE is not consulted): what a
 * host that runs one thread per GPU calls, each thread with its own share of the streams
 * (the reference runs one stream per process, inference.cpp:362-405; streams never
 * exchange data, so the shares need no collective). Every call on a session selects the
 * session's device first, so a session may be driven from any one thread at a time. */
int litnice_b200_session_create_on(const litnice_b200_dims *dims, int32_t max_streams, int32_t device,
                                   litnice_b200_session **out);
void litnice_b200_session_destroy(litnice_b200_session *s);
const char *litnice_b200_last_error(const litnice_b200_session *s);

/* Weights enter as the parameter-arena image (layout of named_layout.cpp:40-161),
 * either from host memory or from a version-6 checkpoint file; mirrors
 * load_checkpoint (checkpoint.cpp:588-652), including its dimension checks. */
int litnice_b200_load_params(litnice_b200_session *s, const void *host_arena, uint64_t bytes);
int litnice_b200_load_checkpoint(litnice_b200_session *s, const char *path);

/* generate_text (inference.cpp:265-296) for n_streams independent streams in
 * lockstep: every step recomputes the whole context (the reference keeps no
 * KV cache), samples on the GPU and appends the token on the GPU. All streams
 * share prompt_len. Stops after max_new tokens or when the context reaches
 * max_seq_len (guard of inference.cpp:278). prompts: [n_streams, prompt_len]
 * host int32; seeds: [n_streams] (inference.seed per stream) or NULL for
 * 12345; out_tokens: [n_streams, max_new] host int32; *out_count receives the
 * tokens produced per stream. Host buffers in, host buffers out. */
int litnice_b200_generate(litnice_b200_session *s, const int32_t *prompts, int32_t n_streams,
                          int32_t prompt_len, int32_t max_new,
                          const litnice_b200_sampling *sampling, const uint32_t *seeds,
                          int32_t *out_tokens, int32_t *out_count);

/* The same loop split in three so that the middle part can be timed with the
 * prompts already resident in HBM: upload, run (returns tokens per stream),
 * download. */
int litnice_b200_upload_prompts(litnice_b200_session *s, const int32_t *prompts,
                                int32_t n_streams, int32_t prompt_len, const uint32_t *seeds);
int litnice_b200_run(litnice_b200_session *s, int32_t max_new,
                     const litnice_b200_sampling *sampling, int32_t *out_count);
int litnice_b200_download_tokens(litnice_b200_session *s, int32_t *out_tokens, int32_t max_new);

/* When enabled, every step of generate/run also keeps its last-row logits
 * ([step][stream][vocab]) for litnice_b200_read_step_logits. Parity runs only. */
int litnice_b200_keep_step_logits(litnice_b200_session *s, int32_t enable);
int litnice_b200_read_step_logits(litnice_b200_session *s, float *out, int64_t max_floats);

/* Transformer::forward (transformer.cpp:70-114) on ids [n_streams, seq_len]:
 * writes logits of every row ([n_streams, seq_len, vocab], all_rows != 0) or of
 * the last row of each stream ([n_streams, vocab]) to host memory. */
int litnice_b200_forward(litnice_b200_session *s, const int32_t *ids, int32_t n_streams,
                         int32_t seq_len, int32_t all_rows, float *out_logits);

/* inspect_distribution (inference.cpp:298-359): next-token probabilities of
 * the last row of each stream, softmax evaluated in double; probs is
 * [n_streams, vocab] host float. */
int litnice_b200_inspect(litnice_b200_session *s, const int32_t *ids, int32_t n_streams,
                         int32_t seq_len, float *probs);

/* select_next_token_sampled (inference.cpp:200-263) alone: one draw per row of
 * host logits [n_rows, vocab] with generator std::mt19937(seeds[row]) advanced
 * `draws` times; out is [n_rows, draws]. Used to check the fused sampler
 * against the host selector on identical logits. */
int litnice_b200_sample_logits(litnice_b200_session *s, const float *logits, int32_t n_rows,
                               const litnice_b200_sampling *sampling, const uint32_t *seeds,
                               int32_t draws, int32_t *out);

int litnice_b200_get_stats(const litnice_b200_session *s, litnice_b200_stats *out);

/* No counterpart in the reference. Few-row product out[m, n] = x[m, k] * W[k, n]
 * (+ bias[n]) for callers that cannot allocate device memory while they run:
 * a host that has already given all device memory to its own arenas, or a
 * loop that cannot afford the device-wide stall of an allocation. It calls no
 * cudaMalloc / cudaFree or any other allocating routine; the split-k partial
 * sums live in a 1.5 MiB array built into the library image (held by every GPU
 * that loads the library until the process exits).
 *   x [m, k], W [k, n] row-major, bias [n] or NULL, out [m, n]: device pointers
 *   owned by the caller; m must be 1, 2, 4 or 8; stream is a cudaStream_t
 *   (NULL = default stream). The call only enqueues work on that stream.
 * Returns 0, LITNICE_B200_EINVAL, LITNICE_B200_ECUDA, or LITNICE_B200_ETOOBIG
 * when m, k, n would need more than the 393216 floats of built-in scratch
 * (a line on stderr says how much was needed). The kernel cuts k into
 * min(ceil(296 / ceil(n / 128)), ceil(k / 64)) ranges when n < 18944 and keeps
 * ranges * m * n partial sums, so in practice only m = 8 is ever refused: with
 * 16385..18816 columns and k > 128 (3 ranges), or 12289..12544 columns and k > 192
 * (4 ranges). Shapes with n >= 18944 or k <= 64 need no scratch at all.
 * The first call on each device looks up the device address of the built-in
 * array (and loads the kernels): make that first call before any stream
 * capture begins. All calls share the one array: it keeps the previous call's
 * partial sums, which is harmless because each call overwrites every entry it
 * later reads, but two calls whose kernels overlap on the GPU (different
 * streams, or different host threads) race on it. */
int litnice_b200_gemv_noalloc(const float *x, int32_t m, const float *w, int32_t k, int32_t n,
                              const float *bias, float *out, void *stream);

/* ------------------------------------------------------------------------ */
/* 3. Diagnostics and measurement aids.                                       */
/*    None of these is part of the token loop and a host binds none of them;  */
/*    the tests, bench.py and the profiling commands call them.               */
/* ------------------------------------------------------------------------ */

/* Runs one step at context length seq_len for n_streams streams with CUDA
 * events around each projection and attention launch, `repeats` times, and
 * fills the gemm_* / attn_* fields of the stats. Measurement aid. */
int litnice_b200_profile_step(litnice_b200_session *s, int32_t n_streams, int32_t seq_len,
                              int32_t repeats);

/* One projection on host buffers: c[m,n] = a[m,k] * w[k,n] (+ bias[n]) (+ residual[m,n])
 * (ReLU when relu != 0), i.e. gemm_ranked_matrix_rhs followed by add_bias_rowwise
 * / add_bias_relu_rowwise / add (device_backend.cpp:1112-1131, 840-908, 752-813).
 * engine 0: fp32 SIMT kernel; engine 1: tcgen05 tensor-core kernel with the
 * three-product TF32 split (needs k % 32 == 0 and n % 64 == 0); engine 2: the
 * same kernel on fp16 pairs with one power-of-two scale per 64 consecutive k of
 * a row (k % 64 == 0), the operand format of the native loop. Allocates and
 * frees its own device buffers; meant for checking the two engines against
 * each other and against the CPU. */
int litnice_b200_projection_host(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                                 const float *bias, const float *residual, int32_t relu, float *c);

/* Measurement aid: the same projection (no epilogue terms) launched `repeats`
 * times back to back on one stream; *avg_us receives the mean device time per
 * launch after the first (CUDA events on that stream). */
int litnice_b200_projection_time(int32_t engine, const float *a, int32_t m, int32_t k, const float *w, int32_t n,
                                 float *c, int32_t repeats, double *avg_us);

/* The few-row product out[m, n] = x[m, k] * W[k, n] (+ bias[n]) (+ residual[m, n])
 * (ReLU when relu != 0), m <= 8, on host buffers: the M <= 8 case of
 * gemm_ranked_matrix_rhs (device_backend.cpp:1112-1131) as the output head uses it
 * on the last rows (output_head.cpp:58-70), followed by add_bias_rowwise / add /
 * relu (:840-908, 752-813, 978-1001). With ln_gamma and ln_beta ([k], both or
 * neither) the rows of x pass through layernorm_forward (:1247-1279) first, inside
 * the same kernel; only shapes the streaming kernel takes (EINVAL otherwise).
 * Allocates and frees its own device buffers. */
int litnice_b200_gemv_host(const float *x, int32_t m, const float *w, int32_t k, int32_t n,
                           const float *bias, const float *residual, int32_t relu, const float *ln_gamma,
                           const float *ln_beta, float *out);

/* Device time of that product. cold_l2 = 2: `repeats` calls back to back between one
 * pair of CUDA events, each on the next of a ring of weight copies larger than three
 * times the L2 (every call reads its matrix from HBM); 1: events around each call
 * with a 256 MB buffer written before it; 0: the same matrix every call. force_tn
 * (0, 128, 256) and force_splits (0 = planned; negative: that many k ranges joined through
 * scratch and a second kernel instead of a thread-block cluster) override the tile plan. *avg_us: mean
 * microseconds per call; *launches: kernels per call. */
int litnice_b200_gemv_time(int32_t m, int32_t k, int32_t n, int32_t repeats, int32_t cold_l2,
                           int32_t force_tn, int32_t force_splits, double *avg_us, int32_t *launches);

/* Self-test of the bounded waits: a one-CTA kernel waits on a barrier that nothing
 * completes, with a limit of limit_us microseconds (1..1000). It must come back on
 * its own with *code == 2 (a wait ran out), *detail == 99 and *waited_us >= limit_us,
 * and the device must stay usable. */
int litnice_b200_selftest_wait_timeout(int32_t limit_us, int32_t *code, int32_t *detail, double *waited_us);

#ifdef __cplusplus
}
#endif
#endif /* LITNICE_BACKEND_B200_H */
