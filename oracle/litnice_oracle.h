/* Test infrastructure, not product code.
 *
 * CPU restatement, in plain C, of the litnicelm inference path: the parameter
 * arena layout, every backend operator the forward pass uses, the forward pass
 * itself and the token selectors. Each function cites the reference lines it
 * follows. Arithmetic is ordered exactly as the reference CPU backend orders it
 * (fp32 products summed in ascending k, fp64 means and softmax sums), and the
 * library is built without FMA contraction, so results are bit-identical to
 * the reference CPU backend; tests/test_oracle_pin.py checks that against the
 * reference compiled from its own sources.
 *
 * Parity status: the reference ships no tests, golden vectors or fixtures for
 * this path, so the pin is "outputs of the reference itself run in the build
 * container" (committed under tests/golden/ with their generator).
 */
#ifndef LITNICE_ORACLE_H
#define LITNICE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LO_MAX_LAYERS 64

typedef struct lo_dims {
  int32_t n_layers, n_heads, d_model, d_ff, vocab, max_seq;
  int64_t alignment; /* memory.alignment_bytes */
} lo_dims;

typedef struct lo_layer_off {
  uint64_t ln1_g, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_g, ln2_b, w1, b1, w2, b2;
} lo_layer_off;

typedef struct lo_layout {
  uint64_t total_bytes, decay_bytes;
  uint64_t tok_emb, pos_emb, lnf_g, lnf_b, lm_head;
  lo_layer_off layer[LO_MAX_LAYERS];
} lo_layout;

/* Byte offsets of every parameter in the arena (named_layout.cpp:40-161). */
int lo_build_layout(const lo_dims *d, lo_layout *out);

/* Operators on dense row-major arrays (device_backend.cpp, lines cited in .c). */
void lo_gemm(const float *a, const float *b, float *out, int64_t m, int64_t k, int64_t n);
void lo_gemm_rhs_t(const float *a, int64_t lda, const float *b, int64_t ldb, float *out,
                   int64_t ldo, int64_t m, int64_t k, int64_t n);
void lo_gemm_strided(const float *a, int64_t lda, const float *b, int64_t ldb, float *out,
                     int64_t ldo, int64_t m, int64_t k, int64_t n);
void lo_layernorm(const float *x, const float *gamma, const float *beta, float *out,
                  int64_t rows, int64_t cols);
void lo_softmax_rows(const float *x, float *out, int64_t rows, int64_t cols);
void lo_scaled_causal_softmax_rows(const float *x, float scale, float *out, int64_t rows,
                                   int64_t cols);
int lo_embedding(const float *table, const int32_t *ids, float *out, int64_t n_ids,
                 int64_t vocab, int64_t d);

/* Transformer::forward for one stream (transformer.cpp:70-114). logits_out has
 * s*V floats, or V floats (the last row) when only_last != 0. Returns 0, or -1
 * on a token id outside [0, V). */
int lo_forward(const lo_dims *d, const void *params, const int32_t *ids, int32_t s,
               float *logits_out, int only_last);

/* Token selectors (inference.cpp:188-263). */
int32_t lo_greedy(const float *row, int32_t v);

typedef struct lo_mt19937 {
  uint32_t mt[624];
  int32_t idx;
} lo_mt19937;
void lo_mt_seed(lo_mt19937 *g, uint32_t seed);
uint32_t lo_mt_next(lo_mt19937 *g);
/* Candidates with exactly equal logits keep ascending-id order (the reference
 * leaves that order to std::sort). Returns -1 for top_p outside (0,1]. */
int32_t lo_sample(const float *row, int32_t v, float temp, uint32_t top_k, float top_p,
                  lo_mt19937 *g);
/* Same, also reporting how many candidates survived top-k / top-p. */
int32_t lo_sample_ex(const float *row, int32_t v, float temp, uint32_t top_k, float top_p,
                     lo_mt19937 *g, int32_t *kept_out);

/* generate_text for one stream (inference.cpp:265-296): returns the number of
 * tokens written to out_ids; optionally stores each step's last-row logits. */
int32_t lo_generate(const lo_dims *d, const void *params, const int32_t *prompt,
                    int32_t prompt_len, int32_t max_new, float temp, uint32_t top_k,
                    float top_p, uint32_t seed, int32_t *out_ids, float *step_logits);

#ifdef __cplusplus
}
#endif
#endif
