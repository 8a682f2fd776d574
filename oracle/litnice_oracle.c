/* Test infrastructure, not product code. See litnice_oracle.h.
 *
 * Citations are paths inside the litnicelm reference tree.
 * Build: gcc -std=c11 -O2 -fopenmp -ffp-contract=off (oracle/Makefile). Rows
 * are independent, so the OpenMP split over rows cannot change any value.
 */
#include "litnice_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

static uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

/* named_layout.cpp:40-161: parameters are declared in model order; the ones
 * with weight decay (embeddings and matrices) are packed first, each aligned,
 * the zone is padded, then the rest (LayerNorm vectors, biases) follow. */
int lo_build_layout(const lo_dims *d, lo_layout *out) {
  if (d->n_layers <= 0 || d->n_layers > LO_MAX_LAYERS || d->alignment <= 0) return -1;
  const uint64_t A = (uint64_t)d->alignment, D = (uint64_t)d->d_model, F = (uint64_t)d->d_ff,
                 V = (uint64_t)d->vocab, S = (uint64_t)d->max_seq;
  uint64_t cur = 0;
#define PUT(field, bytes) do { cur = align_up(cur, A); (field) = cur; cur += (bytes); } while (0)
  PUT(out->tok_emb, 4 * V * D);
  PUT(out->pos_emb, 4 * S * D);
  for (int l = 0; l < d->n_layers; ++l) {
    PUT(out->layer[l].qkv_w, 4 * D * 3 * D);
    PUT(out->layer[l].out_w, 4 * D * D);
    PUT(out->layer[l].w1, 4 * D * F);
    PUT(out->layer[l].w2, 4 * F * D);
  }
  PUT(out->lm_head, 4 * D * V);
  out->decay_bytes = align_up(cur, A);
  cur = out->decay_bytes;
  for (int l = 0; l < d->n_layers; ++l) {
    PUT(out->layer[l].ln1_g, 4 * D);
    PUT(out->layer[l].ln1_b, 4 * D);
    PUT(out->layer[l].qkv_b, 4 * 3 * D);
    PUT(out->layer[l].out_b, 4 * D);
    PUT(out->layer[l].ln2_g, 4 * D);
    PUT(out->layer[l].ln2_b, 4 * D);
    PUT(out->layer[l].b1, 4 * F);
    PUT(out->layer[l].b2, 4 * D);
  }
  PUT(out->lnf_g, 4 * D);
  PUT(out->lnf_b, 4 * D);
#undef PUT
  out->total_bytes = align_up(cur, A);
  return 0;
}

/* device_backend.cpp:1112-1131 (gemm_ranked_matrix_rhs) and :1175-1193
 * (gemm_batched): out[r,c] = sum_k a[r,k]*b[k,c], one fp32 accumulator per
 * element, k ascending. The k-outer/c-inner order below keeps that sequence. */
void lo_gemm_strided(const float *a, int64_t lda, const float *b, int64_t ldb, float *out,
                     int64_t ldo, int64_t m, int64_t k, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float *o = out + r * ldo;
    for (int64_t c = 0; c < n; ++c) o[c] = 0.0f;
    for (int64_t kk = 0; kk < k; ++kk) {
      const float av = a[r * lda + kk];
      const float *brow = b + kk * ldb;
      for (int64_t c = 0; c < n; ++c) o[c] = o[c] + av * brow[c];
    }
  }
}

void lo_gemm(const float *a, const float *b, float *out, int64_t m, int64_t k, int64_t n) {
  lo_gemm_strided(a, k, b, n, out, n, m, k, n);
}

/* device_backend.cpp:1216-1235 (gemm_batched_rhs_t): out[r,c] = sum_k a[r,k]*b[c,k]. */
void lo_gemm_rhs_t(const float *a, int64_t lda, const float *b, int64_t ldb, float *out,
                   int64_t ldo, int64_t m, int64_t k, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < n; ++c) {
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; ++kk) acc = acc + a[r * lda + kk] * b[c * ldb + kk];
      out[r * ldo + c] = acc;
    }
}

/* device_backend.cpp:1247-1279: mean and biased variance in double,
 * inv_std = 1/sqrt(float(var)+1e-5f) in float. */
void lo_layernorm(const float *x, const float *gamma, const float *beta, float *out,
                  int64_t rows, int64_t cols) {
  const float eps = 1e-5f;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    double mean = 0.0;
    for (int64_t c = 0; c < cols; ++c) mean += xr[c];
    mean /= (double)cols;
    double var = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      const double dd = (double)xr[c] - mean;
      var += dd * dd;
    }
    var /= (double)cols;
    const float inv_std = 1.0f / sqrtf((float)var + eps);
    for (int64_t c = 0; c < cols; ++c) {
      const float xn = (xr[c] - (float)mean) * inv_std;
      out[r * cols + c] = xn * gamma[c] + beta[c];
    }
  }
}

/* device_backend.cpp:1466-1494: fp32 max, expf, fp64 sum, inv = float(1/sum). */
void lo_softmax_rows(const float *x, float *out, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *o = out + r * cols;
    float mx = xr[0];
    for (int64_t c = 1; c < cols; ++c) mx = xr[c] > mx ? xr[c] : mx;
    double sum = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      o[c] = expf(xr[c] - mx);
      sum += (double)o[c];
    }
    const float inv = (float)(1.0 / sum);
    for (int64_t c = 0; c < cols; ++c) o[c] = o[c] * inv;
  }
}

/* device_backend.cpp:1554-1592: row r of each [cols,cols] block keeps columns
 * c <= r % cols; max and sum over those; zeros elsewhere. */
void lo_scaled_causal_softmax_rows(const float *x, float scale, float *out, int64_t rows,
                                   int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *o = out + r * cols;
    const int64_t lr = r % cols;
    float mx = -FLT_MAX;
    for (int64_t c = 0; c <= lr; ++c) {
      const float v = xr[c] * scale;
      mx = v > mx ? v : mx;
    }
    double sum = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      float v = 0.0f;
      if (c <= lr) {
        const float sv = xr[c] * scale;
        v = expf(sv - mx);
        sum += (double)v;
      }
      o[c] = v;
    }
    const float inv = (float)(1.0 / sum);
    for (int64_t c = 0; c <= lr; ++c) o[c] = o[c] * inv;
  }
}

/* device_backend.cpp:1345-1366: row gather; an id outside [0,V) is an error. */
int lo_embedding(const float *table, const int32_t *ids, float *out, int64_t n_ids,
                 int64_t vocab, int64_t d) {
  for (int64_t t = 0; t < n_ids; ++t) {
    if (ids[t] < 0 || ids[t] >= vocab) return -1;
    memcpy(out + t * d, table + (int64_t)ids[t] * d, (size_t)d * sizeof(float));
  }
  return 0;
}

static void add_bias(float *x, const float *b, int64_t rows, int64_t cols, int relu) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      const float v = x[r * cols + c] + b[c];
      x[r * cols + c] = relu ? (v > 0.0f ? v : 0.0f) : v;
    }
}

/* transformer.cpp:70-114, transformer_layer.cpp:50-92,
 * self_attention_fused_inplace.cpp:42-103 (the `reference` attention variant,
 * self_attention.cpp:41-102, yields the same values: scale, mask to -1e9 and a
 * full-row softmax give exp()==0 above the diagonal), ffn.cpp:38-66,
 * output_head.cpp:36-74. */
int lo_forward(const lo_dims *d, const void *params, const int32_t *ids, int32_t s,
               float *logits_out, int only_last) {
  lo_layout L;
  if (lo_build_layout(d, &L) != 0) return -2;
  const int64_t D = d->d_model, F = d->d_ff, V = d->vocab, H = d->n_heads, dh = D / H;
  const char *base = (const char *)params;
#define P(off) ((const float *)(base + (off)))
  float *x = malloc(sizeof(float) * s * D), *ln = malloc(sizeof(float) * s * D),
        *qkv = malloc(sizeof(float) * s * 3 * D), *ctx = malloc(sizeof(float) * s * D),
        *tmp = malloc(sizeof(float) * s * D), *y = malloc(sizeof(float) * s * D),
        *h = malloc(sizeof(float) * s * F), *sc = malloc(sizeof(float) * (size_t)s * s),
        *w = malloc(sizeof(float) * (size_t)s * s);
  int rc = 0;
  if (lo_embedding(P(L.tok_emb), ids, x, s, V, D) != 0) { rc = -1; goto done; }
  {
    const float *pos = P(L.pos_emb);
    for (int64_t i = 0; i < (int64_t)s * D; ++i) x[i] = x[i] + pos[i];
  }
  const float scale = 1.0f / sqrtf((float)dh);
  for (int l = 0; l < d->n_layers; ++l) {
    const lo_layer_off *o = &L.layer[l];
    lo_layernorm(x, P(o->ln1_g), P(o->ln1_b), ln, s, D);
    lo_gemm(ln, P(o->qkv_w), qkv, s, D, 3 * D);
    add_bias(qkv, P(o->qkv_b), s, 3 * D, 0);
    for (int64_t hh = 0; hh < H; ++hh) {
      const float *q = qkv + hh * dh, *k = qkv + D + hh * dh, *v = qkv + 2 * D + hh * dh;
      lo_gemm_rhs_t(q, 3 * D, k, 3 * D, sc, s, s, dh, s);
      lo_scaled_causal_softmax_rows(sc, scale, w, s, s);
      lo_gemm_strided(w, s, v, 3 * D, ctx + hh * dh, D, s, s, dh);
    }
    lo_gemm(ctx, P(o->out_w), tmp, s, D, D);
    add_bias(tmp, P(o->out_b), s, D, 0);
    for (int64_t i = 0; i < (int64_t)s * D; ++i) y[i] = x[i] + tmp[i];
    lo_layernorm(y, P(o->ln2_g), P(o->ln2_b), ln, s, D);
    lo_gemm(ln, P(o->w1), h, s, D, F);
    add_bias(h, P(o->b1), s, F, 1);
    lo_gemm(h, P(o->w2), tmp, s, F, D);
    add_bias(tmp, P(o->b2), s, D, 0);
    for (int64_t i = 0; i < (int64_t)s * D; ++i) x[i] = y[i] + tmp[i];
  }
  lo_layernorm(x, P(L.lnf_g), P(L.lnf_b), ln, s, D);
  if (only_last)
    lo_gemm(ln + (int64_t)(s - 1) * D, P(L.lm_head), logits_out, 1, D, V);
  else
    lo_gemm(ln, P(L.lm_head), logits_out, s, D, V);
#undef P
done:
  free(x); free(ln); free(qkv); free(ctx); free(tmp); free(y); free(h); free(sc); free(w);
  return rc;
}

/* inference.cpp:188-198: first index of the maximum (strict '>'). */
int32_t lo_greedy(const float *row, int32_t v) {
  int32_t best = 0;
  float bv = row[0];
  for (int32_t i = 1; i < v; ++i)
    if (row[i] > bv) { bv = row[i]; best = i; }
  return best;
}

/* std::mt19937 as published (Matsumoto & Nishimura), seeded the way
 * std::mersenne_twister_engine::seed(value) does. */
void lo_mt_seed(lo_mt19937 *g, uint32_t seed) {
  g->mt[0] = seed;
  for (int i = 1; i < 624; ++i)
    g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
  g->idx = 624;
}

uint32_t lo_mt_next(lo_mt19937 *g) {
  if (g->idx >= 624) {
    for (int i = 0; i < 624; ++i) {
      const uint32_t yv = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7fffffffu);
      g->mt[i] = g->mt[(i + 397) % 624] ^ (yv >> 1) ^ ((yv & 1u) ? 0x9908b0dfu : 0u);
    }
    g->idx = 0;
  }
  uint32_t yv = g->mt[g->idx++];
  yv ^= yv >> 11;
  yv ^= (yv << 7) & 0x9d2c5680u;
  yv ^= (yv << 15) & 0xefc60000u;
  yv ^= yv >> 18;
  return yv;
}

typedef struct { double x; int32_t id; } cand_t;
static int cand_cmp(const void *pa, const void *pb) {
  const cand_t *a = pa, *b = pb;
  if (a->x > b->x) return -1;
  if (a->x < b->x) return 1;
  return a->id < b->id ? -1 : (a->id > b->id ? 1 : 0);
}

/* inference.cpp:200-263; the draw is libstdc++'s std::discrete_distribution
 * (GCC 13 bits/random.tcc: weights normalised by their sum, running sums, last
 * one forced to 1.0, lower_bound on a canonical double built from two 32-bit
 * outputs; fewer than two weights draws nothing and returns index 0). */
int32_t lo_sample_ex(const float *row, int32_t v, float temp, uint32_t top_k, float top_p,
                     lo_mt19937 *g, int32_t *kept_out) {
  if (kept_out) *kept_out = 1;
  if (temp <= 0.0f || top_k == 1) return lo_greedy(row, v);
  if (!(top_p > 0.0f && top_p <= 1.0f)) return -1;
  cand_t *c = malloc(sizeof(cand_t) * (size_t)v);
  double *w = malloc(sizeof(double) * (size_t)v);
  const double inv_temp = 1.0 / (double)temp;
  for (int32_t i = 0; i < v; ++i) { c[i].id = i; c[i].x = (double)row[i] * inv_temp; }
  qsort(c, (size_t)v, sizeof(cand_t), cand_cmp);
  size_t n = (size_t)v;
  if (top_k > 0 && top_k < n) n = top_k;
  if (top_p < 1.0f) {
    const double mx = c[0].x;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) { w[i] = exp(c[i].x - mx); sum += w[i]; }
    double cum = 0.0;
    size_t keep = 0;
    for (; keep < n; ++keep) {
      cum += w[keep] / sum;
      if (cum >= (double)top_p) { ++keep; break; }
    }
    n = keep < 1 ? 1 : keep;
  }
  if (kept_out) *kept_out = (int32_t)n;
  int32_t result;
  if (n < 2) {
    result = c[0].id;
  } else {
    const double mx = c[0].x;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) { w[i] = exp(c[i].x - mx); sum += w[i]; }
    double run = 0.0;
    for (size_t i = 0; i < n; ++i) { run += w[i] / sum; w[i] = run; }
    w[n - 1] = 1.0;
    const double lo = (double)lo_mt_next(g);
    const double hi = (double)lo_mt_next(g);
    double p = (lo + hi * 4294967296.0) / 18446744073709551616.0;
    if (p >= 1.0) p = nextafter(1.0, 0.0);
    size_t a = 0, b = n; /* lower_bound: first i with w[i] >= p */
    while (a < b) {
      const size_t m = a + (b - a) / 2;
      if (w[m] < p) a = m + 1; else b = m;
    }
    result = c[a].id;
  }
  free(c);
  free(w);
  return result;
}

int32_t lo_sample(const float *row, int32_t v, float temp, uint32_t top_k, float top_p,
                  lo_mt19937 *g) {
  return lo_sample_ex(row, v, temp, top_k, top_p, g, 0);
}

/* inference.cpp:265-296: whole-context forward per token, guard
 * `step < max_new && ids.size() < max_seq_len`, one generator per generation. */
int32_t lo_generate(const lo_dims *d, const void *params, const int32_t *prompt,
                    int32_t prompt_len, int32_t max_new, float temp, uint32_t top_k,
                    float top_p, uint32_t seed, int32_t *out_ids, float *step_logits) {
  int32_t *ids = malloc(sizeof(int32_t) * (size_t)(d->max_seq + 1));
  float *row = malloc(sizeof(float) * (size_t)d->vocab);
  int32_t n = prompt_len;
  if (n == 0) { ids[0] = 0; n = 1; } else memcpy(ids, prompt, sizeof(int32_t) * (size_t)n);
  lo_mt19937 g;
  lo_mt_seed(&g, seed);
  int32_t made = 0;
  for (int32_t step = 0; step < max_new && n < d->max_seq; ++step) {
    if (lo_forward(d, params, ids, n, row, 1) != 0) { made = -1; break; }
    const int32_t next = lo_sample(row, d->vocab, temp, top_k, top_p, &g);
    if (step_logits) memcpy(step_logits + (int64_t)made * d->vocab, row, sizeof(float) * (size_t)d->vocab);
    ids[n++] = next;
    out_ids[made++] = next;
  }
  free(ids);
  free(row);
  return made;
}
