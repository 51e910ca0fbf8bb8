/* CPU oracle for whole decode steps, C restatement.  TEST INFRASTRUCTURE ONLY:
 * built and called by tests/, __graft_entry__.smoke() and bench.py's CPU legs
 * (cpu_baseline, --impl reference); nothing in the product path links or loads it.
 *
 * What each piece restates (reference = unnamedlambda/base):
 *   dense GEMV    the reference's CPU GEMV, lean/algorithms/RowDotBenchAlgorithm.lean:20-150:
 *                 four f32 lane accumulators, acc = acc + (x * w) (separate multiply and add),
 *                 horizontal (e0 + e1) + (e2 + e3), scalar tail; rows in pairs there, which
 *                 does not change a row's arithmetic.  The reference runs it on one thread;
 *                 `threads` > 1 splits ROWS over OpenMP threads (same per-row arithmetic).
 *   MX block dot  lean/lib/AlgorithmLib/ML/QuantMX.lean:56-74, 131-186 (left fold, as moe_oracle.c)
 *   RMSNorm       lean/algorithms/Qwen2Proven.lean:304-333  x * inv * w, inv = 1 / sqrt(mean + eps)
 *   RoPE          Qwen2Proven.lean:487-511 (half-split, two roundings), table built as
 *                 lean/algorithms/Qwen2Common.lean:522-560 (powf, sinf, cosf in f32)
 *   attention     lean/lib/AlgorithmLib/Cuda.lean:313-360 + softmax Qwen2Proven.lean:666-749:
 *                 scores = 0.125 K q, max shift, exp, normalise, P^T V; q heads share kv heads
 *   SiLU gate     Qwen2Proven.lean:71-81;  argmax = first index of the maximum, :926-972
 *   decode        one token per call [token, pos], Qwen2Common.lean:30, 830-864
 * Not in the reference (gpt-oss): sink logit in the softmax denominator, sliding window,
 * bf16 K/V rows, router bias, top-k softmax over the selected logits, clamped SwiGLU.  These
 * follow oracle/gptoss_oracle.py and oracle/moe_oracle.py, which are pinned against the
 * transformers package (tests/golden/); against the reference they are "parity unpinned".
 * This file is checked against those NumPy oracles in tests/test_oracle_model.py.
 *
 * Weights are the seeded synthetic tensors of base_b200/csrc/kernels/synth.cuh
 * (oracle/synth.py is the NumPy twin): pure 32-bit integer functions of (seed, tensor, index).
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off -fopenmp)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- synthetic tensors ------------------------------------------------------------------ */
static inline uint32_t synth_hash(uint32_t i, uint32_t tensor, uint32_t seed) {
  uint32_t h = i * 0x9E3779B1u + tensor * 0x85EBCA77u + seed * 0xC2B2AE3Du;
  h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
  return h;
}
static inline float synth_normal(uint32_t i, uint32_t tensor, uint32_t seed, float c) {
  const uint32_t a = synth_hash(2 * i, tensor, seed), b = synth_hash(2 * i + 1, tensor, seed);
  const int s = (int)((a & 255) + ((a >> 8) & 255) + ((a >> 16) & 255) + (a >> 24) + (b & 255) + ((b >> 8) & 255) +
                      ((b >> 16) & 255) + (b >> 24)) - 1020;
  return (float)s * c;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static inline float bf16_to_f32(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t tid_of(uint32_t layer, uint32_t kind) { return layer * 32u + kind; }
static float sigma_c(double sigma) { return (float)(sigma / 209.0232); }

static uint8_t *gen_bytes(size_t n, uint32_t tensor, uint32_t seed) {
  uint8_t *p = (uint8_t *)malloc(n ? n : 1);
  if (!p) return NULL;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) p[i] = (uint8_t)(synth_hash((uint32_t)i >> 2, tensor, seed) >> (8 * ((uint32_t)i & 3)));
  return p;
}
static uint8_t *gen_scales(size_t n, uint32_t tensor, uint32_t seed, int lo, int span) {
  uint8_t *p = (uint8_t *)malloc(n ? n : 1);
  if (!p) return NULL;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) p[i] = (uint8_t)(lo + synth_hash((uint32_t)i, tensor, seed) % (uint32_t)span);
  return p;
}
static float *gen_normal(size_t n, uint32_t tensor, uint32_t seed, double sigma, int one_plus) {
  float *p = (float *)malloc((n ? n : 1) * sizeof(float));
  const float c = sigma_c(sigma);
  if (!p) return NULL;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) {
    const float v = synth_normal((uint32_t)i, tensor, seed, c);
    p[i] = one_plus ? 1.0f + v : v;
  }
  return p;
}
static uint16_t *gen_normal_bf16(size_t n, uint32_t tensor, uint32_t seed, double sigma) {
  uint16_t *p = (uint16_t *)malloc((n ? n : 1) * sizeof(uint16_t));
  const float c = sigma_c(sigma);
  if (!p) return NULL;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) p[i] = f32_to_bf16(synth_normal((uint32_t)i, tensor, seed, c));
  return p;
}

/* ---- arithmetic --------------------------------------------------------------------------- */
/* RowDotBenchAlgorithm.lean:86-99 (SIMD body), :101-107 (horizontal), :109-121 (scalar tail) */
static float rowdot_f32(const float *w, const float *x, int K) {
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  int j = 0;
  for (; j + 4 <= K; j += 4) {
    a0 = a0 + x[j] * w[j];
    a1 = a1 + x[j + 1] * w[j + 1];
    a2 = a2 + x[j + 2] * w[j + 2];
    a3 = a3 + x[j + 3] * w[j + 3];
  }
  float s = (a0 + a1) + (a2 + a3);
  for (; j < K; ++j) s = s + x[j] * w[j];
  return s;
}
/* the same with bf16 weights (widened exactly) */
static float rowdot_bf16(const uint16_t *w, const float *x, int K) {
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  int j = 0;
  for (; j + 4 <= K; j += 4) {
    a0 = a0 + x[j] * bf16_to_f32(w[j]);
    a1 = a1 + x[j + 1] * bf16_to_f32(w[j + 1]);
    a2 = a2 + x[j + 2] * bf16_to_f32(w[j + 2]);
    a3 = a3 + x[j + 3] * bf16_to_f32(w[j + 3]);
  }
  float s = (a0 + a1) + (a2 + a3);
  for (; j < K; ++j) s = s + x[j] * bf16_to_f32(w[j]);
  return s;
}
static void gemv_f32(const float *W, const float *x, const float *bias, float *y, int rows, int K) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) y[r] = rowdot_f32(W + (size_t)r * K, x, K) + (bias ? bias[r] : 0.0f);
}
static void gemv_bf16(const uint16_t *W, const float *x, const float *bias, float *y, int rows, int K) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) y[r] = rowdot_bf16(W + (size_t)r * K, x, K) + (bias ? bias[r] : 0.0f);
}
/* Exposed for the bit-exact check of the fold above (tests) and for timing the GEMV alone. */
void oracle_rowdot_gemv_f32(const float *W, const float *x, float *y, int rows, int K, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  gemv_f32(W, x, NULL, y, rows, K);
}

/* The reference's committed GPU fold, its own CPU image (applications/warp-check/src/lib.rs:28-116: `butterfly`,
 * `Walk::idx`, `dot_by`): 32 lane accumulators walk the row (walk 0 vec4, 1 strided, 2 blocked), acc += a * b with
 * separate multiply and add, then five xor rounds lane[l] = prev[l] + prev[l ^ m], m = 16, 8, 4, 2, 1, read at lane 0. */
void oracle_warp_fold_gemv(const float *W, const float *x, float *y, int rows, int n, int walk) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float *w = W + (size_t)r * n;
    float lane[32], prev[32];
    const int trips = walk == 0 ? n / 128 : n / 32, width = walk == 0 ? 4 : 1;
    for (int l = 0; l < 32; ++l) {
      float acc = 0.0f;
      for (int t = 0; t < trips; ++t) {
        const int o = walk == 0 ? t * 128 + l * 4 : walk == 1 ? t * 32 + l : l * (n / 32) + t;
        for (int q = 0; q < width; ++q) acc = acc + w[o + q] * x[o + q];
      }
      lane[l] = acc;
    }
    for (int m = 16; m > 0; m >>= 1) {
      memcpy(prev, lane, sizeof(lane));
      for (int l = 0; l < 32; ++l) lane[l] = prev[l] + prev[l ^ m];
    }
    y[r] = lane[0];
  }
}

static void rms_norm(const float *g, const float *x, float *y, int n, float eps) {
  float ss = 0.0f;
  for (int i = 0; i < n; ++i) ss = ss + x[i] * x[i];
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * inv * g[i];
}
static float *rope_table(float theta, int max_seq) {
  float *t = (float *)malloc((size_t)2 * max_seq * 32 * sizeof(float));
  if (!t) return NULL;
  for (int p = 0; p < max_seq; ++p)
    for (int i = 0; i < 32; ++i) {
      const float inv = powf(theta, -((float)i / 32.0f));
      const float ang = (float)p * inv;
      t[(size_t)p * 32 + i] = sinf(ang);
      t[(size_t)max_seq * 32 + (size_t)p * 32 + i] = cosf(ang);
    }
  return t;
}
static void rope_row(float *v, const float *sn, const float *cs) {
  for (int i = 0; i < 32; ++i) {
    const float lo = v[i], hi = v[i + 32];
    v[i] = lo * cs[i] - hi * sn[i];
    v[i + 32] = lo * sn[i] + hi * cs[i];
  }
}
/* One q head over positions [lo, pos] of its kv head's cache (ring of cache_len rows). */
static void attend(const float *q, const float *kc, const float *vc, int cache_len, int lo, int pos, const float *sink,
                   float *scores, float *out) {
  float m = sink ? *sink : -INFINITY;
  for (int p = lo; p <= pos; ++p) {
    const float *k = kc + (size_t)(p % cache_len) * 64;
    float s = 0.0f;
    for (int d = 0; d < 64; ++d) s = s + k[d] * q[d];
    scores[p - lo] = s;
    if (s > m) m = s;
  }
  float den = sink ? expf(*sink - m) : 0.0f;
  for (int p = lo; p <= pos; ++p) { scores[p - lo] = expf(scores[p - lo] - m); den = den + scores[p - lo]; }
  for (int d = 0; d < 64; ++d) out[d] = 0.0f;
  for (int p = lo; p <= pos; ++p) {
    const float w = scores[p - lo] / den;
    const float *v = vc + (size_t)(p % cache_len) * 64;
    for (int d = 0; d < 64; ++d) out[d] = out[d] + w * v[d];
  }
}
static int argmax_first(const float *v, int n) {
  int best = 0;
  for (int i = 1; i < n; ++i)
    if (v[i] > v[best]) best = i;
  return best;
}

/* from moe_oracle.c */
int oracle_moe_ffn(const float *x, int T, int H, int I, int E, int k, float alpha, float limit, const float *Wr,
                   const float *br, const uint8_t *gu_codes, const uint8_t *gu_scales, const float *gu_bias,
                   const uint8_t *dn_codes, const uint8_t *dn_scales, const float *dn_bias, float *y, int32_t *idx_out,
                   float *w_out, int threads);

/* ---- gpt-oss ------------------------------------------------------------------------------ */
enum { kLn1 = 0, kWqkv, kBqkv, kSinks, kWo, kBo, kLn2, kWr, kBr, kGuCodes, kGuScales, kGuBias, kDnCodes, kDnScales,
       kDnBias, kEmbed = 16, kLmHead, kLnF, kKCache, kVCache };

typedef struct {
  float *ln1, *bqkv, *sinks, *bo, *ln2, *wr, *br, *gu_bias, *dn_bias;
  uint16_t *wqkv, *wo;
  uint8_t *gu_codes, *gu_scales, *dn_codes, *dn_scales;
  float *kc, *vc;          /* [n_kv][cache_len][64], values are bf16-representable */
  int cache_len, window;
} GLayer;

typedef struct {
  int layers, H, I, E, k, NQ, NKV, V, window, max_seq;
  float theta, eps, alpha, limit;
  uint32_t seed;
  uint16_t *embed, *lm_head;
  float *lnf, *rope;
  GLayer *ly;
  float *x, *xn, *qkv, *att, *h, *y, *scores, *logits;
  int32_t last_idx[8 * 128];     /* top-k of the last step, per layer */
  double t_dense, t_attn, t_moe, t_head;
} GptOss;

static double now_s(void) {
#ifdef _OPENMP
  return omp_get_wtime();
#else
  return 0.0;
#endif
}

void oracle_gptoss_free(GptOss *m) {
  if (!m) return;
  if (m->ly)
    for (int l = 0; l < m->layers; ++l) {
      GLayer *y = &m->ly[l];
      free(y->ln1); free(y->bqkv); free(y->sinks); free(y->bo); free(y->ln2); free(y->wr); free(y->br);
      free(y->gu_bias); free(y->dn_bias); free(y->wqkv); free(y->wo); free(y->gu_codes); free(y->gu_scales);
      free(y->dn_codes); free(y->dn_scales); free(y->kc); free(y->vc);
    }
  free(m->ly); free(m->embed); free(m->lm_head); free(m->lnf); free(m->rope);
  free(m->x); free(m->xn); free(m->qkv); free(m->att); free(m->h); free(m->y); free(m->scores); free(m->logits);
  free(m);
}

/* ints: layers, hidden, inter, experts, top_k, n_q, n_kv, vocab, window, max_seq; floats: theta, eps, alpha, limit.
 * Sliding layers are the even layers, as in the stage program.  Returns NULL when memory runs out. */
GptOss *oracle_gptoss_new(const int32_t *ci, const float *cf, uint32_t seed, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  GptOss *m = (GptOss *)calloc(1, sizeof(GptOss));
  if (!m) return NULL;
  m->layers = ci[0]; m->H = ci[1]; m->I = ci[2]; m->E = ci[3]; m->k = ci[4]; m->NQ = ci[5]; m->NKV = ci[6];
  m->V = ci[7]; m->window = ci[8]; m->max_seq = ci[9];
  m->theta = cf[0]; m->eps = cf[1]; m->alpha = cf[2]; m->limit = cf[3];
  m->seed = seed;
  if (m->k > 8 || m->layers > 128 || m->E > 128) { free(m); return NULL; }
  const size_t H = m->H, I = m->I, E = m->E, V = m->V;
  const size_t QD = (size_t)m->NQ * 64, KVD = (size_t)m->NKV * 64, QKV = QD + 2 * KVD;
  const uint32_t G = 1000;
  int ok = 1;
  m->embed = gen_normal_bf16(V * H, tid_of(G, kEmbed), seed, 0.02);
  m->lm_head = gen_normal_bf16(V * H, tid_of(G, kLmHead), seed, 0.02);
  m->lnf = gen_normal(H, tid_of(G, kLnF), seed, 0.02, 1);
  m->rope = rope_table(m->theta, m->max_seq);
  m->ly = (GLayer *)calloc((size_t)m->layers, sizeof(GLayer));
  ok = m->embed && m->lm_head && m->lnf && m->rope && m->ly;
  for (int l = 0; l < m->layers && ok; ++l) {
    GLayer *y = &m->ly[l];
    const uint32_t L = (uint32_t)l;
    y->window = (l % 2 == 0) ? m->window : 0;
    y->cache_len = y->window > 0 ? (y->window < m->max_seq ? y->window : m->max_seq) : m->max_seq;
    y->ln1 = gen_normal(H, tid_of(L, kLn1), seed, 0.02, 1);
    y->wqkv = gen_normal_bf16(QKV * H, tid_of(L, kWqkv), seed, 0.02);
    y->bqkv = gen_normal(QKV, tid_of(L, kBqkv), seed, 0.02, 0);
    y->sinks = gen_normal((size_t)m->NQ, tid_of(L, kSinks), seed, 1.0, 0);
    y->wo = gen_normal_bf16(H * QD, tid_of(L, kWo), seed, 0.02);
    y->bo = gen_normal(H, tid_of(L, kBo), seed, 0.02, 0);
    y->ln2 = gen_normal(H, tid_of(L, kLn2), seed, 0.02, 1);
    y->wr = gen_normal(E * H, tid_of(L, kWr), seed, 0.02, 0);
    y->br = gen_normal(E, tid_of(L, kBr), seed, 0.01, 0);
    y->gu_codes = gen_bytes(E * 2 * I * (H / 2), tid_of(L, kGuCodes), seed);
    y->gu_scales = gen_scales(E * 2 * I * (H / 32), tid_of(L, kGuScales), seed, 117, 7);
    y->gu_bias = gen_normal(E * 2 * I, tid_of(L, kGuBias), seed, 0.01, 0);
    y->dn_codes = gen_bytes(E * H * (I / 2), tid_of(L, kDnCodes), seed);
    y->dn_scales = gen_scales(E * H * (I / 32), tid_of(L, kDnScales), seed, 117, 7);
    y->dn_bias = gen_normal(E * H, tid_of(L, kDnBias), seed, 0.01, 0);
    y->kc = (float *)calloc(KVD * (size_t)y->cache_len, sizeof(float));
    y->vc = (float *)calloc(KVD * (size_t)y->cache_len, sizeof(float));
    ok = y->ln1 && y->wqkv && y->bqkv && y->sinks && y->wo && y->bo && y->ln2 && y->wr && y->br && y->gu_codes &&
         y->gu_scales && y->gu_bias && y->dn_codes && y->dn_scales && y->dn_bias && y->kc && y->vc;
  }
  m->x = (float *)malloc(H * 4); m->xn = (float *)malloc(H * 4); m->qkv = (float *)malloc(QKV * 4);
  m->att = (float *)malloc(QD * 4); m->h = (float *)malloc(H * 4); m->y = (float *)malloc(H * 4);
  m->scores = (float *)malloc((size_t)m->NQ * (size_t)m->max_seq * 4); m->logits = (float *)malloc(V * 4);
  ok = ok && m->x && m->xn && m->qkv && m->att && m->h && m->y && m->scores && m->logits;
  if (!ok) { oracle_gptoss_free(m); return NULL; }
  return m;
}

/* The synthetic cache the stage program's `fillKV` extra writes: every K and V row of sequence `seq` of
 * `batch` is bf16 N(0, 1) from (seed, layer * 32 + 19 / 20, index in [batch][n_kv][cache_len][64]). */
void oracle_gptoss_fill_kv(GptOss *m, int seq, int batch) {
  (void)batch;
  const float c = sigma_c(1.0);
  for (int l = 0; l < m->layers; ++l) {
    GLayer *y = &m->ly[l];
    const size_t n = (size_t)m->NKV * y->cache_len * 64, base = (size_t)seq * n;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
      y->kc[i] = bf16_to_f32(f32_to_bf16(synth_normal((uint32_t)(base + i), tid_of((uint32_t)l, kKCache), m->seed, c)));
      y->vc[i] = bf16_to_f32(f32_to_bf16(synth_normal((uint32_t)(base + i), tid_of((uint32_t)l, kVCache), m->seed, c)));
    }
  }
}

/* One decode step of one sequence; positions must come in order (or after oracle_gptoss_fill_kv).
 * logits_out may be null.  Returns the greedy token, or -1. */
int oracle_gptoss_step(GptOss *m, int token, int pos, float *logits_out, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  if (!m || token < 0 || token >= m->V || pos < 0 || pos >= m->max_seq) return -1;
  const int H = m->H, NQ = m->NQ, NKV = m->NKV, QD = NQ * 64, KVD = NKV * 64, QKV = QD + 2 * KVD, Gq = NQ / NKV;
  for (int i = 0; i < H; ++i) m->x[i] = bf16_to_f32(m->embed[(size_t)token * H + i]);
  const float *sn = m->rope + (size_t)pos * 32, *cs = m->rope + (size_t)m->max_seq * 32 + (size_t)pos * 32;
  for (int l = 0; l < m->layers; ++l) {
    GLayer *y = &m->ly[l];
    double t0 = now_s();
    rms_norm(y->ln1, m->x, m->xn, H, m->eps);
    gemv_bf16(y->wqkv, m->xn, y->bqkv, m->qkv, QKV, H);
    double t1 = now_s();
    m->t_dense += t1 - t0;
    for (int h = 0; h < NQ; ++h) {
      rope_row(m->qkv + h * 64, sn, cs);
      for (int d = 0; d < 64; ++d) m->qkv[h * 64 + d] = m->qkv[h * 64 + d] * 0.125f;
    }
    const int slot = pos % y->cache_len;
    for (int h = 0; h < NKV; ++h) {
      float *kr = m->qkv + QD + h * 64, *vr = m->qkv + QD + KVD + h * 64;
      rope_row(kr, sn, cs);
      for (int d = 0; d < 64; ++d) {
        y->kc[((size_t)h * y->cache_len + slot) * 64 + d] = bf16_to_f32(f32_to_bf16(kr[d]));
        y->vc[((size_t)h * y->cache_len + slot) * 64 + d] = bf16_to_f32(f32_to_bf16(vr[d]));
      }
    }
    const int lo = y->window > 0 ? (pos + 1 - y->window > 0 ? pos + 1 - y->window : 0) : 0;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < NQ; ++h)
      attend(m->qkv + h * 64, y->kc + (size_t)(h / Gq) * y->cache_len * 64, y->vc + (size_t)(h / Gq) * y->cache_len * 64,
             y->cache_len, lo, pos, &y->sinks[h], m->scores + (size_t)h * m->max_seq, m->att + h * 64);
    double t2 = now_s();
    m->t_attn += t2 - t1;
    gemv_bf16(y->wo, m->att, y->bo, m->h, H, QD);
    for (int i = 0; i < H; ++i) m->h[i] = m->x[i] + m->h[i];
    rms_norm(y->ln2, m->h, m->xn, H, m->eps);
    double t3 = now_s();
    m->t_dense += t3 - t2;
    float wts[8];
    if (oracle_moe_ffn(m->xn, 1, H, m->I, m->E, m->k, m->alpha, m->limit, y->wr, y->br, y->gu_codes, y->gu_scales,
                       y->gu_bias, y->dn_codes, y->dn_scales, y->dn_bias, m->y, m->last_idx + 8 * l, wts, 0) != 0)
      return -1;
    for (int i = 0; i < H; ++i) m->x[i] = m->h[i] + m->y[i];
    m->t_moe += now_s() - t3;
  }
  double t4 = now_s();
  rms_norm(m->lnf, m->x, m->xn, H, m->eps);
  gemv_bf16(m->lm_head, m->xn, NULL, m->logits, m->V, H);
  const int nxt = argmax_first(m->logits, m->V);
  m->t_head += now_s() - t4;
  if (logits_out) memcpy(logits_out, m->logits, (size_t)m->V * 4);
  return nxt;
}

/* out[0..3] = seconds spent so far in dense GEMVs (qkv, o-proj), attention, the MoE FFN, final norm + lm_head + argmax;
 * out[4 .. 4 + layers * 8) = the experts chosen in the last step as floats (top-k order, 8 per layer). */
void oracle_gptoss_stats(const GptOss *m, double *out) {
  out[0] = m->t_dense; out[1] = m->t_attn; out[2] = m->t_moe; out[3] = m->t_head;
  for (int i = 0; i < m->layers * 8; ++i) out[4 + i] = (double)m->last_idx[i];
}

/* ---- Qwen2 (f32 weights and cache, no sinks, no window; tied lm_head) ------------------------- */
typedef struct {
  float *ln1, *wqkv, *bqkv, *wo, *ln2, *wgu, *wdn, *kc, *vc;
} QLayer;
typedef struct {
  int layers, H, F, NQ, NKV, V, max_seq;
  float theta, eps;
  float *embed, *lnf, *rope;
  QLayer *ly;
  float *x, *xn, *qkv, *att, *h, *gu, *scores, *logits;
} Qwen2;

void oracle_qwen2_free(Qwen2 *m) {
  if (!m) return;
  if (m->ly)
    for (int l = 0; l < m->layers; ++l) {
      QLayer *y = &m->ly[l];
      free(y->ln1); free(y->wqkv); free(y->bqkv); free(y->wo); free(y->ln2); free(y->wgu); free(y->wdn); free(y->kc); free(y->vc);
    }
  free(m->ly); free(m->embed); free(m->lnf); free(m->rope);
  free(m->x); free(m->xn); free(m->qkv); free(m->att); free(m->h); free(m->gu); free(m->scores); free(m->logits);
  free(m);
}

/* ints: layers, hidden, inter, n_q, n_kv, vocab, max_seq; floats: theta, eps.  Tensor kinds as oracle/qwen2_oracle.py. */
Qwen2 *oracle_qwen2_new(const int32_t *ci, const float *cf, uint32_t seed, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  Qwen2 *m = (Qwen2 *)calloc(1, sizeof(Qwen2));
  if (!m) return NULL;
  m->layers = ci[0]; m->H = ci[1]; m->F = ci[2]; m->NQ = ci[3]; m->NKV = ci[4]; m->V = ci[5]; m->max_seq = ci[6];
  m->theta = cf[0]; m->eps = cf[1];
  const size_t H = m->H, F = m->F, V = m->V, QD = (size_t)m->NQ * 64, KVD = (size_t)m->NKV * 64, QKV = QD + 2 * KVD;
  m->embed = gen_normal(V * H, tid_of(1000, 16), seed, 0.02, 0);
  m->lnf = gen_normal(H, tid_of(1000, 17), seed, 0.02, 1);
  m->rope = rope_table(m->theta, m->max_seq);
  m->ly = (QLayer *)calloc((size_t)m->layers, sizeof(QLayer));
  int ok = m->embed && m->lnf && m->rope && m->ly;
  for (int l = 0; l < m->layers && ok; ++l) {
    QLayer *y = &m->ly[l];
    const uint32_t L = (uint32_t)l;
    y->ln1 = gen_normal(H, tid_of(L, 0), seed, 0.02, 1);
    y->wqkv = gen_normal(QKV * H, tid_of(L, 1), seed, 0.02, 0);
    y->bqkv = gen_normal(QKV, tid_of(L, 2), seed, 0.02, 0);
    y->wo = gen_normal(H * QD, tid_of(L, 3), seed, 0.02, 0);
    y->ln2 = gen_normal(H, tid_of(L, 4), seed, 0.02, 1);
    y->wgu = gen_normal(2 * F * H, tid_of(L, 5), seed, 0.02, 0);
    y->wdn = gen_normal(H * F, tid_of(L, 6), seed, 0.02, 0);
    y->kc = (float *)calloc(KVD * (size_t)m->max_seq, sizeof(float));
    y->vc = (float *)calloc(KVD * (size_t)m->max_seq, sizeof(float));
    ok = y->ln1 && y->wqkv && y->bqkv && y->wo && y->ln2 && y->wgu && y->wdn && y->kc && y->vc;
  }
  m->x = (float *)malloc(H * 4); m->xn = (float *)malloc(H * 4); m->qkv = (float *)malloc(QKV * 4);
  m->att = (float *)malloc(QD * 4); m->h = (float *)malloc(H * 4); m->gu = (float *)malloc(2 * F * 4);
  m->scores = (float *)malloc((size_t)m->NQ * (size_t)m->max_seq * 4); m->logits = (float *)malloc(V * 4);
  ok = ok && m->x && m->xn && m->qkv && m->att && m->h && m->gu && m->scores && m->logits;
  if (!ok) { oracle_qwen2_free(m); return NULL; }
  return m;
}

int oracle_qwen2_step(Qwen2 *m, int token, int pos, float *logits_out, int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  if (!m || token < 0 || token >= m->V || pos < 0 || pos >= m->max_seq) return -1;
  const int H = m->H, F = m->F, NQ = m->NQ, NKV = m->NKV, QD = NQ * 64, KVD = NKV * 64, QKV = QD + 2 * KVD, Gq = NQ / NKV;
  memcpy(m->x, m->embed + (size_t)token * H, (size_t)H * 4);
  const float *sn = m->rope + (size_t)pos * 32, *cs = m->rope + (size_t)m->max_seq * 32 + (size_t)pos * 32;
  for (int l = 0; l < m->layers; ++l) {
    QLayer *y = &m->ly[l];
    rms_norm(y->ln1, m->x, m->xn, H, m->eps);
    gemv_f32(y->wqkv, m->xn, y->bqkv, m->qkv, QKV, H);
    for (int h = 0; h < NQ; ++h) {
      rope_row(m->qkv + h * 64, sn, cs);
      for (int d = 0; d < 64; ++d) m->qkv[h * 64 + d] = m->qkv[h * 64 + d] * 0.125f;
    }
    for (int h = 0; h < NKV; ++h) {
      float *kr = m->qkv + QD + h * 64, *vr = m->qkv + QD + KVD + h * 64;
      rope_row(kr, sn, cs);
      memcpy(y->kc + ((size_t)h * m->max_seq + pos) * 64, kr, 256);
      memcpy(y->vc + ((size_t)h * m->max_seq + pos) * 64, vr, 256);
    }
#pragma omp parallel for schedule(static)
    for (int h = 0; h < NQ; ++h)
      attend(m->qkv + h * 64, y->kc + (size_t)(h / Gq) * m->max_seq * 64, y->vc + (size_t)(h / Gq) * m->max_seq * 64,
             m->max_seq, 0, pos, NULL, m->scores + (size_t)h * m->max_seq, m->att + h * 64);
    gemv_f32(y->wo, m->att, NULL, m->h, H, QD);
    for (int i = 0; i < H; ++i) m->h[i] = m->x[i] + m->h[i];
    rms_norm(y->ln2, m->h, m->xn, H, m->eps);
    gemv_f32(y->wgu, m->xn, NULL, m->gu, 2 * F, H);
    for (int i = 0; i < F; ++i) m->gu[i] = (m->gu[i] / (1.0f + expf(-m->gu[i]))) * m->gu[F + i];
    gemv_f32(y->wdn, m->gu, NULL, m->xn, H, F);
    for (int i = 0; i < H; ++i) m->x[i] = m->h[i] + m->xn[i];
  }
  rms_norm(m->lnf, m->x, m->xn, H, m->eps);
  gemv_f32(m->embed, m->xn, NULL, m->logits, m->V, H);
  if (logits_out) memcpy(logits_out, m->logits, (size_t)m->V * 4);
  return argmax_first(m->logits, m->V);
}
