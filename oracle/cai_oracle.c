/*
 * cai_oracle.c - C restatement of the reference's CPU decode path (TEST
 * INFRASTRUCTURE and the timed CPU baseline; never linked into the product).
 *
 * What it restates (paths relative to the reference project root):
 *   int8-code x fp32 dot product with 4 independent 8-lane FMA accumulators over
 *   32-element strips        neural/neuralvolume.pas:1780-1882 (AVXDotProductInt8),
 *                            :12693-12745 (DotProductsTiledInt8: one dot per output row)
 *   Q8_0 / Q4_0 block rules  neural/neuralgguf.pas:1487-1503, 811-845 (x = d*q, x = d*(nib-8));
 *                            the block scale is applied once per 32-block after the raw sum
 *   fp16 decode              neural/neuralvolume.pas:1737-1770
 *   RMSNorm, RoPE, SwiGLU, KV append, decode attention
 *                            neural/neural.cl:1047-1085, 1517-1542, 1213-1263, 2354-2379, 2406-2499
 *   graph order, fused up|gate packing, tied head
 *                            neural/neuralpretrained.pas:16423-16875, 17412-17421, 15655-15671
 * Dense Llama-family models only (the MoE branch is covered by the numpy oracle).
 * Rows are split over OpenMP threads the way the reference's thread pool chunks
 * output neurons (neural/neuralthread.pas:58-110).
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -fopenmp -shared -fPIC).
 */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK 32
enum { CO_F32 = 0, CO_F16 = 1, CO_Q4_0 = 2, CO_Q8_0 = 8 };

static float half_to_float(uint16_t h) {
  const uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
  uint32_t bits;
  float f;
  if (exp == 0) {
    if (man == 0) { bits = sign << 31; memcpy(&f, &bits, 4); return f; }
    f = (float)man * 5.9604644775390625e-8f;
    return sign ? -f : f;
  }
  if (exp == 0x1F) bits = (sign << 31) | (0xFFu << 23) | (man << 13);
  else bits = (sign << 31) | ((exp + 112) << 23) | (man << 13);
  memcpy(&f, &bits, 4);
  return f;
}

static inline float hsum8(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  lo = _mm_hadd_ps(lo, lo);
  lo = _mm_hadd_ps(lo, lo);
  return _mm_cvtss_f32(lo);
}

/* one Q8_0 row (k/32 blocks of 34 bytes) dot x */
static float dot_q8_0(const uint8_t* row, const float* x, int64_t k) {
  __m256 total = _mm256_setzero_ps();
  for (int64_t b = 0; b < k / QK; ++b) {
    const uint8_t* blk = row + b * 34;
    uint16_t hs;
    memcpy(&hs, blk, 2);
    const float d = half_to_float(hs);
    const int8_t* q = (const int8_t*)(blk + 2);
    const float* xb = x + b * QK;
    __m256 a0 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(q)))), _mm256_loadu_ps(xb));
    __m256 a1 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(q + 8)))), _mm256_loadu_ps(xb + 8));
    __m256 a2 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(q + 16)))), _mm256_loadu_ps(xb + 16));
    __m256 a3 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(q + 24)))), _mm256_loadu_ps(xb + 24));
    const __m256 s = _mm256_add_ps(_mm256_add_ps(a0, a1), _mm256_add_ps(a2, a3));
    total = _mm256_fmadd_ps(_mm256_set1_ps(d), s, total);
  }
  return hsum8(total);
}

/* one Q4_0 row (k/32 blocks of 18 bytes) dot x; byte e: low nibble = element e, high = element e+16 */
static float dot_q4_0(const uint8_t* row, const float* x, int64_t k) {
  __m256 total = _mm256_setzero_ps();
  const __m128i mask = _mm_set1_epi8(0x0F);
  const __m256i eight = _mm256_set1_epi32(8);
  for (int64_t b = 0; b < k / QK; ++b) {
    const uint8_t* blk = row + b * 18;
    uint16_t hs;
    memcpy(&hs, blk, 2);
    const float d = half_to_float(hs);
    const __m128i raw = _mm_loadu_si128((const __m128i*)(blk + 2));
    const __m128i lo = _mm_and_si128(raw, mask);
    const __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), mask);
    const float* xb = x + b * QK;
    __m256 a0 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(lo), eight)), _mm256_loadu_ps(xb));
    __m256 a1 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(lo, 8)), eight)), _mm256_loadu_ps(xb + 8));
    __m256 a2 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(hi), eight)), _mm256_loadu_ps(xb + 16));
    __m256 a3 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(hi, 8)), eight)), _mm256_loadu_ps(xb + 24));
    const __m256 s = _mm256_add_ps(_mm256_add_ps(a0, a1), _mm256_add_ps(a2, a3));
    total = _mm256_fmadd_ps(_mm256_set1_ps(d), s, total);
  }
  return hsum8(total);
}

static float dot_f32(const float* w, const float* x, int64_t k) {
  __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
  int64_t i = 0;
  for (; i + 32 <= k; i += 32) {
    a0 = _mm256_fmadd_ps(_mm256_loadu_ps(w + i), _mm256_loadu_ps(x + i), a0);
    a1 = _mm256_fmadd_ps(_mm256_loadu_ps(w + i + 8), _mm256_loadu_ps(x + i + 8), a1);
    a2 = _mm256_fmadd_ps(_mm256_loadu_ps(w + i + 16), _mm256_loadu_ps(x + i + 16), a2);
    a3 = _mm256_fmadd_ps(_mm256_loadu_ps(w + i + 24), _mm256_loadu_ps(x + i + 24), a3);
  }
  float s = hsum8(_mm256_add_ps(_mm256_add_ps(a0, a1), _mm256_add_ps(a2, a3)));
  for (; i < k; ++i) s += w[i] * x[i];
  return s;
}

static size_t row_bytes(int type, int64_t k) {
  switch (type) {
    case CO_Q8_0: return (size_t)(k / QK) * 34;
    case CO_Q4_0: return (size_t)(k / QK) * 18;
    case CO_F16: return (size_t)k * 2;
    default: return (size_t)k * 4;
  }
}

/* y[b*n + a] = W[a] . x[b] (+ bias[a]) for GGUF rows of `type` */
void co_gemv(int type, const void* blocks, int64_t n, int64_t k, const float* x, int batch, const float* bias, float* y) {
  const size_t rb = row_bytes(type, k);
#pragma omp parallel for schedule(static)
  for (int64_t a = 0; a < n; ++a) {
    const uint8_t* row = (const uint8_t*)blocks + (size_t)a * rb;
    for (int b = 0; b < batch; ++b) {
      const float* xb = x + (size_t)b * k;
      float s;
      if (type == CO_Q8_0) s = dot_q8_0(row, xb, k);
      else if (type == CO_Q4_0) s = dot_q4_0(row, xb, k);
      else if (type == CO_F32) s = dot_f32((const float*)row, xb, k);
      else {
        s = 0.f;
        for (int64_t i = 0; i < k; ++i) { uint16_t h; memcpy(&h, row + 2 * i, 2); s += half_to_float(h) * xb[i]; }
      }
      y[(size_t)b * n + a] = s + (bias ? bias[a] : 0.f);
    }
  }
}

void co_dequantize(int type, const void* blocks, int64_t n_elems, float* out) {
  const uint8_t* p = (const uint8_t*)blocks;
  if (type == CO_Q8_0) {
    for (int64_t b = 0; b < n_elems / QK; ++b) {
      uint16_t hs; memcpy(&hs, p + b * 34, 2);
      const float d = half_to_float(hs);
      const int8_t* q = (const int8_t*)(p + b * 34 + 2);
      for (int i = 0; i < QK; ++i) out[b * QK + i] = d * (float)q[i];
    }
  } else if (type == CO_Q4_0) {
    for (int64_t b = 0; b < n_elems / QK; ++b) {
      uint16_t hs; memcpy(&hs, p + b * 18, 2);
      const float d = half_to_float(hs);
      const uint8_t* q = p + b * 18 + 2;
      for (int e = 0; e < QK; ++e) {
        const int nib = (e < 16) ? (q[e] & 0x0F) : ((q[e - 16] >> 4) & 0x0F);
        out[b * QK + e] = d * (float)(nib - 8);
      }
    }
  } else if (type == CO_F16) {
    for (int64_t i = 0; i < n_elems; ++i) { uint16_t h; memcpy(&h, p + 2 * i, 2); out[i] = half_to_float(h); }
  } else {
    memcpy(out, blocks, (size_t)n_elems * 4);
  }
}

/* ------------------------------------------------------------------------ */
/* dense Llama-family model, weights referenced (not copied) in GGUF rows,   */
/* q/k rows already in the in-net interleaved order                          */
/* ------------------------------------------------------------------------ */
typedef struct {
  int32_t hidden, inter, layers, heads, kv_heads, head_dim, vocab;
  float rms_eps, rope_theta;
  int32_t tie_embeddings, qkv_bias;
} co_config;

typedef struct {
  const float *attn_norm, *ffn_norm, *bq, *bk, *bv;
  const void *wq, *wk, *wv, *wo, *wup, *wgate, *wdown;
  int tq, tk, tv, to, tup, tgate, tdown;
} co_layer;

typedef struct {
  co_config cfg;
  co_layer* layers;
  const void* embed; int t_embed;
  const void* head; int t_head;
  const float* final_norm;
  float* theta;
} co_model;

typedef struct {
  co_model* m;
  int max_ctx, len;
  float *k, *v;           /* [layers][kv_heads][max_ctx][hd] */
  float *x, *h, *q, *kk, *vv, *att, *fused, *act, *tmp, *scores;
} co_session;

co_model* co_model_create(const co_config* cfg) {
  co_model* m = (co_model*)calloc(1, sizeof(co_model));
  m->cfg = *cfg;
  m->layers = (co_layer*)calloc((size_t)cfg->layers, sizeof(co_layer));
  m->theta = (float*)malloc(sizeof(float) * (size_t)(cfg->head_dim / 2));
  for (int k = 0; k < cfg->head_dim / 2; ++k)
    m->theta[k] = (float)exp(-2.0 * (double)k / (double)cfg->head_dim * log((double)cfg->rope_theta));
  return m;
}
void co_model_destroy(co_model* m) { if (m) { free(m->layers); free(m->theta); free(m); } }

/* kind: 0 embed 1 head 2 final_norm 3 attn_norm 4 ffn_norm 5 q 6 k 7 v 8 o 9 up 10 gate 11 down 12 bq 13 bk 14 bv */
int co_model_set_tensor(co_model* m, int kind, int layer, int type, const void* data) {
  if (kind >= 3 && (layer < 0 || layer >= m->cfg.layers)) return 1;
  co_layer* L = (kind >= 3) ? &m->layers[layer] : NULL;
  switch (kind) {
    case 0: m->embed = data; m->t_embed = type; if (m->cfg.tie_embeddings) { m->head = data; m->t_head = type; } break;
    case 1: m->head = data; m->t_head = type; break;
    case 2: m->final_norm = (const float*)data; break;
    case 3: L->attn_norm = (const float*)data; break;
    case 4: L->ffn_norm = (const float*)data; break;
    case 5: L->wq = data; L->tq = type; break;
    case 6: L->wk = data; L->tk = type; break;
    case 7: L->wv = data; L->tv = type; break;
    case 8: L->wo = data; L->to = type; break;
    case 9: L->wup = data; L->tup = type; break;
    case 10: L->wgate = data; L->tgate = type; break;
    case 11: L->wdown = data; L->tdown = type; break;
    case 12: L->bq = (const float*)data; break;
    case 13: L->bk = (const float*)data; break;
    case 14: L->bv = (const float*)data; break;
    default: return 1;
  }
  return 0;
}

co_session* co_session_create(co_model* m, int max_ctx) {
  const co_config* c = &m->cfg;
  co_session* s = (co_session*)calloc(1, sizeof(co_session));
  s->m = m; s->max_ctx = max_ctx;
  const size_t cache = (size_t)c->layers * c->kv_heads * max_ctx * c->head_dim;
  s->k = (float*)calloc(cache, 4); s->v = (float*)calloc(cache, 4);
  const int qw = c->heads * c->head_dim, kw = c->kv_heads * c->head_dim;
  s->x = (float*)malloc(4 * (size_t)c->hidden); s->h = (float*)malloc(4 * (size_t)c->hidden);
  s->q = (float*)malloc(4 * (size_t)qw); s->kk = (float*)malloc(4 * (size_t)kw); s->vv = (float*)malloc(4 * (size_t)kw);
  s->att = (float*)malloc(4 * (size_t)qw);
  s->fused = (float*)malloc(4 * (size_t)2 * c->inter); s->act = (float*)malloc(4 * (size_t)c->inter);
  s->tmp = (float*)malloc(4 * (size_t)c->hidden);
  s->scores = (float*)malloc(4 * (size_t)c->heads * max_ctx);
  return s;
}
void co_session_destroy(co_session* s) {
  if (!s) return;
  free(s->k); free(s->v); free(s->x); free(s->h); free(s->q); free(s->kk); free(s->vv); free(s->att);
  free(s->fused); free(s->act); free(s->tmp); free(s->scores); free(s);
}
void co_session_reset(co_session* s) { s->len = 0; }
/* marks `len` cache rows as committed without computing them (timing at a given context) */
void co_session_assume_len(co_session* s, int len) {
  if (len > s->len) {
    /* touch the newly assumed rows with a cheap pattern so the pages are real memory, not the zero page */
    const co_config* c = &s->m->cfg;
    const size_t plane = (size_t)s->max_ctx * c->head_dim;
    for (size_t p = 0; p < (size_t)c->layers * c->kv_heads; ++p)
      for (size_t i = (size_t)s->len * c->head_dim; i < (size_t)len * c->head_dim; ++i) {
        const float v = (float)(((uint32_t)(i + p) * 2654435761u) >> 16) * (1.0f / 65536.0f) - 0.5f;
        s->k[p * plane + i] = v;
        s->v[p * plane + i] = -v;
      }
  }
  s->len = len;
}

static void rmsnorm(const float* x, const float* g, float* y, int n, float eps) {
  float ss = 0.f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = g[i] * (x[i] * inv);
}
static void rope(float* x, int width, int hd, int pos, const float* theta) {
  for (int p = 0; p < width / 2; ++p) {
    const float a = (float)pos * theta[p % (hd / 2)];
    const float s = sinf(a), c = cosf(a);
    const float x0 = x[2 * p], x1 = x[2 * p + 1];
    x[2 * p] = c * x0 - s * x1;
    x[2 * p + 1] = s * x0 + c * x1;
  }
}

/* one width-1 forward at absolute position pos; appends at slot s->len */
int co_session_step(co_session* s, int token, int pos, float* logits) {
  co_model* m = s->m;
  const co_config* c = &m->cfg;
  if (s->len >= s->max_ctx || token < 0 || token >= c->vocab) return 1;
  const int H = c->hidden, hd = c->head_dim, qw = c->heads * hd, kw = c->kv_heads * hd, I = c->inter;
  const int slot = s->len, n = slot + 1, group = c->heads / c->kv_heads;
  const float inv_sqrt = 1.0f / sqrtf((float)hd);
  co_dequantize(m->t_embed, (const uint8_t*)m->embed + (size_t)token * row_bytes(m->t_embed, H), H, s->x);
  for (int l = 0; l < c->layers; ++l) {
    const co_layer* L = &m->layers[l];
    rmsnorm(s->x, L->attn_norm, s->h, H, c->rms_eps);
    co_gemv(L->tq, L->wq, qw, H, s->h, 1, c->qkv_bias ? L->bq : NULL, s->q);
    co_gemv(L->tk, L->wk, kw, H, s->h, 1, c->qkv_bias ? L->bk : NULL, s->kk);
    co_gemv(L->tv, L->wv, kw, H, s->h, 1, c->qkv_bias ? L->bv : NULL, s->vv);
    rope(s->q, qw, hd, pos, m->theta);
    rope(s->kk, kw, hd, pos, m->theta);
    float* kc = s->k + (size_t)l * c->kv_heads * s->max_ctx * hd;
    float* vc = s->v + (size_t)l * c->kv_heads * s->max_ctx * hd;
    for (int g = 0; g < c->kv_heads; ++g) {
      memcpy(kc + ((size_t)g * s->max_ctx + slot) * hd, s->kk + g * hd, 4 * (size_t)hd);
      memcpy(vc + ((size_t)g * s->max_ctx + slot) * hd, s->vv + g * hd, 4 * (size_t)hd);
    }
#pragma omp parallel for schedule(static)
    for (int hq = 0; hq < c->heads; ++hq) {
      const int g = hq / group;
      const float* q = s->q + hq * hd;
      const float* kp = kc + (size_t)g * s->max_ctx * hd;
      const float* vp = vc + (size_t)g * s->max_ctx * hd;
      float* sc = s->scores + (size_t)hq * s->max_ctx;
      float mx = -1e30f;
      for (int j = 0; j < n; ++j) {
        const float acc = dot_f32(kp + (size_t)j * hd, q, hd);
        sc[j] = acc * inv_sqrt;
        if (sc[j] > mx) mx = sc[j];
      }
      float sum = 0.f;
      for (int j = 0; j < n; ++j) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
      float* o = s->att + hq * hd;
      for (int t = 0; t < hd; ++t) o[t] = 0.f;
      for (int j = 0; j < n; ++j) {
        const float p = sc[j];
        const float* vr = vp + (size_t)j * hd;
        for (int t = 0; t < hd; ++t) o[t] += p * vr[t];
      }
      const float invs = sum > 0.f ? 1.0f / sum : 0.f;
      for (int t = 0; t < hd; ++t) o[t] *= invs;
    }
    co_gemv(L->to, L->wo, H, qw, s->att, 1, NULL, s->tmp);
    for (int i = 0; i < H; ++i) s->x[i] += s->tmp[i];
    rmsnorm(s->x, L->ffn_norm, s->h, H, c->rms_eps);
    co_gemv(L->tup, L->wup, I, H, s->h, 1, NULL, s->fused);          /* first half = up   */
    co_gemv(L->tgate, L->wgate, I, H, s->h, 1, NULL, s->fused + I);  /* second half = gate */
    for (int i = 0; i < I; ++i) {
      const float b = s->fused[I + i];
      float sig;
      if (b > 0.f) sig = 1.0f / (1.0f + expf(-b)); else { const float e = expf(b); sig = e / (1.0f + e); }
      s->act[i] = s->fused[i] * (b * sig);
    }
    co_gemv(L->tdown, L->wdown, H, I, s->act, 1, NULL, s->tmp);
    for (int i = 0; i < H; ++i) s->x[i] += s->tmp[i];
  }
  s->len = n;
  if (logits) {
    rmsnorm(s->x, m->final_norm, s->h, H, c->rms_eps);
    co_gemv(m->t_head, m->head, c->vocab, H, s->h, 1, NULL, logits);
  }
  return 0;
}

int co_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void co_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
