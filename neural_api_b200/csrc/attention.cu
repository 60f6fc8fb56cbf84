// KV-cache GQA decode attention with a split over the context.
//
//   rope_append : optional full-width q/k RMSNorm, RoPE on Q (in place) and K,
//                 K,V of the token written at slot cache_len[b] of the head-major
//                 cache [b][kv_head][pos][d].
//   decode      : one CTA per (kv head, context split, sequence). The CTA serves
//                 every query head of the GQA group, so each K/V row is read from
//                 HBM once per group rather than once per query head. Lanes are
//                 grouped LPK = ceil(hd/8) per key (8 channels per lane, two
//                 16-byte loads); every lane group keeps an online-softmax state
//                 (m, l, acc) that is merged lanes -> warps -> splits in a fixed
//                 order. Scores are scaled by 1/sqrt(hd) after the dot product and
//                 the sum is divided once at the end, as in the reference kernel.
//   combine     : merges the per-split partial states.
#include "gemv_common.cuh"      // packed fp32x2 arithmetic
#include <math.h>

struct AttnParams {
  float* qkv; int64_t ld;
  float* k_cache; float* v_cache;
  const int32_t* cache_len;
  int q_heads, kv_heads, head_dim, max_ctx;
  const float* theta; const int32_t* pos;
  const float* q_norm; const float* k_norm; float eps;
  float* out; int64_t ldo;
  float* partial; int nsplit;
  float inv_sqrt_d;
  int min_chunk;          // fewest cached rows a context split covers (set by the launcher for the kernel it picked)
  int8_t* k_codes; int8_t* v_codes; float* k_scales; float* v_scales;     // int8 cache (k_codes != NULL)
  const int32_t* seq_index;                                               // cache sequence of each batch row (NULL = the row itself)
  int* err;               // device-visible error word: 2 = a cache length outside [0, max_ctx) was refused
  int k_blocked;          // K cache block-transposed (cai_k_blocked_index)
  // which cached rows a step sees (TNNetFusedSDPA's Window and EnableEviction):
  int window;             // > 0: only the most recent `window` rows (sliding-window layers, jStart of neural/neural.cl:2437-2438)
  int evict_sinks, evict_window;   // evict_window > 0: StreamingLLM, the first `sinks` rows and the most recent `window` rows live
};

// The number of cached rows comes from a device word the host cannot always vouch for (the allocation-free entry
// point's caller owns it). A length outside [0, max_ctx) would put the appended row, and the rows the decode
// kernels walk, outside the cache: refuse it (no access at all), raise the error word, and let every kernel of the
// step leave in the same way.
// Where the row of a step that finds `len` rows before it goes. Eviction keeps the rows physically as the first `sinks`
// slots plus a ring of `window` slots: the row of position len >= sinks + window overwrites the oldest non-sink row.
// (The reference shifts the surviving rows down by one instead, neural/neuraldecode.pas:1257-1310; the set of live rows
// is the same, and keys keep their original rotation either way.)
__device__ __forceinline__ int attn_slot(const AttnParams& p, int len) {
  const int cap = p.evict_sinks + p.evict_window;
  return (p.evict_window > 0 && len >= cap) ? p.evict_sinks + (len - p.evict_sinks) % p.evict_window : len;
}
// The cached rows [base, n) a step attends over, the new row included.
__device__ __forceinline__ void attn_range(const AttnParams& p, int len, int& base, int& n) {
  n = len + 1; base = 0;
  if (p.evict_window > 0) { const int cap = p.evict_sinks + p.evict_window; if (n > cap) n = cap; }
  else if (p.window > 0 && n > p.window) base = n - p.window;
}
__device__ __forceinline__ bool attn_len_ok(const AttnParams& p, int len) {
  if (len >= 0 && (len < p.max_ctx || p.evict_window > 0)) return true;
  if (threadIdx.x == 0 && p.err) *p.err = 2;
  return false;
}

// Rows per context split: the context spread over nsplit splits, at least min_chunk rows, a multiple of 32.
// Short contexts use few splits; the other CTAs leave at once. Decode and combine kernels both use this.
__device__ __forceinline__ int attn_chunk(int n, int nsplit, int min_chunk) {
  int chunk = (n + nsplit - 1) / nsplit;
  if (chunk < min_chunk) chunk = min_chunk;
  return (chunk + 31) & ~31;
}

__global__ void rope_append_kernel(const AttnParams p) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const int bs = p.seq_index ? p.seq_index[b] : b;     // the cache sequence this row appends to
  const int hd = p.head_dim;
  const int qw = p.q_heads * hd, kw = p.kv_heads * hd;
  float* row = p.qkv + (int64_t)b * p.ld;
  if (!attn_len_ok(p, p.cache_len[b])) return;
  const int slot = attn_slot(p, p.cache_len[b]);
  float inv_q = 1.f, inv_k = 1.f;
  if (p.q_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < qw; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    ss = block_sum(ss, red);
    inv_q = 1.0f / sqrtf(ss / (float)qw + p.eps);
    ss = 0.f;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) ss = fmaf(row[qw + c], row[qw + c], ss);
    ss = block_sum(ss, red);
    inv_k = 1.0f / sqrtf(ss / (float)kw + p.eps);
  }
  const int pos = p.pos ? p.pos[b] : p.cache_len[b];
  const int half_hd = hd >> 1;
  // Q pairs, in place
  for (int pr = threadIdx.x; pr < (qw >> 1); pr += blockDim.x) {
    float x0 = row[2 * pr], x1 = row[2 * pr + 1];
    if (p.q_norm) { x0 = p.q_norm[2 * pr] * (x0 * inv_q); x1 = p.q_norm[2 * pr + 1] * (x1 * inv_q); }
    if (p.theta) {
      float s, c;
      sincosf((float)pos * p.theta[pr % half_hd], &s, &c);
      const float y0 = c * x0 - s * x1, y1 = s * x0 + c * x1;
      x0 = y0; x1 = y1;
    }
    row[2 * pr] = x0; row[2 * pr + 1] = x1;
  }
  // K pairs -> cache; V -> cache
  for (int pr = threadIdx.x; pr < (kw >> 1); pr += blockDim.x) {
    float x0 = row[qw + 2 * pr], x1 = row[qw + 2 * pr + 1];
    if (p.k_norm) { x0 = p.k_norm[2 * pr] * (x0 * inv_k); x1 = p.k_norm[2 * pr + 1] * (x1 * inv_k); }
    if (p.theta) {
      float s, c;
      sincosf((float)pos * p.theta[pr % half_hd], &s, &c);
      const float y0 = c * x0 - s * x1, y1 = s * x0 + c * x1;
      x0 = y0; x1 = y1;
    }
    const int g = (2 * pr) / hd, d = (2 * pr) % hd;
    float* dst = p.k_cache + ((int64_t)bs * p.kv_heads + g) * p.max_ctx * hd +
                 (p.k_blocked ? (int64_t)cai_k_blocked_index(slot, d, hd) : (int64_t)slot * hd + d);
    dst[0] = x0; dst[1] = x1;
  }
  for (int c = threadIdx.x; c < kw; c += blockDim.x) {
    const int g = c / hd, d = c % hd;
    p.v_cache[(((int64_t)bs * p.kv_heads + g) * p.max_ctx + slot) * hd + d] = row[qw + kw + c];
  }
}

// ---------------------------------------------------------------------------
// RoPE + append into the int8 KV cache. Same front end as rope_append_kernel (optional full-width q/k norm, Q
// rotated in place); the rotated K row and the V row of the token are staged in shared memory, then one warp per
// (kv head, K|V) quantizes its row in the reference's cache format: one symmetric fp32 scale per row,
// scale = maxabs / 127 over the finite magnitudes, code = clamp(rint(v * (1 / maxabs) * 127), -127, 127) with the
// multiplications in that order and round-half-to-even; a zero or denormal row maximum gives zero codes and
// scale 1; NaN -> 0, infinities clamp.
// ---------------------------------------------------------------------------
__global__ void rope_append_int8_kernel(const AttnParams p) {
  extern __shared__ float kv_s[];                    // [kw] rotated K, then [kw] V
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const int bs = p.seq_index ? p.seq_index[b] : b;     // the cache sequence this row appends to
  const int hd = p.head_dim;
  const int qw = p.q_heads * hd, kw = p.kv_heads * hd;
  float* row = p.qkv + (int64_t)b * p.ld;
  if (!attn_len_ok(p, p.cache_len[b])) return;
  const int slot = attn_slot(p, p.cache_len[b]);
  float inv_q = 1.f, inv_k = 1.f;
  if (p.q_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < qw; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    ss = block_sum(ss, red);
    inv_q = 1.0f / sqrtf(ss / (float)qw + p.eps);
    ss = 0.f;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) ss = fmaf(row[qw + c], row[qw + c], ss);
    ss = block_sum(ss, red);
    inv_k = 1.0f / sqrtf(ss / (float)kw + p.eps);
  }
  const int pos = p.pos ? p.pos[b] : p.cache_len[b];
  const int half_hd = hd >> 1;
  for (int pr = threadIdx.x; pr < (qw >> 1); pr += blockDim.x) {
    float x0 = row[2 * pr], x1 = row[2 * pr + 1];
    if (p.q_norm) { x0 = p.q_norm[2 * pr] * (x0 * inv_q); x1 = p.q_norm[2 * pr + 1] * (x1 * inv_q); }
    if (p.theta) {
      float s, c;
      sincosf((float)pos * p.theta[pr % half_hd], &s, &c);
      const float y0 = c * x0 - s * x1, y1 = s * x0 + c * x1;
      x0 = y0; x1 = y1;
    }
    row[2 * pr] = x0; row[2 * pr + 1] = x1;
  }
  for (int pr = threadIdx.x; pr < (kw >> 1); pr += blockDim.x) {
    float x0 = row[qw + 2 * pr], x1 = row[qw + 2 * pr + 1];
    if (p.k_norm) { x0 = p.k_norm[2 * pr] * (x0 * inv_k); x1 = p.k_norm[2 * pr + 1] * (x1 * inv_k); }
    if (p.theta) {
      float s, c;
      sincosf((float)pos * p.theta[pr % half_hd], &s, &c);
      const float y0 = c * x0 - s * x1, y1 = s * x0 + c * x1;
      x0 = y0; x1 = y1;
    }
    kv_s[2 * pr] = x0; kv_s[2 * pr + 1] = x1;
  }
  for (int c = threadIdx.x; c < kw; c += blockDim.x) kv_s[kw + c] = row[qw + kw + c];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int task = warp; task < 2 * p.kv_heads; task += nwarps) {
    const int part = task / p.kv_heads, g = task - part * p.kv_heads;     // part 0 = K, 1 = V
    const float* src = kv_s + (size_t)part * kw + (size_t)g * hd;
    float m = 0.f;
    for (int d = lane; d < hd; d += 32) {
      const float a = fabsf(src[d]);
      if (__float_as_uint(a) <= 0x7F7FFFFFu) m = fmaxf(m, a);            // finite magnitudes only
    }
    m = warp_max(m);
    const bool usable = __float_as_uint(m) >= 0x00800000u;                // a normal number
    const float row_scale = usable ? (m / 127.0f) : 1.0f;
    const float recip = usable ? (1.0f / m) : 0.0f;
    const int64_t rowi = ((int64_t)bs * p.kv_heads + g) * p.max_ctx + slot;
    int8_t* codes = (part == 0 ? p.k_codes : p.v_codes) + rowi * hd;
    // block-transposed K codes: the row's codes go to their places inside the position's 32-row block
    int8_t* khead = p.k_codes + ((int64_t)bs * p.kv_heads + g) * p.max_ctx * hd;
    const bool blocked = (part == 0) && p.k_blocked;
    if (lane == 0) (part == 0 ? p.k_scales : p.v_scales)[rowi] = row_scale;
    for (int d = lane; d < hd; d += 32) {
      const float v = src[d];
      float scaled = v * recip * 127.0f;
      if (__float_as_uint(fabsf(v)) > 0x7F800000u) scaled = 0.f;          // NaN
      const int8_t code = (int8_t)fminf(fmaxf(rintf(scaled), -127.0f), 127.0f);
      if (blocked) khead[cai_k_blocked_index_i8(slot, d, hd)] = code;
      else codes[d] = code;
    }
  }
}

__device__ __forceinline__ void load8(const float* __restrict__ ptr, int nd, bool vec, float (&v)[8]) {
  if (vec) {
    const float4 a = *(const float4*)ptr, b = *(const float4*)(ptr + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (i < nd) ? ptr[i] : 0.f;
  }
}

constexpr int ATTN_MIN_CHUNK = 64;
constexpr int ATTN_WARPS = 4;
constexpr int ATTN_KEYS = 2;   // keys in flight per lane group (K and V rows of both are loaded together)

template <int GT>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attn_decode_kernel(const AttnParams p, int lpk) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int hd = p.head_dim;
  const int G = p.q_heads / p.kv_heads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % lpk, kslot = lane / lpk;
  const int kpw = 32 / lpk;
  const int d0 = sub * 8;
  int nd = hd - d0; nd = nd > 8 ? 8 : (nd < 0 ? 0 : nd);
  const bool vec = (nd == 8) && ((hd & 3) == 0);

  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;                                         // the step attends over rows [base, n)
  attn_range(p, p.cache_len[b], base, n);
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (split >= used) return;
  const int j_begin = base + split * chunk;
  int j_end = j_begin + chunk; if (j_end > n) j_end = n;

  float* q_s = smem;                                  // [G][hd]
  float* merge_s = smem + (size_t)G * hd;             // [ATTN_WARPS][GT][hd + 2]
  const float* qrow = p.qkv + (int64_t)b * p.ld + (int64_t)g * G * hd;
  for (int i = threadIdx.x; i < G * hd; i += blockDim.x) q_s[i] = qrow[i];
  __syncthreads();

  const int bs = p.seq_index ? p.seq_index[b] : b;
  const float* kbase = p.k_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * hd;
  const float* vbase = p.v_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * hd;
  const int key_stride = ATTN_WARPS * kpw;

  for (int h0 = 0; h0 < G; h0 += GT) {
    float m[GT], l[GT], acc[GT][8];
#pragma unroll
    for (int t = 0; t < GT; ++t) {
      m[t] = -INFINITY; l[t] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[t][i] = 0.f;
    }
    // The trip count depends on the warp only (not on the lane's key slot): every lane of a
    // warp runs the same iterations, so the full-mask shuffles below are always converged.
    for (int jb = j_begin + warp * kpw; jb < j_end; jb += key_stride * ATTN_KEYS) {
      const int j0 = jb + kslot;
      float kv[ATTN_KEYS][8], vv[ATTN_KEYS][8];
      bool valid[ATTN_KEYS];
      // K and V rows of the keys of this iteration are requested together, before any arithmetic
#pragma unroll
      for (int t = 0; t < ATTN_KEYS; ++t) {
        const int j = j0 + t * key_stride;
        valid[t] = (j < j_end) && (nd > 0);
        if (valid[t]) {
          load8(kbase + (int64_t)j * hd + d0, nd, vec, kv[t]);
          load8(vbase + (int64_t)j * hd + d0, nd, vec, vv[t]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) { kv[t][i] = 0.f; vv[t][i] = 0.f; }
        }
      }
      float s[GT][ATTN_KEYS];
#pragma unroll
      for (int hh = 0; hh < GT; ++hh) {
        const int h = (h0 + hh < G) ? (h0 + hh) : (G - 1);
        float qv[8];
        load8(q_s + h * hd + d0, nd, vec, qv);
#pragma unroll
        for (int t = 0; t < ATTN_KEYS; ++t) {
          float dsum = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) dsum = fmaf(qv[i], kv[t][i], dsum);
          s[hh][t] = dsum;
        }
      }
      // reduce the partial dots across the lanes of a key group
      for (int o = 1; o < lpk; o <<= 1) {
#pragma unroll
        for (int hh = 0; hh < GT; ++hh)
#pragma unroll
          for (int t = 0; t < ATTN_KEYS; ++t) s[hh][t] += __shfl_xor_sync(0xffffffffu, s[hh][t], o);
      }
#pragma unroll
      for (int hh = 0; hh < GT; ++hh) {
        float mx = m[hh];
#pragma unroll
        for (int t = 0; t < ATTN_KEYS; ++t) {
          const int j = j0 + t * key_stride;
          s[hh][t] = (j < j_end) ? s[hh][t] * p.inv_sqrt_d : -INFINITY;
          mx = fmaxf(mx, s[hh][t]);
        }
        if (mx == -INFINITY) continue;
        const float scale = expf(m[hh] - mx);
        float pt[ATTN_KEYS];
        float lsum = 0.f;
#pragma unroll
        for (int t = 0; t < ATTN_KEYS; ++t) { pt[t] = expf(s[hh][t] - mx); lsum += pt[t]; }
        l[hh] = l[hh] * scale + lsum;
        m[hh] = mx;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float a = acc[hh][i] * scale;
#pragma unroll
          for (int t = 0; t < ATTN_KEYS; ++t) a = fmaf(pt[t], vv[t][i], a);
          acc[hh][i] = a;
        }
      }
    }
    // merge the key groups of a warp (lanes with the same `sub`)
    for (int o = lpk; o < 32; o <<= 1) {
#pragma unroll
      for (int hh = 0; hh < GT; ++hh) {
        const float om = __shfl_xor_sync(0xffffffffu, m[hh], o);
        const float ol = __shfl_xor_sync(0xffffffffu, l[hh], o);
        const float mx = fmaxf(m[hh], om);
        const float sa = (mx == -INFINITY) ? 0.f : expf(m[hh] - mx);
        const float sb = (mx == -INFINITY) ? 0.f : expf(om - mx);
        l[hh] = l[hh] * sa + ol * sb;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float oa = __shfl_xor_sync(0xffffffffu, acc[hh][i], o);
          acc[hh][i] = acc[hh][i] * sa + oa * sb;
        }
        m[hh] = mx;
      }
    }
    // warps -> shared memory
    __syncthreads();   // merge_s free (previous head tile consumed)
    if (kslot == 0) {
#pragma unroll
      for (int hh = 0; hh < GT; ++hh) {
        float* dst = merge_s + ((size_t)warp * GT + hh) * (hd + 2);
        if (sub == 0) { dst[0] = m[hh]; dst[1] = l[hh]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) if (i < nd) dst[2 + d0 + i] = acc[hh][i];
      }
    }
    __syncthreads();
    // all threads: merge the warps for (head, d) pairs and write
    for (int idx = threadIdx.x; idx < GT * hd; idx += blockDim.x) {
      const int hh = idx / hd, d = idx % hd;
      if (h0 + hh >= G) continue;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) mx = fmaxf(mx, merge_s[((size_t)w * GT + hh) * (hd + 2)]);
      float lt = 0.f, at = 0.f;
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) {
        const float* src = merge_s + ((size_t)w * GT + hh) * (hd + 2);
        const float sc = (mx == -INFINITY) ? 0.f : expf(src[0] - mx);
        lt += src[1] * sc;
        at += src[2 + d] * sc;
      }
      const int h = g * G + h0 + hh;
      if (used == 1) {
        p.out[(int64_t)b * p.ldo + (int64_t)h * hd + d] = (lt > 0.f) ? at / lt : 0.f;
      } else {
        float* dst = p.partial + (((int64_t)b * p.q_heads + h) * p.nsplit + split) * (hd + 2);
        if (d == 0) { dst[0] = mx; dst[1] = lt; }
        dst[2 + d] = at;
      }
    }
  }
}


// ---------------------------------------------------------------------------
// Decode attention for head_dim 64 / 128 and groups of up to 8 query heads: the kernel the long contexts run on.
// The kernel above spends ~90 warp instructions per cached row (every lane of a 16-lane key group repeats the
// softmax arithmetic, and the dot products cost 4 shuffle stages per key and head); at 1 KB per row that is several
// times what HBM could deliver (measured 1.0 TB/s at context 8192). Here a warp works on tiles of 32 rows and
// changes the meaning of a lane between the two products:
//   Q.K   lane = row: the lane walks its K row with 16-byte loads (eight in flight), q comes from shared memory
//         as a broadcast; no cross-lane reduction, the softmax terms are computed once per row;
//   P.V   lane = 2 or 4 channels: V rows are read coalesced, the probabilities come back from shared memory four rows
//         at a time as broadcasts; the lane keeps acc[head][its channels].
// ~50 instructions per row for 5 heads x 128 channels. Online softmax state (m, l, acc) per warp, merged warps ->
// splits in fixed order exactly like the general kernel (same partial format, same combine kernel).
// ---------------------------------------------------------------------------
constexpr int ATTN_TILE_MIN_CHUNK = 128;   // 4 warps x one tile of 32 rows

// (Four CTAs per SM, i.e. at most 128 registers: a context of 8192 rows makes 520 CTAs for 8 KV heads, which then
// run as one wave of 592 slots; with two or three resident CTAs the tail wave doubled the kernel's time.)
template <int G, int HD>
__global__ void __launch_bounds__(ATTN_WARPS * 32, 4) attn_decode_tile_kernel(const AttnParams p) {
  constexpr int DPL = HD / 32;                         // channels per lane in the P.V phase
  constexpr int DP2 = DPL / 2;                         // ... as packed pairs
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;                                         // the step attends over rows [base, n)
  attn_range(p, p.cache_len[b], base, n);
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (split >= used) return;
  const int j_begin = base + split * chunk;
  int j_end = j_begin + chunk; if (j_end > n) j_end = n;

  // All multiply-adds are packed pairs (fma.rn.f32x2: two IEEE fp32 FMAs per instruction), which halves the
  // instruction count of both products; the probabilities are kept in shared memory as (p, p) pairs for that.
  float* q_s = smem;                                                   // [G][HD]
  f32x2_t* p_s = (f32x2_t*)(q_s + G * HD) + (size_t)warp * G * 32;     // this warp's [G][32] pairs (p, p)
  float* merge_s = smem + G * HD + ATTN_WARPS * G * 64;                // [ATTN_WARPS][G][HD + 2]
  const float* qrow = p.qkv + (int64_t)b * p.ld + (int64_t)g * G * HD;
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) q_s[i] = qrow[i];
  __syncthreads();

  const int bs = p.seq_index ? p.seq_index[b] : b;
  const float* kbase = p.k_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * HD;
  const float* vbase = p.v_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * HD;

  float m[G], l[G];
  f32x2_t acc[G][DP2];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DP2; ++d) acc[h][d] = 0ull;
  }

  for (int tile = j_begin + warp * 32; tile < j_end; tile += ATTN_WARPS * 32) {
    // ---- Q.K, lane = row (rows past the end re-read the last row and are masked below)
    const int j = tile + lane;
    const bool valid = j < j_end;
    const int jr = valid ? j : j_end - 1;
    // row layout: the lane's own row, piece after piece; block-transposed layout: piece p of the 32 rows of the lane's
    // block is 512 contiguous bytes (a fully coalesced load per instruction)
    const ulonglong2* krow = p.k_blocked ? (const ulonglong2*)(kbase + (int64_t)(jr >> 5) * 32 * HD) + (jr & 31)
                                         : (const ulonglong2*)(kbase + (int64_t)jr * HD);
    const int kstep = p.k_blocked ? 32 : 1;              // 16-byte units between consecutive pieces of a row
    f32x2_t s2[G];
#pragma unroll
    for (int h = 0; h < G; ++h) s2[h] = 0ull;
    // 64 channels (16 loads in flight) at a time: few dependent round trips to HBM
#pragma unroll
    for (int c = 0; c < HD / 64; ++c) {
      ulonglong2 k[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) k[i] = krow[(c * 16 + i) * kstep];
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const ulonglong2* q2 = (const ulonglong2*)(q_s + h * HD + c * 64);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const ulonglong2 q = q2[i];
          s2[h] = fma2(q.x, k[i].x, s2[h]);
          s2[h] = fma2(q.y, k[i].y, s2[h]);
        }
      }
    }
    // ---- P.V, lane = DPL channels. The V rows do not depend on the softmax, so the first half of the tile's rows
    //      is requested before it (masked rows re-read the last row and carry probability 0)
    const int last = j_end - 1 - tile;                 // index of the tile's last valid row, >= 0
    f32x2_t v[16][DP2];
    auto load_v = [&](int base) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int r = (base + t <= last) ? (base + t) : last;
        const float* vrow = vbase + (int64_t)(tile + r) * HD + lane * DPL;
        if (DPL == 4) {
          const ulonglong2 x = *(const ulonglong2*)vrow;
          v[t][0] = x.x; v[t][DP2 - 1] = x.y;
        } else {
          v[t][0] = *(const f32x2_t*)vrow;
        }
      }
    };
    auto use_v = [&](int base) {
#pragma unroll
      for (int t2 = 0; t2 < 16; t2 += 2) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const ulonglong2 pr = *(const ulonglong2*)(p_s + h * 32 + base + t2);   // (p, p) of two rows
#pragma unroll
          for (int d = 0; d < DP2; ++d) {
            acc[h][d] = fma2(pr.x, v[t2 + 0][d], acc[h][d]);
            acc[h][d] = fma2(pr.y, v[t2 + 1][d], acc[h][d]);
          }
        }
      }
    };
    load_v(0);
    // ---- softmax terms of the tile, once per row
    __syncwarp();                                      // the previous tile's probabilities have been consumed
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float sc = valid ? sum2(s2[h]) * p.inv_sqrt_d : -INFINITY;
      const float mnew = fmaxf(m[h], warp_max(sc));    // finite: the tile holds at least one row
      const float pj = valid ? expf(sc - mnew) : 0.f;
      const float psum = warp_sum(pj);
      const float corr = expf(m[h] - mnew);            // 0 on the first tile (m = -inf)
      l[h] = l[h] * corr + psum;
      m[h] = mnew;
      const f32x2_t corr2 = pack2(corr, corr);
#pragma unroll
      for (int d = 0; d < DP2; ++d) acc[h][d] = fma2(acc[h][d], corr2, 0ull);
      p_s[h * 32 + lane] = pack2(pj, pj);
    }
    __syncwarp();
    use_v(0);
    if (last >= 16) {
      load_v(16);
      use_v(16);
    }
  }
  // ---- warps -> shared memory -> one state per head (a warp that had no tile contributes m = -inf, l = 0)
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float* dst = merge_s + ((size_t)warp * G + h) * (HD + 2);
    if (lane == 0) { dst[0] = m[h]; dst[1] = l[h]; }
#pragma unroll
    for (int d = 0; d < DP2; ++d) {
      float lo, hi;
      asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[h][d]));
      dst[2 + lane * DPL + 2 * d] = lo;
      dst[2 + lane * DPL + 2 * d + 1] = hi;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int hh = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) mx = fmaxf(mx, merge_s[((size_t)w * G + hh) * (HD + 2)]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) {
      const float* src = merge_s + ((size_t)w * G + hh) * (HD + 2);
      const float sc = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mx);
      lt += src[1] * sc;
      at += src[2 + d] * sc;
    }
    const int h = g * G + hh;
    if (used == 1) {
      p.out[(int64_t)b * p.ldo + (int64_t)h * HD + d] = (lt > 0.f) ? at / lt : 0.f;
    } else {
      float* dst = p.partial + (((int64_t)b * p.q_heads + h) * p.nsplit + split) * (HD + 2);
      if (d == 0) { dst[0] = mx; dst[1] = lt; }
      dst[2 + d] = at;
    }
  }
}

// ---------------------------------------------------------------------------
// The tiled decode kernel over the int8 KV cache (the reference's cai_sdpa_decode_int8 arithmetic): the codes go
// straight into the dot products and each row's scale enters once, outside the element loop:
//   score_j = (sum_d q_d * kcode_jd) * (kscale_j / sqrt(hd)),   out = sum_j (p_j * vscale_j) * vcode_j / sum_j p_j.
// A row is 64 or 128 bytes of codes plus one scale, a quarter of the fp32 cache's traffic. Same tiling as the fp32
// kernel: lane = row for Q.K (the row's codes in 16-byte loads, converted exactly through the 2^23 constant),
// lane = 2 or 4 channels for P.V (one 2- or 4-byte load per row).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float s8_to_float(uint32_t w_xor80, int i) {
  // byte i of a word whose bytes were XOR-ed with 0x80: (0x4B000000 | u) is 8388608 + u, minus 8388736 leaves the int8
  return __uint_as_float(__byte_perm(w_xor80, 0x4B000000u, 0x7650u + (uint32_t)i)) - 8388736.0f;
}

template <int G, int HD>
__global__ void __launch_bounds__(ATTN_WARPS * 32, 4) attn_decode_tile_int8_kernel(const AttnParams p) {
  constexpr int DPL = HD / 32;
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;                                         // the step attends over rows [base, n)
  attn_range(p, p.cache_len[b], base, n);
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (split >= used) return;
  const int j_begin = base + split * chunk;
  int j_end = j_begin + chunk; if (j_end > n) j_end = n;

  float* q_s = smem;                                   // [G][HD]
  float* p_s = q_s + G * HD + (size_t)warp * G * 32;   // this warp's [G][32] probabilities x value scales
  float* merge_s = smem + G * HD + ATTN_WARPS * G * 32;
  const float* qrow = p.qkv + (int64_t)b * p.ld + (int64_t)g * G * HD;
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) q_s[i] = qrow[i];
  __syncthreads();

  const int bs = p.seq_index ? p.seq_index[b] : b;
  const int64_t plane = ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx;
  const int8_t* kbase = p.k_codes + plane * HD;
  const int8_t* vbase = p.v_codes + plane * HD;
  const float* ksc = p.k_scales + plane;
  const float* vsc = p.v_scales + plane;

  // All multiply-adds are packed pairs (fma.rn.f32x2), as in the fp32 kernel: the codes of two neighbouring channels
  // become one register pair (two byte-permutes into the 2^23 constant and ONE packed subtract), which nearly halves
  // the instruction count of a kernel that is bound by instruction issue, not by its quarter-size rows.
  constexpr int DP2 = DPL / 2;
  float m[G], l[G];
  f32x2_t acc[G][DP2];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DP2; ++d) acc[h][d] = 0ull;
  }
  const f32x2_t negc = pack2(-8388736.0f, -8388736.0f);

  for (int tile = j_begin + warp * 32; tile < j_end; tile += ATTN_WARPS * 32) {
    const int j = tile + lane;
    const bool valid = j < j_end;
    const int jr = valid ? j : j_end - 1;              // rows past the end re-read the last row and are masked
    // row layout: the lane's own row; block-transposed: piece i of the block's 32 rows is 512 contiguous bytes
    const uint4* krow = p.k_blocked ? (const uint4*)(kbase + (int64_t)(jr >> 5) * 32 * HD) + (jr & 31) : (const uint4*)(kbase + (int64_t)jr * HD);
    const int kstep = p.k_blocked ? 32 : 1;
    const float kscale = ksc[jr] * p.inv_sqrt_d;
    const float vscale = vsc[jr];
    f32x2_t s2[G];
#pragma unroll
    for (int h = 0; h < G; ++h) s2[h] = 0ull;
    uint4 kw[HD / 16];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) kw[i] = krow[i * kstep];   // the whole row of codes in flight
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) {
      const uint32_t w4[4] = {kw[i].x ^ 0x80808080u, kw[i].y ^ 0x80808080u, kw[i].z ^ 0x80808080u, kw[i].w ^ 0x80808080u};
      f32x2_t kp[8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        kp[2 * t] = add2(pack2(__uint_as_float(__byte_perm(w4[t], 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(w4[t], 0x4B000000u, 0x7651u))), negc);
        kp[2 * t + 1] = add2(pack2(__uint_as_float(__byte_perm(w4[t], 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(w4[t], 0x4B000000u, 0x7653u))), negc);
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const ulonglong2* q2 = (const ulonglong2*)(q_s + h * HD + i * 16);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const ulonglong2 q = q2[t];
          s2[h] = fma2(q.x, kp[2 * t], s2[h]);
          s2[h] = fma2(q.y, kp[2 * t + 1], s2[h]);
        }
      }
    }
    // the tile's V codes: lane = DPL channels, 32 rows (masked rows re-read the last row and carry probability 0)
    const int last = j_end - 1 - tile;
    uint32_t vw[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) {
      const int r = (t <= last) ? t : last;
      const int8_t* vrow = vbase + (int64_t)(tile + r) * HD + lane * DPL;
      vw[t] = (DPL == 4) ? *(const uint32_t*)vrow : (uint32_t)*(const unsigned short*)vrow;
    }
    __syncwarp();
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float sc = valid ? sum2(s2[h]) * kscale : -INFINITY;
      const float mnew = fmaxf(m[h], warp_max(sc));
      const float pj = valid ? expf(sc - mnew) : 0.f;
      const float psum = warp_sum(pj);
      const float corr = expf(m[h] - mnew);
      l[h] = l[h] * corr + psum;
      m[h] = mnew;
      const f32x2_t corr2 = pack2(corr, corr);
#pragma unroll
      for (int d = 0; d < DP2; ++d) acc[h][d] = fma2(acc[h][d], corr2, 0ull);
      p_s[h * 32 + lane] = pj * vscale;                 // the value scale rides with the probability
    }
    __syncwarp();
#pragma unroll
    for (int t4 = 0; t4 < 32; t4 += 4) {
      if (t4 > last) break;
      f32x2_t vf[4][DP2];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t w = vw[t4 + t] ^ 0x80808080u;
        vf[t][0] = add2(pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651u))), negc);
        if (DP2 == 2)
          vf[t][DP2 - 1] = add2(pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653u))), negc);
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float4 pr = *(const float4*)(p_s + h * 32 + t4);
        const f32x2_t p0 = pack2(pr.x, pr.x), p1 = pack2(pr.y, pr.y), p2 = pack2(pr.z, pr.z), p3 = pack2(pr.w, pr.w);
#pragma unroll
        for (int d = 0; d < DP2; ++d) {
          f32x2_t a = acc[h][d];
          a = fma2(p0, vf[0][d], a); a = fma2(p1, vf[1][d], a);
          a = fma2(p2, vf[2][d], a); a = fma2(p3, vf[3][d], a);
          acc[h][d] = a;
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float* dst = merge_s + ((size_t)warp * G + h) * (HD + 2);
    if (lane == 0) { dst[0] = m[h]; dst[1] = l[h]; }
#pragma unroll
    for (int d = 0; d < DP2; ++d) {
      float lo, hi;
      asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[h][d]));
      dst[2 + lane * DPL + 2 * d] = lo;
      dst[2 + lane * DPL + 2 * d + 1] = hi;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int hh = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) mx = fmaxf(mx, merge_s[((size_t)w * G + hh) * (HD + 2)]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) {
      const float* src = merge_s + ((size_t)w * G + hh) * (HD + 2);
      const float sc = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mx);
      lt += src[1] * sc;
      at += src[2 + d] * sc;
    }
    const int h = g * G + hh;
    if (used == 1) {
      p.out[(int64_t)b * p.ldo + (int64_t)h * HD + d] = (lt > 0.f) ? at / lt : 0.f;
    } else {
      float* dst = p.partial + (((int64_t)b * p.q_heads + h) * p.nsplit + split) * (HD + 2);
      if (d == 0) { dst[0] = mx; dst[1] = lt; }
      dst[2 + d] = at;
    }
  }
}

// ---------------------------------------------------------------------------
// The int8 KV cache on the integer tensor-core path (mma.sync m16n8k32, s8 x s8 -> s32), groups of up to 5 query heads.
//
// The kernel above spends ~8 lane instructions per cached code (a byte-permute and half a packed subtract to make it a
// float, G/2 packed multiply-adds): it is bound by instruction issue at a third of the copy rate. Here the codes are
// never unpacked: they ARE the B operand of an integer matrix product, and the fp32 side (q, or p x value scale) is the
// A operand, split exactly into three int8 limbs per head (value = s * (l0 + l1/128 + l2/16384), s a power of two, the
// residue below 2^-21 of the largest magnitude), so the 16 rows of the instruction hold 3 limbs x up to 5 heads.
// Every integer product and sum is exact; the limb split is the only approximation, at fp32's own level.
//
//   Q.K   A = q limbs [16][d], B = K codes [d][8 rows]: a thread's B registers are its 16-byte loads of the rows, used as
//         they arrive (which 32 channels one instruction covers is free as long as A is permuted the same way);
//         scores leave through shared memory to lane = row, where the limbs are summed, the row scale and the head's
//         power of two applied, and the online softmax runs as in the kernels above (fp32).
//   P.V   A = limbs of p_j * vscale_j (scaled per 32-row tile by a power of two above the tile's largest value scale),
//         B = V codes [32 rows][8 channels]: a thread loads 16 (8) bytes of 8 rows and transposes 4x4 byte blocks
//         with byte-permutes (8 per 16 codes); the s32 result of a tile is added into fp32 accumulators, one per
//         (head, limb) row, with the tile's factor; the limb rows are summed once, at the end.
// Work split, masking of the rows past the end, partial format and merge orders are those of the kernel above.
// ---------------------------------------------------------------------------
constexpr int I8M_SROW = 40;                                     // words between score rows in shared memory (conflict-free stores)
constexpr int I8M_THREADS = 64;                                  // two warps: each scores 32 of a tile's 64 rows and owns half of the channels
constexpr int I8M_PROW = 80;                                     // bytes between limb rows (64 used: conflict-free fragment loads)
constexpr int I8M_SCRATCH = 2 * 15 * I8M_SROW * 4 + 16 * I8M_PROW + 2 * 8 * 4 + 8 * 4 + 2 * 8 * 4;   // scores, limb rows, exchange, head factors, sums
static __host__ __device__ inline int i8m_slot_bytes(int HD) { return 64 * HD + 512; }        // 64 rows of codes (the K slot: and the rows' 2 x 64 scales)
static __host__ __device__ inline int i8m_smem_bytes(int HD) { return 16 * HD + 2 * i8m_slot_bytes(HD) + I8M_SCRATCH; }

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// three int8 limbs of t (|t| <= 64): t = l0 + l1/128 + l2/16384 + residue, |residue| <= 2^-15; every step is exact
// (rounding through the 1.5 * 2^23 constant: the sum's low mantissa bits are the rounded integer in two's complement,
// so the limb's byte is the low byte of the sum's bit pattern and no conversion instruction is needed)
__device__ __forceinline__ void i8m_limbs(float t, int& l0, int& l1, int& l2) {
  const float magic = 12582912.0f;
  const float x0 = t + magic;
  float r = (t - (x0 - magic)) * 128.0f;
  const float x1 = r + magic;
  r = (r - (x1 - magic)) * 128.0f;
  const float x2 = r + magic;
  l0 = __float_as_int(x0); l1 = __float_as_int(x1); l2 = __float_as_int(x2);   // only the low byte is the limb
}
// the largest value of a warp in one instruction: floats compare like the integers their bits map to below
__device__ __forceinline__ float i8m_warp_max(float v) {
  int k = __float_as_int(v);
  k ^= (k >> 31) & 0x7FFFFFFF;
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(k));
  r ^= (r >> 31) & 0x7FFFFFFF;
  return __int_as_float(r);
}
__device__ __forceinline__ void i8m_cp4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint2 i8m_lds8(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t i8m_lds4(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// Where 16-byte piece `piece` of tile row `row` sits in a stage. K rows: a thread reads two neighbouring rows' pieces
// {0,2,4,6} + i at once (head_dim 128) or all four pieces of two rows (head_dim 64), and the block-transposed cache
// arrives as one piece of 32 consecutive rows per copy instruction. V rows: a thread reads part of one piece of rows r,
// r + 4, r + 8, r + 12 at once. Both swizzles keep those accesses free of bank conflicts.
template <int HD> __device__ __forceinline__ int i8m_k_slot(int row, int piece) { return HD == 128 ? (piece ^ (row & 7)) : (piece ^ ((row >> 1) & 3)); }
template <int HD> __device__ __forceinline__ int i8m_v_slot(int row, int piece) { return HD == 128 ? (piece ^ (((row >> 2) & 3) << 1)) : (piece ^ (((row >> 2) & 1) << 1)); }

template <int G, int HD>
__global__ void __launch_bounds__(I8M_THREADS, 8) attn_decode_mma_int8_kernel(const AttnParams p) {
  static_assert(3 * G <= 15, "three limbs of every head in the 16 rows of one instruction");
  constexpr int KP = HD / 64;                          // 16-byte pieces of a K row per thread and 8-row tile
  constexpr int KS = HD / 32;                          // K steps of the score product
  constexpr int E = HD / 16;                           // V channels per thread = instructions of the value product per 32 rows
  constexpr int PPR = HD / 16;                         // 16-byte pieces per cached row
  constexpr int SLOT = 64 * HD + 512;                  // a tile's K (or V) rows; the K slot also holds the rows' key and value scales
  extern __shared__ __align__(16) unsigned char smem_i8m[];
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;           // the instruction's row / column group and position in it
  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;
  attn_range(p, p.cache_len[b], base, n);
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (split >= used) return;
  const int j_begin = base + split * chunk;
  int j_end = j_begin + chunk; if (j_end > n) j_end = n;

  int8_t* aq = (int8_t*)smem_i8m;                                            // [16][HD] limbs of q
  unsigned char* ring_p = smem_i8m + 16 * HD;
  const uint32_t k_sl = (uint32_t)__cvta_generic_to_shared(ring_p), v_sl = k_sl + SLOT;   // the K slot and the V slot
  unsigned char* scratch = ring_p + 2 * SLOT;
  int* s_s = (int*)scratch + warp * 15 * I8M_SROW;                           // this warp's scores [15][I8M_SROW]
  int8_t* ap = (int8_t*)(scratch + 2 * 15 * I8M_SROW * 4);                   // limbs of p x vscale [16][I8M_PROW], 64 rows used
  float* xch = (float*)(ap + 16 * I8M_PROW);                                       // [2 warps][8]: maxima of the warp's 32 rows (G scores, 1 value scale)
  float* qs_s = xch + 16;                                                    // [8] power of two of each head's limbs
  float* l_s = qs_s + 8;                                                     // [2 warps][8] sums at the end
  float* st = (float*)ring_p;                                                // after the loop: accumulators [16][HD]

  const int bs = p.seq_index ? p.seq_index[b] : b;
  const int64_t plane = ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx;
  const int8_t* kbase = p.k_codes + plane * HD;
  const int8_t* vbase = p.v_codes + plane * HD;
  const float* ksc = p.k_scales + plane;
  const float* vsc = p.v_scales + plane;

  // One slot each for a tile's K rows and V rows, refilled as soon as its readers are through: the next tile's K rows
  // fly during this tile's softmax and value product, its V rows during the next score product. One commit group per
  // call (rows past the end re-read the last row and are masked; nothing once the tiles are through).
  // The parts of the copy addresses that do not change from tile to tile (whole tiles that start on a block boundary
  // take them; the last, partial tile and a window's odd start go row by row).
  const bool blk = p.k_blocked != 0;
  const int k_src0 = blk ? (tid >> 5) * 32 * HD + (tid & 31) * 16 : (tid / PPR) * HD + (tid % PPR) * 16;
  const int k_sstep = blk ? 512 : (64 / PPR) * HD;                         // source bytes between this thread's copies
  const int k_swz = blk ? (HD == 128 ? (tid & 7) : ((tid >> 1) & 3)) : 0;
  const uint32_t k_dst0 = blk ? (uint32_t)(tid * HD) : (uint32_t)((tid / PPR) * HD + i8m_k_slot<HD>(tid / PPR, tid % PPR) * 16);
  const int v_src0 = (tid / PPR) * HD + (tid % PPR) * 16;
  auto fill_k = [&](int tile) {
    if (tile + 64 <= j_end && (!blk || (tile & 31) == 0)) {
      const int8_t* src = kbase + (int64_t)tile * HD + k_src0;
#pragma unroll
      for (int it = 0; it < PPR; ++it) {
        // block-transposed: row tid, piece it; row-major: row tid / PPR + it * 64 / PPR (same swizzle in every step), piece tid % PPR
        const uint32_t dst = blk ? k_sl + k_dst0 + ((it ^ k_swz) << 4) : k_sl + k_dst0 + it * (64 / PPR) * HD;
        gv_cp_async16(dst, src + it * k_sstep, 16u);
      }
      i8m_cp4(k_sl + 64 * HD + tid * 4, ksc + tile + tid);
      i8m_cp4(k_sl + 64 * HD + 256 + tid * 4, vsc + tile + tid);
    } else if (tile < j_end) {
#pragma unroll
      for (int it = 0; it < PPR; ++it) {
        int row, piece;
        if (p.k_blocked) { row = tid; piece = it; } else { row = (it * 64 + tid) / PPR; piece = (it * 64 + tid) % PPR; }
        int r = tile + row; if (r > j_end - 1) r = j_end - 1;
        const int8_t* src = p.k_blocked ? kbase + (int64_t)(r >> 5) * 32 * HD + piece * 512 + (r & 31) * 16 : kbase + (int64_t)r * HD + piece * 16;
        gv_cp_async16(k_sl + row * HD + i8m_k_slot<HD>(row, piece) * 16, src, 16u);
      }
      int r = tile + tid; if (r > j_end - 1) r = j_end - 1;
      i8m_cp4(k_sl + 64 * HD + tid * 4, ksc + r);
      i8m_cp4(k_sl + 64 * HD + 256 + tid * 4, vsc + r);
    }
    gv_cp_async_commit();
  };
  auto fill_v = [&](int tile) {
    if (tile + 64 <= j_end) {
      const int8_t* src = vbase + (int64_t)tile * HD + v_src0;
#pragma unroll
      for (int it = 0; it < PPR; ++it) {
        const int row = tid / PPR + it * (64 / PPR);
        gv_cp_async16(v_sl + row * HD + i8m_v_slot<HD>(row, tid % PPR) * 16, src + it * (64 / PPR) * HD, 16u);
      }
    } else if (tile < j_end) {
#pragma unroll
      for (int it = 0; it < PPR; ++it) {
        const int row = (it * 64 + tid) / PPR, piece = (it * 64 + tid) % PPR;
        int r = tile + row; if (r > j_end - 1) r = j_end - 1;
        gv_cp_async16(v_sl + row * HD + i8m_v_slot<HD>(row, piece) * 16, vbase + (int64_t)r * HD + piece * 16, 16u);
      }
    }
    gv_cp_async_commit();
  };
  // the first rows start to move before the query is even read
  int tile = j_begin;
  fill_k(tile);

  // q -> limbs (warp w takes heads w, w + 2, ...); rows 3G..15 of both A matrices stay zero
  const float* qrow = p.qkv + (int64_t)b * p.ld + (int64_t)g * G * HD;
  for (int i = tid; i < (16 - 3 * G) * HD; i += I8M_THREADS) aq[3 * G * HD + i] = 0;
  for (int i = tid; i < 16 * I8M_PROW / 4; i += I8M_THREADS) ((uint32_t*)ap)[i] = 0u;
  for (int h = warp; h < G; h += 2) {
    float mx = 0.f;
    for (int d = lane; d < HD; d += 32) mx = fmaxf(mx, fabsf(qrow[h * HD + d]));
    mx = warp_max(mx);
    int e = (mx > 0.f && mx < 3.0e38f) ? ilogbf(mx) - 5 : 0;                // |q| / 2^e < 64
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    const float inv = ldexpf(1.f, -e);
    if (lane == 0) qs_s[h] = ldexpf(1.f, e);
    for (int d = lane; d < HD; d += 32) {
      int l0, l1, l2;
      i8m_limbs(qrow[h * HD + d] * inv, l0, l1, l2);
      aq[(3 * h + 0) * HD + d] = (int8_t)l0;
      aq[(3 * h + 1) * HD + d] = (int8_t)l1;
      aq[(3 * h + 2) * HD + d] = (int8_t)l2;
    }
  }
  __syncthreads();
  // this thread's A registers of the score product: K step s pairs with words 2(s&1), 2(s&1)+1 of the thread's piece
  // 2 tig + (s >> 1) (head_dim 128) or tig (head_dim 64) of the K rows
  uint32_t qa[KS][4];
#pragma unroll
  for (int s = 0; s < KS; ++s) {
    const int word = (KP == 2 ? 2 * tig + (s >> 1) : tig) * 4 + 2 * (s & 1);
    const uint32_t* a32 = (const uint32_t*)aq;
    qa[s][0] = a32[gid * (HD / 4) + word];
    qa[s][1] = a32[(gid + 8) * (HD / 4) + word];
    qa[s][2] = a32[gid * (HD / 4) + word + 1];
    qa[s][3] = a32[(gid + 8) * (HD / 4) + word + 1];
  }
  float qs[G];
#pragma unroll
  for (int h = 0; h < G; ++h) qs[h] = qs_s[h];

  float m[G], l[G];                                    // m: the same in both warps; l: the sum over this lane's rows
  float acc[E][4];
#pragma unroll
  for (int h = 0; h < G; ++h) { m[h] = -INFINITY; l[h] = 0.f; }
#pragma unroll
  for (int e = 0; e < E; ++e) { acc[e][0] = 0.f; acc[e][1] = 0.f; acc[e][2] = 0.f; acc[e][3] = 0.f; }
  // rows gid and gid + 8 of the value product: limb (row % 3) of head (row / 3)
  const int h_lo = gid / 3, h_hi = (gid + 8) / 3;
  const float pw_lo = (gid % 3 == 0) ? 1.f : ((gid % 3 == 1) ? 0.0078125f : 6.103515625e-05f);
  const float pw_hi = ((gid + 8) % 3 == 0) ? 1.f : (((gid + 8) % 3 == 1) ? 0.0078125f : 6.103515625e-05f);

  // where this thread reads its operands in the slots: the swizzles depend on the row only through bits that the row
  // offsets added per step do not touch
  uint32_t k_rd[KP];
#pragma unroll
  for (int i = 0; i < KP; ++i) k_rd[i] = k_sl + (warp * 32 + gid) * HD + i8m_k_slot<HD>(gid, KP == 2 ? 2 * tig + i : tig) * 16;
  const uint32_t v_rd = (E == 8) ? v_sl + (4 * tig) * HD + i8m_v_slot<HD>(4 * tig, warp * 4 + (gid >> 1)) * 16 + (gid & 1) * 8
                                 : v_sl + (4 * tig) * HD + i8m_v_slot<HD>(4 * tig, warp * 2 + (gid >> 2)) * 16 + (gid & 3) * 4;
  for (; tile < j_end; tile += 64) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's copies of the tile's K rows have landed
    __syncthreads();                                    // ... and everybody else's; the V slot's readers are through
    fill_v(tile);
    const int my = warp * 32 + lane;                    // this lane's row of the tile
    const bool valid = tile + my < j_end;
    float kscale, vscale;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(kscale) : "r"(k_sl + 64 * HD + my * 4));
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(vscale) : "r"(k_sl + 64 * HD + 256 + my * 4));
    kscale *= p.inv_sqrt_d;
    // scores of this warp's 32 rows: four 8-row tiles x KS steps
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      int4 kw[KP];
#pragma unroll
      for (int i = 0; i < KP; ++i) kw[i] = gv_lds16(k_rd[i] + nt * 8 * HD);
      int d[4] = {0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const int4 w = kw[s >> 1];
        mma_s8(d, qa[s], (uint32_t)((s & 1) ? w.z : w.x), (uint32_t)((s & 1) ? w.w : w.y), d);
      }
      *(int2*)(s_s + gid * I8M_SROW + nt * 8 + 2 * tig) = make_int2(d[0], d[1]);
      if (gid + 8 < 15) *(int2*)(s_s + (gid + 8) * I8M_SROW + nt * 8 + 2 * tig) = make_int2(d[2], d[3]);
    }
    __syncwarp();
    float sc[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float s0 = (float)s_s[(3 * h) * I8M_SROW + lane], s1 = (float)s_s[(3 * h + 1) * I8M_SROW + lane], s2 = (float)s_s[(3 * h + 2) * I8M_SROW + lane];
      const float dot = fmaf(fmaf(s2, 0.0078125f, s1), 0.0078125f, s0) * qs[h];
      sc[h] = valid ? dot * kscale : -INFINITY;
      const float mx = i8m_warp_max(sc[h]);
      if (lane == 0) xch[warp * 8 + h] = mx;
    }
    {
      const float vmx = i8m_warp_max(valid ? vscale : 0.f);
      if (lane == 0) xch[warp * 8 + 7] = vmx;
    }
    __syncthreads();                                    // the maxima are out; the K slot's readers are through
    fill_k(tile + 64);
    // the power of two all of the tile's p x vscale are scaled by: above the largest value scale (p <= 1)
    const float vmax = fmaxf(xch[7], xch[15]);
    float ts = 1.f;
    if (vmax > 1e-30f && vmax < 1e30f) ts = __uint_as_float((__float_as_uint(vmax) & 0x7F800000u) + 0x00800000u);
    const float to_u = 64.0f / ts;
    bool rescale = false;
    float corr[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float mnew = fmaxf(m[h], fmaxf(xch[h], xch[8 + h]));
      const float pj = valid ? expf(sc[h] - mnew) : 0.f;
      corr[h] = (mnew == m[h]) ? 1.f : expf(m[h] - mnew);     // the same in every thread
      rescale = rescale || (corr[h] != 1.f);
      l[h] = l[h] * corr[h] + pj;                             // this lane's rows only: the lanes are summed once, at the end
      m[h] = mnew;
      int l0, l1, l2;
      i8m_limbs(pj * vscale * to_u, l0, l1, l2);
      ap[(3 * h + 0) * I8M_PROW + my] = (int8_t)l0;
      ap[(3 * h + 1) * I8M_PROW + my] = (int8_t)l1;
      ap[(3 * h + 2) * I8M_PROW + my] = (int8_t)l2;
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this thread's copies of the tile's V rows (the next K rows may still fly)
    __syncthreads();                                    // the limbs are out, the V rows are in
    if (rescale) {                                      // the same in every thread: m and corr come out of the exchanged maxima
      float c_lo = 1.f, c_hi = 1.f;
#pragma unroll
      for (int h = 0; h < G; ++h) { if (h_lo == h) c_lo = corr[h]; if (h_hi == h) c_hi = corr[h]; }
#pragma unroll
      for (int e = 0; e < E; ++e) { acc[e][0] *= c_lo; acc[e][1] *= c_lo; acc[e][2] *= c_hi; acc[e][3] *= c_hi; }
    }
    // the value product over the tile's 64 rows (two K steps summed in s32) for this warp's half of the channels:
    // E channels from byte warp * HD/2 + gid * E on, of rows 4 tig .. 4 tig + 3 and 16 + 4 tig .. + 3 of each 32-row half
    int dv[E][4];
#pragma unroll
    for (int e = 0; e < E; ++e) { dv[e][0] = 0; dv[e][1] = 0; dv[e][2] = 0; dv[e][3] = 0; }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t pa[4];
      pa[0] = ((const uint32_t*)ap)[gid * (I8M_PROW / 4) + ks * 8 + tig];
      pa[1] = ((const uint32_t*)ap)[(gid + 8) * (I8M_PROW / 4) + ks * 8 + tig];
      pa[2] = ((const uint32_t*)ap)[gid * (I8M_PROW / 4) + ks * 8 + 4 + tig];
      pa[3] = ((const uint32_t*)ap)[(gid + 8) * (I8M_PROW / 4) + ks * 8 + 4 + tig];
      uint32_t vw[8][E / 4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row0 = ks * 32 + (i >> 2) * 16 + (i & 3);          // the row is row0 + 4 tig
        if (E == 8) {
          const uint2 v = i8m_lds8(v_rd + row0 * HD);
          vw[i][0] = v.x; vw[i][E / 4 - 1] = v.y;
        } else {
          vw[i][0] = i8m_lds4(v_rd + row0 * HD);
        }
      }
#pragma unroll
      for (int w = 0; w < E / 4; ++w) {
        uint32_t o[2][4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {             // 4 x 4 byte transpose: word w of four rows -> one register per channel
          const uint32_t t0 = __byte_perm(vw[grp * 4 + 0][w], vw[grp * 4 + 1][w], 0x5140), t1 = __byte_perm(vw[grp * 4 + 0][w], vw[grp * 4 + 1][w], 0x7362);
          const uint32_t t2 = __byte_perm(vw[grp * 4 + 2][w], vw[grp * 4 + 3][w], 0x5140), t3 = __byte_perm(vw[grp * 4 + 2][w], vw[grp * 4 + 3][w], 0x7362);
          o[grp][0] = __byte_perm(t0, t2, 0x5410); o[grp][1] = __byte_perm(t0, t2, 0x7632);
          o[grp][2] = __byte_perm(t1, t3, 0x5410); o[grp][3] = __byte_perm(t1, t3, 0x7632);
        }
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) mma_s8(dv[w * 4 + e4], pa, o[0][e4], o[1][e4], dv[w * 4 + e4]);
      }
    }
    const float f_lo = ts * 0.015625f * pw_lo, f_hi = ts * 0.015625f * pw_hi;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      acc[e][0] = fmaf(f_lo, (float)dv[e][0], acc[e][0]);
      acc[e][1] = fmaf(f_lo, (float)dv[e][1], acc[e][1]);
      acc[e][2] = fmaf(f_hi, (float)dv[e][2], acc[e][2]);
      acc[e][3] = fmaf(f_hi, (float)dv[e][3], acc[e][3]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  // accumulators -> [16][HD] over the ring (column n of instruction e is channel warp * HD/2 + n * E + e); the limb
  // rows of a head are summed below
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int c0 = warp * (HD / 2) + (2 * tig) * E + e, c1 = warp * (HD / 2) + (2 * tig + 1) * E + e;
    st[gid * HD + c0] = acc[e][0];
    st[gid * HD + c1] = acc[e][1];
    st[(gid + 8) * HD + c0] = acc[e][2];
    st[(gid + 8) * HD + c1] = acc[e][3];
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const float lw = warp_sum(l[h]);
    if (lane == 0) l_s[warp * 8 + h] = lw;
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += I8M_THREADS) {
    const int hh = idx / HD, d = idx % HD;
    float mh = -INFINITY;                               // m[hh] without a dynamically indexed register array
#pragma unroll
    for (int h = 0; h < G; ++h) if (h == hh) mh = m[h];
    const float lt = l_s[hh] + l_s[8 + hh];
    const float at = (st[(3 * hh) * HD + d] + st[(3 * hh + 1) * HD + d]) + st[(3 * hh + 2) * HD + d];
    const int h = g * G + hh;
    if (used == 1) {
      p.out[(int64_t)b * p.ldo + (int64_t)h * HD + d] = (lt > 0.f) ? at / lt : 0.f;
    } else {
      float* dst = p.partial + (((int64_t)b * p.q_heads + h) * p.nsplit + split) * (HD + 2);
      if (d == 0) { dst[0] = mh; dst[1] = lt; }
      dst[2 + d] = at;
    }
  }
}

// ---------------------------------------------------------------------------
// The same attention with the cached rows staged through shared memory by cp.async instead of ordinary loads.
// The kernel above is a chain of dependent round trips per warp (K pieces, then V rows, then the next tile), so the
// memory pipe idles between them: 3.5 TB/s at context 8192 (long-scoreboard stall of 5 warps per issue). Here every
// warp owns a ring of RING_DEPTH stages of 4 KB and the fill runs RING_DEPTH - 1 stages ahead of the arithmetic,
// straight across tiles: a tile of 32 rows is HD/32 stages of K (32 rows x 32 channels: one contiguous 4 KB run of the
// block-transposed cache, already [piece][row] for conflict-free lane = row reads) followed by its V rows (whole rows).
// Needs the block-transposed K cache and rows [0, n) (no sliding window: its first row is not on a block boundary).
// Same partial format and combine kernel as the kernels above; same fixed merge orders.
// ---------------------------------------------------------------------------
constexpr int RING_STAGE = 4096;
constexpr int RING_DEPTH = 4;
constexpr int RING_WARPS = 4;
static __host__ __device__ inline int ring_rings_offset(int G, int HD) { return ((G * HD * 4 + RING_WARPS * G * 32 * 4) + 127) & ~127; }
static __host__ __device__ inline int ring_smem_bytes(int G, int HD) {
  const int ring = RING_WARPS * RING_DEPTH * RING_STAGE, merge = RING_WARPS * G * (HD + 2) * 4;
  return ring_rings_offset(G, HD) + (ring > merge ? ring : merge);
}

template <int G, int HD>
__global__ void __launch_bounds__(RING_WARPS * 32, 3) attn_decode_ring_kernel(const AttnParams p) {
  constexpr int KS = HD / 32;                    // K stages per tile (32 channels each)
  constexpr int VR = RING_STAGE / (HD * 4);      // rows per V stage
  constexpr int VG = 32 / VR;                    // V stages per tile
  constexpr int SPT = KS + VG;                   // stages per tile
  constexpr int RP = HD / 4;                     // 16-byte pieces per row
  constexpr int DPL = HD / 32;
  constexpr int DP2 = DPL / 2;
  extern __shared__ __align__(128) unsigned char ring_smem[];
  pdl_trigger();
  const int g = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;
  attn_range(p, p.cache_len[b], base, n);              // base == 0 here (the launcher keeps windowed steps off this kernel)
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (split >= used) return;
  const int j_begin = base + split * chunk;
  int j_end = j_begin + chunk; if (j_end > n) j_end = n;

  float* q_s = (float*)ring_smem;                                                   // [G][HD]
  float* p_s = q_s + G * HD + (size_t)warp * G * 32;                                // this warp's [G][32] probabilities
  unsigned char* rings = ring_smem + ring_rings_offset(G, HD);
  float* merge_s = (float*)rings;                                                   // [RING_WARPS][G][HD + 2], after the loop
  const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(rings) + (uint32_t)warp * RING_DEPTH * RING_STAGE;

  const int bs = p.seq_index ? p.seq_index[b] : b;
  const float* kbase = p.k_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * HD;
  const float* vbase = p.v_cache + ((int64_t)bs * p.kv_heads + g) * (int64_t)p.max_ctx * HD;

  float m[G], l[G];
  f32x2_t acc[G][DP2];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DP2; ++d) acc[h][d] = 0ull;
  }
  const int n_tiles = (j_end - j_begin + 31) >> 5;
  const int my_tiles = (warp < n_tiles) ? (n_tiles - warp + RING_WARPS - 1) / RING_WARPS : 0;
  const int total = my_tiles * SPT;
  int fs = 0, fslot = 0, rslot = 0;
  // copies stage `fs` of this warp's sequence into ring slot `fslot` (an empty group past the end)
  auto issue = [&]() {
    if (fs < total) {
      const int ti = fs / SPT, st = fs - ti * SPT;
      const int tile = j_begin + 32 * (warp + RING_WARPS * ti);
      const int last = j_end - 1 - tile;
      const uint32_t dst = ring_a + fslot * RING_STAGE;
      if (st < KS) {
        // pieces 8 st .. 8 st + 7 of the tile's 32-row block: [piece][row] in memory and in the stage alike. (Rows past
        // the filled part of the cache hold whatever was there: their scores are masked and never reach a sum.)
        const float* srcg = kbase + (size_t)(tile >> 5) * 32 * HD + (size_t)st * 1024;
#pragma unroll
        for (int j = 0; j < 8; ++j) gv_cp_async16(dst + (j * 32 + lane) * 16, srcg + (j * 32 + lane) * 4, 16u);
      } else {
        const int v0 = (st - KS) * VR;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int idx = j * 32 + lane;
          const int row = v0 + idx / RP, cp = idx - (idx / RP) * RP;
          const int rc = row <= last ? row : last;
          gv_cp_async16(dst + idx * 16, vbase + (size_t)(tile + rc) * HD + cp * 4, 16u);
        }
      }
      ++fs;
    }
    gv_cp_async_commit();
    fslot = (fslot + 1 == RING_DEPTH) ? 0 : fslot + 1;
  };
  auto next_stage = [&]() -> uint32_t {
    gv_cp_async_wait_depth(RING_DEPTH);
    __syncwarp();
    issue();
    const uint32_t src = ring_a + rslot * RING_STAGE;
    rslot = (rslot + 1 == RING_DEPTH) ? 0 : rslot + 1;
    return src;
  };
#pragma unroll 1
  for (int s = 0; s < RING_DEPTH - 1; ++s) issue();
  // (the cached rows are on their way: now fetch this step's query rows)
  const float* qrow = p.qkv + (int64_t)b * p.ld + (int64_t)g * G * HD;
  for (int i = threadIdx.x; i < G * HD; i += RING_WARPS * 32) q_s[i] = qrow[i];
  __syncthreads();
#pragma unroll 1
  for (int ti = 0; ti < my_tiles; ++ti) {
    const int tile = j_begin + 32 * (warp + RING_WARPS * ti);
    const bool valid = tile + lane < j_end;
    const int last = j_end - 1 - tile;
    f32x2_t s2[G];
#pragma unroll
    for (int h = 0; h < G; ++h) s2[h] = 0ull;
#pragma unroll 1
    for (int st = 0; st < KS; ++st) {
      const uint32_t src = next_stage();
#pragma unroll
      for (int pc = 0; pc < 8; ++pc) {
        ulonglong2 k;
        asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(k.x), "=l"(k.y) : "r"(src + (pc * 32 + lane) * 16));
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const ulonglong2 q = *(const ulonglong2*)(q_s + h * HD + st * 32 + pc * 4);
          s2[h] = fma2(q.x, k.x, s2[h]);
          s2[h] = fma2(q.y, k.y, s2[h]);
        }
      }
    }
    __syncwarp();                                      // the previous tile's probabilities have been consumed
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float sc = valid ? sum2(s2[h]) * p.inv_sqrt_d : -INFINITY;
      const float mnew = fmaxf(m[h], warp_max(sc));    // finite: the tile holds at least one row
      const float pj = valid ? expf(sc - mnew) : 0.f;
      const float psum = warp_sum(pj);
      const float corr = expf(m[h] - mnew);            // 0 on the first tile (m = -inf)
      l[h] = l[h] * corr + psum;
      m[h] = mnew;
      const f32x2_t corr2 = pack2(corr, corr);
#pragma unroll
      for (int d = 0; d < DP2; ++d) acc[h][d] = fma2(acc[h][d], corr2, 0ull);
      p_s[h * 32 + lane] = pj;
    }
    __syncwarp();
#pragma unroll 1
    for (int vg = 0; vg < VG; ++vg) {
      const uint32_t src = next_stage();
      if (vg * VR > last) continue;                    // a whole stage of masked rows
#pragma unroll
      for (int r = 0; r < VR; r += 2) {
        f32x2_t v0[DP2], v1[DP2];
        if (DPL == 4) {
          asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v0[0]), "=l"(v0[DP2 - 1]) : "r"(src + r * (HD * 4) + lane * 16));
          asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v1[0]), "=l"(v1[DP2 - 1]) : "r"(src + (r + 1) * (HD * 4) + lane * 16));
        } else {
          asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v0[0]) : "r"(src + r * (HD * 4) + lane * 8));
          asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v1[0]) : "r"(src + (r + 1) * (HD * 4) + lane * 8));
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float2 pr = *(const float2*)(p_s + h * 32 + vg * VR + r);          // the probabilities of two rows
          const f32x2_t p0 = pack2(pr.x, pr.x), p1 = pack2(pr.y, pr.y);
#pragma unroll
          for (int d = 0; d < DP2; ++d) {
            acc[h][d] = fma2(p0, v0[d], acc[h][d]);
            acc[h][d] = fma2(p1, v1[d], acc[h][d]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");       // the rings become the merge area below
  __syncthreads();
  // ---- warps -> shared memory -> one state per head (a warp that had no tile contributes m = -inf, l = 0)
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float* dst = merge_s + ((size_t)warp * G + h) * (HD + 2);
    if (lane == 0) { dst[0] = m[h]; dst[1] = l[h]; }
#pragma unroll
    for (int d = 0; d < DP2; ++d) {
      float lo, hi;
      asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[h][d]));
      dst[2 + lane * DPL + 2 * d] = lo;
      dst[2 + lane * DPL + 2 * d + 1] = hi;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int hh = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < RING_WARPS; ++w) mx = fmaxf(mx, merge_s[((size_t)w * G + hh) * (HD + 2)]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < RING_WARPS; ++w) {
      const float* src = merge_s + ((size_t)w * G + hh) * (HD + 2);
      const float sc = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mx);
      lt += src[1] * sc;
      at += src[2 + d] * sc;
    }
    const int h = g * G + hh;
    if (used == 1) {
      p.out[(int64_t)b * p.ldo + (int64_t)h * HD + d] = (lt > 0.f) ? at / lt : 0.f;
    } else {
      float* dst = p.partial + (((int64_t)b * p.q_heads + h) * p.nsplit + split) * (HD + 2);
      if (d == 0) { dst[0] = mx; dst[1] = lt; }
      dst[2 + d] = at;
    }
  }
}

template <int G, int HD>
static int launch_ring_one(cai_ctx* ctx, dim3 grid, const AttnParams& p) {
  static bool configured[64] = {false};
  const size_t smem = (size_t)ring_smem_bytes(G, HD);
  const int dev = ctx->device;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    CAI_CUDA(ctx, cudaFuncSetAttribute(attn_decode_ring_kernel<G, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  pdl_launch(ctx, attn_decode_ring_kernel<G, HD>, grid, dim3(RING_WARPS * 32), smem, p);
  return CAI_OK;
}
template <int HD>
static int launch_ring(cai_ctx* ctx, int G, dim3 grid, const AttnParams& p) {
  switch (G) {
    case 1: return launch_ring_one<1, HD>(ctx, grid, p);
    case 2: return launch_ring_one<2, HD>(ctx, grid, p);
    case 3: return launch_ring_one<3, HD>(ctx, grid, p);
    case 4: return launch_ring_one<4, HD>(ctx, grid, p);
    case 5: return launch_ring_one<5, HD>(ctx, grid, p);
    case 6: return launch_ring_one<6, HD>(ctx, grid, p);
    case 7: return launch_ring_one<7, HD>(ctx, grid, p);
    default: return launch_ring_one<8, HD>(ctx, grid, p);
  }
}

template <int HD>
static void launch_tile_int8(cai_ctx* ctx, int G, dim3 grid, size_t smem, const AttnParams& p) {
  switch (G) {
    case 1: pdl_launch(ctx, attn_decode_tile_int8_kernel<1, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 2: pdl_launch(ctx, attn_decode_tile_int8_kernel<2, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 3: pdl_launch(ctx, attn_decode_tile_int8_kernel<3, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 4: pdl_launch(ctx, attn_decode_tile_int8_kernel<4, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 5: pdl_launch(ctx, attn_decode_tile_int8_kernel<5, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 6: pdl_launch(ctx, attn_decode_tile_int8_kernel<6, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 7: pdl_launch(ctx, attn_decode_tile_int8_kernel<7, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    default: pdl_launch(ctx, attn_decode_tile_int8_kernel<8, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
  }
}

template <int G, int HD>
static int launch_mma_int8_one(cai_ctx* ctx, dim3 grid, const AttnParams& p) {
  static bool configured[64] = {false};
  const size_t smem = (size_t)i8m_smem_bytes(HD);
  const int dev = ctx->device;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    CAI_CUDA(ctx, cudaFuncSetAttribute(attn_decode_mma_int8_kernel<G, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  pdl_launch(ctx, attn_decode_mma_int8_kernel<G, HD>, grid, dim3(I8M_THREADS), smem, p);
  return CAI_OK;
}
template <int HD>
static int launch_mma_int8(cai_ctx* ctx, int G, dim3 grid, const AttnParams& p) {
  switch (G) {
    case 1: return launch_mma_int8_one<1, HD>(ctx, grid, p);
    case 2: return launch_mma_int8_one<2, HD>(ctx, grid, p);
    case 3: return launch_mma_int8_one<3, HD>(ctx, grid, p);
    case 4: return launch_mma_int8_one<4, HD>(ctx, grid, p);
    default: return launch_mma_int8_one<5, HD>(ctx, grid, p);
  }
}

template <int HD>
static void launch_tile(cai_ctx* ctx, int G, dim3 grid, size_t smem, const AttnParams& p) {
  switch (G) {
    case 1: pdl_launch(ctx, attn_decode_tile_kernel<1, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 2: pdl_launch(ctx, attn_decode_tile_kernel<2, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 3: pdl_launch(ctx, attn_decode_tile_kernel<3, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 4: pdl_launch(ctx, attn_decode_tile_kernel<4, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 5: pdl_launch(ctx, attn_decode_tile_kernel<5, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 6: pdl_launch(ctx, attn_decode_tile_kernel<6, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    case 7: pdl_launch(ctx, attn_decode_tile_kernel<7, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
    default: pdl_launch(ctx, attn_decode_tile_kernel<8, HD>, grid, dim3(ATTN_WARPS * 32), smem, p); break;
  }
}

__global__ void attn_combine_kernel(const AttnParams p) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y;
  const int hd = p.head_dim;
  const float* src = p.partial + ((int64_t)b * p.q_heads + h) * (int64_t)p.nsplit * (hd + 2);
  if (!attn_len_ok(p, p.cache_len[b])) return;
  int base, n;                                         // the step attends over rows [base, n)
  attn_range(p, p.cache_len[b], base, n);
  const int chunk = attn_chunk(n - base, p.nsplit, p.min_chunk);
  const int used = (n - base + chunk - 1) / chunk;
  if (used == 1) return;                              // the single split wrote the output itself
  float mx = -INFINITY;
  for (int s = 0; s < used; ++s) mx = fmaxf(mx, src[(size_t)s * (hd + 2)]);
  float lt = 0.f;
  for (int s = 0; s < used; ++s) {
    const float ms = src[(size_t)s * (hd + 2)];
    lt += src[(size_t)s * (hd + 2) + 1] * ((ms == -INFINITY) ? 0.f : expf(ms - mx));
  }
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float at = 0.f;
    for (int s = 0; s < used; ++s) {
      const float ms = src[(size_t)s * (hd + 2)];
      at += src[(size_t)s * (hd + 2) + 2 + d] * ((ms == -INFINITY) ? 0.f : expf(ms - mx));
    }
    p.out[(int64_t)b * p.ldo + (int64_t)h * hd + d] = (lt > 0.f) ? at / lt : 0.f;
  }
}

int attn_nsplit(cai_ctx* ctx, int batch, int kv_heads, int max_ctx) {
  int64_t ctas = (int64_t)batch * kv_heads;
  int ns = (int)((6 * (int64_t)ctx->sm_count + ctas - 1) / ctas);   // about 6 CTAs of 4 warps per SM
  const int cap = (max_ctx + 63) / 64;                              // at least 64 rows per split at full context
  if (ns > cap) ns = cap;
  if (ns > 128) ns = 128;
  const int forced = env_int("CAI_ATTN_NSPLIT", 0);                  // tuning knob: the number of context splits
  if (forced > 0) ns = forced < 128 ? forced : 128;
  if (ns < 1) ns = 1;
  return ns;
}
size_t attn_partial_floats(int batch, int q_heads, int nsplit, int head_dim) {
  return (size_t)batch * q_heads * nsplit * (head_dim + 2);
}

static AttnParams to_params(cai_ctx* ctx, const AttnArgs& a) {
  AttnParams p;
  p.err = ctx->err_flag;
  p.qkv = a.qkv; p.ld = a.ld; p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.cache_len = a.cache_len_dev;
  p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.head_dim = a.head_dim; p.max_ctx = a.max_ctx;
  p.theta = a.theta; p.pos = a.pos_dev; p.q_norm = a.q_norm; p.k_norm = a.k_norm; p.eps = a.eps;
  p.out = a.out; p.ldo = a.ldo; p.partial = a.partial; p.nsplit = a.nsplit;
  p.inv_sqrt_d = (float)(1.0 / sqrt((double)a.head_dim));
  p.min_chunk = ATTN_MIN_CHUNK;
  p.k_codes = a.k_codes; p.v_codes = a.v_codes; p.k_scales = a.k_scales; p.v_scales = a.v_scales;
  p.seq_index = a.seq_index_dev;
  p.k_blocked = a.k_blocked;
  p.window = a.window; p.evict_sinks = a.evict_sinks; p.evict_window = a.evict_window;
  return p;
}

// true when the int8 KV cache can serve this shape (the tiled kernels only)
// true when the fp32 K cache of this shape may use the block-transposed layout (the tiled kernel serves it)
bool attn_k_blocked_supported(int q_heads, int kv_heads, int head_dim) {
  static const int use_tile = [] { const char* e = getenv("CAI_ATTN_TILE"); return (e && *e) ? atoi(e) : 1; }();
  return use_tile && kv_heads > 0 && (q_heads % kv_heads) == 0 && (q_heads / kv_heads) <= 8 && (head_dim == 64 || head_dim == 128);
}
bool attn_int8_supported(int q_heads, int kv_heads, int head_dim) {
  return kv_heads > 0 && (q_heads % kv_heads) == 0 && (q_heads / kv_heads) <= 8 && (head_dim == 64 || head_dim == 128);
}

int attn_rope_append(cai_ctx* ctx, const AttnArgs& a) {
  ctx->cur_family = FAM_ATTN;
  if (a.head_dim % 2) return cai_fail(ctx, CAI_ERR_INVALID, "head_dim must be even");
  if (a.k_codes) {
    const size_t smem = (size_t)2 * a.kv_heads * a.head_dim * sizeof(float);
    if (smem > 48 * 1024) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "int8 KV append: %d kv heads x %d dims exceed shared memory", a.kv_heads, a.head_dim);
    pdl_launch(ctx, rope_append_int8_kernel, dim3(a.batch), dim3(256), smem, to_params(ctx, a));
    CAI_LAUNCHED(ctx);
    return CAI_OK;
  }
  pdl_launch(ctx, rope_append_kernel, dim3(a.batch), dim3(256), 0, to_params(ctx, a));
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

int attn_decode(cai_ctx* ctx, const AttnArgs& a) {
  ctx->cur_family = FAM_ATTN;
  if (a.q_heads % a.kv_heads) return cai_fail(ctx, CAI_ERR_INVALID, "q_heads %d not a multiple of kv_heads %d", a.q_heads, a.kv_heads);
  if (a.head_dim > 256 || a.head_dim < 2) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "head_dim %d outside 2..256", a.head_dim);
  if (a.nsplit > 1 && !a.partial) return cai_fail(ctx, CAI_ERR_INVALID, "split attention without scratch");
  const int G = a.q_heads / a.kv_heads;
  int lpk = 1;
  while (lpk * 8 < a.head_dim) lpk <<= 1;
  AttnParams p = to_params(ctx, a);
  dim3 grid(a.kv_heads, a.nsplit, a.batch);
  static const int use_tile = [] { const char* e = getenv("CAI_ATTN_TILE"); return (e && *e) ? atoi(e) : 1; }();
  if (a.k_codes) {
    if (!attn_int8_supported(a.q_heads, a.kv_heads, a.head_dim))
      return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "int8 KV cache: head_dim 64 or 128 and groups of up to 8 query heads");
    p.min_chunk = ATTN_TILE_MIN_CHUNK;
    const size_t tsmem = ((size_t)G * a.head_dim + (size_t)ATTN_WARPS * G * 32 + (size_t)ATTN_WARPS * G * (a.head_dim + 2)) * sizeof(float);
    // Groups of 2 to 5 query heads run on the integer tensor-core kernel when their splits are long. Its cost per cached
    // byte does not depend on the group (the instruction's 16 rows are there anyway) while the CUDA-core kernel's grows
    // with it, and it starts slower (the query's limbs, two warps per CTA). Measured per 64 layers: groups of 5, 64
    // sequences x 8192 rows 28.2 -> 17.9 ms; one sequence in 128-row splits 3.30 -> 3.45 ms; groups of 1 (OLMoE, 64
    // sequences x 2048 rows, 16 layers) 2.13 -> 2.30 ms. So: splits of 512 rows or more at full context and at least
    // two heads per group. CAI_ATTN_I8MMA=1 / 0 forces it on / off; read at every call so that a test can switch it.
    const char* mma_env = getenv("CAI_ATTN_I8MMA");
    const bool use_mma = (mma_env && *mma_env) ? atoi(mma_env) != 0 : (G >= 2 && a.max_ctx / (a.nsplit > 0 ? a.nsplit : 1) >= 512);
    if (use_mma && G <= 5) {
      if (a.head_dim == 128) { CAI_TRY(launch_mma_int8<128>(ctx, G, grid, p)); }
      else { CAI_TRY(launch_mma_int8<64>(ctx, G, grid, p)); }
    } else if (a.head_dim == 128) launch_tile_int8<128>(ctx, G, grid, tsmem, p);
    else launch_tile_int8<64>(ctx, G, grid, tsmem, p);
    CAI_LAUNCHED(ctx);
    if (a.nsplit > 1) {
      dim3 cgrid(a.q_heads, a.batch);
      pdl_launch(ctx, attn_combine_kernel, cgrid, dim3(128), 0, p);
      CAI_LAUNCHED(ctx);
    }
    return CAI_OK;
  }
  if (a.k_blocked && !(use_tile && (a.head_dim == 128 || a.head_dim == 64) && G <= 8 && (a.max_ctx % 32) == 0))
    return cai_fail(ctx, CAI_ERR_STATE, "internal: block-transposed K cache outside the tiled attention kernel");
  static const int use_ring = [] { const char* e = getenv("CAI_ATTN_RING"); return (e && *e) ? atoi(e) : 1; }();
  if (use_tile && use_ring && a.k_blocked && a.window <= 0 && (a.head_dim == 128 || a.head_dim == 64) && G <= 8) {
    // the cp.async kernel: rows [0, n) of the block-transposed cache. Three CTAs fit an SM (64 KB of rings each), so
    // the full context is cut into about that many splits: one wave, every warp walking several tiles through its ring
    p.min_chunk = ATTN_TILE_MIN_CHUNK;
    {
      const int64_t lanes = (int64_t)a.batch * a.kv_heads;
      const int64_t target = (3 * (int64_t)ctx->sm_count) / lanes;
      if (target >= 1) {
        const int mc = (int)((((int64_t)a.max_ctx + target - 1) / target + 31) & ~(int64_t)31);
        if (mc > p.min_chunk) p.min_chunk = mc;
      }
    }
    CAI_TRY(a.head_dim == 128 ? launch_ring<128>(ctx, G, grid, p) : launch_ring<64>(ctx, G, grid, p));
    CAI_LAUNCHED(ctx);
    if (a.nsplit > 1) {
      dim3 cgrid(a.q_heads, a.batch);
      pdl_launch(ctx, attn_combine_kernel, cgrid, dim3(128), 0, p);
      CAI_LAUNCHED(ctx);
    }
    return CAI_OK;
  }
  if (use_tile && (a.head_dim == 128 || a.head_dim == 64) && G <= 8) {
    p.min_chunk = ATTN_TILE_MIN_CHUNK;
    const size_t tsmem = ((size_t)G * a.head_dim + (size_t)ATTN_WARPS * G * 64 + (size_t)ATTN_WARPS * G * (a.head_dim + 2)) * sizeof(float);
    if (a.head_dim == 128) launch_tile<128>(ctx, G, grid, tsmem, p);
    else launch_tile<64>(ctx, G, grid, tsmem, p);
    CAI_LAUNCHED(ctx);
    if (a.nsplit > 1) {
      dim3 cgrid(a.q_heads, a.batch);
      pdl_launch(ctx, attn_combine_kernel, cgrid, dim3(128), 0, p);
      CAI_LAUNCHED(ctx);
    }
    return CAI_OK;
  }
  p.min_chunk = ATTN_MIN_CHUNK;
  const int gt = G >= 8 ? 8 : G;
  const size_t smem = ((size_t)G * a.head_dim + (size_t)ATTN_WARPS * gt * (a.head_dim + 2)) * sizeof(float);
  if (smem > 48 * 1024) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "attention group of %d heads x %d dims exceeds shared memory", G, a.head_dim);
  switch (gt) {
    case 1: pdl_launch(ctx, attn_decode_kernel<1>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 2: pdl_launch(ctx, attn_decode_kernel<2>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 3: pdl_launch(ctx, attn_decode_kernel<3>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 4: pdl_launch(ctx, attn_decode_kernel<4>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 5: pdl_launch(ctx, attn_decode_kernel<5>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 6: pdl_launch(ctx, attn_decode_kernel<6>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    case 7: pdl_launch(ctx, attn_decode_kernel<7>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
    default: pdl_launch(ctx, attn_decode_kernel<8>, grid, dim3(ATTN_WARPS * 32), smem, p, lpk); break;
  }
  CAI_LAUNCHED(ctx);
  if (a.nsplit > 1) {
    dim3 cgrid(a.q_heads, a.batch);
    pdl_launch(ctx, attn_combine_kernel, cgrid, dim3(128), 0, p);
    CAI_LAUNCHED(ctx);
  }
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free decode step.
//
// Some hosts may not allocate device memory when they call into this library:
// a real-time audio or control loop that must not block in the driver's
// allocator, a plugin that was handed a fixed arena by its embedding
// application, or a process whose device-memory budget was fixed at start-up.
// For them the split-context partial results live in the fixed array below,
// which is part of the library image: every GPU that loads the library holds
// these 2 MiB until the process exits.
// ---------------------------------------------------------------------------
#define CAI_SDPA_NOALLOC_MAX_FLOATS (512 * 1024)
static __device__ __align__(256) float g_sdpa_noalloc_scratch[CAI_SDPA_NOALLOC_MAX_FLOATS];

// Device address of the array above, looked up once per device. In host code the symbol
// g_sdpa_noalloc_scratch is only a handle, not an address the GPU can use.
static float* g_sdpa_noalloc_ptr[64] = {nullptr};

extern "C" int cai_sdpa_step_noalloc(cai_ctx* ctx, float* qkv_row_dev, float* k_cache_dev, float* v_cache_dev,
                                     const int32_t* cache_len_dev, int q_heads, int kv_heads, int head_dim, int max_ctx,
                                     float* out_dev) {
  CAI_TRY(cai_bind(ctx));
  if (!qkv_row_dev || !k_cache_dev || !v_cache_dev || !cache_len_dev || !out_dev)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_sdpa_step_noalloc: null buffer");
  if (q_heads < 1 || kv_heads < 1 || (q_heads % kv_heads) || head_dim < 2 || (head_dim % 2) || head_dim > 256 || max_ctx < 1)
    return cai_fail(ctx, CAI_ERR_INVALID, "cai_sdpa_step_noalloc: heads %d/%d head_dim %d ctx %d", q_heads, kv_heads, head_dim, max_ctx);
  if (ctx->device < 0 || ctx->device >= 64) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "cai_sdpa_step_noalloc: device index %d", ctx->device);
  const int nsplit = attn_nsplit(ctx, 1, kv_heads, max_ctx);
  const size_t need = attn_partial_floats(1, q_heads, nsplit, head_dim);
  if (need > (size_t)CAI_SDPA_NOALLOC_MAX_FLOATS)
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED,
                    "cai_sdpa_step_noalloc: %d heads x %d context splits x %d dims need %zu scratch floats, the built-in "
                    "scratch holds %d; use cai_sdpa_create / cai_sdpa_step_dev for this shape",
                    q_heads, nsplit, head_dim, need, CAI_SDPA_NOALLOC_MAX_FLOATS);
  if (!g_sdpa_noalloc_ptr[ctx->device]) {
    // first call on this device (current device == ctx->device after cai_bind)
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_sdpa_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return cai_fail(ctx, CAI_ERR_CUDA, "cudaGetSymbolAddress(scratch) -> %s", cudaGetErrorString(e));
    g_sdpa_noalloc_ptr[ctx->device] = ptr;
  }
  AttnArgs a;
  a.qkv = qkv_row_dev; a.ld = (int64_t)(q_heads + 2 * kv_heads) * head_dim;
  a.k_cache = k_cache_dev; a.v_cache = v_cache_dev; a.cache_len_dev = cache_len_dev;
  a.batch = 1; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.max_ctx = max_ctx;
  a.out = out_dev; a.ldo = (int64_t)q_heads * head_dim;
  a.partial = g_sdpa_noalloc_ptr[ctx->device];   // every slot the combine kernel reads is written first: nothing to clear
  a.nsplit = nsplit;
  CAI_TRY(attn_rope_append(ctx, a));
  CAI_TRY(attn_decode(ctx, a));
  return CAI_OK;
}
