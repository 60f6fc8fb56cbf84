// Token sampling on the device: temperature, top-k, nucleus (top-p) truncation and the weighted draw, so that a sampled
// generation does not ship the whole logits row (600 KB at a 152k vocabulary) to the host for every token, nor sort it
// there.
//
// What is restated: TNNetTemperatureProcessor (logits / T before the softmax, neural/neuralchatengine.pas:1387-1388),
// the candidate window of TNNetSamplerBase (post-softmax scores sorted descending, truncated to the top K:
// SelectTopCandidates, neural/neuralvolume.pas:991-1030) and the draw of TNNetSamplerWeightedTopK.SampleFromSorted
// (:4749-4785): Roll = u * KeptSum, the first candidate whose running sum exceeds Roll. The uniform number u is the
// caller's (cai_session_step_topk hands the window to the host, whose own sampler and Random then decide) or comes from
// a counter-based generator keyed by (seed, step, sequence) that cai_sampling_uniform reproduces on the host.
//
// Two kernels per step and sequence:
//   sample_chunks_kernel  the vocabulary cut into SAMPLE_CHUNKS pieces, one CTA each: the piece's maximum and
//                         sum of exp((x - max) / T), and its k largest logits (k rounds of a block-wide first-maximum);
//   sample_merge_kernel   one CTA per sequence: the k largest of the SAMPLE_CHUNKS * k candidates in descending order
//                         (ties: lowest index first), their probabilities against the full-row denominator, nucleus cut,
//                         the draw; the sampled token replaces the greedy one the step left in the session's words.
#include "cai_common.cuh"
#include <math.h>

#define SAMPLE_CHUNKS 128
#define SAMPLE_MAX_K 64

__host__ __device__ static inline uint64_t sample_mix(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
// uniform in [0, 1) with 24 bits, keyed by (seed, step, sequence)
__host__ __device__ static inline float sample_uniform(uint64_t seed, uint64_t step, uint64_t seq) {
  const uint64_t u = sample_mix(sample_mix(seed ^ (step * 0xD6E8FEB86659FD93ull)) + seq);
  return (float)(u >> 40) * 5.9604644775390625e-8f;
}

__device__ __forceinline__ void first_max_merge(float& best, int& besti, float ob, int oi) {
  if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
}
// block-wide first maximum of (v, i); every thread gets the result. sv/si: 32 entries each.
__device__ __forceinline__ void block_first_max(float& v, int& i, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) first_max_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
  __syncthreads();
  if (lane == 0) { sv[warp] = v; si[warp] = i; }
  __syncthreads();
  v = (lane < nw) ? sv[lane] : -INFINITY;
  i = (lane < nw) ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) first_max_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
}

// grid (SAMPLE_CHUNKS, batch). Dynamic shared memory: the chunk's logits.
__global__ void __launch_bounds__(256) sample_chunks_kernel(const float* __restrict__ logits, int64_t ld, int n, int k, float inv_t,
                                                            float* __restrict__ chunk_max, float* __restrict__ chunk_sum,
                                                            float* __restrict__ cand_val, int* __restrict__ cand_idx) {
  extern __shared__ float xs[];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float red[32];
  const int c = blockIdx.x, b = blockIdx.y;
  const float* row = logits + (int64_t)b * ld;
  const int per = (n + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
  const int lo = c * per;
  int hi = lo + per; if (hi > n) hi = n;
  const int cnt = hi > lo ? hi - lo : 0;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
    float v = row[lo + i];
    if (!(v == v)) v = -INFINITY;                       // a NaN logit can never be drawn
    xs[i] = v;
  }
  __syncthreads();
  // the chunk's maximum (logits may be negative: a first-maximum reduction, not the non-negative block_max)
  {
    float v = -INFINITY; int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) first_max_merge(v, idx, xs[i], lo + i);
    block_first_max(v, idx, sv, si);
    m = v;
  }
  float s = 0.f;
  if (m > -INFINITY)
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) s += expf((xs[i] - m) * inv_t);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    chunk_max[(size_t)b * SAMPLE_CHUNKS + c] = m;
    chunk_sum[(size_t)b * SAMPLE_CHUNKS + c] = s;
  }
  // the chunk's k largest, descending, ties to the lower index
  for (int j = 0; j < k; ++j) {
    float v = -INFINITY; int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) first_max_merge(v, idx, xs[i], lo + i);
    block_first_max(v, idx, sv, si);
    if (threadIdx.x == 0) {
      cand_val[((size_t)b * SAMPLE_CHUNKS + c) * SAMPLE_MAX_K + j] = v;
      cand_idx[((size_t)b * SAMPLE_CHUNKS + c) * SAMPLE_MAX_K + j] = (v > -INFINITY) ? idx : -1;
      if (v > -INFINITY) xs[idx - lo] = -INFINITY;      // taken
    }
    __syncthreads();
  }
}

struct SampleMergeParams {
  const float* chunk_max; const float* chunk_sum; const float* cand_val; const int* cand_idx;
  int k; float inv_t; float top_p;
  unsigned long long seed;
  const float* uniforms;        // optional [batch]: the caller's uniform numbers instead of the generator's
  int32_t* ids_out; float* probs_out;       // optional [batch][k]: the window itself
  // optional: write the drawn token into the session's words (replacing the greedy token of the step just finished)
  int32_t* tokens; int32_t* trace; const int32_t* trace_count; int batch; long long trace_cap;
  int32_t* drawn_out;           // optional [batch]
};

// grid (batch), 1024 threads.
__global__ void __launch_bounds__(1024) sample_merge_kernel(const SampleMergeParams p) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float red[32];
  __shared__ float win_v[SAMPLE_MAX_K];
  __shared__ int win_i[SAMPLE_MAX_K];
  const int b = blockIdx.x;
  const float* cmax = p.chunk_max + (size_t)b * SAMPLE_CHUNKS;
  const float* csum = p.chunk_sum + (size_t)b * SAMPLE_CHUNKS;
  const float* cval = p.cand_val + (size_t)b * SAMPLE_CHUNKS * SAMPLE_MAX_K;
  const int* cidx = p.cand_idx + (size_t)b * SAMPLE_CHUNKS * SAMPLE_MAX_K;
  // full-row maximum and denominator of softmax(x / T)
  float M = -INFINITY;
  for (int c = threadIdx.x; c < SAMPLE_CHUNKS; c += blockDim.x) M = fmaxf(M, cmax[c]);
  { int dummy = 0; float v = M; block_first_max(v, dummy, sv, si); M = v; }
  float S = 0.f;
  for (int c = threadIdx.x; c < SAMPLE_CHUNKS; c += blockDim.x)
    if (cmax[c] > -INFINITY) S += csum[c] * expf((cmax[c] - M) * p.inv_t);
  S = block_sum(S, red);
  // The k largest of the chunks' candidates. A chunk's list is descending, so its next untaken entry is its best:
  // thread c < SAMPLE_CHUNKS keeps a cursor into chunk c's list; k rounds of a first-maximum over the cursors.
  int cur = 0;
  for (int j = 0; j < p.k; ++j) {
    float v = -INFINITY; int idx = 0x7fffffff;
    if (threadIdx.x < SAMPLE_CHUNKS && cur < p.k) {
      const int id = cidx[threadIdx.x * SAMPLE_MAX_K + cur];
      if (id >= 0) { v = cval[threadIdx.x * SAMPLE_MAX_K + cur]; idx = id; }
    }
    const int mine = idx;
    block_first_max(v, idx, sv, si);
    if (threadIdx.x < SAMPLE_CHUNKS && mine == idx && idx != 0x7fffffff) ++cur;
    if (threadIdx.x == 0) { win_v[j] = v; win_i[j] = (v > -INFINITY) ? idx : -1; }
    __syncthreads();
  }
  if (threadIdx.x != 0) return;
  // probabilities of the window against the full-row denominator; nucleus cut; the weighted draw
  float probs[SAMPLE_MAX_K];
  int kept = 0;
  for (int j = 0; j < p.k; ++j) {
    if (win_i[j] < 0) break;
    probs[j] = expf((win_v[j] - M) * p.inv_t) / S;
    ++kept;
  }
  if (p.ids_out) {
    for (int j = 0; j < p.k; ++j) {
      p.ids_out[(size_t)b * p.k + j] = j < kept ? win_i[j] : -1;
      p.probs_out[(size_t)b * p.k + j] = j < kept ? probs[j] : 0.f;
    }
  }
  if (!p.tokens && !p.drawn_out) return;
  int n_keep = kept;
  if (p.top_p > 0.f && p.top_p < 1.f) {
    float cum = 0.f;
    for (int j = 0; j < kept; ++j) {
      cum += probs[j];
      if (cum > p.top_p) { n_keep = j + 1; break; }     // the candidate that crosses the mass stays in
    }
  }
  float kept_sum = 0.f;
  for (int j = 0; j < n_keep; ++j) kept_sum += probs[j];
  int pick = kept > 0 ? win_i[0] : 0;
  if (kept_sum > 0.f) {
    unsigned long long step = p.trace_count ? (unsigned long long)*p.trace_count : 0ull;
    const float u = p.uniforms ? p.uniforms[b] : sample_uniform(p.seed, step, (unsigned long long)b);
    const float roll = u * kept_sum;
    float cum = 0.f;
    pick = win_i[n_keep - 1];                           // numeric-safety fallback
    for (int j = 0; j < n_keep; ++j) {
      cum += probs[j];
      if (roll < cum) { pick = win_i[j]; break; }
    }
  }
  if (p.drawn_out) p.drawn_out[b] = pick;
  if (p.tokens) {
    p.tokens[b] = pick;
    const int cnt = *p.trace_count;                     // the step has already counted itself
    if (cnt >= 1 && (long long)cnt * p.batch <= p.trace_cap) p.trace[(long long)(cnt - 1) * p.batch + b] = pick;
  }
}

int sample_scratch_floats(int batch) { return batch * SAMPLE_CHUNKS * (2 + 2 * SAMPLE_MAX_K); }

// logits [batch][ld] on the device; scratch: sample_scratch_floats(batch) floats.
int sample_launch(cai_ctx* ctx, const float* logits, int64_t ld, int batch, int vocab, int k, float temperature, float top_p,
                  unsigned long long seed, const float* uniforms_dev, float* scratch, int32_t* ids_out_dev, float* probs_out_dev,
                  int32_t* tokens_dev, int32_t* trace_dev, const int32_t* trace_count_dev, long long trace_cap, int32_t* drawn_out_dev) {
  if (k < 1 || k > SAMPLE_MAX_K) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "sampling window of %d candidates: 1..%d", k, SAMPLE_MAX_K);
  if (!(temperature > 0.f)) return cai_fail(ctx, CAI_ERR_INVALID, "temperature %g must be positive", (double)temperature);
  const int per = (vocab + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
  if ((size_t)per * 4 > 40 * 1024) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "vocabulary of %d rows exceeds the sampler's chunks", vocab);
  float* chunk_max = scratch;
  float* chunk_sum = chunk_max + (size_t)batch * SAMPLE_CHUNKS;
  float* cand_val = chunk_sum + (size_t)batch * SAMPLE_CHUNKS;
  int* cand_idx = (int*)(cand_val + (size_t)batch * SAMPLE_CHUNKS * SAMPLE_MAX_K);
  ctx->cur_family = FAM_OTHER;
  sample_chunks_kernel<<<dim3(SAMPLE_CHUNKS, batch), 256, (size_t)per * 4, ctx->stream>>>(logits, ld, vocab, k, 1.0f / temperature, chunk_max,
                                                                                         chunk_sum, cand_val, cand_idx);
  CAI_LAUNCHED(ctx);
  SampleMergeParams p;
  memset(&p, 0, sizeof(p));
  p.chunk_max = chunk_max; p.chunk_sum = chunk_sum; p.cand_val = cand_val; p.cand_idx = cand_idx;
  p.k = k; p.inv_t = 1.0f / temperature; p.top_p = top_p; p.seed = seed; p.uniforms = uniforms_dev;
  p.ids_out = ids_out_dev; p.probs_out = probs_out_dev; p.tokens = tokens_dev; p.trace = trace_dev; p.trace_count = trace_count_dev;
  p.batch = batch; p.trace_cap = trace_cap; p.drawn_out = drawn_out_dev;
  sample_merge_kernel<<<batch, 1024, 0, ctx->stream>>>(p);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

extern "C" int cai_sampling_uniform(uint64_t seed, uint64_t step, uint64_t seq, float* out_u) {
  if (!out_u) return CAI_ERR_INVALID;
  *out_u = sample_uniform(seed, step, seq);
  return CAI_OK;
}
