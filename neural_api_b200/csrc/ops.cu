// Small per-token operators of the decode step: embedding gather, RMSNorm, RoPE,
// SwiGLU, router softmax/top-k, argmax, MoE combine.
#include "cai_common.cuh"
#include "gguf_blocks.cuh"
#include <math.h>

// ---------------------------------------------------------------------------
// embedding gather: out[b][c] = dequant(table[token_b][c])   (EncodeZero = 1:
// token 0 is a real row)
// ---------------------------------------------------------------------------
__global__ void embed_kernel(int type, const void* __restrict__ codes, const __half* __restrict__ scales,
                             int64_t sstride, int64_t k, int64_t n_rows, const int32_t* __restrict__ tokens, float* __restrict__ out, int64_t ld,
                             const float* __restrict__ rscale, int* err) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  int64_t tok = tokens[b];
  if ((tok < 0 || tok >= n_rows) && threadIdx.x == 0) cai_report_index(err, CAI_SITE_EMBED_TOKEN, tok, n_rows);
  if (tok < 0) tok = 0;
  if (tok >= n_rows) tok = n_rows - 1;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    float v;
    const int64_t i = tok * k + c;
    if (type == CAI_TYPE_Q8_0) v = __half2float(scales[tok * sstride + c / CAI_QK]) * (float)((int)((const uint8_t*)codes)[i] - 128);
    else if (type == CAI_TYPE_Q4_0) {
      const int64_t blk = i / CAI_QK;
      const int e = (int)(i % CAI_QK);
      const uint8_t byte = ((const uint8_t*)codes)[blk * 16 + (e & 15)];
      const int nib = (e < 16) ? (byte & 0x0F) : (byte >> 4);
      v = __half2float(scales[tok * sstride + c / CAI_QK]) * (float)(nib - 8);
    } else if (type == CAI_TYPE_I8ROW) v = rscale[tok] * (float)((int)((const uint8_t*)codes)[i] - 128);
    else if (type == CAI_TYPE_F16) v = __half2float(((const __half*)codes)[i]);
    else if (type == CAI_TYPE_Q4_K || type == CAI_TYPE_Q5_K || type == CAI_TYPE_Q6_K) {
      const int bb = type == CAI_TYPE_Q4_K ? 144 : (type == CAI_TYPE_Q5_K ? 176 : 210);
      v = ggufdev::decode_element(type, (const uint8_t*)codes + (i >> 8) * bb, (int)(i & 255));
    }
    else v = ((const float*)codes)[i];
    out[(int64_t)b * ld + c] = v;
  }
}

int op_embed(cai_ctx* ctx, const QWeight* t, const int32_t* tokens_dev, int batch, float* out, int64_t ld) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, embed_kernel, dim3(batch), dim3(256), 0, t->type, (const void*)t->codes, (const __half*)t->scales, t->sstride, t->k, t->n, tokens_dev, out, ld, (const float*)t->rscale, ctx->err_flag);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// RMSNorm per token: inv = 1/sqrt(mean(x^2) + eps); y = gain * (x * inv)
// ---------------------------------------------------------------------------
__global__ void rmsnorm_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ gain,
                               float* __restrict__ y, int64_t ldy, int depth, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const float* xr = x + (int64_t)blockIdx.x * ldx;
  float* yr = y + (int64_t)blockIdx.x * ldy;
  float ss = 0.f;
  for (int c = threadIdx.x; c < depth; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)depth + eps);
  for (int c = threadIdx.x; c < depth; c += blockDim.x) yr[c] = gain[c] * (xr[c] * inv);
}

int op_rmsnorm(cai_ctx* ctx, const float* x, int64_t ldx, const float* gain, float* y, int64_t ldy, int tokens, int depth, float eps) {
  ctx->cur_family = FAM_OTHER;
  int threads = depth >= 2048 ? 512 : (depth >= 512 ? 256 : 128);
  pdl_launch(ctx, rmsnorm_kernel, dim3(tokens), dim3(threads), 0, x, ldx, gain, y, ldy, depth, eps);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// RoPE on interleaved pairs (2k, 2k+1); angle = (float)pos * theta[k] in fp32,
// full-range sincosf.
// ---------------------------------------------------------------------------
__global__ void rope_theta_kernel(float* theta, int half, int head_dim, double log_base) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k < half) theta[k] = (float)exp(-2.0 * (double)k / (double)head_dim * log_base);
}
int op_rope_theta_table(cai_ctx* ctx, float* theta_dev, int head_dim, float base) {
  ctx->cur_family = FAM_OTHER;
  const int half = head_dim / 2;
  rope_theta_kernel<<<(half + 127) / 128, 128, 0, ctx->stream>>>(theta_dev, half, head_dim, log((double)base));
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

__global__ void rope_kernel(float* __restrict__ x, int64_t ldx, int depth, int head_dim, const float* __restrict__ theta,
                            const int32_t* __restrict__ pos_dev, int pos_stride, int pos_offset) {
  const int t = blockIdx.x;
  const int pos = (pos_dev ? pos_dev[t * pos_stride] : t) + pos_offset;
  const int half_hd = head_dim >> 1;
  float* xr = x + (int64_t)t * ldx;
  for (int pr = threadIdx.x; pr < (depth >> 1); pr += blockDim.x) {
    const int k = pr % half_hd;
    const float angle = (float)pos * theta[k];
    float s, c;
    sincosf(angle, &s, &c);
    const float x0 = xr[2 * pr], x1 = xr[2 * pr + 1];
    xr[2 * pr] = c * x0 - s * x1;
    xr[2 * pr + 1] = s * x0 + c * x1;
  }
}

int op_rope(cai_ctx* ctx, float* x, int64_t ldx, int tokens, int depth, int head_dim, const float* theta_dev,
            const int32_t* pos_dev, int pos_stride, int pos_offset) {
  ctx->cur_family = FAM_OTHER;
  rope_kernel<<<tokens, 128, 0, ctx->stream>>>(x, ldx, depth, head_dim, theta_dev, pos_dev, pos_stride, pos_offset);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// SwiGLU: y[d] = x[d] * swish(x[half + d])   (first half = up, second = gate)
// ---------------------------------------------------------------------------
__global__ void swiglu_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy, int half) {
  const float* xr = x + (int64_t)blockIdx.y * ldx;
  float* yr = y + (int64_t)blockIdx.y * ldy;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= half) return;
  const float a = xr[d], b = xr[half + d];
  float sig;
  if (b > 0.f) sig = 1.0f / (1.0f + expf(-b));
  else { const float s = expf(b); sig = s / (1.0f + s); }
  yr[d] = a * (b * sig);
}
int op_swiglu(cai_ctx* ctx, const float* x, int64_t ldx, float* y, int64_t ldy, int tokens, int half) {
  ctx->cur_family = FAM_OTHER;
  dim3 grid((half + 255) / 256, tokens);
  swiglu_kernel<<<grid, 256, 0, ctx->stream>>>(x, ldx, y, ldy, half);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// Router: softmax over all experts, keep top-k (ties: lowest index), optional
// renormalisation of the survivors. One warp per token.
// ---------------------------------------------------------------------------
__global__ void topk_gate_kernel(const float* __restrict__ logits, int tokens, int n_experts, int top_k, int renorm,
                                 int32_t* __restrict__ ids, float* __restrict__ gates, int* __restrict__ err) {
  extern __shared__ float probs_all[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* probs = probs_all + (size_t)warp * n_experts;
  const float* row = logits + (int64_t)t * n_experts;
  float m = -INFINITY;
  for (int e = lane; e < n_experts; e += 32) m = fmaxf(m, row[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < n_experts; e += 32) { const float v = expf(row[e] - m); probs[e] = v; sum += v; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < n_experts; e += 32) probs[e] = probs[e] / sum;
  __syncwarp();
  float kept_sum = 0.f;
  for (int s = 0; s < top_k; ++s) {
    float best = -INFINITY; int besti = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = probs[e];
      if (v >= 0.f && (v > best || (v == best && e < besti))) { best = v; besti = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (besti == 0x7fffffff) {
      // No candidate: the row holds NaN (or only -inf) logits, so no probability compares >= 0. Keep the ids in
      // range (slot s takes expert s, which no earlier slot can hold when the whole row is unusable; otherwise the
      // lowest untaken expert), give the slot no weight, and raise the error word: one non-finite activation
      // must end as a status, not as an out-of-range expert index in the kernels that follow.
      int pick = 0;
      for (int e = 0; e < n_experts; ++e) if (probs[e] != -1.0f) { pick = e; break; }
      besti = pick; best = 0.f;
      if (lane == 0 && err) *err = 3;
    }
    if (lane == 0) {
      ids[(int64_t)t * top_k + s] = besti;
      gates[(int64_t)t * top_k + s] = best;
      probs[besti] = -1.0f;   // taken
    }
    kept_sum += best;
    __syncwarp();
  }
  if (renorm && lane == 0 && kept_sum > 0.f)
    for (int s = 0; s < top_k; ++s) gates[(int64_t)t * top_k + s] = gates[(int64_t)t * top_k + s] / kept_sum;
}

int op_topk_gate(cai_ctx* ctx, const float* logits, int tokens, int n_experts, int top_k, int renorm,
                 int32_t* ids, float* gates) {
  ctx->cur_family = FAM_OTHER;
  if (top_k < 1 || top_k > n_experts) return cai_fail(ctx, CAI_ERR_INVALID, "top_k %d of %d experts", top_k, n_experts);
  const int warps = 4;
  const size_t smem = (size_t)warps * n_experts * sizeof(float);
  if (smem > 48 * 1024) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "router with %d experts exceeds the kernel's shared memory", n_experts);
  pdl_launch(ctx, topk_gate_kernel, dim3((tokens + warps - 1) / warps), dim3(warps * 32), smem, logits, tokens, n_experts, top_k, renorm, ids, gates, ctx->err_flag);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// argmax: first index of the maximum of each row. The row is cut into ARGMAX_CHUNKS pieces, one CTA
// each; the last CTA of a row to finish (atomic ticket, no waiting) merges the per-chunk winners in
// chunk order, so the result does not depend on timing. Tickets reset themselves.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void argmax_merge(float& best, int& besti, float ob, int oi) {
  if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
}
__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int n, int32_t* __restrict__ out_idx,
                              float* __restrict__ out_val, float* __restrict__ part_val, int* __restrict__ part_idx,
                              int* __restrict__ tickets) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_last;
  pdl_trigger();
  pdl_wait();
  const int row_id = blockIdx.y, chunk = blockIdx.x, chunks = gridDim.x;
  const float* row = logits + (int64_t)row_id * ld;
  const int per = (n + chunks - 1) / chunks;
  const int lo = chunk * per;
  int hi = lo + per; if (hi > n) hi = n;
  float best = -INFINITY; int besti = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; besti = i; }      // strided scan keeps the first index per thread
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, besti, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, besti, o));
  if (lane == 0) { sv[warp] = best; si[warp] = besti; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = (lane < nw) ? sv[lane] : -INFINITY;
    besti = (lane < nw) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_merge(best, besti, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, besti, o));
    if (lane == 0) {
      __stcg(part_val + (size_t)row_id * chunks + chunk, best);
      __stcg(part_idx + (size_t)row_id * chunks + chunk, besti);
      __threadfence();
      const int old = atomicAdd(tickets + row_id, 1);
      s_last = (old == chunks - 1) ? 1 : 0;
      if (old == chunks - 1) tickets[row_id] = 0;
    }
  }
  __syncthreads();
  if (!s_last || warp != 0) return;
  __threadfence();
  best = -INFINITY; besti = 0x7fffffff;
  for (int c = lane; c < chunks; c += 32)
    argmax_merge(best, besti, __ldcg(part_val + (size_t)row_id * chunks + c), __ldcg(part_idx + (size_t)row_id * chunks + c));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, besti, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, besti, o));
  if (lane == 0) {
    if (besti == 0x7fffffff) besti = 0;          // every entry NaN or -inf: index 0, like a scan that never updates
    out_idx[row_id] = besti;
    if (out_val) out_val[row_id] = best;
  }
}
int op_argmax(cai_ctx* ctx, const float* logits, int64_t ld, int batch, int n, int32_t* out_idx, float* out_val,
              float* part_val, int* part_idx, int* tickets) {
  ctx->cur_family = FAM_OTHER;
  int chunks = (n + 2047) / 2048;
  if (chunks > CAI_ARGMAX_CHUNKS) chunks = CAI_ARGMAX_CHUNKS;
  if (chunks < 1) chunks = 1;
  pdl_launch(ctx, argmax_kernel, dim3(chunks, batch), dim3(256), 0, logits, ld, n, out_idx, out_val, part_val, part_idx, tickets);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// cos/sin of (float)pos * theta[k] for every sequence of the step: the same values serve every layer
// and head, so the full-range sincosf (slow for large angles) runs once per step, not once per layer.
__global__ void rope_table_kernel(const float* __restrict__ theta, const int32_t* __restrict__ pos, int half, float* __restrict__ cs) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  for (int k = threadIdx.x; k < half; k += blockDim.x) {
    float s, c;
    sincosf((float)pos[b] * theta[k], &s, &c);
    cs[((size_t)b * half + k) * 2] = c;
    cs[((size_t)b * half + k) * 2 + 1] = s;
  }
}
int op_rope_table(cai_ctx* ctx, const float* theta_dev, const int32_t* pos_dev, int batch, int half, float* cs_dev) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, rope_table_kernel, dim3(batch), dim3(128), 0, theta_dev, pos_dev, half, cs_dev);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// MoE combine: x[t] += sum_s gate[t][s] * pair_out[t*k + s]   (slot order)
// ---------------------------------------------------------------------------
__global__ void moe_combine_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ pair_out, int64_t ldp,
                                   const float* __restrict__ gates, int top_k, int depth) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= depth) return;
  float y = 0.f;
  for (int s = 0; s < top_k; ++s)
    y = y + gates[(int64_t)t * top_k + s] * pair_out[((int64_t)t * top_k + s) * ldp + c];
  x[(int64_t)t * ldx + c] += y;
}
int op_moe_combine(cai_ctx* ctx, float* x, int64_t ldx, const float* pair_out, int64_t ldp, const float* gates,
                   int tokens, int top_k, int depth) {
  ctx->cur_family = FAM_OTHER;
  dim3 grid((depth + 255) / 256, tokens);
  pdl_launch(ctx, moe_combine_kernel, grid, dim3(256), 0, x, ldx, pair_out, ldp, gates, top_k, depth);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += y[i];
}
int op_add_inplace(cai_ctx* ctx, float* x, const float* y, int64_t n) {
  ctx->cur_family = FAM_OTHER;
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, y, n);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// Groups the (token, expert) pairs of a mixture-of-experts layer by expert, into tiles of up to `tile_rows` pairs
// that share one expert: tile_expert[t] (-1 = unused tile) and tile_pairs[t * tile_rows + i] (-1 = unused slot).
// Pairs keep their order inside an expert and experts come in index order, so the lists are deterministic.
// One CTA; pairs <= 4096, experts <= 1024.
// ---------------------------------------------------------------------------
__global__ void moe_group_kernel(const int32_t* __restrict__ ids, int pairs, int n_experts, int tile_rows, int max_tiles,
                                 int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_pairs, int expert_lo, int expert_hi, int* err) {
  extern __shared__ int32_t sh[];
  int32_t* s_ids = sh;                       // [pairs]
  int32_t* s_cnt = sh + pairs;               // [n_experts]
  int32_t* s_base = s_cnt + n_experts;       // [n_experts + 1] first tile of each expert
  pdl_trigger();
  pdl_wait();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= n_experts) cai_report_index(err, CAI_SITE_MOE_EXPERT, e, n_experts);
    s_ids[i] = (e >= expert_lo && e < expert_hi) ? e : -1;     // -1: another rank's expert (or no expert at all)
  }
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) s_cnt[e] = 0;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) tile_pairs[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x)
    if (s_ids[i] >= 0) atomicAdd(&s_cnt[s_ids[i]], 1);      // counts only: order does not matter
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < n_experts; ++e) { s_base[e] = t; t += (s_cnt[e] + tile_rows - 1) / tile_rows; }
    s_base[n_experts] = t;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = s_ids[i];
    if (e < 0) continue;
    int rank = 0;                             // pairs of the same expert before this one
    for (int q = 0; q < i; ++q) rank += (s_ids[q] == e) ? 1 : 0;
    const int t = s_base[e] + rank / tile_rows;
    if (t < max_tiles) {
      tile_pairs[(size_t)t * tile_rows + (rank % tile_rows)] = i;
      if (rank % tile_rows == 0) tile_expert[t] = e;
    }
  }
}

int op_moe_group(cai_ctx* ctx, const int32_t* expert_ids, int pairs, int n_experts, int tile_rows, int max_tiles,
                 int32_t* tile_expert, int32_t* tile_pairs, int expert_lo, int expert_hi) {
  ctx->cur_family = FAM_OTHER;
  if (pairs < 1 || pairs > 4096 || n_experts < 1 || n_experts > 1024)
    return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "moe grouping: %d pairs, %d experts", pairs, n_experts);
  const size_t smem = ((size_t)pairs + 2 * (size_t)n_experts + 1) * sizeof(int32_t);
  pdl_launch(ctx, moe_group_kernel, dim3(1), dim3(512), smem, expert_ids, pairs, n_experts, tile_rows, max_tiles, tile_expert, tile_pairs,
             expert_lo, expert_hi, ctx->err_flag);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// Expert parallelism helpers. A rank's tokens travel as rows [hidden floats | top_k ids (bit-cast) | top_k gates].
// ---------------------------------------------------------------------------
__global__ void moe_pack_kernel(const float* __restrict__ h, int64_t ldh, const int32_t* __restrict__ ids, const float* __restrict__ gates,
                                int hidden, int top_k, int stride, float* __restrict__ packed) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float* row = packed + (size_t)t * stride;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) row[c] = h[(int64_t)t * ldh + c];
  for (int k = threadIdx.x; k < top_k; k += blockDim.x) {
    row[hidden + k] = __int_as_float(ids[t * top_k + k]);
    row[hidden + top_k + k] = gates[t * top_k + k];
  }
}
int op_moe_pack(cai_ctx* ctx, const float* h, int64_t ldh, const int32_t* ids, const float* gates, int tokens, int hidden, int top_k, int stride,
                float* packed) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, moe_pack_kernel, dim3(tokens), dim3(256), 0, h, ldh, ids, gates, hidden, top_k, stride, packed);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
__global__ void moe_unpack_ids_kernel(const float* __restrict__ packed, int tokens, int hidden, int top_k, int stride,
                                      int32_t* __restrict__ ids, float* __restrict__ gates) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * top_k) return;
  const int t = i / top_k, k = i - t * top_k;
  const float* row = packed + (size_t)t * stride;
  ids[i] = __float_as_int(row[hidden + k]);
  gates[i] = row[hidden + top_k + k];
}
int op_moe_unpack_ids(cai_ctx* ctx, const float* packed, int tokens, int hidden, int top_k, int stride, int32_t* ids, float* gates) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, moe_unpack_ids_kernel, dim3((tokens * top_k + 255) / 256), dim3(256), 0, packed, tokens, hidden, top_k, stride, ids, gates);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
__global__ void moe_combine_partial_kernel(const float* __restrict__ pair_out, int64_t ldp, const int32_t* __restrict__ ids,
                                           const float* __restrict__ gates, int top_k, int hidden, int expert_lo, int expert_hi,
                                           float* __restrict__ y, int64_t ldy) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top_k; ++k) {                       // slots in order: the sum does not depend on the rank count
      const int e = ids[t * top_k + k];
      if (e >= expert_lo && e < expert_hi) acc += gates[t * top_k + k] * pair_out[(int64_t)(t * top_k + k) * ldp + c];
    }
    y[(int64_t)t * ldy + c] = acc;
  }
}
int op_moe_combine_partial(cai_ctx* ctx, const float* pair_out, int64_t ldp, const int32_t* ids, const float* gates, int tokens, int top_k,
                           int hidden, int expert_lo, int expert_hi, float* y, int64_t ldy) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, moe_combine_partial_kernel, dim3(tokens), dim3(256), 0, pair_out, ldp, ids, gates, top_k, hidden, expert_lo, expert_hi, y, ldy);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
__global__ void add_rows_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ y, int64_t ldy, int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) x[(int64_t)t * ldx + c] += y[(int64_t)t * ldy + c];
}
int op_add_rows(cai_ctx* ctx, float* x, int64_t ldx, const float* y, int64_t ldy, int tokens, int width) {
  ctx->cur_family = FAM_OTHER;
  pdl_launch(ctx, add_rows_kernel, dim3(tokens), dim3(256), 0, x, ldx, y, ldy, width);
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
