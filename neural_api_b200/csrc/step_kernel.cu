// One persistent kernel per decode step.
//
// The launch-per-operator step (model.cu: enqueue_step) pays ~5-10 us of drain, activation staging and tail per
// launch; a Qwen2.5-0.5B step is 149 such launches for 80 us of memory traffic. Here the whole step of a dense model
// (one sequence, Q8_0 weights, fp32 KV cache) is ONE cooperative kernel, one 16-warp CTA per SM, that walks the
// layers phase by phase:
//
//   [q|k|v] product (RMSNorm fused into the staging, RoPE + KV append in the epilogue) | attention over the cache,
//   split over the context | (merge of the splits) | O product + residual | [up|gate] product (RMSNorm, SwiGLU) |
//   down product + residual | ... | LM head (final norm) + argmax | advance
//
// with a grid-wide barrier between phases: a counter in global memory that only grows during a launch; every CTA
// adds one and polls until the count reaches the phase's target. The poll is bounded on the global timer: a CTA
// that gives up raises the context's error word and an abort word that makes every other CTA leave too.
//
// Weights never wait for a barrier. Every warp owns a cp.async ring in shared memory (stages of 4 rows x 512 codes
// + their 4 x 16 scales) and a FILL CURSOR that walks the warp's whole tile list of the step - matrix after matrix,
// straight across phase boundaries - ring_depth-1 stages ahead of the arithmetic. While a barrier settles, the
// activations are staged and the attention runs, the first tiles of the next matrix are already in shared memory.
//
// Work split of a product: a row group is 4 output rows (2 (up, gate) pairs for SwiGLU); the row groups of a matrix
// are dealt to the CTAs in contiguous, balanced ranges; inside a CTA a row group is cut into `ksplit` K-parts of
// `cpp` 512-code chunks, the (row group, part) tiles are dealt round-robin to the 16 warps, a warp reduces its tile
// over the lanes and leaves 4 partial sums in shared memory, and after a CTA barrier one thread per output row adds
// the parts in part order and applies the epilogue. The host picks ksplit per matrix kind to balance the warps.
// Reduction orders are fixed: results do not depend on timing.
//
// The residual stream is handed from the O and down products to the next phase without a grid barrier: every value
// travels as a (value, tag) pair that the readers poll (sk_row_handover). Tensor parallel: the CTA that owns an output
// row pushes its partial sum to every rank with plain stores over mapped peer memory and adds the ranks' sums of its
// rows in rank order. No separate all-reduce launches, no library call, no cluster-scope copy of any kind.
#include "gemv_common.cuh"
#include "step_kernel.cuh"
#include <math.h>
#include <stdlib.h>
#include <new>

namespace {

constexpr int SK_THREADS = 512;
constexpr int SK_WARPS = 16;
constexpr int SK_RPW = 4;
constexpr int SK_STAGE = SK_RPW * (512 + 32);        // bytes of one ring stage: 4 x 512 codes + 4 x 16 fp16 scales
constexpr int SK_XU = 4;                             // float4 pieces per thread of a normed row (hidden <= 8192)
constexpr int SK_FOLD_FLOATS = 49152;                // splits x q_width up to which the O staging merges the splits itself
constexpr int SK_FOLD_MAX_CHUNK = 512;               // ... and the longest split worth accepting for that (one 32-row tile per warp)
constexpr int SK_FOLD_MAX_SPLITS = 8;                // ... and the most splits: the fold walks them one after the other in every CTA
                                                     // (measured: 64 splits cost the O staging 13 us, the merge phase + its barrier 5)
constexpr int SK_MIN_CHUNK = 64;                     // fewest cached rows of a context split
enum { MK_QKV = 0, MK_O = 1, MK_GU = 2, MK_DOWN = 3, MK_HEAD = 4 };

struct SkMat {
  int K, KC;            // columns, 512-code chunks per row
  int sstride;          // halves between scale rows
  int n_rg;             // row groups of the matrix
  int ksplit, cpp;      // K-parts per row group, chunks per part
  int half;             // > 0: SwiGLU pairing, rows (j, half + j)
  int n_rows;
};
struct SkPtrs { const uint8_t* codes; const __half* scales; };
struct SkLayerDev { const float* attn_norm; const float* ffn_norm; const float* qkv_bias; float* k_cache; float* v_cache; };

struct SkTp {
  int rank, world;
  float* peer_ll1[8];      // every rank's row-exchange area: pairs [2 parities][world][hidden] of (partial sum, tag)
  int* my_flags;
  int* peer_flags[8];
  float* my_slots;
  const float* peer_slots[8];
  long long max_elems;
  int* seq;
  int* gave_up;
  int vocab_offset;
  int argmax_site;         // slot of the (value, index) exchange at the end of the step
};

struct SkParams {
  SkMat mat[5];
  const SkPtrs* ptrs;            // [4 * layers + 1]
  const SkLayerDev* lay;         // [layers]
  int layers, n_mats;
  int hidden, qw, kw, inter, q_heads, kv_heads, max_ctx, vocab;
  float eps, inv_sqrt_d;
  const uint8_t* emb_codes; const __half* emb_scales; int emb_sstride, emb_rows;
  const float* final_norm; const float* theta;
  int32_t *tokens, *pos, *len;
  float *xres, *qbuf, *att, *act, *logits, *partial;
  int nsplit_max;
  float* cand_val; int* cand_idx;
  int32_t* amax_idx; float* amax_val; int32_t* trace; int32_t* trace_count; long long trace_cap;
  int use_ll;                    // hand the residual stream over as tagged pairs (else: store, grid barrier, load)
  float* ll2;                    // pairs [2 parities][hidden] of (residual stream value, tag): the row every CTA stages next
  unsigned* sync;                // [0] arrivals of this launch, [1] abort word, [2] tags handed out so far
  int* err; unsigned limit_us;
  unsigned long long* ts;        // optional phase trace: [0] entries, then (time, family) pairs
  int fine;                      // also stamp inside the phases (families 4 staged, 5 products done, 6 epilogue done)
  int ring_depth;
  int off_xs, off_slots, off_misc, off_tab, off_ring;     // byte offsets in dynamic shared memory
  int at_warps, at_depth;        // attention: warps that take tiles, stages of their rings
  SkTp tp;
};

// ---------------------------------------------------------------------------------------------------------------
// grid barrier
// ---------------------------------------------------------------------------------------------------------------
// Adds this CTA's arrival and (wait = true) polls until `target` arrivals are in. Returns false when the step is
// being abandoned (this CTA's wait ran out, or another CTA's did).
__device__ __forceinline__ bool sk_barrier(const SkParams& P, unsigned target, int* s_flag, bool wait) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.sync) : "memory");
    int ok = 1;
    if (wait) {
      unsigned long long t0 = 0;
      const unsigned long long limit = (unsigned long long)P.limit_us * 1000ull;
      unsigned polls = 0;
      while (true) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.sync) : "memory");
        if (v >= target) break;
        if ((++polls & 127u) == 0) {
          if (*(volatile unsigned*)(P.sync + 1)) { ok = 0; break; }
          const unsigned long long now = gtime_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > limit) { ok = 0; *(volatile unsigned*)(P.sync + 1) = 1u; *P.err = 1; break; }
        }
      }
    }
    *s_flag = ok;
  }
  __syncthreads();
  return *s_flag != 0;
}

__device__ __forceinline__ void sk_trace(const SkParams& P, int& n, int family) {
  if (P.ts && blockIdx.x == 0 && threadIdx.x == 0) {
    P.ts[1 + 2 * n] = gtime_ns();
    P.ts[2 + 2 * n] = (unsigned long long)family;
    ++n;
    P.ts[0] = (unsigned long long)n;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// weight ring
// ---------------------------------------------------------------------------------------------------------------
struct SkFill {
  int gi, kind, t, T, c, c_end, rg0, slot, k_lane, s_idx;
  int hold;                      // the cursor stopped in front of an O matrix (the attention phase borrows the rings)
  const uint8_t* codes; const __half* scales;
  const uint8_t* wp[SK_RPW];
  const __half* sp;
};

__device__ __forceinline__ int sk_row_of(const SkMat& M, int rg, int r) {
  if (M.half > 0) {
    int j = 2 * rg + (r >> 1);
    if (j >= M.half) j = M.half - 1;
    return (r & 1) ? M.half + j : j;
  }
  const int row = 4 * rg + r;
  return row >= M.n_rows ? M.n_rows - 1 : row;
}
__device__ __forceinline__ int sk_rg_begin(int n_rg, int cta, int grid) { return (int)(((long long)cta * n_rg) / grid); }

__device__ __forceinline__ void sk_tile_setup(const SkParams& P, SkFill& f, int lane) {
  const SkMat& M = P.mat[f.kind];
  const int rgl = f.t / M.ksplit, kp = f.t - rgl * M.ksplit;
  f.c = kp * M.cpp;
  f.c_end = min(M.KC, f.c + M.cpp);
  const int rg = f.rg0 + rgl;
#pragma unroll
  for (int r = 0; r < SK_RPW; ++r) f.wp[r] = f.codes + (size_t)sk_row_of(M, rg, r) * (size_t)M.K + (size_t)f.c * 512 + lane * 16;
  f.sp = f.scales + (size_t)sk_row_of(M, rg, (lane >> 1) & 3) * (size_t)M.sstride + f.c * 16 + (lane & 1) * 8;
  f.s_idx = f.c * 16 + (lane & 1) * 8;
  f.k_lane = f.c * 512 + lane * 16;
}

// cross_o = false: the cursor stops in front of an O matrix (f.hold): the attention phase that precedes it uses
// the rings' shared memory for the K and V rows, and the step resumes the cursor when that phase is over.
__device__ __forceinline__ void sk_next_matrix(const SkParams& P, SkFill& f, const SkPtrs* tab, int lane, int warp, bool cross_o = false) {
  while (true) {
    if (!cross_o && f.gi + 1 < P.n_mats - 1 && ((f.gi + 1) & 3) == MK_O) { f.hold = 1; return; }
    cross_o = false;
    ++f.gi;
    if (f.gi >= P.n_mats) return;
    f.kind = (f.gi == P.n_mats - 1) ? MK_HEAD : (f.gi & 3);
    const SkMat& M = P.mat[f.kind];
    f.rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x);
    f.T = (sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x) - f.rg0) * M.ksplit;
    f.t = warp;
    if (f.t < f.T) {
      f.codes = tab[f.gi].codes;
      f.scales = tab[f.gi].scales;
      sk_tile_setup(P, f, lane);
      return;
    }
  }
}

// Copies the cursor's next chunk into the ring (one commit group per call, empty once the step's tiles are through).
__device__ __forceinline__ void sk_fill_one(const SkParams& P, SkFill& f, const SkPtrs* tab, uint32_t ring_w, int lane, int warp) {
  if (!f.hold && f.gi < P.n_mats) {
    const int K = P.mat[f.kind].K;
    const uint32_t ok = (f.k_lane < K) ? 16u : 0u;
    const uint32_t dst = ring_w + f.slot * SK_STAGE + lane * 16;
#pragma unroll
    for (int r = 0; r < SK_RPW; ++r) {
      gv_cp_async16(dst + r * 512, ok ? (const void*)f.wp[r] : (const void*)f.codes, ok);
      f.wp[r] += 512;
    }
    if (lane < 2 * SK_RPW) {
      const uint32_t sok = (f.s_idx < (K >> 5)) ? 16u : 0u;
      gv_cp_async16(ring_w + f.slot * SK_STAGE + SK_RPW * 512 + lane * 16, sok ? (const void*)f.sp : (const void*)f.scales, sok);
    }
    f.sp += 16; f.s_idx += 16; f.k_lane += 512;
    if (++f.c == f.c_end) {
      f.t += SK_WARPS;
      if (f.t < f.T) sk_tile_setup(P, f, lane);
      else sk_next_matrix(P, f, tab, lane, warp);
    }
  }
  gv_cp_async_commit();
  f.slot = (f.slot + 1 == P.ring_depth) ? 0 : f.slot + 1;
}

// The products of one phase: this warp's tiles of matrix kind `kind`, partial sums into slots[(rgl * ksplit + kp) * 4 + r].
__device__ __forceinline__ void sk_gemv(const SkParams& P, const int kind, SkFill& f, int& rd_slot, const SkPtrs* tab, uint32_t ring_w,
                                        const float* xs, float* slots, int lane, int warp) {
  const SkMat& M = P.mat[kind];
  const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x);
  const int T = (sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x) - rg0) * M.ksplit;
  const int xsw = (lane >> 1) & 3;
  for (int t = warp; t < T; t += SK_WARPS) {
    const int rgl = t / M.ksplit, kp = t - rgl * M.ksplit;
    const int c0 = kp * M.cpp, c1 = min(M.KC, c0 + M.cpp);
    f32x2_t acc2[SK_RPW];
#pragma unroll
    for (int r = 0; r < SK_RPW; ++r) acc2[r] = 0ull;
    for (int c = c0; c < c1; ++c) {
      gv_cp_async_wait_depth(P.ring_depth);      // this lane's copies of the stage have landed
      __syncwarp();                              // ... and the scales the copy lanes fetched
      sk_fill_one(P, f, tab, ring_w, lane, warp);   // refills the stage read in the previous iteration
      const uint32_t src = ring_w + rd_slot * SK_STAGE;
      rd_slot = (rd_slot + 1 == P.ring_depth) ? 0 : rd_slot + 1;
      const int k_lane = c * 512 + lane * 16;
      if (k_lane < M.K) {
        int4 wv[SK_RPW];
        uint32_t sv[SK_RPW];
#pragma unroll
        for (int r = 0; r < SK_RPW; ++r) {
          wv[r] = gv_lds16(src + r * 512 + lane * 16);
          sv[r] = gv_lds_u16(src + SK_RPW * 512 + r * 32 + (lane >> 1) * 2);
        }
        const float* xr = xs + k_lane;
        f32x2_t part[SK_RPW];
#pragma unroll
        for (int r = 0; r < SK_RPW; ++r) part[r] = 0ull;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 xv = *(const float4*)(xr + 4 * (i ^ xsw));
#pragma unroll
          for (int r = 0; r < SK_RPW; ++r) part[r] = q8_word_fma(((const uint32_t*)&wv[r])[i], xv, part[r]);
        }
#pragma unroll
        for (int r = 0; r < SK_RPW; ++r) {
          const float d = half_bits_to_float(sv[r]);
          acc2[r] = fma2(pack2(d, d), part[r], acc2[r]);
        }
      }
    }
    float a[SK_RPW];
#pragma unroll
    for (int r = 0; r < SK_RPW; ++r) a[r] = warp_sum(sum2(acc2[r]));
    if (lane < SK_RPW) {
      const float v = lane == 0 ? a[0] : (lane == 1 ? a[1] : (lane == 2 ? a[2] : a[3]));
      slots[(rgl * M.ksplit + kp) * SK_RPW + lane] = v;
    }
  }
}

__device__ __forceinline__ float sk_slot_sum(const float* slots, int rgl, int ksplit, int r) {
  float s = 0.f;
  for (int kp = 0; kp < ksplit; ++kp) s += slots[(rgl * ksplit + kp) * SK_RPW + r];
  return s;
}

// ---------------------------------------------------------------------------------------------------------------
// activation staging (every CTA holds the whole input row of the phase, swizzled like the GEMV kernels' rows)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 sk_ldcg4(const float* p) { return __ldcg((const float4*)p); }
__device__ __forceinline__ bool sk_pair_wait2(const SkParams& P, const float* p, int tag, float& v0, float& v1);

// x = gain * (src * inv_rms(src)); src is row emb_tok of the embedding table, dequantized on the fly (emb_tok >= 0), or
// the residual stream (emb_tok < 0): as tagged pairs (`src` points at the pairs, `tag` != 0 is the hand-over waited
// for) or, tag == 0, as a plain row.
// keep_raw (CTA 0 at layer 0): also store the raw row as the residual stream. False when a poll ran out of time.
template <bool LL>
__device__ __forceinline__ bool sk_stage_normed(const SkParams& P, float* xs, float* red, const float* src, int emb_tok,
                                                const float* gain, float* keep_raw, int tag = 0) {
  bool ok = true;
  const int K = P.hidden, K4 = K >> 2;
  float4 xv[SK_XU], gv[SK_XU];
#pragma unroll
  for (int u = 0; u < SK_XU; ++u) {
    const int c4 = threadIdx.x + u * SK_THREADS;
    xv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    gv[u] = xv[u];
    if (c4 < K4) {
      gv[u] = __ldg((const float4*)gain + c4);
      if (emb_tok < 0) {
        if constexpr (LL) {
          ok = sk_pair_wait2(P, src + 8 * c4, tag, xv[u].x, xv[u].y) && ok;
          ok = sk_pair_wait2(P, src + 8 * c4 + 4, tag, xv[u].z, xv[u].w) && ok;
        } else {
          xv[u] = sk_ldcg4(src + 4 * c4);            // plain row in global memory (a grid barrier came before)
        }
      } else {
        const uint32_t w = __ldg((const uint32_t*)(P.emb_codes + (size_t)emb_tok * K) + c4);
        const float d = __half2float(__ldg(P.emb_scales + (size_t)emb_tok * P.emb_sstride + (c4 >> 3)));
        xv[u].x = d * (float)((int)(w & 255u) - 128);
        xv[u].y = d * (float)((int)((w >> 8) & 255u) - 128);
        xv[u].z = d * (float)((int)((w >> 16) & 255u) - 128);
        xv[u].w = d * (float)((int)(w >> 24) - 128);
      }
    }
  }
  if (keep_raw) {
#pragma unroll
    for (int u = 0; u < SK_XU; ++u) {
      const int c4 = threadIdx.x + u * SK_THREADS;
      if (c4 < K4) *((float4*)keep_raw + c4) = xv[u];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < SK_XU; ++u) {
    ss = fmaf(xv[u].x, xv[u].x, ss); ss = fmaf(xv[u].y, xv[u].y, ss);
    ss = fmaf(xv[u].z, xv[u].z, ss); ss = fmaf(xv[u].w, xv[u].w, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)K + P.eps);
#pragma unroll
  for (int u = 0; u < SK_XU; ++u) {
    const int c4 = threadIdx.x + u * SK_THREADS;
    if (c4 < K4) {
      float4 y;
      y.x = gv[u].x * (xv[u].x * inv); y.y = gv[u].y * (xv[u].y * inv);
      y.z = gv[u].z * (xv[u].z * inv); y.w = gv[u].w * (xv[u].w * inv);
      *(float4*)(xs + x_phys<CAI_TYPE_Q8_0>((int64_t)c4 * 4)) = y;
    }
  }
  if constexpr (LL) return __syncthreads_and(ok ? 1 : 0) != 0;
  __syncthreads();
  return true;
}

__device__ __forceinline__ void sk_stage_copy(float* xs, const float* src, int K) {
  const int K4 = K >> 2;
  for (int base = 0; base < K4; base += SK_THREADS * 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c4 = base + u * SK_THREADS + threadIdx.x;
      if (c4 < K4) v[u] = sk_ldcg4(src + 4 * c4);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c4 = base + u * SK_THREADS + threadIdx.x;
      if (c4 < K4) *(float4*)(xs + x_phys<CAI_TYPE_Q8_0>((int64_t)c4 * 4)) = v[u];
    }
  }
  __syncthreads();
}

// Merge of the context splits of every head straight into the staged row (short contexts: few splits).
template <int HD>
__device__ __forceinline__ void sk_stage_merge(const SkParams& P, float* xs, int used) {
  const int K4 = P.qw >> 2;
  for (int c4 = threadIdx.x; c4 < K4; c4 += SK_THREADS) {
    const int h = (c4 * 4) / HD, d = (c4 * 4) - h * HD;
    const float* src = P.partial + (size_t)h * P.nsplit_max * (HD + 2);
    float mx = -INFINITY;
    for (int s = 0; s < used; ++s) mx = fmaxf(mx, __ldcg(src + (size_t)s * (HD + 2)));
    float lt = 0.f;
    float4 at = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < used; ++s) {
      const float2 ml = __ldcg((const float2*)(src + (size_t)s * (HD + 2)));
      const float sc = (ml.x == -INFINITY) ? 0.f : expf(ml.x - mx);
      const float2 a0 = __ldcg((const float2*)(src + (size_t)s * (HD + 2) + 2 + d));
      const float2 a1 = __ldcg((const float2*)(src + (size_t)s * (HD + 2) + 4 + d));
      lt += ml.y * sc;
      at.x += a0.x * sc; at.y += a0.y * sc; at.z += a1.x * sc; at.w += a1.y * sc;
    }
    float4 y;
    y.x = (lt > 0.f) ? at.x / lt : 0.f; y.y = (lt > 0.f) ? at.y / lt : 0.f;
    y.z = (lt > 0.f) ? at.z / lt : 0.f; y.w = (lt > 0.f) ? at.w / lt : 0.f;
    *(float4*)(xs + x_phys<CAI_TYPE_Q8_0>((int64_t)c4 * 4)) = y;
  }
  __syncthreads();
}

// The same merge as its own phase (long contexts): one warp per 4 outputs, the lanes take the splits (lane, lane + 32,
// ...), each lane merges its own splits in order and the lanes are then combined with one max and five sums over the
// warp. The outputs are dealt over all warps of the grid; result to P.att.
template <int HD>
__device__ __forceinline__ void sk_merge_phase(const SkParams& P, int used) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int K4 = P.qw >> 2;
  for (int c4 = blockIdx.x + gridDim.x * warp; c4 < K4; c4 += gridDim.x * SK_WARPS) {
    const int h = (c4 * 4) / HD, d = (c4 * 4) - h * HD;
    const float* src = P.partial + (size_t)h * P.nsplit_max * (HD + 2);
    float mx = -INFINITY, lt = 0.f;
    float4 at = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = lane; s < used; s += 32) {
      const float2 ml = __ldcg((const float2*)(src + (size_t)s * (HD + 2)));
      const float2 a0 = __ldcg((const float2*)(src + (size_t)s * (HD + 2) + 2 + d));
      const float2 a1 = __ldcg((const float2*)(src + (size_t)s * (HD + 2) + 4 + d));
      if (ml.x == -INFINITY) continue;
      const float mnew = fmaxf(mx, ml.x);
      const float ca = (mx == -INFINITY) ? 0.f : expf(mx - mnew), cb = expf(ml.x - mnew);
      lt = lt * ca + ml.y * cb;
      at.x = at.x * ca + a0.x * cb; at.y = at.y * ca + a0.y * cb; at.z = at.z * ca + a1.x * cb; at.w = at.w * ca + a1.y * cb;
      mx = mnew;
    }
    const float mall = warp_max(mx);
    const float sc = (mx == -INFINITY) ? 0.f : expf(mx - mall);
    lt = warp_sum(lt * sc);
    at.x = warp_sum(at.x * sc); at.y = warp_sum(at.y * sc); at.z = warp_sum(at.z * sc); at.w = warp_sum(at.w * sc);
    if (lane == 0) {
      float4 y;
      y.x = (lt > 0.f) ? at.x / lt : 0.f; y.y = (lt > 0.f) ? at.y / lt : 0.f;
      y.z = (lt > 0.f) ? at.z / lt : 0.f; y.w = (lt > 0.f) ? at.w / lt : 0.f;
      *((float4*)P.att + c4) = y;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// attention over the cache: items (kv head, context split) dealt to the CTAs; inside an item 8 warps take tiles of
// 32 rows (lane = row for Q.K, lane = 2 or 4 channels for P.V), online softmax per warp, warps merged in warp order.
//
// With this kernel's shared-memory carve-out the L1 cache is a few tens of KB: ordinary loads of K and V rows cannot
// keep enough lines in flight (measured: 2.2 TB/s). So the rows come in through cp.async, which needs no L1 line:
// every attention warp owns a ring of 4 KB stages. A tile is KS stages of K (32 rows x 32 channels: in the sessions'
// block-transposed K cache that is one contiguous 4 KB run, already laid out [piece][row] for conflict-free lane = row
// reads) followed by VG stages of V (whole
// rows, as they lie in the cache). The fill runs AT_DEPTH - 1 stages ahead of the arithmetic, straight across tiles.
// Rows past the end of the split are fetched from the split's last row (finite values) and carry probability 0.
// ---------------------------------------------------------------------------------------------------------------
constexpr int AT_STAGE = 4096;

// shared memory of the phase: q [G][HD] | probabilities [warps][G][32] | rings [warps][depth][AT_STAGE], which become
// the merge area [warps][G][HD + 2] once the rows are through
static __host__ __device__ inline int at_rings_offset(int G, int HD, int warps) { return ((G * HD * 4 + warps * G * 32 * 4) + 127) & ~127; }
static __host__ __device__ inline int at_smem_bytes(int G, int HD, int warps, int depth) {
  const int ring = warps * depth * AT_STAGE, merge = warps * G * (HD + 2) * 4;
  return at_rings_offset(G, HD, warps) + (ring > merge ? ring : merge);
}

template <int G, int HD>
__device__ __forceinline__ void sk_attention(const SkParams& P, const SkLayerDev& L, unsigned char* smem, int n, int chunk, int used,
                                             int lane, int warp) {
  constexpr int KS = HD / 32;                    // K stages per tile (32 channels each)
  constexpr int VR = AT_STAGE / (HD * 4);        // rows per V stage
  constexpr int VG = 32 / VR;                    // V stages per tile
  constexpr int SPT = KS + VG;                   // stages per tile
  constexpr int RP = HD / 4;                     // 16-byte pieces per row
  constexpr int DPL = HD / 32;
  constexpr int DP2 = DPL / 2;
  const int AT_WARPS = P.at_warps, AT_DEPTH = P.at_depth;
  const int aw = warp < AT_WARPS ? warp : 0;
  float* q_s = (float*)smem;                                                        // [G][HD]
  float* p_s = q_s + G * HD + (size_t)aw * G * 32;                                  // this warp's [G][32] probabilities
  unsigned char* rings = smem + at_rings_offset(G, HD, AT_WARPS);
  float* merge_s = (float*)rings;                                                   // [AT_WARPS][G][HD + 2], after the loop
  const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(rings) + (uint32_t)aw * AT_DEPTH * AT_STAGE;
  const int items = P.kv_heads * used;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int g = item / used, split = item - g * used;
    const int j_begin = split * chunk;
    int j_end = j_begin + chunk; if (j_end > n) j_end = n;
    __syncthreads();                                                     // the previous item's shared memory is free
    float m[G], l[G];
    f32x2_t acc[G][DP2];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
      for (int d = 0; d < DP2; ++d) acc[h][d] = 0ull;
    }
    if (warp < AT_WARPS) {
      const float* kbase = L.k_cache + (size_t)g * (size_t)P.max_ctx * HD;
      const float* vbase = L.v_cache + (size_t)g * (size_t)P.max_ctx * HD;
      const int n_tiles = (j_end - j_begin + 31) >> 5;
      const int my_tiles = (warp < n_tiles) ? (n_tiles - warp + AT_WARPS - 1) / AT_WARPS : 0;
      const int total = my_tiles * SPT;
      int fs = 0, fslot = 0, rslot = 0;
      // copies stage `fs` of this warp's sequence into ring slot `fslot` (an empty group past the end)
      auto issue = [&]() {
        if (fs < total) {
          const int ti = fs / SPT, st = fs - ti * SPT;
          const int tile = j_begin + 32 * (warp + AT_WARPS * ti);
          const int last = j_end - 1 - tile;
          const uint32_t dst = ring_a + fslot * AT_STAGE;
          if (st < KS) {
            // pieces 8 st .. 8 st + 7 of the tile's 32-row block: one contiguous 4 KB run, [piece][row] in memory and
            // in the stage alike. (Rows past the end of the cache's filled part hold whatever was there: their scores
            // are masked and never reach a sum.)
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
        fslot = (fslot + 1 == AT_DEPTH) ? 0 : fslot + 1;
      };
      auto next_stage = [&]() -> uint32_t {
        gv_cp_async_wait_depth(AT_DEPTH);
        __syncwarp();
        issue();
        const uint32_t src = ring_a + rslot * AT_STAGE;
        rslot = (rslot + 1 == AT_DEPTH) ? 0 : rslot + 1;
        return src;
      };
#pragma unroll 1
      for (int s = 0; s < AT_DEPTH - 1; ++s) issue();
      // (the cached rows are on their way: now fetch this step's query rows)
      for (int i = threadIdx.x; i < G * HD; i += AT_WARPS * 32) q_s[i] = __ldcg(P.qbuf + (size_t)g * G * HD + i);
      asm volatile("bar.sync 1, %0;" ::"r"(AT_WARPS * 32) : "memory");       // the attention warps only
#pragma unroll 1
      for (int ti = 0; ti < my_tiles; ++ti) {
        const int tile = j_begin + 32 * (warp + AT_WARPS * ti);
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
          const float sc = valid ? sum2(s2[h]) * P.inv_sqrt_d : -INFINITY;
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
      asm volatile("cp.async.wait_all;" ::: "memory");     // the rings become the merge area below
    }
    __syncthreads();
    const int n_tiles_all = (j_end - j_begin + 31) >> 5;
    const int nw = n_tiles_all < AT_WARPS ? n_tiles_all : AT_WARPS;      // warps that had a tile
    if (warp < nw) {
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
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += SK_THREADS) {
      const int hh = idx / HD, d = idx - hh * HD;
      float mx = -INFINITY;
      for (int w = 0; w < nw; ++w) mx = fmaxf(mx, merge_s[((size_t)w * G + hh) * (HD + 2)]);
      float lt = 0.f, at = 0.f;
      for (int w = 0; w < nw; ++w) {
        const float* src = merge_s + ((size_t)w * G + hh) * (HD + 2);
        const float sc = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mx);
        lt += src[1] * sc;
        at += src[2 + d] * sc;
      }
      float* dst = P.partial + ((size_t)(g * G + hh) * P.nsplit_max + split) * (HD + 2);
      if (d == 0) { dst[0] = mx; dst[1] = lt; }
      dst[2 + d] = at;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// hand-over of the residual stream between phases without a grid barrier
//
// The O and down products end in the residual stream x (hidden floats), and the next phase needs ALL of x on EVERY
// CTA. Instead of "store, grid barrier, load" each value travels as an 8-byte pair (value, tag) written with one store
// (8-byte stores are single-copy atomic, so a reader sees the value and its tag together); the tag is a number that is
// new for every hand-over of every step, and a reader simply re-reads a pair until the tag is the one it waits for.
// One store-to-load latency replaces barrier + load, and a CTA whose rows are done does not wait for the slowest CTA
// before it starts to collect the others' rows.
//   one GPU:  the CTA that owns row r writes x[r] = x[r] + sum_r and the pair (x[r], tag) into `ll2`; every CTA's
//             staging polls the hidden pairs of ll2.
//   N GPUs:   the owner first pushes (sum_r, tag) into EVERY rank's `ll1[parity][its rank][r]` (plain stores over
//             mapped peer memory), then collects the N partial sums of its own rows from its own ll1 (the owners of
//             the same rows on the other ranks pushed them), adds them in rank order to x[r], and continues as above.
// Two parities alternate: a pair is rewritten two hand-overs later, which no rank can reach before every CTA of every
// rank has read the earlier one (each hand-over needs rows from all CTAs of all ranks, and a CTA sends its rows only
// after its own staging of the previous hand-over). Every poll is bounded on the global timer.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void sk_pair_store(float* p, float v, int tag) {
  asm volatile("st.volatile.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v), "f"(__int_as_float(tag)) : "memory");
}
// Polls one pair until its tag is `tag`; false when the time limit ran out (or the step is being abandoned).
__device__ __forceinline__ bool sk_pair_wait(const SkParams& P, const float* p, int tag, float& v) {
  float a, t;
  asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(t) : "l"(p) : "memory");
  if (__float_as_int(t) == tag) { v = a; return true; }
  const unsigned long long t0 = gtime_ns(), limit = (unsigned long long)P.limit_us * 1000ull;
  unsigned polls = 0;
  while (true) {
    asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(t) : "l"(p) : "memory");
    if (__float_as_int(t) == tag) { v = a; return true; }
    if ((++polls & 63u) == 0) {
      if (*(volatile unsigned*)(P.sync + 1)) return false;
      if (gtime_ns() - t0 > limit) { *(volatile unsigned*)(P.sync + 1) = 1u; *P.err = 1; return false; }
    }
  }
}

// Two neighbouring pairs with one 16-byte load.
__device__ __forceinline__ bool sk_pair_wait2(const SkParams& P, const float* p, int tag, float& v0, float& v1) {
  float a, ta, b, tb;
  const unsigned long long t0 = gtime_ns(), limit = (unsigned long long)P.limit_us * 1000ull;
  unsigned polls = 0;
  while (true) {
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a), "=f"(ta), "=f"(b), "=f"(tb) : "l"(p) : "memory");
    if (__float_as_int(ta) == tag && __float_as_int(tb) == tag) { v0 = a; v1 = b; return true; }
    if ((++polls & 63u) == 0) {
      if (*(volatile unsigned*)(P.sync + 1)) return false;
      if (gtime_ns() - t0 > limit) { *(volatile unsigned*)(P.sync + 1) = 1u; *P.err = 1; return false; }
    }
  }
}

// End of an O / down phase for output row `row` with this rank's sum `v`: returns false on a time-out.
__device__ __forceinline__ bool sk_row_handover(const SkParams& P, int row, float v, int tag) {
  const int par = tag & 1;
  float x = __ldcg(P.xres + row);
  bool ok = true;
  if (P.tp.world > 1) {
    const size_t at = ((size_t)(par * P.tp.world + P.tp.rank) * P.hidden + row) * 2;
    for (int r = 0; r < P.tp.world; ++r) sk_pair_store(P.tp.peer_ll1[r] + at, v, tag);
    const float* mine = P.tp.peer_ll1[P.tp.rank];
    for (int r = 0; r < P.tp.world; ++r) {
      float part = 0.f;
      ok = sk_pair_wait(P, mine + ((size_t)(par * P.tp.world + r) * P.hidden + row) * 2, tag, part) && ok;
      x += part;
    }
  } else {
    x += v;
  }
  P.xres[row] = x;
  sk_pair_store(P.ll2 + ((size_t)par * P.hidden + row) * 2, x, tag);
  return ok;
}

// ---------------------------------------------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------------------------------------------
#define SK_SYNC(wait_flag)                                                                    \
  do {                                                                                        \
    ++epoch;                                                                                  \
    if (!sk_barrier(P, epoch * gridDim.x, s_flag, (wait_flag))) { sk_drain(); return; }       \
  } while (0)

__device__ __forceinline__ void sk_drain() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int G, int HD, bool LL>
__global__ void __launch_bounds__(SK_THREADS, 1) step_kernel(const SkParams P) {
  extern __shared__ __align__(16) unsigned char sk_smem[];
  float* xs = (float*)(sk_smem + P.off_xs);                        // staged input row (the attention phase uses everything from here up)
  float* slots = (float*)(sk_smem + P.off_slots);
  float* red = (float*)(sk_smem + P.off_misc);                     // [32]
  int* s_flag = (int*)(sk_smem + P.off_misc + 128);
  float* s_best_v = (float*)(sk_smem + P.off_misc + 192);          // [16]
  int* s_best_i = (int*)(sk_smem + P.off_misc + 256);              // [16]
  float* cs = (float*)(sk_smem + P.off_misc + 320);                // [HD / 2][2] cos, sin of this step's position
  const SkLayerDev* tab_lay = (const SkLayerDev*)(sk_smem + P.off_tab);
  const SkPtrs* tab = (const SkPtrs*)(sk_smem + P.off_tab + ((P.layers * (int)sizeof(SkLayerDev) + 15) & ~15));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ring_w = (uint32_t)__cvta_generic_to_shared(sk_smem + P.off_ring) + warp * P.ring_depth * SK_STAGE;

  const int len = P.len[0];
  if (len < 0 || len >= P.max_ctx) {                               // no room for the row this step appends: touch nothing
    if (blockIdx.x == 0 && threadIdx.x == 0) *P.err = 2;
    return;
  }
  int token = P.tokens[0];
#if CAI_CHECKED_BUILD
  if ((token < 0 || token >= P.emb_rows) && blockIdx.x == 0 && threadIdx.x == 0) cai_report_index(P.err, CAI_SITE_STEP_TOKEN, token, P.emb_rows);
#endif
  if (token < 0) token = 0;
  if (token >= P.emb_rows) token = P.emb_rows - 1;
  const int pos = P.pos[0];
  const int tp_seq0 = (P.tp.world > 1) ? *(volatile int*)P.tp.seq : 0;
  const int tag0 = LL ? (int)*(volatile unsigned*)(P.sync + 2) : 0;   // tags handed out by the steps before this one

  // pointer tables and this step's RoPE table into shared memory, then the ring is primed
  {
    // (the layer table is allocated with 16 bytes of slack, so whole 16-byte loads stay inside it)
    const int n16 = (((P.layers * (int)sizeof(SkLayerDev) + 15) & ~15)) / 16;
    int4* dst = (int4*)(sk_smem + P.off_tab);
    for (int i = threadIdx.x; i < n16; i += SK_THREADS) dst[i] = __ldg((const int4*)P.lay + i);
    int4* dst2 = (int4*)tab;
    for (int i = threadIdx.x; i < P.n_mats; i += SK_THREADS) dst2[i] = __ldg((const int4*)P.ptrs + i);
    for (int k = threadIdx.x; k < HD / 2; k += SK_THREADS) {
      float s, c;
      sincosf((float)pos * __ldg(P.theta + k), &s, &c);
      cs[2 * k] = c; cs[2 * k + 1] = s;
    }
  }
  __syncthreads();

  SkFill f;
  f.gi = -1; f.slot = 0; f.kind = 0; f.hold = 0; f.t = 0; f.T = 0; f.c = 0; f.c_end = 0; f.rg0 = 0; f.k_lane = 0; f.s_idx = 0;
  f.codes = nullptr; f.scales = nullptr; f.sp = nullptr;
#pragma unroll
  for (int r = 0; r < SK_RPW; ++r) f.wp[r] = nullptr;
  sk_next_matrix(P, f, tab, lane, warp);
  for (int s = 0; s < P.ring_depth - 1; ++s) sk_fill_one(P, f, tab, ring_w, lane, warp);
  int rd_slot = 0;
  unsigned epoch = 0;
  int nts = 0;
  int tp_k = 0;
  sk_trace(P, nts, FAM_OTHER);

  // context splits of this step (the same on every CTA)
  const int n = len + 1;
  int chunk = (n + P.nsplit_max - 1) / P.nsplit_max;
  if (chunk < SK_MIN_CHUNK) chunk = SK_MIN_CHUNK;
  chunk = (chunk + 31) & ~31;
  {
    // Fewer, longer splits when that lets the O staging merge them itself: a phase of this kernel costs microseconds
    // whatever it moves, so the separate merge phase (and its grid barrier) is worth more than the last bit of
    // parallelism over the context, as long as a split stays within one 32-row tile per warp.
    int max_fold = SK_FOLD_FLOATS / P.qw;
    if (max_fold > SK_FOLD_MAX_SPLITS) max_fold = SK_FOLD_MAX_SPLITS;
    if (max_fold >= 1) {
      const int c2 = (((n + max_fold - 1) / max_fold) + 31) & ~31;
      if (c2 > chunk && c2 <= SK_FOLD_MAX_CHUNK) chunk = c2;
    }
  }
  const int used = (n + chunk - 1) / chunk;
  const bool fold = used <= SK_FOLD_MAX_SPLITS && used * P.qw <= SK_FOLD_FLOATS;
  const bool tp = P.tp.world > 1;

  for (int l = 0; l < P.layers; ++l) {
    const SkLayerDev L = tab_lay[l];
    // ---- [q|k|v]: RMSNorm in the staging; RoPE and the KV append in the epilogue
    if (!sk_stage_normed<LL>(P, xs, red, LL ? P.ll2 + (size_t)((tag0 + 2 * l) & 1) * P.hidden * 2 : P.xres, l == 0 ? token : -1,
                             L.attn_norm, (l == 0 && blockIdx.x == 0) ? P.xres : nullptr, tag0 + 2 * l)) { sk_drain(); return; }
    if (P.fine) sk_trace(P, nts, 4);
    sk_gemv(P, MK_QKV, f, rd_slot, tab, ring_w, xs, slots, lane, warp);
    if (P.fine) sk_trace(P, nts, 5);
    __syncthreads();
    {
      const SkMat& M = P.mat[MK_QKV];
      const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x), rg1 = sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x);
      for (int p = threadIdx.x; p < (rg1 - rg0) * 2; p += SK_THREADS) {
        const int rgl = p >> 1, r0 = (p & 1) * 2;
        const int row = 4 * (rg0 + rgl) + r0;
        if (row + 1 < M.n_rows) {
          float v0 = sk_slot_sum(slots, rgl, M.ksplit, r0), v1 = sk_slot_sum(slots, rgl, M.ksplit, r0 + 1);
          if (L.qkv_bias) { v0 += __ldg(L.qkv_bias + row); v1 += __ldg(L.qkv_bias + row + 1); }
          if (row < P.qw + P.kw) {
            const int rr = (row < P.qw) ? row : row - P.qw;
            const int k = (rr % HD) >> 1;
            const float c = cs[2 * k], s = cs[2 * k + 1];
            const float y0 = c * v0 - s * v1, y1 = s * v0 + c * v1;
            v0 = y0; v1 = y1;
          }
          if (row < P.qw) {
            *(float2*)(P.qbuf + row) = make_float2(v0, v1);
          } else {
            const bool is_k = row < P.qw + P.kw;
            const int rr = row - P.qw - (is_k ? 0 : P.kw);
            const int g = rr / HD, d = rr - g * HD;
            float* dst = is_k ? L.k_cache + (size_t)g * P.max_ctx * HD + cai_k_blocked_index(len, d, HD)
                              : L.v_cache + ((size_t)g * P.max_ctx + len) * HD + d;
            *(float2*)dst = make_float2(v0, v1);
          }
        }
      }
    }
    if (P.fine) sk_trace(P, nts, 6);
    SK_SYNC(true);
    sk_trace(P, nts, FAM_LINEAR);
    // ---- attention over the cache
    sk_drain();                                                      // (the cursor is on hold: nothing of the rings is in flight or unread)
    sk_attention<G, HD>(P, L, (unsigned char*)xs, n, chunk, used, lane, warp);
    // the rings are the weights' again: resume the cursor at the O matrix and prime
    __syncthreads();
    f.hold = 0; f.slot = rd_slot;
    sk_next_matrix(P, f, tab, lane, warp, true);
    for (int s = 0; s < P.ring_depth - 1; ++s) sk_fill_one(P, f, tab, ring_w, lane, warp);
    if (P.fine) sk_trace(P, nts, 6);
    SK_SYNC(true);
    sk_trace(P, nts, FAM_ATTN);
    if (!fold) {
      sk_merge_phase<HD>(P, used);
      SK_SYNC(true);
      sk_trace(P, nts, FAM_ATTN);
      sk_stage_copy(xs, P.att, P.qw);
    } else {
      sk_stage_merge<HD>(P, xs, used);
    }
    // ---- O + residual
    if (P.fine) sk_trace(P, nts, 4);
    sk_gemv(P, MK_O, f, rd_slot, tab, ring_w, xs, slots, lane, warp);
    if (P.fine) sk_trace(P, nts, 5);
    __syncthreads();
    {
      const SkMat& M = P.mat[MK_O];
      const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x), rg1 = sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x);
      if constexpr (LL) {
        bool ok = true;
        for (int i = threadIdx.x; i < (rg1 - rg0) * 4; i += SK_THREADS) {
          const int row = 4 * rg0 + i;
          if (row < M.n_rows) ok = sk_row_handover(P, row, sk_slot_sum(slots, i >> 2, M.ksplit, i & 3), tag0 + 2 * l + 1) && ok;
        }
        if (__syncthreads_or(ok ? 0 : 1)) { sk_drain(); return; }
      } else {
        for (int i = threadIdx.x; i < (rg1 - rg0) * 4; i += SK_THREADS) {
          const int row = 4 * rg0 + i;
          if (row < M.n_rows) P.xres[row] = sk_slot_sum(slots, i >> 2, M.ksplit, i & 3) + __ldcg(P.xres + row);
        }
      }
    }
    if constexpr (!LL) SK_SYNC(true);
    sk_trace(P, nts, FAM_LINEAR);
    // ---- [up|gate]: RMSNorm in the staging, SwiGLU in the epilogue
    if (!sk_stage_normed<LL>(P, xs, red, LL ? P.ll2 + (size_t)((tag0 + 2 * l + 1) & 1) * P.hidden * 2 : P.xres, -1, L.ffn_norm, nullptr,
                             tag0 + 2 * l + 1)) { sk_drain(); return; }
    sk_gemv(P, MK_GU, f, rd_slot, tab, ring_w, xs, slots, lane, warp);
    __syncthreads();
    {
      const SkMat& M = P.mat[MK_GU];
      const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x), rg1 = sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x);
      for (int u = threadIdx.x; u < (rg1 - rg0) * 2; u += SK_THREADS) {
        const int rgl = u >> 1, r0 = (u & 1) * 2;
        const int j = 2 * (rg0 + rgl) + (u & 1);
        if (j < M.half) {
          const float up = sk_slot_sum(slots, rgl, M.ksplit, r0), gate = sk_slot_sum(slots, rgl, M.ksplit, r0 + 1);
          P.act[j] = up * swish(gate);
        }
      }
    }
    SK_SYNC(true);
    sk_trace(P, nts, FAM_LINEAR);
    // ---- down + residual
    sk_stage_copy(xs, P.act, P.inter);
    sk_gemv(P, MK_DOWN, f, rd_slot, tab, ring_w, xs, slots, lane, warp);
    __syncthreads();
    {
      const SkMat& M = P.mat[MK_DOWN];
      const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x), rg1 = sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x);
      if constexpr (LL) {
        bool ok = true;
        for (int i = threadIdx.x; i < (rg1 - rg0) * 4; i += SK_THREADS) {
          const int row = 4 * rg0 + i;
          if (row < M.n_rows) ok = sk_row_handover(P, row, sk_slot_sum(slots, i >> 2, M.ksplit, i & 3), tag0 + 2 * l + 2) && ok;
        }
        if (__syncthreads_or(ok ? 0 : 1)) { sk_drain(); return; }
      } else {
        for (int i = threadIdx.x; i < (rg1 - rg0) * 4; i += SK_THREADS) {
          const int row = 4 * rg0 + i;
          if (row < M.n_rows) P.xres[row] = sk_slot_sum(slots, i >> 2, M.ksplit, i & 3) + __ldcg(P.xres + row);
        }
      }
    }
    if constexpr (!LL) SK_SYNC(true);
    sk_trace(P, nts, FAM_LINEAR);
  }

  // ---- LM head (final norm in the staging) + this CTA's first maximum
  if (!sk_stage_normed<LL>(P, xs, red, LL ? P.ll2 + (size_t)((tag0 + 2 * P.layers) & 1) * P.hidden * 2 : P.xres, -1, P.final_norm, nullptr,
                           tag0 + 2 * P.layers)) { sk_drain(); return; }
  sk_gemv(P, MK_HEAD, f, rd_slot, tab, ring_w, xs, slots, lane, warp);
  __syncthreads();
  {
    const SkMat& M = P.mat[MK_HEAD];
    const int rg0 = sk_rg_begin(M.n_rg, blockIdx.x, gridDim.x), rg1 = sk_rg_begin(M.n_rg, blockIdx.x + 1, gridDim.x);
    float best = -INFINITY; int besti = 0x7fffffff;
    for (int i = threadIdx.x; i < (rg1 - rg0) * 4; i += SK_THREADS) {
      const int row = 4 * rg0 + i;
      if (row < M.n_rows) {
        const float v = sk_slot_sum(slots, i >> 2, M.ksplit, i & 3);
        P.logits[row] = v;
        if (v > best) { best = v; besti = row; }                   // rows ascend per thread: the first maximum stays
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) { s_best_v[warp] = best; s_best_i[warp] = besti; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < SK_WARPS; ++w)
        if (s_best_v[w] > best || (s_best_v[w] == best && s_best_i[w] < besti)) { best = s_best_v[w]; besti = s_best_i[w]; }
      P.cand_val[blockIdx.x] = best;
      P.cand_idx[blockIdx.x] = besti;
    }
  }
  sk_drain();
  // ---- last barrier: the other CTAs arrive and leave, CTA 0 waits, picks the token and advances the session
  ++epoch;
  if (!sk_barrier(P, epoch * gridDim.x, s_flag, blockIdx.x == 0)) return;
  if (blockIdx.x != 0) return;
  sk_trace(P, nts, FAM_LINEAR);
  if (warp == 0) {
    float best = -INFINITY; int besti = 0x7fffffff;
    for (int c = lane; c < (int)gridDim.x; c += 32) {
      const float v = __ldcg(P.cand_val + c);
      const int i = __ldcg(P.cand_idx + c);
      if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (besti == 0x7fffffff) besti = 0;
    bool ok = true;
    if (tp) {
      // every rank's (value, global index) through the last slot; all ranks pick the same winner
      const int site = P.tp.argmax_site;
      besti += P.tp.vocab_offset;
      if (lane == 0) {
        float* mine = P.tp.my_slots + (size_t)site * P.tp.max_elems;
        mine[0] = best; mine[1] = __int_as_float(besti);
      }
      __syncwarp();
      __threadfence_system();
      const int seq = tp_seq0 + (++tp_k);
      if (lane < P.tp.world) *(volatile int*)(P.tp.peer_flags[lane] + P.tp.rank) = seq;
      if (lane < P.tp.world) {
        const volatile int* fl = (const volatile int*)(P.tp.my_flags + lane);
        bool got = *fl >= seq;
        if (!got && *(volatile int*)P.tp.gave_up == 0) {
          const unsigned long long t0 = gtime_ns(), limit = (unsigned long long)P.limit_us * 1000ull;
          while (true) {
            if (*fl >= seq) { got = true; break; }
            if (gtime_ns() - t0 > limit) break;
          }
        }
        if (!got) { *P.err = 1; *(volatile int*)P.tp.gave_up = 1; }
        ok = got;
      }
      ok = __all_sync(0xffffffffu, ok);
      __threadfence_system();
      if (ok) {
        best = -INFINITY; besti = 0x7fffffff;
        for (int r = 0; r < P.tp.world; ++r) {
          const volatile float* src = (const volatile float*)(P.tp.peer_slots[r] + (size_t)site * P.tp.max_elems);
          const float v = src[0];
          const int i = __float_as_int(src[1]);
          if (v > best || (v == best && i < besti)) { best = v; besti = i; }
        }
        if (besti == 0x7fffffff) besti = 0;
      }
    }
    if (lane == 0 && ok) {
      P.amax_idx[0] = besti;
      P.amax_val[0] = best;
      P.tokens[0] = besti;
      P.pos[0] = pos + 1;
      P.len[0] = len + 1;
      const int cnt = *P.trace_count;
      if ((long long)(cnt + 1) <= P.trace_cap) P.trace[cnt] = besti;
      *P.trace_count = cnt + 1;
      if (tp) *(volatile int*)P.tp.seq = tp_seq0 + tp_k;
    }
    if (LL && lane == 0) *(volatile unsigned*)(P.sync + 2) = (unsigned)(tag0 + 2 * P.layers);   // (every CTA read tag0 before the first barrier)
    if (lane == 0) {
      __threadfence();
      *(volatile unsigned*)P.sync = 0u;                             // every other CTA has arrived and left
    }
  }
  sk_trace(P, nts, FAM_OTHER);
}

// A two-CTA kernel whose barrier expects one arrival more than there are CTAs: the wait must run out, raise the
// error word and return. Exercises the time-out branch of sk_barrier without hanging anything.
__global__ void step_barrier_timeout_kernel(const SkParams P) {
  __shared__ int s_flag;
  sk_barrier(P, gridDim.x + 1, &s_flag, true);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
struct StepPlan {
  SkParams P;
  int grid = 0;
  size_t smem = 0;
  void (*fn)(const SkParams) = nullptr;
  SkPtrs* ptrs_dev = nullptr;
  SkLayerDev* lay_dev = nullptr;
  float* cand_val = nullptr;
  int* cand_idx = nullptr;
  float* ll2 = nullptr;
  unsigned* sync_dev = nullptr;
  int trace_len = 0;
};

typedef void (*StepFn)(const SkParams);
static StepFn pick_kernel(int G, int HD, bool ll) {
#define SK_CASE(g, hd) if (G == g && HD == hd) return ll ? step_kernel<g, hd, true> : step_kernel<g, hd, false>
  SK_CASE(1, 64); SK_CASE(2, 64); SK_CASE(4, 64); SK_CASE(7, 64); SK_CASE(8, 64);
  SK_CASE(1, 128); SK_CASE(2, 128); SK_CASE(4, 128); SK_CASE(5, 128); SK_CASE(8, 128);
#undef SK_CASE
  return nullptr;
}

static bool q8_ok(const QWeight* w) {
  return w && w->type == CAI_TYPE_Q8_0 && w->codes && w->scales && (w->k % 32) == 0 && (w->sstride % 8) == 0 &&
         ((uintptr_t)w->codes % 16) == 0 && ((uintptr_t)w->scales % 16) == 0 && (w->k % 16) == 0;
}

// K-parts per row group that balance the 16 warps of the busiest CTA (cost in chunk times; a tile's lane reduction
// and bookkeeping count as a third of a chunk).
static void pick_ksplit(SkMat& M, int grid) {
  const int max_local = (M.n_rg + grid - 1) / grid;
  double best_cost = 1e30;
  int best_s = 1, best_cpp = M.KC;
  for (int s = 1; s <= M.KC; ++s) {
    const int cpp = (M.KC + s - 1) / s;
    const int s_eff = (M.KC + cpp - 1) / cpp;
    const int tiles = max_local * s_eff;
    const int rounds = (tiles + SK_WARPS - 1) / SK_WARPS;
    const double cost = rounds * (cpp + 0.35);
    if (cost < best_cost - 1e-9) { best_cost = cost; best_s = s_eff; best_cpp = cpp; }
  }
  M.ksplit = best_s; M.cpp = best_cpp;
}

static SkMat make_mat(const QWeight* w, int half, int grid) {
  SkMat M;
  M.K = (int)w->k; M.KC = (int)((w->k + 511) / 512); M.sstride = (int)w->sstride; M.n_rows = (int)w->n; M.half = half;
  M.n_rg = half > 0 ? (half + 1) / 2 : (int)((w->n + 3) / 4);
  pick_ksplit(M, grid);
  return M;
}

void step_plan_destroy(StepPlan* p) {
  if (!p) return;
  if (p->ptrs_dev) cudaFree(p->ptrs_dev);
  if (p->lay_dev) cudaFree(p->lay_dev);
  if (p->cand_val) cudaFree(p->cand_val);
  if (p->cand_idx) cudaFree(p->cand_idx);
  if (p->ll2) cudaFree(p->ll2);
  if (p->sync_dev) cudaFree(p->sync_dev);
  delete p;
}

int step_plan_create(cai_ctx* ctx, const StepSetup& s, StepPlan** out) {
  *out = nullptr;
  if (env_int("CAI_STEP_KERNEL", -1) == 0) return CAI_ERR_UNSUPPORTED;
  if (s.kv_heads < 1 || (s.q_heads % s.kv_heads)) return CAI_ERR_UNSUPPORTED;
  const int G = s.q_heads / s.kv_heads, HD = s.head_dim;
  // Tagged-pair hand-over of the residual stream: always between GPUs (it replaces a flag exchange and two grid
  // barriers per sum over the ranks); on one GPU it measured 4 % faster on the Qwen2.5-0.5B shape and 4 % slower on the
  // Qwen2.5-32B shape than the grid barrier, so there it serves small layers only. CAI_STEP_LL=0/1 forces it on one GPU.
  const bool use_ll = s.tp_world > 1 || env_int("CAI_STEP_LL", ((int64_t)s.hidden * s.inter * 3 < ((int64_t)24 << 20)) ? 1 : 0) != 0;
  StepFn fn = pick_kernel(G, HD, use_ll);
  if (!fn) return CAI_ERR_UNSUPPORTED;
  if (s.hidden > SK_THREADS * SK_XU * 4 || (s.hidden % 32) || (s.inter % 32) || s.layers < 1) return CAI_ERR_UNSUPPORTED;
  if (!q8_ok(s.embed) || !q8_ok(s.lm_head) || s.embed->k != s.hidden || s.lm_head->k != s.hidden) return CAI_ERR_UNSUPPORTED;
  if (s.lm_head->bias) return CAI_ERR_UNSUPPORTED;
  const int qw = s.q_heads * HD, kw = s.kv_heads * HD;
  for (const auto& L : s.layer) {
    if (!q8_ok(L.wqkv) || !q8_ok(L.wo) || !q8_ok(L.wgu) || !q8_ok(L.wdown)) return CAI_ERR_UNSUPPORTED;
    if (L.wqkv->n != qw + 2 * kw || L.wqkv->k != s.hidden || L.wo->n != s.hidden || L.wo->k != qw ||
        L.wgu->n != 2 * (int64_t)s.inter || L.wgu->k != s.hidden || L.wdown->n != s.hidden || L.wdown->k != s.inter)
      return CAI_ERR_UNSUPPORTED;
    if (L.wo->bias || L.wgu->bias || L.wdown->bias) return CAI_ERR_UNSUPPORTED;
    if (L.wqkv->sstride != s.layer[0].wqkv->sstride || L.wo->sstride != s.layer[0].wo->sstride ||
        L.wgu->sstride != s.layer[0].wgu->sstride || L.wdown->sstride != s.layer[0].wdown->sstride)
      return CAI_ERR_UNSUPPORTED;
    if (((uintptr_t)L.k_cache % 16) || ((uintptr_t)L.v_cache % 16) || ((uintptr_t)L.attn_norm % 16) || ((uintptr_t)L.ffn_norm % 16))
      return CAI_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)s.final_norm % 16) || (qw % 4) || (s.hidden % 4)) return CAI_ERR_UNSUPPORTED;
  if (s.tp_world > 1 && (!s.ar || s.tp_world > 8)) return CAI_ERR_UNSUPPORTED;
  if (!s.k_blocked || (s.max_ctx % 32)) return CAI_ERR_UNSUPPORTED;

  StepPlan* p = new (std::nothrow) StepPlan();
  if (!p) return CAI_ERR_OOM;
  memset(&p->P, 0, sizeof(p->P));
  p->fn = fn;
  p->grid = ctx->sm_count;
  SkParams& P = p->P;
  const int grid = p->grid;
  P.mat[MK_QKV] = make_mat(s.layer[0].wqkv, 0, grid);
  P.mat[MK_O] = make_mat(s.layer[0].wo, 0, grid);
  P.mat[MK_GU] = make_mat(s.layer[0].wgu, s.inter, grid);
  P.mat[MK_DOWN] = make_mat(s.layer[0].wdown, 0, grid);
  P.mat[MK_HEAD] = make_mat(s.lm_head, 0, grid);
  P.layers = s.layers; P.n_mats = 4 * s.layers + 1;
  P.hidden = s.hidden; P.qw = qw; P.kw = kw; P.inter = s.inter; P.q_heads = s.q_heads; P.kv_heads = s.kv_heads;
  P.max_ctx = s.max_ctx; P.vocab = s.vocab;
  P.eps = s.rms_eps; P.inv_sqrt_d = (float)(1.0 / sqrt((double)HD));
  P.emb_codes = (const uint8_t*)s.embed->codes; P.emb_scales = s.embed->scales; P.emb_sstride = (int)s.embed->sstride; P.emb_rows = (int)s.embed->n;
  P.final_norm = s.final_norm; P.theta = s.theta;
  P.tokens = s.tokens; P.pos = s.pos; P.len = s.len;
  P.xres = s.xres; P.qbuf = s.qbuf; P.att = s.att; P.act = s.act; P.logits = s.logits; P.partial = s.partial;
  P.amax_idx = s.amax_idx; P.amax_val = s.amax_val; P.trace = s.trace; P.trace_count = s.trace_count; P.trace_cap = s.trace_cap;
  P.err = ctx->err_flag; P.limit_us = ctx->wait_limit_us;
  // context splits: about one (kv head, split) item per CTA, at least one 32-row tile each at full context, and what
  // the session's scratch holds
  {
    int ns = grid / s.kv_heads;
    const int cap_rows = (s.max_ctx + 31) / 32;
    if (ns > cap_rows) ns = cap_rows;
    const size_t per_split = (size_t)s.q_heads * (HD + 2);
    if ((size_t)ns * per_split > s.partial_floats) ns = (int)(s.partial_floats / per_split);
    if (ns < 1) { delete p; return CAI_ERR_UNSUPPORTED; }
    P.nsplit_max = ns;
  }
  // shared memory: staged row (or the attention scratch), partial-sum slots, small words, pointer tables, rings
  size_t slot_floats = 0;
  int kmax = s.hidden;
  if (qw > kmax) kmax = qw;
  if (s.inter > kmax) kmax = s.inter;
  for (int k = 0; k < 5; ++k) {
    const size_t need = (size_t)((P.mat[k].n_rg + grid - 1) / grid) * P.mat[k].ksplit * SK_RPW;
    if (need > slot_floats) slot_floats = need;
  }
  // layout: small words | pointer tables | staged row | partial-sum slots | weight rings. The attention phase takes
  // everything from the staged row up (the fill cursor is on hold then, nothing else lives there).
  int max_smem = 0;
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
  const size_t misc_bytes = 320 + (size_t)HD * 4;
  const size_t tab_bytes = (((size_t)s.layers * sizeof(SkLayerDev) + 15) & ~(size_t)15) + (size_t)P.n_mats * sizeof(SkPtrs);
  P.off_misc = 0;
  P.off_tab = (int)((misc_bytes + 15) & ~(size_t)15);
  P.off_xs = (int)(((size_t)P.off_tab + tab_bytes + 127) & ~(size_t)127);
  const size_t xs_bytes = ((size_t)kmax * 4 + 15) & ~(size_t)15;
  const size_t slot_bytes = (slot_floats * 4 + 15) & ~(size_t)15;
  P.off_slots = (int)(P.off_xs + xs_bytes);
  P.off_ring = (int)(((size_t)P.off_slots + slot_bytes + 127) & ~(size_t)127);
  const size_t stage_all = (size_t)SK_WARPS * SK_STAGE;
  int depth = ((size_t)P.off_ring < (size_t)max_smem) ? (int)(((size_t)max_smem - (size_t)P.off_ring) / stage_all) : 0;
  const int want = env_int("CAI_STEP_RING", 4);
  if (depth > want) depth = want;
  if (depth > 8) depth = 8;
  if (depth < 2) { delete p; return CAI_ERR_UNSUPPORTED; }
  P.ring_depth = depth;
  p->smem = (size_t)max_smem;                          // one CTA per SM in any case: the attention phase uses what the rings leave
  {
    const int avail = max_smem - P.off_xs;
    // Tiles of 32 rows an item holds at full context. Few of them (tensor-parallel shards: few KV heads, so many short
    // splits): a handful of warps with rings deep enough to have ALL stages of a tile in flight at once, because the
    // phase is then one round trip to memory; many: every warp, as deep as fits.
    int chunk_full = (s.max_ctx + P.nsplit_max - 1) / P.nsplit_max;
    if (chunk_full < SK_MIN_CHUNK) chunk_full = SK_MIN_CHUNK;
    const int tiles_item = (chunk_full + 31) / 32;
    int aw = SK_WARPS, ad = 0;
    if (tiles_item <= 4) {
      aw = 4;
      for (ad = 8; ad >= 2; --ad) if (at_smem_bytes(G, HD, aw, ad) <= avail) break;
    } else {
      for (; aw >= 4; aw >>= 1) {
        for (ad = 4; ad >= 2; --ad) if (at_smem_bytes(G, HD, aw, ad) <= avail) break;
        if (ad >= 3 || (aw == 4 && ad >= 2)) break;
      }
    }
    if (aw < 4 || ad < 2) { delete p; return CAI_ERR_UNSUPPORTED; }
    aw = env_int("CAI_STEP_AT_WARPS", aw); ad = env_int("CAI_STEP_AT_DEPTH", ad);
    if ((aw != 4 && aw != 8 && aw != 16) || ad < 2 || ad > 8 || at_smem_bytes(G, HD, aw, ad) > avail) { delete p; return CAI_ERR_UNSUPPORTED; }
    P.at_warps = aw; P.at_depth = ad;
  }

  // device tables
  std::vector<SkPtrs> ptrs((size_t)P.n_mats);
  std::vector<SkLayerDev> lay((size_t)s.layers);
  for (int l = 0; l < s.layers; ++l) {
    const StepLayerSetup& L = s.layer[(size_t)l];
    const QWeight* ws[4] = {L.wqkv, L.wo, L.wgu, L.wdown};
    for (int j = 0; j < 4; ++j) { ptrs[(size_t)(4 * l + j)].codes = (const uint8_t*)ws[j]->codes; ptrs[(size_t)(4 * l + j)].scales = ws[j]->scales; }
    lay[(size_t)l].attn_norm = L.attn_norm; lay[(size_t)l].ffn_norm = L.ffn_norm; lay[(size_t)l].qkv_bias = L.wqkv->bias;
    lay[(size_t)l].k_cache = L.k_cache; lay[(size_t)l].v_cache = L.v_cache;
  }
  ptrs[(size_t)(4 * s.layers)].codes = (const uint8_t*)s.lm_head->codes;
  ptrs[(size_t)(4 * s.layers)].scales = s.lm_head->scales;
  bool ok = cudaMalloc((void**)&p->ptrs_dev, ptrs.size() * sizeof(SkPtrs)) == cudaSuccess &&
            cudaMalloc((void**)&p->lay_dev, lay.size() * sizeof(SkLayerDev) + 16) == cudaSuccess &&
            cudaMalloc((void**)&p->cand_val, (size_t)grid * 4) == cudaSuccess &&
            cudaMalloc((void**)&p->cand_idx, (size_t)grid * 4) == cudaSuccess &&
            cudaMalloc((void**)&p->sync_dev, 16) == cudaSuccess &&
            cudaMalloc((void**)&p->ll2, (size_t)4 * s.hidden * sizeof(float)) == cudaSuccess;
  if (ok) {
    ok = cudaMemcpyAsync(p->ptrs_dev, ptrs.data(), ptrs.size() * sizeof(SkPtrs), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
         cudaMemcpyAsync(p->lay_dev, lay.data(), lay.size() * sizeof(SkLayerDev), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
         cudaMemsetAsync(p->sync_dev, 0, 16, ctx->stream) == cudaSuccess &&
         cudaMemsetAsync(p->ll2, 0, (size_t)4 * s.hidden * sizeof(float), ctx->stream) == cudaSuccess && cudaStreamSynchronize(ctx->stream) == cudaSuccess;
  }
  if (ok) ok = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p->smem) == cudaSuccess;
  if (ok) {
    int nblk = 0;
    ok = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nblk, (const void*)fn, SK_THREADS, p->smem) == cudaSuccess && nblk >= 1;
  }
  if (!ok) { cudaGetLastError(); step_plan_destroy(p); return CAI_ERR_UNSUPPORTED; }
  P.ptrs = p->ptrs_dev; P.lay = p->lay_dev; P.cand_val = p->cand_val; P.cand_idx = p->cand_idx; P.sync = p->sync_dev; P.ll2 = p->ll2;
  P.use_ll = use_ll ? 1 : 0;
  P.tp.world = 1; P.tp.rank = 0;
  if (s.tp_world > 1) {
    TpExchange ex;
    if (comm_ar_exchange(s.ar, &ex) != CAI_OK || ex.sites < 2 || ex.max_elems < s.hidden || (ex.max_elems % 4)) {
      step_plan_destroy(p);
      return CAI_ERR_UNSUPPORTED;
    }
    P.tp.rank = ex.rank; P.tp.world = ex.world; P.tp.my_flags = ex.my_flags; P.tp.my_slots = ex.my_slots;
    for (int r = 0; r < 8; ++r) { P.tp.peer_flags[r] = ex.peer_flags[r]; P.tp.peer_slots[r] = ex.peer_slots[r]; }
    P.tp.max_elems = ex.max_elems; P.tp.seq = ex.seq; P.tp.gave_up = ex.gave_up; P.tp.vocab_offset = s.vocab_offset;
    // the row exchange lives at the start of the slot area, the argmax exchange in the last slot
    P.tp.argmax_site = ex.sites - 1;
    if ((int64_t)(ex.sites - 1) * ex.max_elems < (int64_t)4 * ex.world * s.hidden) { step_plan_destroy(p); return CAI_ERR_UNSUPPORTED; }
    for (int r = 0; r < ex.world; ++r) P.tp.peer_ll1[r] = (float*)ex.peer_slots[r];
  }
  // phases per step: per layer 4 products + attention (+ merge) (+ 2 exchanges), head, advance, start
  p->trace_len = 1 + 2 * (s.layers * 16 + 4);
  *out = p;
  return CAI_OK;
}

int step_plan_trace_len(const StepPlan* p) { return p->trace_len; }

int step_plan_enqueue(cai_ctx* ctx, StepPlan* p, unsigned long long* ts_dev) {
  SkParams P = p->P;
  P.ts = ts_dev;
  P.fine = (ts_dev && env_int("CAI_STEP_TRACE_FINE", 0)) ? 1 : 0;
  P.limit_us = ctx->wait_limit_us;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)p->grid); cfg.blockDim = dim3(SK_THREADS); cfg.dynamicSmemBytes = p->smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  void* args[1] = {(void*)&P};
  cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)p->fn, args);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "step kernel launch -> %s", cudaGetErrorString(e));
  ctx->launches++;
  if (CAI_CHECKED_BUILD) return cai_checked_after_launch(ctx, __FILE__, __LINE__);
  return CAI_OK;
}

int step_plan_reset_sync(cai_ctx* ctx, StepPlan* p) {
  CAI_CUDA(ctx, cudaMemsetAsync(p->sync_dev, 0, 8, ctx->stream));     // arrivals and the abort word; the tag counter keeps counting
  CAI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return CAI_OK;
}

// Runs the grid barrier of the step kernel with one arrival missing (2 CTAs, 3 expected): it must give up after
// limit_us, raise the error word and return. The status is what cai_check_device_error then reports.
int step_barrier_selftest(cai_ctx* ctx, unsigned limit_us) {
  unsigned* sync_dev = nullptr;
  CAI_CUDA(ctx, cudaMalloc((void**)&sync_dev, 16));
  CAI_CUDA(ctx, cudaMemsetAsync(sync_dev, 0, 16, ctx->stream));
  SkParams P;
  memset(&P, 0, sizeof(P));
  P.sync = sync_dev; P.err = ctx->err_flag; P.limit_us = limit_us;
  step_barrier_timeout_kernel<<<2, 64, 0, ctx->stream>>>(P);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(sync_dev);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "barrier self-test -> %s", cudaGetErrorString(e));
  ctx->launches++;
  return cai_check_device_error(ctx);
}
