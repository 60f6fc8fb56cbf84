// Dequant-fused GEMV for GGUF Q8_0 / Q4_0 weights (small batch), plus a generic
// warp-per-row kernel for F32 / F16 weights of any width.
//
//   y[b][a] = epilogue( sum_i W[a][i] * x[b][i] ),  W[a][i] = d(a, i/32) * code(a, i)
//
// The sum is formed per 32-block as d * (sum code*x) in fp32: one multiply by the
// block scale per 16 codes instead of one per code. Codes become floats exactly
// (integer -> float through the 2^23 constant), accumulation is fp32 in packed
// fp32x2 instructions, the reduction order is fixed (no atomics), so results are
// reproducible run to run.
//
// Work split: a warp owns RPW output rows and walks K in 512-code (Q8_0) or
// 1024-code (Q4_0) strides, one 16-byte streaming load per lane per row, the next
// stride's loads issued before the current one is consumed; KSPLIT warps of a CTA
// may share the same rows (small-N / large-K shapes) and are combined in shared
// memory in a fixed order. Activations are staged once per CTA in shared memory
// when they fit.
#include "gemv_common.cuh"
#include "gguf_blocks.cuh"
#include <stdlib.h>

// RING = false: a lane keeps the next stride's codes in registers while it consumes the current one.
// RING = true: every warp owns a ring of p.ring_depth stages in shared memory (per stage RPW x 512 bytes of codes
// and the RPW x CHUNK scales that go with them) filled by cp.async, depth-1 strides ahead of the arithmetic: three
// to five times the bytes in flight per SM at no register cost. A lane copies and reads back its own 16 code
// bytes; the scales are copied by the first lanes and read by all (hence the warp barrier per stride).
template <int TYPE, int NB, int RPW, int MINB, bool RING>
__global__ void __launch_bounds__(256, MINB) gemv_quant_kernel(const GemvParams p) {
  extern __shared__ __align__(16) float smem_f[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_cta = blockDim.x >> 5;
  const int groups_per_cta = warps_per_cta / p.ksplit;
  const int group = warp / p.ksplit;
  const int kpart = warp - group * p.ksplit;
  // codes per lane chunk (one 16-byte load) and per warp stride
  // (CAI_TYPE_I8ROW rows are stored like Q8_0 codes, int8 + 128, without a scale plane: the row's fp32 scale multiplies
  // the finished sum, the way DotProductsTiledInt8 applies Scales[a] after the raw code reduction)
  constexpr int CHUNK = (TYPE != CAI_TYPE_Q4_0) ? 16 : 32;
  constexpr int CODE_SHIFT = (TYPE != CAI_TYPE_Q4_0) ? 0 : 1;     // bytes = codes >> shift
  constexpr bool HAS_BLOCK_SCALES = (TYPE != CAI_TYPE_I8ROW);
  const int64_t K = p.k;
  const int64_t row_bytes = K >> CODE_SHIFT;
  const int64_t stride = (int64_t)p.ksplit * 32 * CHUNK;
  const int64_t stride_b = stride >> CODE_SHIFT;                  // bytes of codes per stride
  const int64_t stride_s = stride >> 5;                           // scales per stride
  const int64_t k_first = ((int64_t)kpart * 32 + lane) * CHUNK;
  const int iters = (k_first < K) ? (int)((K - k_first + stride - 1) / stride) : 0;
  // ring variant: warp-uniform trip count (lane 0's), stage geometry, this warp's ring
  constexpr int SC16 = CHUNK * 2 / 16;                            // 16-byte pieces of one row's scales per stride
  constexpr int STAGE_BYTES = RPW * (512 + CHUNK * 2);
  const int64_t k_first_w = (int64_t)kpart * 32 * CHUNK;
  const int iters_w = (k_first_w < K) ? (int)((K - k_first_w + stride - 1) / stride) : 0;
  const uint32_t ring_w = (uint32_t)__cvta_generic_to_shared((char*)smem_f + p.ring_off) + warp * p.ring_depth * STAGE_BYTES;
  const bool swiglu = (p.epi == EPI_SWIGLU);
  const int64_t units_total = swiglu ? (p.n >> 1) : p.n;
  const int units_per_group = swiglu ? (RPW / 2) : RPW;


  // Ring variant: the fill cursor runs ring_depth-1 strides ahead of the arithmetic, straight across row-block
  // boundaries, and is primed before the wait on the preceding kernel: weights are constants, only the
  // activations depend on it, so the first strides stream in while the activations are staged and normed.
  int64_t fcb = blockIdx.x;           // row block being fetched, and the stride within it
  int fit = 0, fill_slot = 0, read_slot = 0;
  const char* fwp[RPW];
  const char* fscp = nullptr;         // copy lanes: this lane's 16-byte piece of one row's scales
  int64_t fsc_idx = 0;                // its first scale index within the row
  const uint32_t fsc_dst = ring_w + RPW * 512 + (lane / SC16) * (CHUNK * 2) + (lane % SC16) * 16;
  auto block_row = [&](int64_t cb, int r) -> int64_t {
    const int64_t unit0 = (cb * groups_per_cta + group) * units_per_group;
    if (swiglu) {
      const int64_t half = p.n >> 1;
      int64_t j = unit0 + (r >> 1);
      if (j >= half) j = half - 1;
      return (r & 1) ? half + j : j;
    }
    const int64_t row = unit0 + r;
    return row >= p.n ? p.n - 1 : row;
  };
  auto fill_setup = [&]() {
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = block_row(fcb, r);
      fwp[r] = (const char*)p.codes + row * row_bytes + (k_first >> CODE_SHIFT);
      if (lane / SC16 == r) {
        fsc_idx = (k_first_w >> 5) + (lane % SC16) * 8;
        fscp = (const char*)((const unsigned short*)p.scales + row * p.sstride + fsc_idx);
      }
    }
  };
  auto fill_one = [&]() {
    if (fcb < p.cta_blocks && iters_w > 0) {
      const uint32_t ok = (fit < iters) ? 16u : 0u;
      const uint32_t dst = ring_w + fill_slot * STAGE_BYTES + lane * 16;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        gv_cp_async16(dst + r * 512, ok ? fwp[r] : (const char*)p.codes, ok);
        fwp[r] += stride_b;
      }
      if (lane < RPW * SC16) {
        const uint32_t sok = (fsc_idx < (K >> 5)) ? 16u : 0u;
        gv_cp_async16(fsc_dst + fill_slot * STAGE_BYTES, sok ? fscp : (const char*)p.scales, sok);
        fscp += stride_s * 2;
        fsc_idx += stride_s;
      }
      if (++fit == iters_w) {
        fit = 0;
        fcb += gridDim.x;
        if (fcb < p.cta_blocks) fill_setup();
      }
    }
    gv_cp_async_commit();               // one group per stride, empty past the end
    fill_slot = (fill_slot + 1 == p.ring_depth) ? 0 : fill_slot + 1;
  };

  pdl_trigger();
  if constexpr (RING) {
    if (fcb < p.cta_blocks && iters_w > 0) fill_setup();
    for (int s = 0; s < p.ring_depth - 1; ++s) fill_one();
  }
  // One-pass staging (rows of up to threads * XU float4): a thread holds its XU pieces of the row in registers, so
  // the loads are all in flight at once and the RMSNorm needs no second trip through shared memory. The norm gains
  // are constants and are fetched here, ahead of the wait on the preceding kernel.
  constexpr int XU = 8;
  const int K4 = (int)(K >> 2);
  const int nthreads = blockDim.x;
  constexpr int GU = 8;                 // pieces per thread when the norm is fused (the gains ride along in registers)
  const bool one_pass = p.x_in_smem && K4 <= nthreads * (p.norm_gain ? GU : XU) && ((uintptr_t)p.norm_gain & 15) == 0;
  float4 gain4[GU];
  if (one_pass && p.norm_gain) {
#pragma unroll
    for (int u = 0; u < GU; ++u) {
      const int c4 = threadIdx.x + u * nthreads;
      gain4[u] = (c4 < K4) ? __ldg((const float4*)p.norm_gain + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();

  // operand selection
  const char* codes = (const char*)p.codes;
  const __half* scales = p.scales;
  const float* bias = p.bias;
  int b0 = blockIdx.y * NB;
  int pair = 0;
  const float* x = p.x;
  if (p.expert_ids) {
    pair = blockIdx.y;
    int e = p.expert_ids[pair];
    if (e < 0 || e >= p.bank_count) {
      if (threadIdx.x == 0) cai_report_index(p.err_flag, CAI_SITE_MOE_EXPERT, e, p.bank_count);
      e = e < 0 ? 0 : p.bank_count - 1;
    }
    codes = (const char*)p.bank_codes[e];
    scales = p.bank_scales[e];
    bias = nullptr;
    x = p.x + (int64_t)(pair / p.x_row_div) * p.ldx;
    b0 = 0;
  } else {
    x = p.x + (int64_t)b0 * p.ldx;
  }

  // Activations -> shared memory ONCE per CTA (the CTA then walks many row blocks), with the per-token
  // RMSNorm of the reference applied on the way when asked: y = gain * (x * inv). Rows beyond the batch
  // repeat row 0 and are never stored.
  const float* xbase[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) xbase[b] = x + (int64_t)((b0 + b < p.batch) ? b : 0) * p.ldx;
  float* red = smem_f;
  if (p.x_in_smem) {
    // A lane reads the 16 (Q8_0) or 32 (Q4_0) activations of its codes as 16-byte pieces; with the natural layout
    // the lanes of a quarter-warp are 64 or 128 bytes apart and collide on 2 or 1 of the 8 bank groups (measured:
    // 70 % of the shared-memory wavefronts of this kernel were conflict replays). So the pieces of a lane's
    // segment are stored XOR-ed with the segment index: x_phys() below, undone in the reads by `xsw`.
    red = smem_f + (int64_t)NB * K;
    float* nred = red + (size_t)2 * warps_per_cta * (RPW * NB);
    if (one_pass) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float* xg = x + (int64_t)((b0 + b < p.batch) ? b : 0) * p.ldx;
        float4 xv[XU];
#pragma unroll
        for (int u = 0; u < XU; ++u) {
          const int c4 = threadIdx.x + u * nthreads;
          xv[u] = (c4 < K4) ? __ldcg((const float4*)xg + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (p.norm_gain) {
          float ss = 0.f;
#pragma unroll
          for (int u = 0; u < GU; ++u) {
            ss = fmaf(xv[u].x, xv[u].x, ss); ss = fmaf(xv[u].y, xv[u].y, ss);
            ss = fmaf(xv[u].z, xv[u].z, ss); ss = fmaf(xv[u].w, xv[u].w, ss);
          }
          ss = block_sum(ss, nred);
          const float inv = 1.0f / sqrtf(ss / (float)K + p.norm_eps);
#pragma unroll
          for (int u = 0; u < GU; ++u) {
            xv[u].x = gain4[u].x * (xv[u].x * inv); xv[u].y = gain4[u].y * (xv[u].y * inv);
            xv[u].z = gain4[u].z * (xv[u].z * inv); xv[u].w = gain4[u].w * (xv[u].w * inv);
          }
        }
#pragma unroll
        for (int u = 0; u < XU; ++u) {
          const int c4 = threadIdx.x + u * nthreads;
          if (c4 < K4) *(float4*)(smem_f + (int64_t)b * K + x_phys<TYPE>((int64_t)c4 * 4)) = xv[u];
        }
      }
      __syncthreads();
    } else {
      for (int64_t i = (int64_t)threadIdx.x * 4; i < (int64_t)NB * K; i += (int64_t)blockDim.x * 4) {
        const int b = (int)(i / K);
        const int64_t c = i - (int64_t)b * K;
        const int bb = (b0 + b < p.batch) ? b : 0;
        *(float4*)(smem_f + (int64_t)b * K + x_phys<TYPE>(c)) = *(const float4*)(x + (int64_t)bb * p.ldx + c);
      }
      __syncthreads();
      if (p.norm_gain) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float* xb = smem_f + (int64_t)b * K;
          float ss = 0.f;
          for (int64_t c = threadIdx.x; c < K; c += blockDim.x) { const float v = xb[x_phys<TYPE>(c)]; ss = fmaf(v, v, ss); }
          ss = block_sum(ss, nred);
          const float inv = 1.0f / sqrtf(ss / (float)K + p.norm_eps);
          for (int64_t c = threadIdx.x; c < K; c += blockDim.x) { float* e = xb + x_phys<TYPE>(c); *e = p.norm_gain[c] * (*e * inv); }
        }
        __syncthreads();
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) xbase[b] = smem_f + (int64_t)b * K;
  }

  // persistent: this CTA takes row blocks blockIdx.x, blockIdx.x + gridDim.x, ...
  int slot_set = 0;
  for (int64_t cb = blockIdx.x; cb < p.cta_blocks; cb += gridDim.x) {
    const int64_t gidx = cb * groups_per_cta + group;
    const int64_t unit0 = gidx * units_per_group;
    // the residual a lane will add in the epilogue, fetched now so that its latency hides behind the strides
    float resid_pre = 0.f;
    if (p.epi == EPI_RESID && kpart == 0 && lane < RPW * NB) {
      const int r = lane / NB, b = lane - r * NB;
      if (unit0 + r < p.n && b0 + b < p.batch)
        resid_pre = __ldcg(p.resid + (int64_t)(p.expert_ids ? pair : (b0 + b)) * p.ldy + unit0 + r);
    }
    int64_t rows[RPW];
    if (swiglu) {
      const int64_t half = p.n >> 1;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        int64_t j = unit0 + (r >> 1);
        if (j >= half) j = half - 1;
        rows[r] = (r & 1) ? half + j : j;
      }
    } else {
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        int64_t row = unit0 + r;
        if (row >= p.n) row = p.n - 1;
        rows[r] = row;
      }
    }
    // per-row pointers advance by a fixed stride: no address multiplications inside the loop
    const char* wp[RPW];
    const unsigned short* sp[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      wp[r] = codes + rows[r] * row_bytes + (k_first >> CODE_SHIFT);
      sp[r] = HAS_BLOCK_SCALES ? (const unsigned short*)scales + rows[r] * p.sstride + (k_first >> 5) : nullptr;
    }
    int4 wv[RPW], wn[RPW];
    uint32_t sv[RPW], sn[RPW];
    if constexpr (!RING) {
#pragma unroll
      for (int r = 0; r < RPW; ++r) { wn[r] = make_int4(0, 0, 0, 0); sn[r] = 0; }
      if (iters > 0) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          wn[r] = ldg_stream16(wp[r]);
          if (HAS_BLOCK_SCALES) sn[r] = __ldg(sp[r]);
        }
      }
    }
    f32x2_t acc2[RPW][NB];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc2[r][b] = 0ull;
    const float* xr[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) xr[b] = xbase[b] + k_first;
    // the XOR the staging applied to this lane's 16-byte pieces (0 when the activations are read from global memory);
    // k_first and the stride are whole multiples of 32 segments, so it is the same for every stride
    const int xsw = p.x_in_smem ? ((TYPE != CAI_TYPE_Q4_0) ? ((lane >> 1) & 3) : (lane & 7)) : 0;

    for (int it = 0; it < (RING ? iters_w : iters); ++it) {
      if constexpr (RING) {
        gv_cp_async_wait_depth(p.ring_depth);     // stage `it` of this lane has landed
        __syncwarp();                             // ... and so have the scales the copy lanes fetched
        fill_one();                               // refills the slot read in the previous stride
        const uint32_t src = ring_w + read_slot * STAGE_BYTES;
        read_slot = (read_slot + 1 == p.ring_depth) ? 0 : read_slot + 1;
        if (it >= iters) continue;                // this lane's codes lie beyond K in the last stride
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          wv[r] = gv_lds16(src + r * 512 + lane * 16);
          sv[r] = gv_lds_u16(src + RPW * 512 + r * (CHUNK * 2) + ((lane * CHUNK) >> 5) * 2);
        }
      } else {
#pragma unroll
        for (int r = 0; r < RPW; ++r) { wv[r] = wn[r]; sv[r] = sn[r]; }
        if (it + 1 < iters) {
#pragma unroll
          for (int r = 0; r < RPW; ++r) {
            wp[r] += stride_b;
            wn[r] = ldg_stream16(wp[r]);
            if (HAS_BLOCK_SCALES) { sp[r] += stride_s; sn[r] = __ldg(sp[r]); }
          }
        }
      }
      f32x2_t part[RPW][NB];
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) part[r][b] = 0ull;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (TYPE != CAI_TYPE_Q4_0) {
          float4 xv[NB];
#pragma unroll
          for (int b = 0; b < NB; ++b) xv[b] = *(const float4*)(xr[b] + 4 * (i ^ xsw));
#pragma unroll
          for (int r = 0; r < RPW; ++r) {
            const uint32_t w = ((const uint32_t*)&wv[r])[i];
#pragma unroll
            for (int b = 0; b < NB; ++b) part[r][b] = q8_word_fma(w, xv[b], part[r][b]);
          }
        } else {
          float4 xlo[NB], xhi[NB];
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            xlo[b] = *(const float4*)(xr[b] + 4 * (i ^ xsw));
            xhi[b] = *(const float4*)(xr[b] + 4 * ((4 + i) ^ xsw));
          }
#pragma unroll
          for (int r = 0; r < RPW; ++r) {
            const uint32_t w = ((const uint32_t*)&wv[r])[i];
#pragma unroll
            for (int b = 0; b < NB; ++b) part[r][b] = q4_word_fma(w, xlo[b], xhi[b], part[r][b]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float d = HAS_BLOCK_SCALES ? half_bits_to_float(sv[r]) : 1.0f;
        const f32x2_t d2 = pack2(d, d);
#pragma unroll
        for (int b = 0; b < NB; ++b) acc2[r][b] = fma2(d2, part[r][b], acc2[r][b]);
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) xr[b] += stride;
    }

    // lanes -> one value per (row, batch)
    float acc[RPW][NB];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(sum2(acc2[r][b]));

    bool store = (unit0 < units_total);
    if (p.ksplit > 1) {
      // fixed-order combine of the KSPLIT warps of a group through shared memory
      // (two sets of slots, alternating per row block: the warps that only contribute go straight on to the next
      // block, whose partial sums land in the other set, so one barrier per block is enough)
      const float* set = red + (size_t)slot_set * warps_per_cta * (RPW * NB);
      float* slot = red + ((size_t)slot_set * warps_per_cta + warp) * (RPW * NB);
      slot_set ^= 1;
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b) slot[r * NB + b] = acc[r][b];
      }
      __syncthreads();
      if (kpart == 0) {
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float sum = 0.f;
            for (int q = 0; q < p.ksplit; ++q) sum += set[(size_t)(group * p.ksplit + q) * (RPW * NB) + r * NB + b];
            acc[r][b] = sum;
          }
      } else {
        store = false;
      }
    }
    if (store && !HAS_BLOCK_SCALES) {
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float rs = p.out_scale[rows[r]];
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] *= rs;
      }
    }
    if (store) gemv_epilogue<NB, RPW>(p, acc, unit0, b0, pair, bias, resid_pre, true);
  }
}

// Generic path: F32 / F16 weights, any K (scalar loads), warp per row (pair of rows for SwiGLU).
template <int NB>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const GemvParams p, int type) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_cta = blockDim.x >> 5;
  const char* codes = (const char*)p.codes;
  const float* bias = p.bias;
  int b0 = blockIdx.y * NB;
  int pair = 0;
  const float* x;
  if (p.expert_ids) {
    pair = blockIdx.y;
    int e = p.expert_ids[pair];
    if (e < 0 || e >= p.bank_count) {
      if (threadIdx.x == 0) cai_report_index(p.err_flag, CAI_SITE_MOE_EXPERT, e, p.bank_count);
      e = e < 0 ? 0 : p.bank_count - 1;
    }
    codes = (const char*)p.bank_codes[e];
    bias = nullptr;
    x = p.x + (int64_t)(pair / p.x_row_div) * p.ldx;
    b0 = 0;
  } else {
    x = p.x + (int64_t)b0 * p.ldx;
  }
  constexpr int RPW = 2;
  const int64_t gidx = (int64_t)blockIdx.x * warps_per_cta + warp;
  const bool sw = (p.epi == EPI_SWIGLU);
  const int64_t half = p.n >> 1;
  const int64_t unit0 = sw ? gidx : gidx * RPW;
  if (unit0 >= (sw ? half : p.n)) return;
  int64_t rows[RPW];
  if (sw) { rows[0] = unit0; rows[1] = half + unit0; }
  else { rows[0] = unit0; rows[1] = (unit0 + 1 < p.n) ? unit0 + 1 : unit0; }
  float acc[RPW][NB];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
  // rows whose width and addresses allow it go four elements per lane and step (16-byte loads of fp32 rows, 8-byte
  // loads of fp16 rows): a file's Q2_K / Q3_K / Q4_1 / Q5_x matrix, decoded to fp32 at load, is a large matrix
  int64_t i0 = 0;
  const bool vec4 = (p.k % 4) == 0 && (p.ldx % 4) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)codes % 16) == 0;
  if (vec4) {
    const int64_t k4 = p.k >> 2;
    for (int64_t i4 = lane; i4 < k4; i4 += 32) {
      float4 w[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (type == CAI_TYPE_F16) {
          const uint2 h = *(const uint2*)((const __half*)codes + rows[r] * p.k + 4 * i4);
          const float2 a = __half22float2(*(const __half2*)&h.x), c = __half22float2(*(const __half2*)&h.y);
          w[r] = make_float4(a.x, a.y, c.x, c.y);
        } else {
          w[r] = *(const float4*)((const float*)codes + rows[r] * p.k + 4 * i4);
        }
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int bb = (b0 + b < p.batch) ? b : 0;
        const float4 xv = *(const float4*)(x + (int64_t)bb * p.ldx + 4 * i4);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          float a = acc[r][b];
          a = fmaf(w[r].x, xv.x, a); a = fmaf(w[r].y, xv.y, a); a = fmaf(w[r].z, xv.z, a); a = fmaf(w[r].w, xv.w, a);
          acc[r][b] = a;
        }
      }
    }
    i0 = p.k;
  }
  for (int64_t i = i0 + lane; i < p.k; i += 32) {
    float w[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
      w[r] = (type == CAI_TYPE_F16) ? __half2float(((const __half*)codes)[rows[r] * p.k + i])
                                    : ((const float*)codes)[rows[r] * p.k + i];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const int bb = (b0 + b < p.batch) ? b : 0;
      const float xv = x[(int64_t)bb * p.ldx + i];
#pragma unroll
      for (int r = 0; r < RPW; ++r) acc[r][b] = fmaf(w[r], xv, acc[r][b]);
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(acc[r][b]);
  gemv_epilogue<NB, RPW>(p, acc, unit0, b0, pair, bias);
}

// K-quant path (Q4_K / Q5_K / Q6_K resident as the file's raw super-blocks): a warp owns a pair of rows and walks
// their super-blocks; per super-block a lane holds two runs of four codes of each row. As for Q8_0 / Q4_0 the block
// arithmetic is regrouped so that the scale meets a sum instead of every code:
//     sum_t (dl * code_t - ml) * x_t  =  dl * (sum_t code_t * x_t)  -  ml * (sum_t x_t),
// with dl = d * sc and ml = dmin * mn rounded once each, exactly as the reference's decoders form them
// (neural/neuralgguf.pas:448-738); codes become floats exactly (byte-permute into the 2^23 constant), the sums are
// packed fp32 FMAs, and sum_t x_t is shared by the two rows. Traffic is the file's 4.5 / 5.5 / 6.6 bits per weight instead of the 32 of a tensor
// decoded at load. Same epilogues as the other GEMVs.
// four codes (one per byte of w, minus `bias`) times four activations -> sum
template <int TYPE>
__device__ __forceinline__ float kq_dot4(uint32_t w, const float4& x) {
  const float c = -(8388608.0f + ggufdev::KQBias<TYPE>::value);
  const f32x2_t negc = pack2(c, c);
  const f32x2_t f01 = add2(pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651u))), negc);
  const f32x2_t f23 = add2(pack2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652u)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653u))), negc);
  f32x2_t s = fma2(f01, pack2(x.x, x.y), 0ull);
  s = fma2(f23, pack2(x.z, x.w), s);
  return sum2(s);
}

template <int TYPE, int NB>
__global__ void __launch_bounds__(256) gemv_kq_kernel(const GemvParams p) {
  constexpr int BB = ggufdev::KQ<TYPE>::BB;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_cta = blockDim.x >> 5;
  const uint8_t* codes = (const uint8_t*)p.codes;
  const float* bias = p.bias;
  int b0 = blockIdx.y * NB;
  int pair = 0;
  const float* x;
  if (p.expert_ids) {
    pair = blockIdx.y;
    int e = p.expert_ids[pair];
    if (e < 0 || e >= p.bank_count) {
      if (threadIdx.x == 0) cai_report_index(p.err_flag, CAI_SITE_MOE_EXPERT, e, p.bank_count);
      e = e < 0 ? 0 : p.bank_count - 1;
    }
    codes = (const uint8_t*)p.bank_codes[e];
    bias = nullptr;
    x = p.x + (int64_t)(pair / p.x_row_div) * p.ldx;
    b0 = 0;
  } else {
    x = p.x + (int64_t)b0 * p.ldx;
  }
  constexpr int RPW = 2;
  const int64_t gidx = (int64_t)blockIdx.x * warps_per_cta + warp;
  const bool sw = (p.epi == EPI_SWIGLU);
  const int64_t half = p.n >> 1;
  const int64_t unit0 = sw ? gidx : gidx * RPW;
  if (unit0 >= (sw ? half : p.n)) return;
  int64_t rows[RPW];
  if (sw) { rows[0] = unit0; rows[1] = half + unit0; }
  else { rows[0] = unit0; rows[1] = (unit0 + 1 < p.n) ? unit0 + 1 : unit0; }
  const int64_t n_sb = p.k >> 8;
  const int64_t row_bytes = n_sb * BB;
  int ea, eb;
  ggufdev::kq_lane_elements<TYPE>(lane, ea, eb);
  float acc[RPW][NB];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
  const uint8_t* rowp[RPW];
#pragma unroll
  for (int r = 0; r < RPW; ++r) rowp[r] = codes + rows[r] * row_bytes;
  // U super-blocks of both rows are requested together (a lane's share of a super-block is ~36 bytes: one at a time
  // leaves the memory pipe nearly empty), then consumed
  constexpr int U = (NB == 1) ? 4 : 2;
  for (int64_t sb0 = 0; sb0 < n_sb; sb0 += U) {
    ggufdev::KQRaw raw[U][RPW];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t sb = (sb0 + u < n_sb) ? sb0 + u : n_sb - 1;
#pragma unroll
      for (int r = 0; r < RPW; ++r) ggufdev::kq_fetch<TYPE>(rowp[r] + sb * BB, lane, raw[u][r]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (sb0 + u < n_sb) {
        const int64_t sb = sb0 + u;
        float4 xa[NB], xb[NB];
        float sxa[NB], sxb[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int bb = (b0 + b < p.batch) ? b : 0;
          const float* xr = x + (int64_t)bb * p.ldx + (sb << 8);
          xa[b] = *(const float4*)(xr + ea);
          xb[b] = *(const float4*)(xr + eb);
          sxa[b] = (xa[b].x + xa[b].y) + (xa[b].z + xa[b].w);
          sxb[b] = (xb[b].x + xb[b].y) + (xb[b].z + xb[b].w);
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          uint32_t wa, wb;
          float dla, mla, dlb, mlb;
          ggufdev::kq_runs<TYPE>(raw[u][r], lane, wa, wb, dla, mla, dlb, mlb);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float a = acc[r][b];
            a = fmaf(dla, kq_dot4<TYPE>(wa, xa[b]), a);
            a = fmaf(dlb, kq_dot4<TYPE>(wb, xb[b]), a);
            if (TYPE != CAI_TYPE_Q6_K) { a = fmaf(-mla, sxa[b], a); a = fmaf(-mlb, sxb[b], a); }
            acc[r][b] = a;
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(acc[r][b]);
  gemv_epilogue<NB, RPW>(p, acc, unit0, b0, pair, bias);
}

// ---------------------------------------------------------------------------
// Q4_K / Q5_K on integer dot products (dp4a). The kernel above turns every 4.5-bit code into a float before it multiplies
// (11 lane instructions per weight: bound by the integer pipe at 0.15 of the HBM rate). Here the codes stay integers:
//   * the CTA splits the activation row once into three exact int8 limbs per 32-wide sub-block (x = s_j * (l0 + l1/128 +
//     l2/16384), s_j a power of two, what is left below 2^-21 of the sub-block's largest magnitude), with the
//     sub-block's fp32 sum beside them, in shared memory, laid out so that a warp's 16-byte reads are conflict-free;
//   * a lane owns one pair of sub-blocks of a super-block (32 code bytes: low nibbles = sub-block 2c, high nibbles =
//     2c + 1), four lanes a super-block, a warp eight super-blocks of two rows per step; a word of four codes is one
//     mask (and one shift) and three dp4a per sub-block;
//   * per sub-block the three integer sums are combined in fp32 and enter the row's sum as in the regrouped form
//     above:  d * sc_j * s_j * sum(code * limbs) - dmin * m_j * sum(x);
//   * the raw super-blocks come through a per-warp cp.async ring (a stage = the step's eight super-blocks of both rows)
//     whose fill runs two stages ahead, across the warp's row pairs, and starts before the activation row is even read
//     (the weights do not depend on the kernel before this one).
// Every integer sum is exact, the block scales are formed as the reference forms them (d * sc rounded once).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void kqi_limbs4(const float4& v, float inv, uint32_t& w0, uint32_t& w1, uint32_t& w2) {
  const float magic = 12582912.0f;                        // 1.5 * 2^23: the sum's low byte is the rounded integer
  const float t[4] = {v.x * inv, v.y * inv, v.z * inv, v.w * inv};
  w0 = w1 = w2 = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float x0 = t[i] + magic;
    float r = (t[i] - (x0 - magic)) * 128.0f;
    const float x1 = r + magic;
    r = (r - (x1 - magic)) * 128.0f;
    const float x2 = r + magic;
    w0 |= (__float_as_uint(x0) & 0xFFu) << (8 * i);
    w1 |= (__float_as_uint(x1) & 0xFFu) << (8 * i);
    w2 |= (__float_as_uint(x2) & 0xFFu) << (8 * i);
  }
}
constexpr int KQI_SBS = 8;                                  // super-blocks of a row per step of a warp (four lanes each)
constexpr int KQI_DEPTH = 3;                                // stages of a warp's ring of raw super-blocks
static __host__ __device__ inline size_t kqi_x_bytes(int64_t k) { return (size_t)(3 * k + 2 * (k / 32) * 4); }   // limbs, scales, sums (a multiple of 16)
static __host__ __device__ inline size_t kqi_smem_bytes(int64_t k, int bb) { return kqi_x_bytes(k) + (size_t)8 * KQI_DEPTH * 2 * KQI_SBS * bb; }

template <int TYPE>
__global__ void __launch_bounds__(256, 2) gemv_kqi_kernel(const GemvParams p) {
  constexpr int BB = ggufdev::KQ<TYPE>::BB;
  constexpr int QOFF = (TYPE == CAI_TYPE_Q4_K) ? 16 : 48;          // where the nibbles start in a super-block
  constexpr int ROWSTEP = KQI_SBS * BB;                            // bytes of one row in a stage
  constexpr int STAGE = 2 * ROWSTEP;
  extern __shared__ __align__(16) unsigned char kqi_smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint8_t* codes = (const uint8_t*)p.codes;
  const float* bias = p.bias;
  const int b0 = p.expert_ids ? 0 : blockIdx.y;
  int pair = 0;
  if (p.expert_ids) {
    pdl_wait();                                                    // the expert ids are the predecessor's output
    pair = blockIdx.y;
    int e = p.expert_ids[pair];
    if (e < 0 || e >= p.bank_count) {
      if (threadIdx.x == 0) cai_report_index(p.err_flag, CAI_SITE_MOE_EXPERT, e, p.bank_count);
      e = e < 0 ? 0 : p.bank_count - 1;
    }
    codes = (const uint8_t*)p.bank_codes[e];
    bias = nullptr;
  }
  const int K = (int)p.k, npairs = K >> 6, nsub = K >> 5;
  unsigned char* xl = kqi_smem;                                    // limbs: [limb 3][16-byte piece 4][pair][16 bytes]
  float* xs = (float*)(kqi_smem + 3 * (size_t)K);                  // [nsub] power of two of the sub-block's limbs
  float* xsum = xs + nsub;                                         // [nsub] sum of the sub-block's activations
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(kqi_smem + kqi_x_bytes(K)) + (uint32_t)warp * KQI_DEPTH * STAGE;

  const bool sw = (p.epi == EPI_SWIGLU);
  const int64_t half = p.n >> 1;
  const int64_t n_units = sw ? half : (p.n + 1) / 2;
  const int64_t n_sb = p.k >> 8;
  const int64_t row_bytes = n_sb * BB;
  const int n_steps = (int)((n_sb + KQI_SBS - 1) / KQI_SBS);
  const int64_t unit_first = (int64_t)blockIdx.x * 8 + warp, unit_stride = (int64_t)gridDim.x * 8;
  const int my_units = unit_first < n_units ? (int)((n_units - unit_first + unit_stride - 1) / unit_stride) : 0;
  const int total_items = my_units * n_steps;
  // One commit group per call: the raw super-blocks of item `fi` (row pair fi / n_steps of this warp, step fi % n_steps).
  int fi = 0, fslot = 0, f_st = 0;
  int64_t f_unit = unit_first;
  const uint8_t *f_src0 = codes, *f_src1 = codes;                  // the cursor's two rows, at the lane's first piece
  auto fill = [&]() {
    if (fi < total_items) {
      if (f_st == 0) {
        const int64_t r0 = sw ? f_unit : 2 * f_unit, r1 = sw ? half + f_unit : ((2 * f_unit + 1 < p.n) ? 2 * f_unit + 1 : 2 * f_unit);
        f_src0 = codes + r0 * row_bytes + lane * 16;
        f_src1 = codes + r1 * row_bytes + lane * 16;
      }
      const int64_t s0 = (int64_t)f_st * KQI_SBS;
      const int np = (int)((n_sb - s0 < KQI_SBS) ? (n_sb - s0) : KQI_SBS) * (BB / 16);
      const uint32_t dst = ring + fslot * STAGE + lane * 16;
#pragma unroll
      for (int i = 0; i < (KQI_SBS * BB / 16 + 31) / 32; ++i) {
        if (lane + 32 * i < np) {
          gv_cp_async16(dst + i * 512, f_src0 + i * 512, 16u);
          gv_cp_async16(dst + ROWSTEP + i * 512, f_src1 + i * 512, 16u);
        }
      }
      f_src0 += ROWSTEP; f_src1 += ROWSTEP;
      ++fi;
      if (++f_st == n_steps) { f_st = 0; f_unit += unit_stride; }
    }
    gv_cp_async_commit();
    fslot = (fslot + 1 == KQI_DEPTH) ? 0 : fslot + 1;
  };
#pragma unroll 1
  for (int d = 0; d < KQI_DEPTH - 1; ++d) fill();
  if (!p.expert_ids) pdl_wait();                                   // the activations are the predecessor's output
  const float* x = p.expert_ids ? p.x + (int64_t)(pair / p.x_row_div) * p.ldx : p.x + (int64_t)b0 * p.ldx;
  // ---- the activation row -> limbs: eight lanes per sub-block, four values each
  for (int j4 = warp; j4 * 4 < nsub; j4 += 8) {
    const int j = j4 * 4 + (lane >> 3), i4 = (lane & 7) * 4;
    const float4 v = *(const float4*)(x + (size_t)j * 32 + i4);
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    float sm = (v.x + v.y) + (v.z + v.w);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      sm += __shfl_xor_sync(0xffffffffu, sm, o);
    }
    int e = (mx > 0.f && mx < 3.0e38f) ? ilogbf(mx) - 5 : 0;       // |x| / 2^e < 64
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    uint32_t w0, w1, w2;
    kqi_limbs4(v, __int_as_float((127 - e) << 23), w0, w1, w2);
    const int kk = j * 32 + i4, pr = kk >> 6, q = (kk & 63) >> 4, byte = kk & 15;
    *(uint32_t*)(xl + ((size_t)(0 * 4 + q) * npairs + pr) * 16 + byte) = w0;
    *(uint32_t*)(xl + ((size_t)(1 * 4 + q) * npairs + pr) * 16 + byte) = w1;
    *(uint32_t*)(xl + ((size_t)(2 * 4 + q) * npairs + pr) * 16 + byte) = w2;
    if ((lane & 7) == 0) {
      xs[j] = (mx < 3.0e38f) ? __int_as_float((127 + e) << 23) : __int_as_float(0x7FC00000);   // a row with inf / NaN gives NaN
      xsum[j] = sm;
    }
  }
  __syncthreads();

  const int c = lane & 3;                                          // the lane's pair of sub-blocks in its super-block
  int rslot = 0;
  for (int uk = 0; uk < my_units; ++uk) {
    const int64_t unit = unit_first + (int64_t)uk * unit_stride;
    float acc[2][1] = {{0.f}, {0.f}};
    for (int st = 0; st < n_steps; ++st) {
      gv_cp_async_wait_depth(KQI_DEPTH);                           // this lane's copies of the oldest stage have landed
      __syncwarp();                                                // ... and every lane's; the stage read last time is free
      fill();
      const uint32_t stage = ring + rslot * STAGE;
      rslot = (rslot + 1 == KQI_DEPTH) ? 0 : rslot + 1;
      const int64_t sb = (int64_t)st * KQI_SBS + (lane >> 2);
      if (sb < n_sb) {
        const int pr = (int)sb * 4 + c;
        int4 head[2], qa[2], qb[2], ha[2], hb[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t blk = stage + r * ROWSTEP + (lane >> 2) * BB;
          head[r] = gv_lds16(blk);
          qa[r] = gv_lds16(blk + QOFF + c * 32);
          qb[r] = gv_lds16(blk + QOFF + c * 32 + 16);
          if (TYPE == CAI_TYPE_Q5_K) { ha[r] = gv_lds16(blk + 16); hb[r] = gv_lds16(blk + 32); }
        }
        int al[2][3], ah[2][3];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int L = 0; L < 3; ++L) { al[r][L] = 0; ah[r][L] = 0; }
#pragma unroll
        for (int t = 0; t < 2; ++t) {                              // code bytes 16 t .. 16 t + 15 of the pair
          int4 xlo[3], xhi[3];
#pragma unroll
          for (int L = 0; L < 3; ++L) {
            xlo[L] = *(const int4*)(xl + ((size_t)(L * 4 + t) * npairs + pr) * 16);
            xhi[L] = *(const int4*)(xl + ((size_t)(L * 4 + 2 + t) * npairs + pr) * 16);
          }
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int4 qv = t ? qb[r] : qa[r];
            const int4 hv = t ? hb[r] : ha[r];
            const uint32_t qw[4] = {(uint32_t)qv.x, (uint32_t)qv.y, (uint32_t)qv.z, (uint32_t)qv.w};
            const uint32_t hw[4] = {(uint32_t)hv.x, (uint32_t)hv.y, (uint32_t)hv.z, (uint32_t)hv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t lo = qw[i] & 0x0F0F0F0Fu, hi = (qw[i] >> 4) & 0x0F0F0F0Fu;
              if (TYPE == CAI_TYPE_Q5_K) {                         // the fifth bit of sub-block j is bit j of the plane's byte
                lo |= ((hw[i] >> (2 * c)) & 0x01010101u) << 4;
                hi |= ((hw[i] >> (2 * c + 1)) & 0x01010101u) << 4;
              }
#pragma unroll
              for (int L = 0; L < 3; ++L) {
                al[r][L] = __dp4a((int)lo, ((const int*)&xlo[L])[i], al[r][L]);
                ah[r][L] = __dp4a((int)hi, ((const int*)&xhi[L])[i], ah[r][L]);
              }
            }
          }
        }
        const float2 s2 = *(const float2*)(xs + 2 * pr), m2 = *(const float2*)(xsum + 2 * pr);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          // scales and mins of sub-blocks 2c and 2c + 1 (DequantizeQ4KScaleMin, neural/neuralgguf.pas:448-472)
          const uint32_t hx = (uint32_t)head[r].x;
          const float d = __half2float(__ushort_as_half((unsigned short)(hx & 0xFFFF)));
          const float dmin = __half2float(__ushort_as_half((unsigned short)(hx >> 16)));
          // both sub-blocks at once, as byte pairs: sub-blocks 0..3 are six bits of the first two byte groups, 4..7 splice
          // the third group's nibbles under the top bits of the first two (no branch: c differs inside a warp)
          const int sh = (2 * c & 3) * 8;
          const uint32_t dd = (uint32_t)head[r].y >> sh, mm = (uint32_t)head[r].z >> sh, md = (uint32_t)head[r].w >> sh;
          const uint32_t sc2 = (c < 2) ? (dd & 0x3F3Fu) : ((md & 0x0F0Fu) | ((dd >> 2) & 0x3030u));
          const uint32_t mn2 = (c < 2) ? (mm & 0x3F3Fu) : (((md >> 4) & 0x0F0Fu) | ((mm >> 2) & 0x3030u));
          const float dl0 = __fmul_rn(d, (float)(sc2 & 0xFFu)), ml0 = __fmul_rn(dmin, (float)(mn2 & 0xFFu));
          const float dl1 = __fmul_rn(d, (float)(sc2 >> 8)), ml1 = __fmul_rn(dmin, (float)(mn2 >> 8));
          const float f = 0.0078125f;
          const float dot0 = fmaf(fmaf((float)al[r][2], f, (float)al[r][1]), f, (float)al[r][0]) * s2.x;
          const float dot1 = fmaf(fmaf((float)ah[r][2], f, (float)ah[r][1]), f, (float)ah[r][0]) * s2.y;
          float a = acc[r][0];
          a = fmaf(dl0, dot0, a); a = fmaf(-ml0, m2.x, a);
          a = fmaf(dl1, dot1, a); a = fmaf(-ml1, m2.y, a);
          acc[r][0] = a;
        }
      }
    }
    acc[0][0] = warp_sum(acc[0][0]);
    acc[1][0] = warp_sum(acc[1][0]);
    gemv_epilogue<1, 2>(p, acc, sw ? unit : 2 * unit, b0, pair, bias);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Q6_K on integer dot products: the same scheme for the 210-byte super-block (128 bytes of low nibbles, 64 bytes of
// high bit pairs, sixteen int8 group scales, one fp16 d; weight = d * sc_g * (code - 32), groups of 16). A lane owns
// the 32 low-nibble bytes of one half of one half-block and with them two 32-wide runs of weights (the low and the
// high nibbles) whose top bits share 32 bytes of the bit-pair plane. Differences to the kernel above:
//   * super-blocks are only 2-byte aligned, so a stage copies the 16-byte pieces that cover the step's bytes and the
//     lane reads aligned 4-byte words, joining neighbours with a funnel shift when its bytes start on a half word
//     (the weight buffers are allocated with 64 spare bytes, so the last piece may reach past the matrix);
//   * sum((code - 32) * limb) = sum(code * limb) - 32 * sum(limb): the limb sums of every 16 activations are kept
//     beside the limbs;
//   * one scale per 16 weights: four integer sums per limb and lane instead of two, no offsets.
// ---------------------------------------------------------------------------
constexpr int KQI6_ROWSTEP = 1712;                          // 8 x 210 bytes + up to 15 bytes of lead-in, a multiple of 16
static __host__ __device__ inline size_t kqi6_x_bytes(int64_t k) { return (size_t)(3 * k + 2 * (k / 32) * 4 + k); }   // limbs, scales, sums, limb sums [k/16][4]
static __host__ __device__ inline size_t kqi6_smem_bytes(int64_t k) { return kqi6_x_bytes(k) + (size_t)8 * KQI_DEPTH * 2 * KQI6_ROWSTEP; }

__global__ void __launch_bounds__(256, 2) gemv_kqi6_kernel(const GemvParams p) {
  constexpr int BB = 210;
  constexpr int ROWSTEP = KQI6_ROWSTEP;
  constexpr int STAGE = 2 * ROWSTEP;
  extern __shared__ __align__(16) unsigned char kqi_smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint8_t* codes = (const uint8_t*)p.codes;
  const float* bias = p.bias;
  const int b0 = p.expert_ids ? 0 : blockIdx.y;
  int pair = 0;
  if (p.expert_ids) {
    pdl_wait();                                                    // the expert ids are the predecessor's output
    pair = blockIdx.y;
    int e = p.expert_ids[pair];
    if (e < 0 || e >= p.bank_count) {
      if (threadIdx.x == 0) cai_report_index(p.err_flag, CAI_SITE_MOE_EXPERT, e, p.bank_count);
      e = e < 0 ? 0 : p.bank_count - 1;
    }
    codes = (const uint8_t*)p.bank_codes[e];
    bias = nullptr;
  }
  const int K = (int)p.k, npairs = K >> 6, nsub = K >> 5;
  unsigned char* xl = kqi_smem;                                    // limbs: [limb 3][16-byte piece 4][pair][16 bytes]
  float* xs = (float*)(kqi_smem + 3 * (size_t)K);                  // [nsub] power of two of the sub-block's limbs
  float* xsum = xs + nsub;                                         // [nsub] (unused here: Q6_K has no offsets)
  int4* lsum = (int4*)(kqi_smem + 3 * (size_t)K + 2 * (size_t)nsub * 4);   // [K / 16] sums of the three limbs over 16 activations
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(kqi_smem + kqi6_x_bytes(K)) + (uint32_t)warp * KQI_DEPTH * STAGE;

  const bool sw = (p.epi == EPI_SWIGLU);
  const int64_t half = p.n >> 1;
  const int64_t n_units = sw ? half : (p.n + 1) / 2;
  const int64_t n_sb = p.k >> 8;
  const int64_t row_bytes = n_sb * BB;
  const int n_steps = (int)((n_sb + KQI_SBS - 1) / KQI_SBS);
  const int64_t unit_first = (int64_t)blockIdx.x * 8 + warp, unit_stride = (int64_t)gridDim.x * 8;
  const int my_units = unit_first < n_units ? (int)((n_units - unit_first + unit_stride - 1) / unit_stride) : 0;
  const int total_items = my_units * n_steps;
  // One commit group per call: the 16-byte pieces that cover the item's super-blocks of both rows. A row's bytes keep
  // their position modulo 16 (byte `start & 15` of the stage row is the first byte of the step's first super-block).
  int fi = 0, fslot = 0, f_st = 0;
  int64_t f_unit = unit_first;
  int64_t f_off0 = 0, f_off1 = 0;                                  // byte offsets of the cursor's two rows in the matrix
  auto fill = [&]() {
    if (fi < total_items) {
      if (f_st == 0) {
        const int64_t r0 = sw ? f_unit : 2 * f_unit, r1 = sw ? half + f_unit : ((2 * f_unit + 1 < p.n) ? 2 * f_unit + 1 : 2 * f_unit);
        f_off0 = r0 * row_bytes; f_off1 = r1 * row_bytes;
      }
      const int64_t s0 = (int64_t)f_st * KQI_SBS;
      const int nbytes = (int)((n_sb - s0 < KQI_SBS) ? (n_sb - s0) : KQI_SBS) * BB;
      const uint32_t dst = ring + fslot * STAGE + lane * 16;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int64_t start = (r ? f_off1 : f_off0) + s0 * BB;
        const int np = (int)(((start & 15) + nbytes + 15) >> 4);   // <= 107 pieces
        const uint8_t* src = codes + (start & ~(int64_t)15) + lane * 16;
#pragma unroll
        for (int i = 0; i < (ROWSTEP / 16 + 31) / 32; ++i)
          if (lane + 32 * i < np) gv_cp_async16(dst + r * ROWSTEP + i * 512, src + i * 512, 16u);
      }
      ++fi;
      if (++f_st == n_steps) { f_st = 0; f_unit += unit_stride; }
    }
    gv_cp_async_commit();
    fslot = (fslot + 1 == KQI_DEPTH) ? 0 : fslot + 1;
  };
#pragma unroll 1
  for (int d = 0; d < KQI_DEPTH - 1; ++d) fill();
  if (!p.expert_ids) pdl_wait();                                   // the activations are the predecessor's output
  const float* x = p.expert_ids ? p.x + (int64_t)(pair / p.x_row_div) * p.ldx : p.x + (int64_t)b0 * p.ldx;
  // ---- the activation row -> limbs (as above), plus the limb sums of every 16 activations
  for (int j4 = warp; j4 * 4 < nsub; j4 += 8) {
    const int j = j4 * 4 + (lane >> 3), i4 = (lane & 7) * 4;
    const float4 v = *(const float4*)(x + (size_t)j * 32 + i4);
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    int e = (mx > 0.f && mx < 3.0e38f) ? ilogbf(mx) - 5 : 0;       // |x| / 2^e < 64
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    uint32_t w0, w1, w2;
    kqi_limbs4(v, __int_as_float((127 - e) << 23), w0, w1, w2);
    const int kk = j * 32 + i4, pr = kk >> 6, q = (kk & 63) >> 4, byte = kk & 15;
    *(uint32_t*)(xl + ((size_t)(0 * 4 + q) * npairs + pr) * 16 + byte) = w0;
    *(uint32_t*)(xl + ((size_t)(1 * 4 + q) * npairs + pr) * 16 + byte) = w1;
    *(uint32_t*)(xl + ((size_t)(2 * 4 + q) * npairs + pr) * 16 + byte) = w2;
    int l0 = __dp4a((int)w0, 0x01010101, 0), l1 = __dp4a((int)w1, 0x01010101, 0), l2 = __dp4a((int)w2, 0x01010101, 0);
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, o);
      l1 += __shfl_xor_sync(0xffffffffu, l1, o);
      l2 += __shfl_xor_sync(0xffffffffu, l2, o);
    }
    if ((lane & 3) == 0) lsum[kk >> 4] = make_int4(l0, l1, l2, 0);
    if ((lane & 7) == 0) {
      xs[j] = (mx < 3.0e38f) ? __int_as_float((127 + e) << 23) : __int_as_float(0x7FC00000);   // a row with inf / NaN gives NaN
      xsum[j] = 0.f;
    }
  }
  __syncthreads();

  const int c = lane & 3, hh = c >> 1, ps = c & 1;                 // the lane's half-block and its half of that
  int rslot = 0;
  for (int uk = 0; uk < my_units; ++uk) {
    const int64_t unit = unit_first + (int64_t)uk * unit_stride;
    const int64_t r0 = sw ? unit : 2 * unit, r1 = sw ? half + unit : ((2 * unit + 1 < p.n) ? 2 * unit + 1 : 2 * unit);
    float acc[2][1] = {{0.f}, {0.f}};
    for (int st = 0; st < n_steps; ++st) {
      gv_cp_async_wait_depth(KQI_DEPTH);                           // this lane's copies of the oldest stage have landed
      __syncwarp();                                                // ... and every lane's; the stage read last time is free
      fill();
      const uint32_t stage = ring + rslot * STAGE;
      rslot = (rslot + 1 == KQI_DEPTH) ? 0 : rslot + 1;
      const int64_t sb = (int64_t)st * KQI_SBS + (lane >> 2);
      if (sb < n_sb) {
        // the two 32-wide runs of this lane: activations of sub-blocks j_lo (low nibbles) and j_hi (high nibbles)
        const int j_lo = (int)sb * 8 + 4 * hh + ps, j_hi = j_lo + 2;
        int al[2][3][2], ah[2][3][2];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int L = 0; L < 3; ++L) { al[r][L][0] = 0; al[r][L][1] = 0; ah[r][L][0] = 0; ah[r][L][1] = 0; }
        uint32_t blk[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int64_t start = (r ? r1 : r0) * row_bytes + (int64_t)st * KQI_SBS * BB;
          blk[r] = stage + r * ROWSTEP + (uint32_t)(start & 15) + (uint32_t)(lane >> 2) * BB;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {                              // code bytes 16 t .. 16 t + 15 of the lane's 32
          int4 xlo[3], xhi[3];
#pragma unroll
          for (int L = 0; L < 3; ++L) {
            xlo[L] = *(const int4*)(xl + ((size_t)(L * 4 + (j_lo & 1) * 2 + t) * npairs + (j_lo >> 1)) * 16);
            xhi[L] = *(const int4*)(xl + ((size_t)(L * 4 + (j_hi & 1) * 2 + t) * npairs + (j_hi >> 1)) * 16);
          }
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            // 16 bytes of low nibbles and of bit pairs from a 2-byte aligned place: five aligned words each
            const uint32_t qa = blk[r] + hh * 64 + ps * 32 + t * 16, ha = blk[r] + 128 + hh * 32 + t * 16;
            const uint32_t qsh = (qa & 2u) * 8u, hsh = (ha & 2u) * 8u;
            uint32_t qv[5], hv[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) {
              asm volatile("ld.shared.u32 %0, [%1];" : "=r"(qv[i]) : "r"((qa & ~3u) + 4 * i));
              asm volatile("ld.shared.u32 %0, [%1];" : "=r"(hv[i]) : "r"((ha & ~3u) + 4 * i));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t qw = __funnelshift_r(qv[i], qv[i + 1], qsh), hw = __funnelshift_r(hv[i], hv[i + 1], hsh);
              const uint32_t lo = (qw & 0x0F0F0F0Fu) | (((hw >> (2 * ps)) & 0x03030303u) << 4);
              const uint32_t hi = ((qw >> 4) & 0x0F0F0F0Fu) | (((hw >> (4 + 2 * ps)) & 0x03030303u) << 4);
#pragma unroll
              for (int L = 0; L < 3; ++L) {
                al[r][L][t] = __dp4a((int)lo, ((const int*)&xlo[L])[i], al[r][L][t]);
                ah[r][L][t] = __dp4a((int)hi, ((const int*)&xhi[L])[i], ah[r][L][t]);
              }
            }
          }
        }
        const float s_lo = xs[j_lo], s_hi = xs[j_hi];
        const int4 ls_lo0 = lsum[2 * j_lo], ls_lo1 = lsum[2 * j_lo + 1], ls_hi0 = lsum[2 * j_hi], ls_hi1 = lsum[2 * j_hi + 1];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          // group scales 8 hh + 2 ps + {0, 1} (low nibbles) and + 4 (high nibbles); d at byte 208
          const uint32_t sa = blk[r] + 192 + 8 * hh + 2 * ps;
          unsigned short s01, s45, dh;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s01) : "r"(sa));
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s45) : "r"(sa + 4));
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(dh) : "r"(blk[r] + 208));
          const float d = __half2float(__ushort_as_half(dh));
          const float f = 0.0078125f;
          float a = acc[r][0];
#pragma unroll
          for (int g = 0; g < 4; ++g) {                            // low nibbles: groups 0, 1; high nibbles: groups 2, 3
            const int4 ls = g == 0 ? ls_lo0 : (g == 1 ? ls_lo1 : (g == 2 ? ls_hi0 : ls_hi1));
            const int a0 = (g < 2 ? al[r][0][g & 1] : ah[r][0][g & 1]) - 32 * ls.x;
            const int a1 = (g < 2 ? al[r][1][g & 1] : ah[r][1][g & 1]) - 32 * ls.y;
            const int a2 = (g < 2 ? al[r][2][g & 1] : ah[r][2][g & 1]) - 32 * ls.z;
            const int sc = (int)(int8_t)(((g < 2 ? s01 : s45) >> (8 * (g & 1))) & 0xFF);
            const float dot = fmaf(fmaf((float)a2, f, (float)a1), f, (float)a0) * (g < 2 ? s_lo : s_hi);
            a = fmaf(__fmul_rn(d, (float)sc), dot, a);
          }
          acc[r][0] = a;
        }
      }
    }
    acc[0][0] = warp_sum(acc[0][0]);
    acc[1][0] = warp_sum(acc[1][0]);
    gemv_epilogue<1, 2>(p, acc, sw ? unit : 2 * unit, b0, pair, bias);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static int launch_kqi6(cai_ctx* ctx, const GemvParams& p, int64_t n_units, unsigned grid_y) {
  const size_t smem = kqi6_smem_bytes(p.k);
  static size_t configured[64] = {0};
  const int dev = ctx->device;
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && configured[dev] < smem) {
    CAI_CUDA(ctx, cudaFuncSetAttribute(gemv_kqi6_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  int64_t ctas = (n_units + 7) / 8;
  const int64_t resident = (smem > 110 * 1024 ? 1 : 2) * (int64_t)ctx->sm_count;
  if (ctas * grid_y > resident) ctas = resident / grid_y > 0 ? resident / grid_y : 1;
  pdl_launch(ctx, gemv_kqi6_kernel, dim3((unsigned)ctas, grid_y), dim3(256), smem, p);
  return CAI_OK;
}

// ---------------------------------------------------------------------------
// Q4_0 at batch 1 on integer dot products: the scheme of the K-quant kernels on the planar Q4_0 layout (16 code
// bytes per 32-weight block, byte e = elements e and e + 16; one fp16 scale per block in its own plane;
// weight = d * (code - 8)). The float kernel spends a byte-permute and half a packed multiply-add per code and is bound
// by the integer pipe at 0.4 of the HBM rate on the largest matrices; here a word of eight codes is one mask, one
// shift and six dp4a against the three int8 limbs of the activations, and per block
//   d * s_j * (sum(code * limbs) - 8 * sum(limbs))
// enters the row's fp32 sum. A lane owns two blocks of a row per step, a warp 64 blocks of two rows; codes and scales
// come through the per-warp cp.async ring; the optional RMSNorm of the activation row is applied while it is split.
// ---------------------------------------------------------------------------
constexpr int Q4I_BPS = 64;                                 // blocks of a row per step
constexpr int Q4I_ROW = Q4I_BPS * 16 + Q4I_BPS * 2;         // a row's share of a stage: code bytes, then the blocks' scales
constexpr int Q4I_STAGE = 2 * Q4I_ROW;
static __host__ __device__ inline size_t q4i_xs_bytes(int64_t k) { return (size_t)(((k / 32) * 4 + 15) & ~(int64_t)15); }     // the blocks' powers of two, padded to 16 bytes
static __host__ __device__ inline size_t q4i_x_bytes(int64_t k) { return (size_t)(3 * k) + q4i_xs_bytes(k) + (size_t)(k / 32) * 16; }   // limbs, scales, limb sums
static __host__ __device__ inline size_t q4i_smem_bytes(int64_t k) { return q4i_x_bytes(k) + (size_t)8 * KQI_DEPTH * Q4I_STAGE; }

__global__ void __launch_bounds__(256, 2) gemv_q4i_kernel(const GemvParams p) {
  constexpr int STAGE = Q4I_STAGE, ROW = Q4I_ROW;
  extern __shared__ __align__(16) unsigned char kqi_smem[];
  __shared__ float red[32];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint8_t* codes = (const uint8_t*)p.codes;
  const unsigned short* scales = (const unsigned short*)p.scales;
  const int b0 = blockIdx.y;
  const int K = (int)p.k, npairs = K >> 6, nblk = K >> 5;
  unsigned char* xl = kqi_smem;                                    // limbs: [limb 3][16-byte piece 4][pair][16 bytes]
  float* xs = (float*)(kqi_smem + 3 * (size_t)K);                  // [nblk] power of two of the block's limbs
  int4* lsum = (int4*)(kqi_smem + 3 * (size_t)K + q4i_xs_bytes(K));    // [nblk] sums of the three limbs over the block
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(kqi_smem + q4i_x_bytes(K)) + (uint32_t)warp * KQI_DEPTH * STAGE;

  const bool sw = (p.epi == EPI_SWIGLU);
  const int64_t half = p.n >> 1;
  const int64_t n_units = sw ? half : (p.n + 1) / 2;
  const int64_t code_row = p.k >> 1;                               // code bytes of a row
  const int n_steps = (nblk + Q4I_BPS - 1) / Q4I_BPS;
  const int64_t unit_first = (int64_t)blockIdx.x * 8 + warp, unit_stride = (int64_t)gridDim.x * 8;
  const int my_units = unit_first < n_units ? (int)((n_units - unit_first + unit_stride - 1) / unit_stride) : 0;
  const int total_items = my_units * n_steps;
  // One commit group per call: step f_st of the cursor's two rows: up to 64 blocks of codes (a piece each) and their
  // scales (16-byte pieces of the scale rows, which are padded to whole pieces).
  int fi = 0, fslot = 0, f_st = 0;
  int64_t f_unit = unit_first, f_r0 = 0, f_r1 = 0;
  auto fill = [&]() {
    if (fi < total_items) {
      if (f_st == 0) {
        f_r0 = sw ? f_unit : 2 * f_unit;
        f_r1 = sw ? half + f_unit : ((2 * f_unit + 1 < p.n) ? 2 * f_unit + 1 : 2 * f_unit);
      }
      const int s0 = f_st * Q4I_BPS;
      const int nb = (nblk - s0 < Q4I_BPS) ? (nblk - s0) : Q4I_BPS;
      const uint32_t dst = ring + fslot * STAGE;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int64_t row = r ? f_r1 : f_r0;
        const uint8_t* csrc = codes + row * code_row + (int64_t)s0 * 16;
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if (lane + 32 * i < nb) gv_cp_async16(dst + r * ROW + (lane + 32 * i) * 16, csrc + (lane + 32 * i) * 16, 16u);
        if (lane * 8 < nb) gv_cp_async16(dst + r * ROW + Q4I_BPS * 16 + lane * 16, scales + row * p.sstride + s0 + lane * 8, 16u);
      }
      ++fi;
      if (++f_st == n_steps) { f_st = 0; f_unit += unit_stride; }
    }
    gv_cp_async_commit();
    fslot = (fslot + 1 == KQI_DEPTH) ? 0 : fslot + 1;
  };
#pragma unroll 1
  for (int d = 0; d < KQI_DEPTH - 1; ++d) fill();
  pdl_wait();                                                      // the activations are the predecessor's output
  const float* x = p.x + (int64_t)b0 * p.ldx;
  // ---- the activation row (normed if asked) -> limbs: eight lanes per block, four values each
  float inv = 1.f;
  if (p.norm_gain) {
    float ss = 0.f;
    for (int c4 = threadIdx.x; c4 < (K >> 2); c4 += blockDim.x) {
      const float4 v = *(const float4*)(x + 4 * c4);
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)K + p.norm_eps);
  }
  for (int j4 = warp; j4 * 4 < nblk; j4 += 8) {
    const int j = j4 * 4 + (lane >> 3), i4 = (lane & 7) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < nblk) {
      v = *(const float4*)(x + (size_t)j * 32 + i4);
      if (p.norm_gain) {
        const float4 g4 = *(const float4*)(p.norm_gain + (size_t)j * 32 + i4);
        v.x = g4.x * (v.x * inv); v.y = g4.y * (v.y * inv); v.z = g4.z * (v.z * inv); v.w = g4.w * (v.w * inv);
      }
    }
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    int e = (mx > 0.f && mx < 3.0e38f) ? ilogbf(mx) - 5 : 0;       // |x| / 2^e < 64
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    uint32_t w0, w1, w2;
    kqi_limbs4(v, __int_as_float((127 - e) << 23), w0, w1, w2);
    int l0 = __dp4a((int)w0, 0x01010101, 0), l1 = __dp4a((int)w1, 0x01010101, 0), l2 = __dp4a((int)w2, 0x01010101, 0);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, o);
      l1 += __shfl_xor_sync(0xffffffffu, l1, o);
      l2 += __shfl_xor_sync(0xffffffffu, l2, o);
    }
    if (j < nblk) {
      const int kk = j * 32 + i4, pr = kk >> 6, q = (kk & 63) >> 4, byte = kk & 15;
      *(uint32_t*)(xl + ((size_t)(0 * 4 + q) * npairs + pr) * 16 + byte) = w0;
      *(uint32_t*)(xl + ((size_t)(1 * 4 + q) * npairs + pr) * 16 + byte) = w1;
      *(uint32_t*)(xl + ((size_t)(2 * 4 + q) * npairs + pr) * 16 + byte) = w2;
      if ((lane & 7) == 0) {
        xs[j] = (mx < 3.0e38f) ? __int_as_float((127 + e) << 23) : __int_as_float(0x7FC00000);   // a row with inf / NaN gives NaN
        lsum[j] = make_int4(l0, l1, l2, 0);
      }
    }
  }
  __syncthreads();

  int rslot = 0;
  for (int uk = 0; uk < my_units; ++uk) {
    const int64_t unit = unit_first + (int64_t)uk * unit_stride;
    float acc[2][1] = {{0.f}, {0.f}};
    for (int st = 0; st < n_steps; ++st) {
      gv_cp_async_wait_depth(KQI_DEPTH);                           // this lane's copies of the oldest stage have landed
      __syncwarp();                                                // ... and every lane's; the stage read last time is free
      fill();
      const uint32_t stage = ring + rslot * STAGE;
      rslot = (rslot + 1 == KQI_DEPTH) ? 0 : rslot + 1;
      const int j0 = st * Q4I_BPS + 2 * lane;                      // the lane's two blocks: j0, j0 + 1 (the block count is even)
      if (j0 < nblk) {
        const int pr = j0 >> 1;
        uint32_t sc2[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc2[r]) : "r"(stage + r * ROW + Q4I_BPS * 16 + lane * 4));
        const float2 s2 = *(const float2*)(xs + j0);
#pragma unroll
        for (int b = 0; b < 2; ++b) {                              // block j0 + b: low nibbles = piece 2b, high nibbles = piece 2b + 1 of the pair
          int4 xlo[3], xhi[3];
#pragma unroll
          for (int L = 0; L < 3; ++L) {
            xlo[L] = *(const int4*)(xl + ((size_t)(L * 4 + 2 * b) * npairs + pr) * 16);
            xhi[L] = *(const int4*)(xl + ((size_t)(L * 4 + 2 * b + 1) * npairs + pr) * 16);
          }
          const int4 ls = lsum[j0 + b];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int4 qv = gv_lds16(stage + r * ROW + (2 * lane + b) * 16);
            const uint32_t qw[4] = {(uint32_t)qv.x, (uint32_t)qv.y, (uint32_t)qv.z, (uint32_t)qv.w};
            int a0 = -8 * ls.x, a1 = -8 * ls.y, a2 = -8 * ls.z;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t lo = qw[i] & 0x0F0F0F0Fu, hi = (qw[i] >> 4) & 0x0F0F0F0Fu;
              a0 = __dp4a((int)lo, ((const int*)&xlo[0])[i], a0); a0 = __dp4a((int)hi, ((const int*)&xhi[0])[i], a0);
              a1 = __dp4a((int)lo, ((const int*)&xlo[1])[i], a1); a1 = __dp4a((int)hi, ((const int*)&xhi[1])[i], a1);
              a2 = __dp4a((int)lo, ((const int*)&xlo[2])[i], a2); a2 = __dp4a((int)hi, ((const int*)&xhi[2])[i], a2);
            }
            const float d = __half2float(__ushort_as_half((unsigned short)(b ? (sc2[r] >> 16) : (sc2[r] & 0xFFFFu))));
            const float f = 0.0078125f;
            const float dot = fmaf(fmaf((float)a2, f, (float)a1), f, (float)a0) * (b ? s2.y : s2.x);
            acc[r][0] = fmaf(d, dot, acc[r][0]);
          }
        }
      }
    }
    acc[0][0] = warp_sum(acc[0][0]);
    acc[1][0] = warp_sum(acc[1][0]);
    gemv_epilogue<1, 2>(p, acc, sw ? unit : 2 * unit, b0, 0, p.bias);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static int launch_q4i(cai_ctx* ctx, const GemvParams& p, int64_t n_units, unsigned grid_y) {
  const size_t smem = q4i_smem_bytes(p.k);
  static size_t configured[64] = {0};
  const int dev = ctx->device;
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && configured[dev] < smem) {
    CAI_CUDA(ctx, cudaFuncSetAttribute(gemv_q4i_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  int64_t ctas = (n_units + 7) / 8;
  const int64_t resident = (smem > 110 * 1024 ? 1 : 2) * (int64_t)ctx->sm_count;
  if (ctas * grid_y > resident) ctas = resident / grid_y > 0 ? resident / grid_y : 1;
  pdl_launch(ctx, gemv_q4i_kernel, dim3((unsigned)ctas, grid_y), dim3(256), smem, p);
  return CAI_OK;
}

template <int TYPE>
static int launch_kqi(cai_ctx* ctx, const GemvParams& p, int64_t n_units, unsigned grid_y) {
  const size_t smem = kqi_smem_bytes(p.k, ggufdev::KQ<TYPE>::BB);
  static size_t configured[64] = {0};
  const int dev = ctx->device;
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && configured[dev] < smem) {   // (one of these per instantiation)
    CAI_CUDA(ctx, cudaFuncSetAttribute(gemv_kqi_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  int64_t ctas = (n_units + 7) / 8;
  const int64_t resident = 2 * (int64_t)ctx->sm_count;             // every CTA splits the activation row itself: no more CTAs than run at once
  if (ctas * grid_y > resident) ctas = resident / grid_y > 0 ? resident / grid_y : 1;
  pdl_launch(ctx, gemv_kqi_kernel<TYPE>, dim3((unsigned)ctas, grid_y), dim3(256), smem, p);
  return CAI_OK;
}

template <int TYPE>
static void launch_kq(cai_ctx* ctx, int nb, dim3 grid, int threads, const GemvParams& p) {
  if (nb == 4) pdl_launch(ctx, gemv_kq_kernel<TYPE, 4>, grid, dim3(threads), 0, p);
  else pdl_launch(ctx, gemv_kq_kernel<TYPE, 1>, grid, dim3(threads), 0, p);
}

int gemm_tc_launch(cai_ctx* ctx, const GemvParams& g, int type);      // gemm_tc.cu

int env_int(const char* name, int dflt) {
  const char* s = getenv(name);
  return (s && *s) ? atoi(s) : dflt;
}

template <int TYPE, int NB, int RPW, int MINB, bool RING = false>
static cudaError_t launch_one_b(cai_ctx* ctx, const GemvParams& p, dim3 grid, int threads, size_t smem) {
  // (single caller thread per context: the function-local cache below needs no lock)
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gemv_quant_kernel<TYPE, NB, RPW, MINB, RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  // persistent grid: exactly the CTAs that can be resident at once (a host-side query, cached per
  // instantiation, device and shared-memory size), each walking several row blocks with the activations staged once
  static int cached_blocks = 0;
  static size_t cached_smem = (size_t)-1;
  static int cached_threads = 0;
  static int cached_device = -1;
  if (cached_smem != smem || cached_threads != threads || cached_device != ctx->device) {
    int nblk = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nblk, gemv_quant_kernel<TYPE, NB, RPW, MINB, RING>, threads, smem);
    if (e != cudaSuccess) return e;
    cached_blocks = nblk < 1 ? 1 : nblk;
    cached_smem = smem;
    cached_threads = threads;
    cached_device = ctx->device;
  }
  const int64_t resident = (int64_t)ctx->sm_count * cached_blocks;
  int64_t gx = grid.x;
  if (gx * grid.y > resident) gx = resident / grid.y;
  if (gx < 1) gx = 1;
  grid.x = (unsigned)gx;
  return pdl_launch(ctx, gemv_quant_kernel<TYPE, NB, RPW, MINB, RING>, grid, dim3(threads), smem, p);
}
// MINB = CTAs per SM the compiler must leave room for (register cap). Measured on B200 for the batch-1,
// 4-rows-per-warp kernel: 2 (<= 128 registers, none spilled) 4.4 TB/s; 3 (80 registers, spills) 3.5 TB/s;
// 1 (no cap) 2.7 TB/s. CAI_GEMV_MINB=3 selects the tighter cap for experiments.
template <int TYPE, int NB, int RPW>
static cudaError_t launch_one(cai_ctx* ctx, const GemvParams& p, dim3 grid, int threads, size_t smem) {
  if constexpr (NB <= 2) {
    if (p.ring_depth > 0) return launch_one_b<TYPE, NB, RPW, 2, true>(ctx, p, grid, threads, smem);
  }
  if (NB == 1 && RPW == 4 && env_int("CAI_GEMV_MINB", 2) == 3) return launch_one_b<TYPE, NB, RPW, (NB == 1 && RPW == 4) ? 3 : 2>(ctx, p, grid, threads, smem);
  return launch_one_b<TYPE, NB, RPW, (NB <= 2) ? 2 : 1>(ctx, p, grid, threads, smem);
}
template <int TYPE, int NB>
static cudaError_t launch_quant(cai_ctx* ctx, const GemvParams& p, int rpw, dim3 grid, int threads, size_t smem) {
  if constexpr (NB <= 2) {                       // wider batch tiles never take 4 rows per warp (the dispatcher caps them at 2)
    if (rpw == 4) return launch_one<TYPE, NB, 4>(ctx, p, grid, threads, smem);
  }
  if (rpw == 2) return launch_one<TYPE, NB, 2>(ctx, p, grid, threads, smem);
  return launch_one<TYPE, NB, 1>(ctx, p, grid, threads, smem);
}
template <int TYPE>
static cudaError_t launch_quant_nb(cai_ctx* ctx, const GemvParams& p, int nb, int rpw, dim3 grid, int threads, size_t smem) {
  if (nb == 1) return launch_quant<TYPE, 1>(ctx, p, rpw, grid, threads, smem);
  if (nb == 2) return launch_quant<TYPE, 2>(ctx, p, rpw, grid, threads, smem);
  if (nb == 4) return launch_quant<TYPE, 4>(ctx, p, rpw, grid, threads, smem);
  return launch_quant<TYPE, 8>(ctx, p, rpw, grid, threads, smem);
}

// Batches the dispatcher sends to the tensor-core GEMM when nothing forces a path.
bool linear_uses_tensor_cores(const QWeight* w, int batch) {
  if (!w || (w->type != CAI_TYPE_Q8_0 && w->type != CAI_TYPE_Q4_0)) return false;
  if (batch > 64) return false;
  if (batch >= 9) return true;
  return batch >= 3 && w->n * w->k >= ((int64_t)32 << 20);
}

bool linear_can_fuse_norm(const QWeight* w, int batch) {
  if (!w || (w->type != CAI_TYPE_Q8_0 && w->type != CAI_TYPE_Q4_0 && w->type != CAI_TYPE_I8ROW)) return false;
  if (env_int("CAI_FUSE_NORM", 1) == 0) return false;
  const int nb = batch >= 5 ? 8 : (batch >= 3 ? 4 : (batch == 2 ? 2 : 1));
  if (batch > 8) return false;       // several batch tiles would each redo the norm; keep the separate kernel
  return (size_t)nb * (size_t)w->k * 4 <= (size_t)env_int("CAI_GEMV_XSMEM", 64 * 1024);
}

int linear_launch(cai_ctx* ctx, const LinearArgs& a) {
  const QWeight* w = a.w;
  ctx->cur_family = FAM_LINEAR;
  if (!w || !a.x || !a.y) return cai_fail(ctx, CAI_ERR_INVALID, "linear: null operand");
  if (a.batch < 1) return cai_fail(ctx, CAI_ERR_INVALID, "linear: batch %d", a.batch);
  if (a.epilogue == EPI_SWIGLU && (w->n % 2)) return cai_fail(ctx, CAI_ERR_INVALID, "SwiGLU epilogue needs an even row count");
  if (a.epilogue == EPI_RESID && !a.resid) return cai_fail(ctx, CAI_ERR_INVALID, "residual epilogue without residual");
  const bool indexed = a.expert_ids_dev != nullptr;
  if (indexed && a.bank_count < 1) return cai_fail(ctx, CAI_ERR_INVALID, "indexed linear: bank of %d matrices", a.bank_count);
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.err_flag = ctx->err_flag;
  p.codes = w->codes; p.scales = w->scales; p.bias = w->bias;
  p.x = a.x; p.ldx = a.ldx; p.y = a.y; p.ldy = a.ldy; p.resid = a.resid;
  p.n = w->n; p.k = w->k; p.sstride = w->sstride; p.batch = a.batch; p.act = a.act; p.epi = a.epilogue;
  p.bank_codes = a.bank_codes_dev; p.bank_scales = a.bank_scales_dev; p.expert_ids = a.expert_ids_dev; p.bank_count = a.bank_count;
  p.x_row_div = a.x_row_div < 1 ? 1 : a.x_row_div; p.row_scale = a.row_scale_dev;
  p.ksplit = 1;
  if (a.epilogue == EPI_QKV_ROPE) {
    if (!a.rope_cs || !a.k_cache || !a.v_cache || !a.cache_len_dev || a.rope_head_dim < 2 || (a.rope_head_dim % 2) || indexed ||
        a.rope_q_width + 2 * a.rope_kv_width != w->n || (a.rope_q_width % a.rope_head_dim) || (a.rope_kv_width % a.rope_head_dim))
      return cai_fail(ctx, CAI_ERR_INVALID, "linear: inconsistent fused RoPE / KV-append arguments");
    p.rope_cs = a.rope_cs; p.rope_q_width = a.rope_q_width; p.rope_kv_width = a.rope_kv_width; p.rope_head_dim = a.rope_head_dim;
    p.rope_kv_heads = a.rope_kv_heads; p.rope_max_ctx = a.rope_max_ctx; p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.k_blocked = a.k_blocked;
    p.cache_len = a.cache_len_dev;
  }
  const int64_t units = (a.epilogue == EPI_SWIGLU) ? w->n / 2 : w->n;
  const bool quant = (w->type == CAI_TYPE_Q8_0 || w->type == CAI_TYPE_Q4_0 || w->type == CAI_TYPE_I8ROW);
  p.out_scale = w->rscale;
  if (!quant) {
    const int threads = 128;
    const int wpc = threads / 32;
    const int64_t groups = (a.epilogue == EPI_SWIGLU) ? units : (units + 1) / 2;
    const int nb = indexed ? 1 : (a.batch >= 4 ? 4 : 1);
    dim3 grid((unsigned)((groups + wpc - 1) / wpc), indexed ? a.batch : (unsigned)((a.batch + nb - 1) / nb));
    if (a.norm_gain) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "linear: fused RMSNorm needs quantized weights");
    if (cai_type_is_kquant(w->type)) {
      if ((a.ldx % 4) || ((uintptr_t)a.x % 16)) return cai_fail(ctx, CAI_ERR_INVALID, "linear: activations must be 16-byte aligned with ldx %% 4 == 0");
      // Q4_K / Q5_K: the integer-dot kernel, one batch row (or expert pair) per grid row (CAI_GEMV_KQI=0: the float kernel)
      if ((w->type == CAI_TYPE_Q4_K || w->type == CAI_TYPE_Q5_K) && a.batch <= 8 && kqi_smem_bytes(w->k, 176) <= 112 * 1024 &&
          env_int("CAI_GEMV_KQI", 1) != 0) {
        if (w->type == CAI_TYPE_Q4_K) { CAI_TRY(launch_kqi<CAI_TYPE_Q4_K>(ctx, p, groups, (unsigned)a.batch)); }
        else { CAI_TRY(launch_kqi<CAI_TYPE_Q5_K>(ctx, p, groups, (unsigned)a.batch)); }
      }
      else if (w->type == CAI_TYPE_Q6_K && a.batch <= 8 && kqi6_smem_bytes(w->k) <= 160 * 1024 && env_int("CAI_GEMV_KQI", 1) != 0 &&
               ((uintptr_t)w->codes % 16) == 0) {
        CAI_TRY(launch_kqi6(ctx, p, groups, (unsigned)a.batch));
      }
      else if (w->type == CAI_TYPE_Q4_K) launch_kq<CAI_TYPE_Q4_K>(ctx, nb, grid, threads, p);
      else if (w->type == CAI_TYPE_Q5_K) launch_kq<CAI_TYPE_Q5_K>(ctx, nb, grid, threads, p);
      else launch_kq<CAI_TYPE_Q6_K>(ctx, nb, grid, threads, p);
    }
    else if (nb == 4) pdl_launch(ctx, gemv_generic_kernel<4>, grid, dim3(threads), 0, p, w->type);
    else pdl_launch(ctx, gemv_generic_kernel<1>, grid, dim3(threads), 0, p, w->type);
    CAI_LAUNCHED(ctx);
    return CAI_OK;
  }
  if ((a.ldx % 4) || ((uintptr_t)a.x % 16)) return cai_fail(ctx, CAI_ERR_INVALID, "linear: activations must be 16-byte aligned with ldx %% 4 == 0");
  // batches of 9..64 rows are a real contraction: tensor cores (tcgen05), unless the call needs a fused
  // epilogue only the CUDA-core kernel has, or CAI_GEMM_TC=0. Batches of 3..8 rows go there too when the matrix
  // is large (measured on 5120 x 27648 Q8_0: 78 us on the tensor cores for up to 16 rows, against 180 us at 4 rows
  // and 316 us at 8 rows for the CUDA-core kernel; 52 us at 2 rows stays); small matrices stay, the tensor-core
  // path has a floor of ~17 us (two launches, pipeline fill).
  if (!indexed && a.batch <= 64 && a.path != 1 && env_int("CAI_GEMM_TC", 1) != 0 &&
      (a.path == 2 || linear_uses_tensor_cores(w, a.batch))) {
    GemvParams pt = p;
    pt.norm_gain = a.norm_gain; pt.norm_eps = a.norm_eps;        // the activation-split kernel applies the norm
    const int st = gemm_tc_launch(ctx, pt, w->type);
    if (st != CAI_ERR_UNSUPPORTED) return st;
  }
  if (a.path == 2) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "linear: the tensor-core path covers batches of up to 64 rows with plain or residual epilogues");
  // Q4_0 at batch 1: integer dot products (CAI_GEMV_Q4I=0: the float kernel below). Measured against that kernel:
  // 5120 x 27648 30.3 -> 28.7 us, 4096 x 14336 18.5 -> 16.2, 3584 x 18944 18.5 -> 16.5, 896 x 4864 equal; at batch 2
  // (one grid row per batch row: the weights cross L2 twice) 41.2 -> 47.2 us, so two rows stay on the float kernel.
  if (w->type == CAI_TYPE_Q4_0 && !indexed && a.batch == 1 && (w->k % 64) == 0 && q4i_smem_bytes(w->k) <= 160 * 1024 &&
      (!a.norm_gain || ((uintptr_t)a.norm_gain % 16) == 0) && env_int("CAI_GEMV_Q4I", 1) != 0) {
    GemvParams pq = p;
    pq.norm_gain = a.norm_gain; pq.norm_eps = a.norm_eps;
    CAI_TRY(launch_q4i(ctx, pq, (a.epilogue == EPI_SWIGLU) ? units : (units + 1) / 2, (unsigned)a.batch));
    CAI_LAUNCHED(ctx);
    return CAI_OK;
  }
  // batch tile
  int nb = 1;
  if (!indexed) nb = a.batch >= 5 ? 8 : (a.batch >= 3 ? 4 : (a.batch == 2 ? 2 : 1));
  // Rows per warp / warps per row group: every CTA of the launch should be resident at once (one wave)
  // with as many 16-byte loads in flight as possible; small-N / large-K shapes split K over the warps of a CTA.
  const int64_t lane_chunk = (w->type != CAI_TYPE_Q4_0) ? 16 : 32;
  const int64_t k_iters_1 = (w->k + lane_chunk * 32 - 1) / (lane_chunk * 32);   // strides of one warp alone
  int rpw, ksplit;
  const int64_t target_groups = (int64_t)ctx->sm_count * 16;   // warps' worth of row groups for a full machine
  // measured on B200 (Q8_0, batch 1): 4 rows per warp wins from N = 5120 up (it shares each activation
  // load between 4 rows); K is split over the warps of a CTA until the launch has a machine's worth of warps
  if (units >= 2048) rpw = 4;
  else if (units >= 512) rpw = 2;
  else rpw = (a.epilogue == EPI_SWIGLU || a.epilogue == EPI_QKV_ROPE) ? 2 : 1;
  if (nb >= 4 && rpw == 4) rpw = 2;
  {
    const int upg = (a.epilogue == EPI_SWIGLU) ? rpw / 2 : rpw;
    const int64_t groups = (units + upg - 1) / upg;
    ksplit = 1;
    while (ksplit < 8 && groups * ksplit * 2 <= target_groups && k_iters_1 >= 2 * ksplit) ksplit *= 2;
    // long rows: let the warps of a CTA share them (more loads in flight per row) while each keeps >= 4 strides
    while (ksplit < 8 && k_iters_1 >= 12 * ksplit && groups * ksplit < 4 * target_groups) ksplit *= 2;
  }
  rpw = env_int("CAI_GEMV_RPW", rpw);
  ksplit = env_int("CAI_GEMV_KSPLIT", ksplit);
  if (rpw != 1 && rpw != 2 && rpw != 4) rpw = 2;
  if ((a.epilogue == EPI_SWIGLU || a.epilogue == EPI_QKV_ROPE) && rpw == 1) rpw = 2;
  if (nb >= 4 && rpw == 4) rpw = 2;
  if (ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) ksplit = 1;
  p.ksplit = ksplit;
  const int units_per_group = (a.epilogue == EPI_SWIGLU) ? rpw / 2 : rpw;
  const int64_t groups = (units + units_per_group - 1) / units_per_group;
  const int64_t ydim = indexed ? a.batch : (a.batch + nb - 1) / nb;
  // activations in shared memory when they fit beside a healthy number of resident CTAs
  const size_t x_bytes = (size_t)nb * (size_t)w->k * 4;
  p.x_in_smem = (x_bytes <= (size_t)env_int("CAI_GEMV_XSMEM", 64 * 1024)) ? 1 : 0;
  const bool ring_ok = w->type != CAI_TYPE_I8ROW && !indexed && nb <= 2 && (w->k % 32) == 0 && (w->sstride % 8) == 0 && ((uintptr_t)w->scales % 16) == 0 &&
                       ((uintptr_t)w->codes % 16) == 0;
  int want = env_int("CAI_GEMV_RING", -1);
  const size_t stage_warp = (size_t)rpw * (512 + lane_chunk * 2);      // ring bytes of one warp and stage
  const int threads = 256;
  const size_t smem_budget = 108 * 1024;         // two CTAs per SM
  const int wpc = threads / 32;
  const int groups_per_cta = wpc / ksplit;
  p.cta_blocks = (groups + groups_per_cta - 1) / groups_per_cta;
  // persistent grid: at most a few CTAs per SM, each walking several row blocks with the activations staged once
  dim3 grid((unsigned)p.cta_blocks, (unsigned)ydim);     // x is cut down to the resident CTA count at launch
  if (a.norm_gain) {
    if (!p.x_in_smem) return cai_fail(ctx, CAI_ERR_UNSUPPORTED, "linear: fused RMSNorm needs the activations to fit in shared memory");
    p.norm_gain = a.norm_gain; p.norm_eps = a.norm_eps;
  }
  size_t smem = (p.x_in_smem ? x_bytes + 32 * sizeof(float) : 0) + (size_t)2 * wpc * rpw * nb * sizeof(float);
  // Ring variant: by default for single-row Q8_0 products, 4 stages when the activations sit in shared memory,
  // 3 when they are read through L1 (K = 27648: deeper rings take the L1 capacity the 108 KB row needs).
  // Measured on B200 against the register prefetch: 5120 x 152064 0.74 -> 0.84 of the copy peak, 5120 x 55296
  // 0.70 -> 0.77, 27648 x 5120 0.55 -> 0.58; slower for 2-row tiles and for Q4_0, which stay on registers.
  // CAI_GEMV_RING=0 turns it off, N >= 2 forces up to N stages on every shape the variant covers (batch tiles of
  // 1 and 2 rows, as many stages as fit). Also measured and not kept: an L2 prefetch of the first row block ahead
  // of the dependency wait (-4 % on the whole 32B step), one 16-warp CTA per SM with the long row staged once
  // (no gain), 9..13-warp CTAs for matrices between one and two 8-warp CTAs per SM (qkv slower, wo equal).
  {
    if (want < 0) want = (nb == 1 && w->type == CAI_TYPE_Q8_0) ? (p.x_in_smem ? 4 : 3) : 0;
    const size_t stage = (size_t)wpc * stage_warp;
    const size_t base = (smem + 15) & ~(size_t)15;
    int depth = 0;
    if (want >= 2 && ring_ok && base + 2 * stage <= smem_budget) {
      depth = (int)((smem_budget - base) / stage);
      if (depth > want) depth = want;
      if (depth > 8) depth = 8;
    }
    if (depth >= 2) { p.ring_depth = depth; p.ring_off = (int)base; smem = base + (size_t)depth * stage; }
  }
  cudaError_t e;
  if (w->type == CAI_TYPE_Q8_0) e = launch_quant_nb<CAI_TYPE_Q8_0>(ctx, p, nb, rpw, grid, threads, smem);
  else if (w->type == CAI_TYPE_I8ROW) e = launch_quant_nb<CAI_TYPE_I8ROW>(ctx, p, nb, rpw, grid, threads, smem);
  else e = launch_quant_nb<CAI_TYPE_Q4_0>(ctx, p, nb, rpw, grid, threads, smem);
  if (e != cudaSuccess) return cai_fail(ctx, CAI_ERR_CUDA, "gemv launch setup -> %s", cudaGetErrorString(e));
  CAI_LAUNCHED(ctx);
  return CAI_OK;
}
